/**
 * Runs tfjs-core's own op suites against the 'cuda' backend, the way
 * tfjs-backend-wasm/src/setup_test.ts does for 'wasm': register a test env and
 * filter the shared suites down to what this backend implements.
 */
import './index';
// tslint:disable-next-line:no-imports-from-dist
import {setTestEnvs, setupTestFilters, TestFilter} from '@tensorflow/tfjs-core/dist/jasmine_util';

setTestEnvs([{name: 'cuda', backendName: 'cuda', isDataSync: true}]);

const excludes = ['gradient', 'derivative', 'complex', 'string', 'NCHW', 'throws when'];
const suites = [
  'fused conv2d', 'fused matmul', 'fused depthwiseConv2D', 'matmul ', 'matmulBatch', 'conv2d ',
  'depthwiseConv2D ', 'maxPool ', 'avgPool ', 'softmax', 'gather ', 'argmax ', 'mean ', 'sum ',
  'max ', 'add ', 'sub ', 'mul ', 'div ', 'relu', 'relu6', 'elu', 'sigmoid', 'leakyrelu', 'prelu',
  'erf', 'exp ', 'sqrt', 'rsqrt', 'square', 'tanh', 'neg ', 'clipByValue', 'transpose', 'concat1d',
  'concat2d', 'concat3d', 'concat4d', 'slice ', 'pad1d', 'pad2d', 'pad3d', 'pad4d', 'tile ',
  'batchNorm2D', 'batchNorm3D', 'batchNorm4D', 'cast'
];
const filters: TestFilter[] = suites.map(startsWith => ({startsWith, excludes}));
setupTestFilters(filters, () => false);
