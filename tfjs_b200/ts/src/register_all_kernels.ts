/** Registers every kernel of the 'cuda' backend (cf. tfjs-backend-cpu/src/register_all_kernels.ts). */
import {registerKernel} from '@tensorflow/tfjs-core';

import {convConfigs} from './kernels/conv';
import {elementwiseConfigs} from './kernels/elementwise';
import {fusedGraphOpConfigs} from './kernels/fused_graph_ops';
import {matMulConfigs} from './kernels/matmul';
import {otherConfigs} from './kernels/pool_reduce_movement';

for (const config of [...convConfigs, ...matMulConfigs, ...elementwiseConfigs, ...otherConfigs,
                      ...fusedGraphOpConfigs]) {
  registerKernel(config);
}
