/** Registers the backend on import, like tfjs-backend-cpu/src/base.ts does for 'cpu'. */
import {registerBackend} from '@tensorflow/tfjs-core';
import {CudaBackend} from './backend_cuda';

registerBackend(
    'cuda',
    () => new CudaBackend(Number(process.env['TFJS_CUDA_DEVICE_ORDINAL'] ?? 0)),
    3 /* above webgl's 2 */);

export {CudaBackend};
