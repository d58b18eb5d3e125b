import './base';
import './register_all_kernels';
export {CudaBackend} from './backend_cuda';
export {CudaGraphModel, loadGraphModelCuda} from './graph_model_cuda';
export {registerGraphOps, rewriteArtifacts} from './graph_rewrites';
export {cudaIO, loadWeightFiles} from './io_cuda';
