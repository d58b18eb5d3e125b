import './base';
import './register_all_kernels';
export {CudaBackend} from './backend_cuda';
export {cudaIO} from './io_cuda';
