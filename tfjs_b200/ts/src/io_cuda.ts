/**
 * An `io` namespace whose decodeWeights leaves uint8 / uint16 affine-quantised
 * weights quantised across PCIe and dequantises them on the GPU, once, at load.
 * GraphModel takes the io namespace as a constructor argument and calls
 * `this.io.decodeWeights` (tfjs-converter/src/executor/graph_model.ts:104-107, :177):
 *
 *     const model = await tf.loadGraphModel(url, {}, cudaIO);
 *
 * Python twin: tfjs_b200/io.py.
 */
import {engine, io, NamedTensorMap, Tensor, util} from '@tensorflow/tfjs-core';

import {CudaBackend} from './backend_cuda';
import {binding, DTYPE} from './binding';

function decodeWeights(weightData: io.WeightData, specs: io.WeightsManifestEntry[]): NamedTensorMap {
  const buffer = weightData instanceof ArrayBuffer ? weightData : io.concatenateArrayBuffers(weightData as ArrayBuffer[]);
  const backend = engine().backend as CudaBackend;
  const out: NamedTensorMap = {};
  let offset = 0;
  for (const spec of specs) {
    const size = util.sizeFromShape(spec.shape);
    const q = spec.quantization;
    if (q != null && (q.dtype === 'uint8' || q.dtype === 'uint16')) {
      if (q.min == null || q.scale == null) {
        throw new Error(`Weight ${spec.name} with quantization ${q.dtype} ` +
                        `doesn't have corresponding metadata min and scale.`);
      }
      const qBytes = q.dtype === 'uint8' ? 1 : 2;
      const nbytes = size * qBytes;
      const qId = binding.alloc(backend.ctx, nbytes);
      binding.write(backend.ctx, qId, new Uint8Array(buffer, offset, nbytes), nbytes);
      const info = backend.makeOutput(spec.shape, spec.dtype as 'float32' | 'int32');
      binding.dequantize(backend.ctx, qBytes, DTYPE[spec.dtype], qId, q.scale, q.min, size,
                         backend.deviceId(info));
      binding.free(backend.ctx, qId);
      out[spec.name] = engine().makeTensorFromTensorInfo(info) as Tensor;
      offset += nbytes;
    } else if (q != null && q.dtype === 'float16' && spec.dtype === 'float32') {
      // half-precision storage: upload the raw bits, widen on the device
      const nbytes = size * 2;
      const qId = binding.alloc(backend.ctx, nbytes);
      binding.write(backend.ctx, qId, new Uint8Array(buffer, offset, nbytes), nbytes);
      const info = backend.makeOutput(spec.shape, 'float32');
      binding.decodeFloat16(backend.ctx, qId, size, backend.deviceId(info));
      binding.free(backend.ctx, qId);
      out[spec.name] = engine().makeTensorFromTensorInfo(info) as Tensor;
      offset += nbytes;
    } else {
      // unquantised entries: the stock decoder, one entry at a time
      const bytes = size * (q != null ? 2 : (spec.dtype === 'bool' ? 1 : 4));
      Object.assign(out, io.decodeWeights(buffer.slice(offset, offset + bytes), [spec]));
      offset += bytes;
    }
  }
  return out;
}

export const cudaIO = {...io, decodeWeights};
