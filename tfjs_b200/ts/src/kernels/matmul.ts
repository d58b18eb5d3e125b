/** _FusedMatMul and BatchMatMul.  Python twin: tfjs_b200/kernels/matmul.py. */
import {_FusedMatMul, BatchMatMul, broadcast_util, KernelConfig, KernelFunc, TensorInfo,
        util} from '@tensorflow/tfjs-core';

import {CudaBackend} from '../backend_cuda';
import {ACTIVATION, binding, packMatMulParams} from '../binding';
import {PendingMatMul} from '../pending';
import {perChannelLen} from './conv';
import {applyActivation, binaryImpl} from './elementwise';

/**
 * Deferred: products that share `a` and these dimensions launch as one group when the first
 * of them is needed (the Q, K and V projections of an attention layer); null when this
 * product does not qualify (batched operands, a transposed `a`, narrow outputs, PReLU, a bias
 * that is not one value per column).
 */
export function deferMatMul(
    backend: CudaBackend, a: TensorInfo, b: TensorInfo, bias: TensorInfo|undefined, activation: string,
    alpha: number, transposeA: boolean, transposeB: boolean, batchA: number, batchB: number, m: number,
    n: number, k: number, biasLen: number|null, heads: [number, number, number]|null,
    outShape: number[]): TensorInfo|null {
  if (!(backend.lazyFusion && backend.groupMatMuls && biasLen != null && batchA === 1 && batchB === 1 &&
        !transposeA && k % 4 === 0 && n > 128 && activation !== 'prelu' &&
        (bias == null || biasLen === n) &&
        // a heads-permuted store the library may decline is refused at the call, where the
        // node executor can still fall back to product + Reshape + Transpose
        (heads == null || (heads[0] === 1 && backend.mathMode === 'tf32' && heads[1] % 32 === 0 &&
                           heads[2] % 32 === 0)) &&
        util.sizeFromShape(outShape) > 0)) {
    return null;
  }
  const inputShapes: {[key: string]: number[]} = {a: a.shape, b: b.shape};
  if (bias != null) inputShapes['bias'] = bias.shape;
  const desc = {name: heads == null ? _FusedMatMul : '_MatMulHeads', inputShapes, outputShapes: [outShape]};
  return backend.defer(outShape, 'float32', new PendingMatMul(
      packMatMulParams(1, 1, m, n, k, false, transposeB, ACTIVATION[activation], biasLen, 0, alpha),
      a.dataId, b.dataId, bias != null ? bias.dataId : null, heads, [desc]));
}

function matMulImpl(
    backend: CudaBackend, a: TensorInfo, b: TensorInfo, transposeA: boolean, transposeB: boolean,
    bias?: TensorInfo, prelu?: TensorInfo, activation = 'linear', alpha = 0.2,
    gelu?: [number, number, number, boolean]): TensorInfo {
  const ar = a.shape.length, br = b.shape.length;
  const innerA = transposeA ? a.shape[ar - 2] : a.shape[ar - 1];
  const innerB = transposeB ? b.shape[br - 1] : b.shape[br - 2];
  const outerA = transposeA ? a.shape[ar - 1] : a.shape[ar - 2];
  const outerB = transposeB ? b.shape[br - 2] : b.shape[br - 1];
  util.assert(innerA === innerB, () =>
      `Error in matMul: inner shapes (${innerA}) and (${innerB}) of Tensors with shapes ` +
      `${a.shape} and ${b.shape} and transposeA=${transposeA} and transposeB=${transposeB} must match.`);
  const batchA = util.sizeFromShape(a.shape.slice(0, -2));
  const batchB = util.sizeFromShape(b.shape.slice(0, -2));
  const outShape = broadcast_util.assertAndGetBroadcastShape(a.shape.slice(0, -2), b.shape.slice(0, -2))
                       .concat([outerA, outerB]);
  const biasLen = perChannelLen(bias, outerB);
  const preluLen = activation === 'prelu' ? perChannelLen(prelu, outerB) : 0;
  const fuseBias = biasLen != null;
  const fuseAct = fuseBias && (activation !== 'prelu' || preluLen != null);
  if (activation === 'gelu_erf' && !(fuseAct && gelu != null)) {
    // only exists as a fused epilogue (graph_rewrites.fuseGeluIntoMatMul)
    throw new Error('matMul: gelu_erf needs a fusable bias');
  }
  const deferred = activation === 'gelu_erf' ? null : deferMatMul(backend, a, b, bias, activation, alpha, transposeA, transposeB,
                               batchA, batchB, outerA, outerB, innerA, fuseBias && fuseAct ? biasLen : null,
                               null, outShape);
  if (deferred != null) return deferred;
  let out = backend.makeOutput(outShape, 'float32');
  if (util.sizeFromShape(outShape) > 0) {
    binding.fusedMatMul(
        backend.ctx,
        packMatMulParams(batchA, batchB, outerA, outerB, innerA, transposeA, transposeB,
                         ACTIVATION[fuseAct ? activation : 'linear'], fuseBias ? biasLen : 0,
                         fuseAct ? (preluLen ?? 0) : 0, alpha, activation === 'gelu_erf' ? gelu : undefined),
        backend.deviceId(a), backend.deviceId(b), fuseBias ? backend.deviceId(bias) : 0,
        fuseAct && activation === 'prelu' ? backend.deviceId(prelu) : 0, backend.deviceId(out));
  }
  if (!fuseBias) {
    const added = binaryImpl(backend, 'Add', out, bias);
    backend.disposeData(out.dataId);
    out = added;
  }
  if (!fuseAct) {
    const act = applyActivation(backend, out, activation, prelu, alpha);
    backend.disposeData(out.dataId);
    out = act;
  }
  return out;
}

type Args = {inputs: {[k: string]: TensorInfo}, attrs: {[k: string]: unknown}, backend: CudaBackend};

export const matMulConfigs: KernelConfig[] = [
  {kernelName: _FusedMatMul, backendName: 'cuda',
   kernelFunc: (({inputs, attrs, backend}: Args) => matMulImpl(
       backend, inputs['a'], inputs['b'], !!attrs['transposeA'], !!attrs['transposeB'], inputs['bias'],
       inputs['preluActivationWeights'], (attrs['activation'] as string) ?? 'linear',
       (attrs['leakyreluAlpha'] as number) ?? 0.2,
       attrs['geluParams'] as [number, number, number, boolean]|undefined)) as unknown as KernelFunc},
  {kernelName: BatchMatMul, backendName: 'cuda',
   kernelFunc: (({inputs, attrs, backend}: Args) => matMulImpl(
       backend, inputs['a'], inputs['b'], !!attrs['transposeA'], !!attrs['transposeB'])) as unknown as KernelFunc},
];
