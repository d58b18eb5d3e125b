/**
 * Kernels behind the three plan rewrites of graph_rewrites.ts, plus Pack:
 *   _FusedLayerNorm       the nine-node layer normalisation of a converted graph (ten with
 *                         the residual Add in front) in one launch
 *   _MatMulHeads          matMul whose result is stored through the permutation that splits
 *                         or merges attention heads
 *   _SoftmaxScaledMasked  softmax(x * scale + mask)
 *   _FusedAttention       softmax(q k^T * scale + mask) v with the heads merged
 * Python twins: _fused_layer_norm / _softmax_scaled_masked in tfjs_b200/kernels/reduce.py,
 * matmul_heads in tfjs_b200/kernels/matmul.py, _pack in movement.py.
 */
import {KernelConfig, KernelFunc, TensorInfo, util} from '@tensorflow/tfjs-core';

import {CudaBackend} from '../backend_cuda';
import {ACTIVATION, binding, packMatMulParams} from '../binding';
import {perChannelLen} from './conv';
import {deferMatMul} from './matmul';

type Args = {inputs: {[k: string]: TensorInfo}, attrs: {[k: string]: unknown}, backend: CudaBackend};
const asFunc = (f: (a: Args) => TensorInfo) => f as unknown as KernelFunc;

/** Shapes the one-launch layer normalisation takes: rows of a multiple of 4 floats, at most
 * 1024, gamma and beta one value per column. */
export function layerNormSupported(x: number[], gamma: number[], beta: number[]): boolean {
  if (x.length === 0) return false;
  const cols = x[x.length - 1];
  const perCol = (s: number[]) => util.sizeFromShape(s) === cols && (s.length === 0 || s[s.length - 1] === cols);
  return cols % 4 === 0 && cols > 0 && cols <= 1024 && perCol(gamma) && perCol(beta);
}

/** rows_per_mask for a mask that broadcasts against x over whole rows, else null. */
export function softmaxMaskRows(x: number[], mask: number[]): number|null {
  const rank = x.length;
  if (mask.length > rank || rank === 0) return null;
  const m = [...new Array(rank - mask.length).fill(1), ...mask];
  if (m[rank - 1] !== x[rank - 1]) return null;
  let lead = 0;
  while (lead < rank - 1 && m[lead] === x[lead]) ++lead;
  if (m.slice(lead, rank - 1).some(d => d !== 1)) return null;
  return Math.max(util.sizeFromShape(x.slice(lead, rank - 1)), 1);
}

export class UnsupportedByLibrary extends Error {}

export const fusedGraphOpConfigs: KernelConfig[] = [
  {kernelName: '_FusedLayerNorm', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const {x, gamma, beta, residual} = inputs;
    if (!layerNormSupported(x.shape, gamma.shape, beta.shape)) {
      throw new Error(`_FusedLayerNorm: unsupported shapes ${x.shape} ${gamma.shape} ${beta.shape}`);
    }
    const cols = x.shape[x.shape.length - 1];
    const out = backend.makeOutput(x.shape, 'float32');
    binding.layerNorm(backend.ctx, backend.deviceId(x), backend.deviceId(residual),
                      backend.deviceId(gamma), backend.deviceId(beta),
                      util.sizeFromShape(x.shape) / cols, cols, Math.fround(attrs['epsilon'] as number),
                      backend.deviceId(out));
    return out;
  })},
  {kernelName: '_SoftmaxScaledMasked', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const x = inputs['logits'], mask = inputs['mask'];
    const scale = attrs['scale'] as number|undefined;
    const cols = x.shape[x.shape.length - 1];
    let rowsPerMask = 1;
    if (mask != null) {
      const rpm = softmaxMaskRows(x.shape, mask.shape);
      if (rpm == null || mask.dtype !== 'float32') {
        throw new Error(`_SoftmaxScaledMasked: mask ${mask.shape} does not broadcast over rows of ${x.shape}`);
      }
      rowsPerMask = rpm;
    }
    const out = backend.makeOutput(x.shape, 'float32');
    binding.softmaxScaledMasked(backend.ctx, backend.deviceId(x), util.sizeFromShape(x.shape) / cols, cols,
                                scale != null ? 1 : 0, Math.fround(scale ?? 1), backend.deviceId(mask),
                                rowsPerMask, backend.deviceId(out));
    return out;
  })},
  {kernelName: '_FusedAttention', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    // softmax(q k^T * scale + mask) v for q, k, v of shape [B, H, S, D], stored [B, S, H, D]
    const {q, k, v, mask} = inputs;
    const scale = attrs['scale'] as number|undefined;
    const same = (a: number[], b: number[]) => a.length === b.length && a.every((d, i) => d === b[i]);
    if (q.shape.length !== 4 || !same(k.shape, q.shape) || !same(v.shape, q.shape) ||
        [q, k, v].some(t => t.dtype !== 'float32')) {
      throw new UnsupportedByLibrary('_FusedAttention: q, k, v of one 4-D shape');
    }
    const [B, H, S, D] = q.shape;
    let unitsPerMask = 1;
    if (mask != null) {
      const rpm = mask.dtype === 'float32' ? softmaxMaskRows([B, H, S, S], mask.shape) : null;
      if (rpm == null || rpm % S !== 0) {
        throw new UnsupportedByLibrary(`_FusedAttention: mask ${mask.shape} is not one row per head`);
      }
      unitsPerMask = rpm / S;
    }
    const out = backend.makeOutput([B, S, H, D], 'float32');
    let taken = false;
    try {
      taken = binding.fusedAttention(backend.ctx, backend.deviceId(q), backend.deviceId(k), backend.deviceId(v),
                                     backend.deviceId(mask), scale != null ? 1 : 0, Math.fround(scale ?? 1),
                                     B, H, S, D, unitsPerMask, backend.deviceId(out));
    } finally {
      if (!taken) backend.disposeData(out.dataId);
    }
    if (!taken) throw new UnsupportedByLibrary('_FusedAttention: shape not taken by the library');
    return out;
  })},
  {kernelName: '_MatMulHeads', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const {a, b, bias} = inputs;
    const [B, S, H, D] = attrs['heads'] as number[];
    const ta = !!attrs['transposeA'], tb = !!attrs['transposeB'];
    const ar = a.shape.length, br = b.shape.length;
    const m = ta ? a.shape[ar - 1] : a.shape[ar - 2], k = ta ? a.shape[ar - 2] : a.shape[ar - 1];
    const n = tb ? b.shape[br - 2] : b.shape[br - 1];
    const batchA = util.sizeFromShape(a.shape.slice(0, -2)), batchB = util.sizeFromShape(b.shape.slice(0, -2));
    const split = attrs['layout'] === 'split';
    const ok = split ? batchA === 1 && batchB === 1 && m === B * S && n === H * D :
                       batchA === B * H && batchB === B * H && m === S && n === D;
    if (!ok) throw new UnsupportedByLibrary(`matMul heads: ${a.shape} x ${b.shape} do not give ${[B, S, H, D]}`);
    const biasLen = perChannelLen(bias, n);
    if (biasLen == null) throw new UnsupportedByLibrary('matMul heads: bias shape');
    const outShape = split ? [B, H, S, D] : [B, S, H, D];
    const activation = (attrs['activation'] as string) ?? 'linear';
    const deferred = deferMatMul(backend, a, b, bias, activation, 0.2, ta, tb, batchA, batchB, m, n, k,
                                 biasLen, [split ? 1 : 2, split ? S : H, D], outShape);
    if (deferred != null) return deferred;
    const out = backend.makeOutput(outShape, 'float32');
    try {
      binding.fusedMatMulHeads(
          backend.ctx,
          packMatMulParams(batchA, batchB, m, n, k, ta, tb, ACTIVATION[(attrs['activation'] as string) ?? 'linear'],
                           biasLen, 0),
          backend.deviceId(a), backend.deviceId(b), backend.deviceId(bias), 0, split ? 1 : 2,
          split ? S : H, D, backend.deviceId(out));
    } catch (e) {
      backend.disposeData(out.dataId);
      throw e;     // TFJS_CUDA_UNSUPPORTED: the node executor runs product, Reshape, Transpose
    }
    return out;
  })},
  {kernelName: 'Pack', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    // Pack.ts: expandDims each input along `axis`, then concat
    const tensors = Object.keys(inputs).sort((p, q) => Number(p) - Number(q)).map(key => inputs[key]);
    let axis = (attrs['axis'] as number) ?? 0;
    const shape = [...tensors[0].shape];
    if (axis < 0) axis += shape.length + 1;
    shape.splice(axis, 0, 1);
    const outShape = [...shape];
    outShape[axis] = tensors.length;
    const out = backend.makeOutput(outShape, tensors[0].dtype);
    const strides = (s: number[]) => s.map((_, i) => util.sizeFromShape(s.slice(i + 1)));
    const i64 = (v: number[]) => BigInt64Array.from((v.length ? v : [0]).map(x => BigInt(x)));
    const os = strides(outShape);
    tensors.forEach((t, pos) => {
      if (util.sizeFromShape(shape) > 0) {
        binding.copyStrided(backend.ctx, t.dtype === 'bool' ? 1 : 4, shape.length, i64(shape),
                            backend.deviceId(t), 0, i64(strides(shape)), i64(shape), backend.deviceId(out),
                            pos * os[axis], i64(os));
      }
    });
    return out;
  })},
];
