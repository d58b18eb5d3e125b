/**
 * Unary and broadcasting binary kernels, Cast, FusedBatchNorm.
 * Python twin: tfjs_b200/kernels/elementwise.py.
 */
import {broadcast_util, DataType, KernelConfig, KernelFunc, TensorInfo, upcastType,
        util} from '@tensorflow/tfjs-core';

import {CudaBackend} from '../backend_cuda';
import {BINARY_OP, binding, DTYPE, EW, i64, UNARY_OP} from '../binding';
import {Desc, EwOp, PendingConv, PendingDepthwise, PendingEw, PendingTile, Ref} from '../pending';

export function castImpl(backend: CudaBackend, x: TensorInfo, dtype: DataType): TensorInfo {
  if (x.dtype === dtype) return backend.view(x, x.shape);
  const out = backend.makeOutput(x.shape, dtype);
  binding.cast(backend.ctx, DTYPE[x.dtype], DTYPE[dtype], backend.deviceId(x),
               util.sizeFromShape(x.shape), backend.deviceId(out));
  return out;
}

export function unaryImpl(backend: CudaBackend, op: keyof typeof UNARY_OP, x: TensorInfo,
                          p0 = 0, p1 = 0): TensorInfo {
  const xf = x.dtype === 'float32' ? x : castImpl(backend, x, 'float32');
  const out = backend.makeOutput(x.shape, 'float32');
  binding.unary(backend.ctx, UNARY_OP[op], p0, p1, backend.deviceId(xf), util.sizeFromShape(x.shape),
                backend.deviceId(out));
  if (xf !== x) backend.disposeData(xf.dataId);
  return out;
}

export function binaryImpl(backend: CudaBackend, op: keyof typeof BINARY_OP, a: TensorInfo,
                           b: TensorInfo): TensorInfo {
  let dtype = upcastType(a.dtype, b.dtype);
  if (dtype === 'bool') dtype = 'int32';
  if (op === 'RealDiv' || op === 'Prelu') dtype = 'float32';
  const ac = a.dtype === dtype ? a : castImpl(backend, a, dtype);
  const bc = b.dtype === dtype ? b : castImpl(backend, b, dtype);
  const outShape = broadcast_util.assertAndGetBroadcastShape(a.shape, b.shape);
  const rank = outShape.length;
  const pad = (s: number[]) => new Array(rank - s.length).fill(1).concat(s);
  const out = backend.makeOutput(outShape, dtype);
  binding.binary(backend.ctx, BINARY_OP[op], DTYPE[dtype], rank, backend.deviceId(ac), i64(pad(a.shape)),
                 backend.deviceId(bc), i64(pad(b.shape)), backend.deviceId(out), i64(outShape));
  if (ac !== a) backend.disposeData(ac.dataId);
  if (bc !== b) backend.disposeData(bc.dataId);
  return out;
}

/** tfjs-backend-cpu/src/utils/fused_utils.ts:29-49. */
export function applyActivation(backend: CudaBackend, x: TensorInfo, activation: string,
                                prelu?: TensorInfo, alpha = 0.2): TensorInfo {
  switch (activation) {
    case 'linear': return backend.view(x, x.shape);
    case 'relu': return unaryImpl(backend, 'Relu', x);
    case 'relu6': return unaryImpl(backend, 'Relu6', x);
    case 'elu': return unaryImpl(backend, 'Elu', x);
    case 'sigmoid': return unaryImpl(backend, 'Sigmoid', x);
    case 'leakyrelu': return unaryImpl(backend, 'LeakyRelu', x, alpha);
    case 'prelu': return binaryImpl(backend, 'Prelu', x, prelu);
    default: throw new Error(`Activation ${activation} has not been implemented for the CUDA backend.`);
  }
}

// ------------------------------------------------------------ deferred launches --
// Python twin: _fold_activation, _conv_residual, _depthwise_bias, deferred_elementwise and
// _batch_norm_rows in tfjs_b200/kernels/elementwise.py.
const EW_BINARY = ['Add', 'Sub', 'Multiply', 'RealDiv', 'Maximum', 'Minimum', 'SquaredDifference'];
const EW_UNARY = ['Relu', 'Relu6', 'Elu', 'Sigmoid', 'Exp', 'Sqrt', 'Rsqrt', 'Square', 'Tanh', 'Neg',
                  'Erf', 'Abs', 'Log'];
const sameShape = (a: number[], b: number[]) => a.length === b.length && a.every((v, i) => v === b[i]);

/** Relu / Relu6 over a pending convolution become the last step of its epilogue; so do
 * Minimum(6, .) and ClipByValue(., 0, 6) after a Relu, the two ways tfjs-layers spells
 * relu6 (activations.ts:83-89, layers/advanced_activations.ts). */
function foldActivation(backend: CudaBackend, name: string, x: TensorInfo,
                        attrs?: {[k: string]: unknown}, other?: TensorInfo): TensorInfo|null {
  const pend = backend.pendingOf(x);
  if (!(pend instanceof PendingConv || pend instanceof PendingDepthwise) || x.dtype !== 'float32') {
    return null;
  }
  let act: 'relu'|'relu6'|null = null;
  if (name === 'Relu' && pend.act === 'linear') {
    act = 'relu';
  } else if (name === 'Relu6' && pend.act !== 'relu6') {
    act = 'relu6';
  } else if (name === 'ClipByValue' && pend.act !== 'relu6' &&
             attrs!['clipValueMin'] === 0 && attrs!['clipValueMax'] === 6) {
    act = 'relu6';
  } else if (name === 'Minimum' && pend.act === 'relu' && other != null) {
    const six = backend.hostValues(other);
    if (other.dtype === 'float32' && util.sizeFromShape(other.shape) === 1 && six != null &&
        six[0] === 6) {
      act = 'relu6';
    }
  }
  if (act == null) return null;
  return backend.withActivation(x, act, {name, inputShapes: {}, outputShapes: [x.shape]});
}

/** Add of a pending convolution and an equal-shape tensor: the block's shortcut. */
function convResidual(backend: CudaBackend, a: TensorInfo, b: TensorInfo): TensorInfo|null {
  if (a.dtype !== 'float32' || b.dtype !== 'float32' || !sameShape(a.shape, b.shape)) return null;
  for (const [conv, other] of [[a, b], [b, a]]) {
    const pend = backend.pendingOf(conv);
    if (pend instanceof PendingConv && pend.residual == null && pend.act === 'linear') {
      const desc: Desc = {name: 'Add', inputShapes: {b: other.shape}, outputShapes: [a.shape]};
      return backend.defer(a.shape, 'float32', pend.withResidual(other.dataId, desc));
    }
  }
  return null;
}

/** Add of a pending depthwise convolution and a per-channel operand: K.biasAdd. */
function depthwiseBias(backend: CudaBackend, a: TensorInfo, b: TensorInfo): TensorInfo|null {
  for (const [conv, other] of [[a, b], [b, a]]) {
    const pend = backend.pendingOf(conv);
    if (!(pend instanceof PendingDepthwise) || pend.bias != null || pend.act !== 'linear' ||
        other.dtype !== 'float32' || backend.pendingOf(other) != null) {
      continue;
    }
    const channels = conv.shape[conv.shape.length - 1];
    const n = util.sizeFromShape(other.shape);
    const perChannel = n === channels && other.shape.length <= conv.shape.length &&
        other.shape[other.shape.length - 1] === channels;
    if (n !== 1 && !perChannel) continue;
    const desc: Desc = {name: 'Add', inputShapes: {b: other.shape}, outputShapes: [conv.shape]};
    return backend.defer(conv.shape, 'float32',
                         pend.withBias(other.dataId, n === 1 ? 1 : channels, desc));
  }
  return null;
}

function ewOperand(backend: CudaBackend, t: TensorInfo, leaves: object[], leafShapes: number[][],
                   ops: EwOp[], outN: number, budget: number): {ref: Ref, desc: Desc[]|null} {
  const pend = backend.pendingOf(t);
  if (pend instanceof PendingEw && util.sizeFromShape(pend.shape) === outN &&
      (pend.consumed === 0 || pend.cheap()) && ops.length + pend.ops.length <= budget &&
      new Set([...leaves, ...pend.leaves]).size <= EW.MAX_INPUTS) {
    const remap = pend.leaves.map((leaf, k) => {
      if (!leaves.includes(leaf)) {
        leaves.push(leaf);
        leafShapes.push(pend.leafShapes[k]);
      }
      return leaves.indexOf(leaf);
    });
    const base = ops.length;
    const ref = (r: Ref): Ref => r[0] === 'in' ? ['in', remap[r[1]]] : ['op', base + r[1]];
    for (const [code, a, b] of pend.ops) ops.push([code, ref(a), ref(b)]);
    pend.consumed++;
    return {ref: ['op', ops.length - 1], desc: pend.desc};
  }
  if (!leaves.includes(t.dataId)) {
    leaves.push(t.dataId);
    leafShapes.push(t.shape);
  }
  return {ref: ['in', leaves.indexOf(t.dataId)], desc: null};
}

/** The float32 kernel `name` as a deferred launch joined to the pending chains of its
 * operands; null when it has to run at once. */
function deferredElementwise(backend: CudaBackend, name: string, a: TensorInfo,
                             b?: TensorInfo): TensorInfo|null {
  if (!backend.lazyFusion || a.dtype !== 'float32' || (b != null && b.dtype !== 'float32')) return null;
  const outShape = b == null ? a.shape : broadcast_util.assertAndGetBroadcastShape(a.shape, b.shape);
  const n = util.sizeFromShape(outShape);
  if (n === 0 || outShape.length > 6) return null;
  let depth = 1;
  for (const t of [a, b]) {
    const pend = t != null ? backend.pendingOf(t) : undefined;
    if (pend instanceof PendingEw) {
      if (pend.depth >= 32) backend.deviceId(t);     // keep the recursion of launches shallow
      else depth = Math.max(depth, pend.depth + 1);
    }
  }
  const leaves: object[] = [], leafShapes: number[][] = [], ops: EwOp[] = [];
  const budget = EW.MAX_OPS - 2;
  const ra = ewOperand(backend, a, leaves, leafShapes, ops, n, budget);
  const rb = b == null ? ra : ewOperand(backend, b, leaves, leafShapes, ops, n, budget);
  if (leaves.length > EW.MAX_INPUTS) return null;
  const code = b != null ? BINARY_OP[name as keyof typeof BINARY_OP] :
                           EW.UNARY + UNARY_OP[name as keyof typeof UNARY_OP];
  ops.push([code, ra.ref, rb.ref]);
  const descs: Desc[] = [...(ra.desc ?? []), ...(b != null ? rb.desc ?? [] : [])];
  const inputShapes: {[k: string]: number[]} = {};
  if (ra.ref[0] === 'in') inputShapes[b != null ? 'a' : 'x'] = a.shape;
  if (b != null && rb.ref[0] === 'in' && rb.ref[1] !== ra.ref[1]) inputShapes['b'] = b.shape;
  descs.push({name, inputShapes, outputShapes: [outShape]});
  return backend.defer(outShape, 'float32', new PendingEw(
      leaves, leafShapes, ops, outShape, descs,
      {code, a: a.dataId, aShape: a.shape, b: b != null ? b.dataId : null,
       bShape: b != null ? b.shape : null}, depth));
}

function unaryKernel(backend: CudaBackend, name: keyof typeof UNARY_OP, x: TensorInfo,
                     attrs: {[k: string]: unknown}, p0 = 0, p1 = 0): TensorInfo {
  if (x.dtype === 'float32' && backend.lazyFusion) {
    if (name === 'Relu' || name === 'Relu6' || name === 'ClipByValue') {
      const folded = foldActivation(backend, name, x, attrs);
      if (folded != null) return folded;
    }
    if (EW_UNARY.includes(name)) {
      const out = deferredElementwise(backend, name, x);
      if (out != null) return out;
    }
  }
  return unaryImpl(backend, name, x, p0, p1);
}

function binaryKernel(backend: CudaBackend, name: keyof typeof BINARY_OP, a: TensorInfo,
                      b: TensorInfo): TensorInfo {
  if (backend.lazyFusion) {
    let out: TensorInfo|null = null;
    if (name === 'Add') out = convResidual(backend, a, b) ?? depthwiseBias(backend, a, b);
    if (name === 'Minimum') {
      out = foldActivation(backend, name, a, undefined, b) ?? foldActivation(backend, name, b, undefined, a);
    }
    if (out == null && EW_BINARY.includes(name)) out = deferredElementwise(backend, name, a, b);
    if (out != null) return out;
  }
  return binaryImpl(backend, name, a, b);
}

/** FusedBatchNorm whose parameters are pending Tiles of rows / columns of x: tfjs-layers'
 * LayerNormalization (layers/normalization.ts:578-622).  The kernel indexes the untiled
 * tensors and the tiles are never made; null when the parameters are not of that form. */
function batchNormRows(backend: CudaBackend, x: TensorInfo, params: Array<TensorInfo|undefined>,
                       eps: number): TensorInfo|null {
  if (x.dtype !== 'float32' || x.shape.length < 1 || util.sizeFromShape(x.shape) === 0) return null;
  const rank = x.shape.length, cols = x.shape[rank - 1];
  const rows = util.sizeFromShape(x.shape) / cols;
  const rowShape = [...x.shape.slice(0, -1), 1];
  const colShape = [...new Array(rank - 1).fill(1), cols];
  const ids: Array<object|null> = [], modes: number[] = [];
  let anyTile = false;
  for (const t of params) {
    if (t == null) { ids.push(null); modes.push(0); continue; }
    if (t.dtype !== 'float32') return null;
    const pend = backend.pendingOf(t);
    let src = t.dataId, shape = t.shape;
    if (pend instanceof PendingTile && sameShape(pend.shape, x.shape)) {
      src = pend.src; shape = pend.srcShape; anyTile = true;
    } else if (pend != null) {
      return null;
    }
    if (shape.length > rank) return null;
    const padded = [...new Array(rank - shape.length).fill(1), ...shape];
    const mode = util.sizeFromShape(shape) === 1 ? 4 : sameShape(padded, x.shape) ? 3 :
        sameShape(padded, rowShape) ? 2 : sameShape(padded, colShape) ? 1 : -1;
    if (mode < 0) return null;
    ids.push(src);
    modes.push(mode);
  }
  if (!anyTile) return null;
  const out = backend.makeOutput(x.shape, 'float32');
  const d = ids.map(i => i != null ? backend.deviceIdOf(i) : 0);
  binding.batchNormRows(backend.ctx, backend.deviceId(x), rows, cols, d[0], modes[0], d[1], modes[1],
                        d[2], modes[2], d[3], modes[3], eps, backend.deviceId(out));
  return out;
}

type Args = {inputs: {[k: string]: TensorInfo}, attrs: {[k: string]: unknown}, backend: CudaBackend};
const asFunc = (f: (a: Args) => TensorInfo) => f as unknown as KernelFunc;

const unaryNames: Array<keyof typeof UNARY_OP> =
    ['Relu', 'Relu6', 'Elu', 'Sigmoid', 'Exp', 'Sqrt', 'Rsqrt', 'Square', 'Tanh', 'Neg', 'Erf', 'Abs', 'Log'];
const binaryNames: Array<keyof typeof BINARY_OP> =
    ['Add', 'Sub', 'Multiply', 'RealDiv', 'Maximum', 'Minimum', 'Pow', 'SquaredDifference'];

export const elementwiseConfigs: KernelConfig[] = [
  ...unaryNames.map(name => ({kernelName: name, backendName: 'cuda',
      kernelFunc: asFunc(({inputs, attrs, backend}) => unaryKernel(backend, name, inputs['x'], attrs))})),
  {kernelName: 'LeakyRelu', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) =>
      unaryImpl(backend, 'LeakyRelu', inputs['x'], (attrs['alpha'] as number) ?? 0.2))},
  {kernelName: 'ClipByValue', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) =>
      unaryKernel(backend, 'ClipByValue', inputs['x'], attrs, attrs['clipValueMin'] as number,
                  attrs['clipValueMax'] as number))},
  ...binaryNames.map(name => ({kernelName: name, backendName: 'cuda',
      kernelFunc: asFunc(({inputs, backend}) => binaryKernel(backend, name, inputs['a'], inputs['b']))})),
  {kernelName: 'Prelu', backendName: 'cuda', kernelFunc: asFunc(({inputs, backend}) =>
      binaryImpl(backend, 'Prelu', inputs['x'], inputs['alpha']))},
  {kernelName: 'Cast', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) =>
      castImpl(backend, inputs['x'], attrs['dtype'] as DataType))},
  {kernelName: 'FusedBatchNorm', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const {x, mean, variance, scale, offset} = inputs;
    const eps = (attrs['varianceEpsilon'] as number) ?? 0.001;
    const rowsForm = batchNormRows(backend, x, [mean, variance, scale, offset], eps);
    if (rowsForm != null) return rowsForm;
    const n = (t?: TensorInfo) => t == null ? 0 : util.sizeFromShape(t.shape);
    const out = backend.makeOutput(x.shape, 'float32');
    binding.batchNorm(backend.ctx, backend.deviceId(x), n(x), backend.deviceId(mean), n(mean),
                      backend.deviceId(variance), n(variance), backend.deviceId(scale), n(scale),
                      backend.deviceId(offset), n(offset), (attrs['varianceEpsilon'] as number) ?? 0.001,
                      backend.deviceId(out));
    return out;
  })},
];
