/**
 * MaxPool, AvgPool, Softmax, Sum, Mean, Max, ArgMax, Reshape, Identity, ExpandDims,
 * Transpose, GatherV2, Concat, Slice, PadV2, Tile.
 * Python twins: tfjs_b200/kernels/pool.py, reduce.py, movement.py.
 */
import {backend_util, KernelConfig, KernelFunc, slice_util, TensorInfo, util} from '@tensorflow/tfjs-core';

import {CudaBackend} from '../backend_cuda';
import {binding, i64, packConvParams, REDUCE_OP} from '../binding';
import {PendingTile} from '../pending';
import {castImpl} from './elementwise';

type Args = {inputs: {[k: string]: TensorInfo}, attrs: {[k: string]: unknown}, backend: CudaBackend};
const asFunc = (f: (a: Args) => TensorInfo) => f as unknown as KernelFunc;
const elemBytes = (t: TensorInfo) => t.dtype === 'bool' ? 1 : 4;

function pool(isMax: boolean) {
  return asFunc(({inputs, attrs, backend}) => {
    const x = inputs['x'];
    const ci = backend_util.computePool2DInfo(
        x.shape as [number, number, number, number], attrs['filterSize'] as number,
        attrs['strides'] as number, 1, attrs['pad'] as 'same' | 'valid',
        attrs['dimRoundingMode'] as 'floor');
    if (ci.filterWidth === 1 && ci.filterHeight === 1 && util.arraysEqual(ci.inShape, ci.outShape)) {
      return backend.view(x, x.shape);
    }
    const out = backend.makeOutput(ci.outShape, 'float32');
    binding.pool2d(backend.ctx,
                   packConvParams({...ci, outChannels: ci.inChannels}, 0, 0, 0, 0.2, true,
                                  [ci.effectiveFilterHeight, ci.effectiveFilterWidth]),
                   isMax ? 1 : 0, backend.deviceId(x), backend.deviceId(out));
    return out;
  });
}

export function transposeImpl(backend: CudaBackend, x: TensorInfo, perm: number[]): TensorInfo {
  const out = backend.makeOutput(perm.map(p => x.shape[p]), x.dtype);
  binding.transpose(backend.ctx, elemBytes(x), x.shape.length, backend.deviceId(x), i64(x.shape),
                    Int32Array.from(perm), backend.deviceId(out));
  return out;
}

function reduce(op: keyof typeof REDUCE_OP, axisAttr: string) {
  return asFunc(({inputs, attrs, backend}) => {
    let x = inputs['x'];
    const tmp: TensorInfo[] = [];
    if (x.dtype !== 'float32') { x = castImpl(backend, x, 'float32'); tmp.push(x); }
    let axes = util.parseAxisParam(attrs[axisAttr] as number[], x.shape).sort((a, b) => a - b);
    const [outShape] = backend_util.computeOutAndReduceShapes(x.shape, axes);
    const contiguous = axes.every((a, i) => i === 0 || a === axes[i - 1] + 1);
    if (!contiguous) {
      x = transposeImpl(backend, x, backend_util.getAxesPermutation(axes, x.shape.length));
      tmp.push(x);
      axes = backend_util.getInnerMostAxes(axes.length, x.shape.length);
    }
    const outer = util.sizeFromShape(x.shape.slice(0, axes[0]));
    const red = util.sizeFromShape(x.shape.slice(axes[0], axes[axes.length - 1] + 1));
    const inner = util.sizeFromShape(x.shape.slice(axes[axes.length - 1] + 1));
    const shape = attrs['keepDims'] ? backend_util.expandShapeToKeepDim(outShape, axes) : outShape;
    const out = backend.makeOutput(shape, 'float32');
    binding.reduce(backend.ctx, REDUCE_OP[op], backend.deviceId(x), outer, red, inner, backend.deviceId(out));
    tmp.forEach(t => backend.disposeData(t.dataId));
    return out;
  });
}

function copyStrided(backend: CudaBackend, x: TensorInfo, xOff: number, out: TensorInfo, oOff: number,
                     oStrides: number[], extent: number[]) {
  const full = (s: number[]) => s.map((_, i) => util.sizeFromShape(s.slice(i + 1)));
  binding.copyStrided(backend.ctx, elemBytes(x), extent.length, i64(extent), backend.deviceId(x), xOff,
                      i64(full(x.shape)), i64(x.shape), backend.deviceId(out), oOff, i64(oStrides));
}
const strides = (s: number[]) => s.map((_, i) => util.sizeFromShape(s.slice(i + 1)));

export const otherConfigs: KernelConfig[] = [
  {kernelName: 'MaxPool', backendName: 'cuda', kernelFunc: pool(true)},
  {kernelName: 'AvgPool', backendName: 'cuda', kernelFunc: pool(false)},
  {kernelName: 'Sum', backendName: 'cuda', kernelFunc: reduce('Sum', 'axis')},
  {kernelName: 'Mean', backendName: 'cuda', kernelFunc: reduce('Mean', 'axis')},
  {kernelName: 'Max', backendName: 'cuda', kernelFunc: reduce('Max', 'reductionIndices')},
  {kernelName: 'ArgMax', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const x = inputs['x'];
    const axis = util.parseAxisParam(attrs['axis'] as number, x.shape)[0];
    const [outShape] = backend_util.computeOutAndReduceShapes(x.shape, [axis]);
    const out = backend.makeOutput(outShape, 'int32');
    binding.argMax(backend.ctx, backend.deviceId(x), util.sizeFromShape(x.shape.slice(0, axis)),
                   x.shape[axis], util.sizeFromShape(x.shape.slice(axis + 1)), backend.deviceId(out));
    return out;
  })},
  {kernelName: 'Softmax', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const logits = inputs['logits'];
    const rank = logits.shape.length;
    const dim = attrs['dim'] === -1 ? rank - 1 : attrs['dim'] as number;
    if (dim !== rank - 1) {
      throw Error('Softmax along a non-last dimension is not yet supported. ' +
                  `Logits was rank ${rank} and dim was ${dim}`);
    }
    const out = backend.makeOutput(logits.shape, 'float32');
    binding.softmax(backend.ctx, backend.deviceId(logits), util.sizeFromShape(logits.shape.slice(0, -1)),
                    logits.shape[rank - 1], backend.deviceId(out));
    return out;
  })},
  {kernelName: 'Reshape', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const x = inputs['x'];
    const shape = util.inferFromImplicitShape(attrs['shape'] as number[], util.sizeFromShape(x.shape));
    return backend.view(x, shape);
  })},
  {kernelName: 'Identity', backendName: 'cuda',
   kernelFunc: asFunc(({inputs, backend}) => backend.view(inputs['x'], inputs['x'].shape))},
  {kernelName: 'ExpandDims', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const x = inputs['input'];
    let dim = attrs['dim'] as number;
    if (dim < 0) dim = x.shape.length + dim + 1;
    const shape = x.shape.slice();
    shape.splice(dim, 0, 1);
    return backend.view(x, shape);
  })},
  {kernelName: 'Transpose', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) =>
      transposeImpl(backend, inputs['x'], attrs['perm'] as number[]))},
  {kernelName: 'GatherV2', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const {x, indices} = inputs;
    const axis = util.parseAxisParam(attrs['axis'] as number, x.shape)[0];
    const info = backend_util.segment_util.collectGatherOpShapeInfo(
        x as never, indices as never, axis, (attrs['batchDims'] as number) ?? 0);
    const host = backend.hostValues(indices);
    if (host != null) {   // GatherV2.ts:36-46: an index outside [0, dim-1] throws
      for (const v of host as Int32Array) {
        util.assert(v >= 0 && v <= info.dimSize - 1,
                    () => `GatherV2: the index value ${v} is not in [0, ${info.dimSize - 1}]`);
      }
    }
    const out = backend.makeOutput(info.outputShape, x.dtype);
    binding.gather(backend.ctx, elemBytes(x), backend.deviceId(x), backend.deviceId(indices), info.batchSize,
                   info.outerSize, info.dimSize, info.sliceSize,
                   util.sizeFromShape(indices.shape) / Math.max(info.batchSize, 1), backend.deviceId(out),
                   host == null ? 1 : 0);
    return out;
  })},
  {kernelName: 'Concat', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const tensors = Object.keys(inputs).sort((a, b) => Number(a) - Number(b)).map(k => inputs[k]);
    const axis = util.parseAxisParam(attrs['axis'] as number, tensors[0].shape)[0];
    const outShape = backend_util.computeOutShape(tensors.map(t => t.shape), axis);
    const out = backend.makeOutput(outShape, tensors[0].dtype);
    const os = strides(outShape);
    let pos = 0;
    for (const t of tensors) {
      if (util.sizeFromShape(t.shape) > 0) copyStrided(backend, t, 0, out, pos * os[axis], os, t.shape);
      pos += t.shape[axis];
    }
    return out;
  })},
  {kernelName: 'Slice', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const x = inputs['x'];
    const [begin, size] = slice_util.parseSliceParams(x as never, attrs['begin'] as number[], attrs['size'] as number[]);
    slice_util.assertParamsValid(x as never, begin, size);
    const out = backend.makeOutput(size, x.dtype);
    const xs = strides(x.shape);
    if (util.sizeFromShape(size) > 0) {
      copyStrided(backend, x, begin.reduce((s, b, i) => s + b * xs[i], 0), out, 0, strides(size), size);
    }
    return out;
  })},
  {kernelName: 'PadV2', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const x = inputs['x'];
    const paddings = attrs['paddings'] as Array<[number, number]>;
    const outShape = paddings.map((p, i) => p[0] + x.shape[i] + p[1]);
    const out = backend.makeOutput(outShape, x.dtype);
    const c = (attrs['constantValue'] as number) ?? 0;
    const bits = x.dtype === 'float32' ? new Uint32Array(new Float32Array([c]).buffer)[0] : (c >>> 0);
    binding.fill(backend.ctx, elemBytes(x), bits, backend.deviceId(out), util.sizeFromShape(outShape));
    const os = strides(outShape);
    if (util.sizeFromShape(x.shape) > 0) {
      copyStrided(backend, x, 0, out, paddings.reduce((s, p, i) => s + p[0] * os[i], 0), os, x.shape);
    }
    return out;
  })},
  {kernelName: 'Tile', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const x = inputs['x'];
    const reps = attrs['reps'] as number[];
    const outShape = x.shape.map((s, i) => s * reps[i]);
    if (backend.lazyFusion && x.dtype === 'float32' && util.sizeFromShape(outShape) > 0 &&
        outShape.length <= 6 && backend.pendingOf(x) == null) {
      // Deferred: a batch normalisation that can index the untiled tensor never needs it
      return backend.defer(outShape, x.dtype, new PendingTile(
          x.dataId, x.shape, reps, outShape, x.dtype,
          [{name: 'Tile', inputShapes: {x: x.shape}, outputShapes: [outShape]}]));
    }
    const out = backend.makeOutput(outShape, x.dtype);
    if (util.sizeFromShape(outShape) > 0) copyStrided(backend, x, 0, out, 0, strides(outShape), outShape);
    return out;
  })},
];
