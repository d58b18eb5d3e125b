/**
 * Unary and broadcasting binary kernels, Cast, FusedBatchNorm.
 * Python twin: tfjs_b200/kernels/elementwise.py.
 */
import {broadcast_util, DataType, KernelConfig, KernelFunc, TensorInfo, upcastType,
        util} from '@tensorflow/tfjs-core';

import {CudaBackend} from '../backend_cuda';
import {BINARY_OP, binding, DTYPE, i64, UNARY_OP} from '../binding';

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

type Args = {inputs: {[k: string]: TensorInfo}, attrs: {[k: string]: unknown}, backend: CudaBackend};
const asFunc = (f: (a: Args) => TensorInfo) => f as unknown as KernelFunc;

const unaryNames: Array<keyof typeof UNARY_OP> =
    ['Relu', 'Relu6', 'Elu', 'Sigmoid', 'Exp', 'Sqrt', 'Rsqrt', 'Square', 'Tanh', 'Neg', 'Erf', 'Abs', 'Log'];
const binaryNames: Array<keyof typeof BINARY_OP> =
    ['Add', 'Sub', 'Multiply', 'RealDiv', 'Maximum', 'Minimum', 'Pow', 'SquaredDifference'];

export const elementwiseConfigs: KernelConfig[] = [
  ...unaryNames.map(name => ({kernelName: name, backendName: 'cuda',
      kernelFunc: asFunc(({inputs, backend}) => unaryImpl(backend, name, inputs['x']))})),
  {kernelName: 'LeakyRelu', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) =>
      unaryImpl(backend, 'LeakyRelu', inputs['x'], (attrs['alpha'] as number) ?? 0.2))},
  {kernelName: 'ClipByValue', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) =>
      unaryImpl(backend, 'ClipByValue', inputs['x'], attrs['clipValueMin'] as number,
                attrs['clipValueMax'] as number))},
  ...binaryNames.map(name => ({kernelName: name, backendName: 'cuda',
      kernelFunc: asFunc(({inputs, backend}) => binaryImpl(backend, name, inputs['a'], inputs['b']))})),
  {kernelName: 'Prelu', backendName: 'cuda', kernelFunc: asFunc(({inputs, backend}) =>
      binaryImpl(backend, 'Prelu', inputs['x'], inputs['alpha']))},
  {kernelName: 'Cast', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) =>
      castImpl(backend, inputs['x'], attrs['dtype'] as DataType))},
  {kernelName: 'FusedBatchNorm', backendName: 'cuda', kernelFunc: asFunc(({inputs, attrs, backend}) => {
    const {x, mean, variance, scale, offset} = inputs;
    const n = (t?: TensorInfo) => t == null ? 0 : util.sizeFromShape(t.shape);
    const out = backend.makeOutput(x.shape, 'float32');
    binding.batchNorm(backend.ctx, backend.deviceId(x), n(x), backend.deviceId(mean), n(mean),
                      backend.deviceId(variance), n(variance), backend.deviceId(scale), n(scale),
                      backend.deviceId(offset), n(offset), (attrs['varianceEpsilon'] as number) ?? 0.001,
                      backend.deviceId(out));
    return out;
  })},
];
