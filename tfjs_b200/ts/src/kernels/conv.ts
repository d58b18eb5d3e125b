/**
 * FusedConv2D, Conv2D, FusedDepthwiseConv2D, DepthwiseConv2dNative.
 * Python twin: tfjs_b200/kernels/conv.py.  NHWC only in this TypeScript version.
 */
import {backend_util, Conv2D, DepthwiseConv2dNative, FusedConv2D, FusedDepthwiseConv2D,
        KernelConfig, KernelFunc, TensorInfo, util} from '@tensorflow/tfjs-core';

import {CudaBackend} from '../backend_cuda';
import {ACTIVATION, binding, packConvParams} from '../binding';
import {PendingConv, PendingDepthwise} from '../pending';
import {applyActivation, binaryImpl} from './elementwise';

/** 1 for a scalar, `channels` when the tensor broadcasts along the last axis, else null. */
export function perChannelLen(t: TensorInfo|undefined, channels: number): number|null {
  if (t == null) return 0;
  const n = util.sizeFromShape(t.shape);
  if (n === 1) return 1;
  return n === channels && t.shape[t.shape.length - 1] === channels ? channels : null;
}

function convImpl(
    backend: CudaBackend, x: TensorInfo, filter: TensorInfo, bias: TensorInfo|undefined,
    prelu: TensorInfo|undefined, attrs: {[k: string]: unknown}, activation: string,
    depthwise: boolean): TensorInfo {
  if ((attrs['dataFormat'] ?? 'NHWC') !== 'NHWC') {
    throw new Error('tfjs-backend-cuda: conv kernels take NHWC tensors');
  }
  const convInfo = backend_util.computeConv2DInfo(
      x.shape as [number, number, number, number],
      filter.shape as [number, number, number, number],
      attrs['strides'] as number | [number, number],
      (attrs['dilations'] ?? [1, 1]) as number | [number, number],
      attrs['pad'] as 'same' | 'valid' | number,
      attrs['dimRoundingMode'] as 'floor' | 'round' | 'ceil', depthwise);
  const biasLen = perChannelLen(bias, convInfo.outChannels);
  const preluLen = activation === 'prelu' ? perChannelLen(prelu, convInfo.outChannels) : 0;
  const fuseBias = biasLen != null;
  const fuseAct = fuseBias && (activation !== 'prelu' || preluLen != null);
  const params = packConvParams(
      convInfo, ACTIVATION[fuseAct ? activation : 'linear'], fuseBias ? biasLen : 0,
      fuseAct ? (preluLen ?? 0) : 0, (attrs['leakyreluAlpha'] as number) ?? 0.2);
  // A depthwise convolution is deferred with its relu / relu6 too: the 1x1 convolution that
  // consumes it (the projection of an inverted-residual block) absorbs it into its launch.
  const deferrable = activation === 'linear' ||
      (depthwise && (activation === 'relu' || activation === 'relu6'));
  if (backend.lazyFusion && fuseBias && deferrable &&
      util.sizeFromShape(convInfo.outShape) > 0) {
    // Deferred: a following Add (residual, or the bias of a depthwise convolution) and
    // Relu / Relu6 / clip fold into this launch's epilogue (kernels/elementwise.ts).
    const inputShapes: {[k: string]: number[]} = {x: x.shape, filter: filter.shape};
    if (bias != null) inputShapes['bias'] = bias.shape;
    const desc = {
      name: depthwise ? (bias != null ? FusedDepthwiseConv2D : DepthwiseConv2dNative) : FusedConv2D,
      inputShapes, outputShapes: [convInfo.outShape]
    };
    const pending = depthwise ?
        new PendingDepthwise(params, x.dataId, filter.dataId, bias != null ? bias.dataId : null, [desc],
                             activation as 'linear'|'relu'|'relu6') :
        new PendingConv(params, x.dataId, filter.dataId, bias != null ? bias.dataId : null, null, [desc]);
    return backend.defer(convInfo.outShape, 'float32', pending);
  }
  let out = backend.makeOutput(convInfo.outShape, 'float32');
  const launch = depthwise ? binding.fusedDepthwiseConv2d : binding.fusedConv2d;
  launch(backend.ctx, params, backend.deviceId(x), backend.deviceId(filter),
         fuseBias ? backend.deviceId(bias) : 0,
         fuseAct && activation === 'prelu' ? backend.deviceId(prelu) : 0, backend.deviceId(out));
  // Unfused tail in the reference's order: Add, then the activation
  // (tfjs-backend-cpu/src/kernels/FusedConv2D.ts:49-92).
  if (!fuseBias) {
    const added = binaryImpl(backend, 'Add', out, bias);
    backend.disposeData(out.dataId);
    out = added;
  }
  if (!fuseAct) {
    const act = applyActivation(backend, out, activation, prelu, attrs['leakyreluAlpha'] as number);
    backend.disposeData(out.dataId);
    out = act;
  }
  return out;
}

function config(kernelName: string, fused: boolean, depthwise: boolean): KernelConfig {
  const kernelFunc = ({inputs, attrs, backend}: {inputs: {[k: string]: TensorInfo},
                       attrs: {[k: string]: unknown}, backend: CudaBackend}) =>
      convImpl(backend, inputs['x'], inputs['filter'], fused ? inputs['bias'] : undefined,
               fused ? inputs['preluActivationWeights'] : undefined, attrs,
               fused ? ((attrs['activation'] as string) ?? 'linear') : 'linear', depthwise);
  return {kernelName, backendName: 'cuda', kernelFunc: kernelFunc as unknown as KernelFunc};
}

export const convConfigs: KernelConfig[] = [
  config(FusedConv2D, true, false), config(Conv2D, false, false),
  config(FusedDepthwiseConv2D, true, true), config(DepthwiseConv2dNative, false, true)
];
