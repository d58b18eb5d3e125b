/**
 * Typed view of the N-API addon (binding/tfjs_cuda_binding.cc), one function per
 * entry point of include/tfjs_cuda.h.
 */
// tslint:disable-next-line:no-require-imports
const addon = require('../build/Release/tfjs_cuda_binding.node');

export type Ctx = unknown;

export interface CudaBinding {
  create(deviceOrdinal: number): Ctx;
  alloc(ctx: Ctx, nbytes: number): number;
  free(ctx: Ctx, id: number): void;
  write(ctx: Ctx, id: number, data: ArrayBufferView, nbytes: number): void;
  read(ctx: Ctx, id: number, out: ArrayBufferView, nbytes: number): void;
  fusedElementwise(ctx: Ctx, program: ArrayBuffer, out: number): void;
  fusedElementwiseCatalogued(ctx: Ctx, program: ArrayBuffer): number;
  decodeFloat16(ctx: Ctx, q: number, n: number, out: number): void;
  captureBegin(ctx: Ctx, arenaBytes: number): void;
  captureEnd(ctx: Ctx, abandon: number): number;
  graphLaunch(ctx: Ctx, graph: number): void;
  graphDestroy(ctx: Ctx, graph: number): void;
  copy(ctx: Ctx, src: number, dst: number, nbytes: number): void;
  highWaterReset(ctx: Ctx): void;
  readBegin(ctx: Ctx, id: number, out: ArrayBufferView, nbytes: number): number;
  readWait(ctx: Ctx, ticket: number): void;
  sync(ctx: Ctx): void;
  memory(ctx: Ctx): {numBytesInGPU: number, numBytesInGPUAllocated: number,
                     poolHighWater: number, numDeviceBuffers: number};
  timeBegin(ctx: Ctx): void;
  timeEnd(ctx: Ctx): number;
  setMathMode(ctx: Ctx, mode: number): void;
  fusedConv2d(ctx: Ctx, params: ArrayBuffer, x: number, filter: number, bias: number,
              prelu: number, out: number): void;
  fusedConv2dResidual(ctx: Ctx, params: ArrayBuffer, x: number, filter: number, bias: number,
                      prelu: number, residual: number, postActivation: number,
                      out: number): void;
  /** false when the library does not take the shapes: launch the two kernels separately. */
  fusedDepthwiseProject(ctx: Ctx, dwParams: ArrayBuffer, pwParams: ArrayBuffer, x: number,
                        dwFilter: number, dwBias: number, pwFilter: number, pwBias: number,
                        residual: number, postActivation: number, out: number): boolean;
  addActivation(ctx: Ctx, activation: number, a: number, b: number, n: number,
                out: number): void;
  fusedDepthwiseConv2d(ctx: Ctx, params: ArrayBuffer, x: number, filter: number, bias: number,
                       prelu: number, out: number): void;
  fusedMatMul(ctx: Ctx, params: ArrayBuffer, a: number, b: number, bias: number, prelu: number,
              out: number): void;
  fusedMatMulHeads(ctx: Ctx, params: ArrayBuffer, a: number, b: number, bias: number,
                   prelu: number, layout: number, rowsOrHeads: number, headDim: number,
                   out: number): void;
  /** Products sharing `a`; false when the library does not take the group (launch the
   * members one by one). */
  fusedMatMulGroup(ctx: Ctx, params: ArrayBuffer, a: number, b: Int32Array, bias: Int32Array|null,
                   layout: number, rowsOrHeads: number, headDim: number, out: Int32Array): boolean;
  pool2d(ctx: Ctx, params: ArrayBuffer, isMax: number, x: number, out: number): void;
  binary(ctx: Ctx, op: number, dtype: number, rank: number, a: number, aShape: BigInt64Array,
         b: number, bShape: BigInt64Array, out: number, outShape: BigInt64Array): void;
  unary(ctx: Ctx, op: number, p0: number, p1: number, x: number, n: number, out: number): void;
  softmax(ctx: Ctx, x: number, rows: number, cols: number, out: number): void;
  softmaxScaledMasked(ctx: Ctx, x: number, rows: number, cols: number, hasScale: number,
                      scale: number, mask: number, rowsPerMask: number, out: number): void;
  /** softmax(q k^T * scale + mask) v for [batch, heads, seq, headDim] operands, stored with
   * the heads merged; false when the library does not take the shape (nothing launched). */
  fusedAttention(ctx: Ctx, q: number, k: number, v: number, mask: number, hasScale: number,
                 scale: number, batch: number, heads: number, seq: number, headDim: number,
                 unitsPerMask: number, out: number): boolean;
  layerNorm(ctx: Ctx, x: number, residual: number, gamma: number, beta: number, rows: number,
            cols: number, epsilon: number, out: number): void;
  reduce(ctx: Ctx, op: number, x: number, outer: number, reduce: number, inner: number,
         out: number): void;
  argMax(ctx: Ctx, x: number, outer: number, reduce: number, inner: number, out: number): void;
  transpose(ctx: Ctx, elemBytes: number, rank: number, x: number, xShape: BigInt64Array,
            perm: Int32Array, out: number): void;
  gather(ctx: Ctx, elemBytes: number, x: number, indices: number, batch: number, outer: number,
         dim: number, slice: number, nIdx: number, out: number, check: number): number;
  cast(ctx: Ctx, from: number, to: number, x: number, n: number, out: number): void;
  copyStrided(ctx: Ctx, elemBytes: number, rank: number, extent: BigInt64Array, x: number,
              xOff: number, xStrides: BigInt64Array, xWrap: BigInt64Array, out: number,
              oOff: number, oStrides: BigInt64Array): void;
  fill(ctx: Ctx, elemBytes: number, bits: number, out: number, n: number): void;
  batchNorm(ctx: Ctx, x: number, n: number, mean: number, nMean: number, variance: number,
            nVar: number, scale: number, nScale: number, offset: number, nOffset: number,
            eps: number, out: number): void;
  dequantize(ctx: Ctx, qBytes: number, toDtype: number, q: number, scale: number, min: number,
             n: number, out: number): void;
  dequantizeStatic(ctx: Ctx, qBytes: number, toDtype: number, q: number, scale: number,
                   min: number, n: number, out: number): void;
  batchNormRows(ctx: Ctx, x: number, rows: number, cols: number, mean: number, meanMode: number,
                variance: number, varMode: number, scale: number, scaleMode: number,
                offset: number, offsetMode: number, eps: number, out: number): void;
  deviceCount(): number;
  upload(ctx: Ctx, data: ArrayBufferView, nbytes: number): number;
  readAsync(ctx: Ctx, id: number, out: ArrayBufferView, nbytes: number): void;
  sizeOf(ctx: Ctx, id: number): number;
  devicePtr(ctx: Ctx, id: number): bigint;
  trim(ctx: Ctx): void;
  hostAlloc(ctx: Ctx, nbytes: number): ArrayBuffer;
  hostFree(ctx: Ctx, buffer: ArrayBuffer): void;
  eventRecord(ctx: Ctx, slot: number): void;
  eventElapsed(ctx: Ctx, slotBegin: number, slotEnd: number): number;
  launchCount(ctx: Ctx): number;
  launchLog(ctx: Ctx, enable: number): void;
  launchLogTake(ctx: Ctx): string;
  flushL2(ctx: Ctx): void;
  weightsBegin(ctx: Ctx, specs: ArrayBuffer): number;
  weightsPush(ctx: Ctx, loader: number, chunk: ArrayBufferView|ArrayBuffer): void;
  weightsPushFile(ctx: Ctx, loader: number, path: string): void;
  weightsEnd(ctx: Ctx, loader: number, ids: Int32Array|null): number;
}

export const binding = addon as CudaBinding;

/** Enum values of include/tfjs_cuda.h. */
export const ACTIVATION: {[name: string]: number} =
    {linear: 0, relu: 1, relu6: 2, prelu: 3, leakyrelu: 4, sigmoid: 5, elu: 6, gelu_erf: 7};
export const DTYPE: {[name: string]: number} = {float32: 0, int32: 1, bool: 2};
export const BINARY_OP = {Add: 0, Sub: 1, Multiply: 2, RealDiv: 3, Maximum: 4, Minimum: 5, Pow: 6,
                          SquaredDifference: 7, Prelu: 8};
export const UNARY_OP = {Relu: 0, Relu6: 1, Elu: 2, Sigmoid: 3, LeakyRelu: 4, Exp: 5, Sqrt: 6,
                         Rsqrt: 7, Square: 8, Tanh: 9, Neg: 10, ClipByValue: 11, Erf: 12, Abs: 13,
                         Log: 14};
export const REDUCE_OP = {Sum: 0, Mean: 1, Max: 2};
export const WEIGHT_STORAGE = {raw: 0, uint8: 1, uint16: 2, float16: 3};
export const EW = {FULL: 0, PERIODIC: 1, ROW: 2, SCALAR: 3, BATCHED: 4, MAX_INPUTS: 8,
                   MAX_OPS: 24, UNARY: 32};
export const STATUS_UNSUPPORTED = 5;

/** tfjs_cuda_weight_spec: u64 n, i32 storage, i32 dtype, f64 scale, f64 min, i32 skip,
 * i32 reserved = 40 bytes per entry. */
export function packWeightSpecs(
    entries: Array<{n: number, storage: number, dtype: number, scale: number, min: number,
                    skip: boolean}>): ArrayBuffer {
  const buf = new ArrayBuffer(40 * entries.length);
  const v = new DataView(buf);
  entries.forEach((e, i) => {
    const o = 40 * i;
    v.setBigUint64(o, BigInt(e.n), true);
    v.setInt32(o + 8, e.storage, true);
    v.setInt32(o + 12, e.dtype, true);
    v.setFloat64(o + 16, e.scale, true);
    v.setFloat64(o + 24, e.min, true);
    v.setInt32(o + 32, e.skip ? 1 : 0, true);
  });
  return buf;
}

/** tfjs_cuda_ew_program: i32 n_inputs, i32 n_ops, u64 n, u32 cols, u32 reserved, then
 * input_id[8], input_mode[8], input_period[8], input_aux[8] (4 bytes each) and 24 ops of
 * {i16 opcode, u8 a, u8 b, f32 p0, f32 p1} = 24 + 4 * 32 + 24 * 12 = 440 bytes. */
export function packEwProgram(p: {
  n: number, cols: number, inputs: Array<{id: number, mode: number, period: number, aux: number}>,
  ops: Array<{opcode: number, a: number, b: number}>
}): ArrayBuffer {
  const buf = new ArrayBuffer(440);
  const v = new DataView(buf);
  v.setInt32(0, p.inputs.length, true);
  v.setInt32(4, p.ops.length, true);
  v.setBigUint64(8, BigInt(p.n), true);
  v.setUint32(16, p.cols, true);
  p.inputs.forEach((inp, k) => {
    v.setInt32(24 + 4 * k, inp.id, true);
    v.setInt32(56 + 4 * k, inp.mode, true);
    v.setUint32(88 + 4 * k, inp.period, true);
    v.setUint32(120 + 4 * k, inp.aux, true);
  });
  p.ops.forEach((op, j) => {
    const o = 152 + 12 * j;
    v.setInt16(o, op.opcode, true);
    v.setUint8(o + 2, op.a);
    v.setUint8(o + 3, op.b);
  });
  return buf;
}

/** tfjs_cuda_conv2d_params: 18 int32 fields, 4 bytes of padding, one double. */
export function packConvParams(
    ci: {batchSize: number, inHeight: number, inWidth: number, inChannels: number,
         outHeight: number, outWidth: number, outChannels: number, filterHeight: number,
         filterWidth: number, strideHeight: number, strideWidth: number, dilationHeight: number,
         dilationWidth: number, padInfo: {top: number, left: number}},
    activation: number, biasLen: number, preluLen: number, leakyreluAlpha = 0.2,
    effective = false, effFilter?: [number, number]): ArrayBuffer {
  const buf = new ArrayBuffer(80);
  const v = new DataView(buf);
  const f = effective && effFilter ? effFilter : [ci.filterHeight, ci.filterWidth];
  [ci.batchSize, ci.inHeight, ci.inWidth, ci.inChannels, ci.outHeight, ci.outWidth,
   ci.outChannels, f[0], f[1], ci.strideHeight, ci.strideWidth, ci.dilationHeight,
   ci.dilationWidth, ci.padInfo.top, ci.padInfo.left, activation, biasLen, preluLen]
      .forEach((x, i) => v.setInt32(4 * i, x, true));
  v.setFloat64(72, leakyreluAlpha, true);
  return buf;
}

/** tfjs_cuda_matmul_params: 10 int32 fields, one double, then the constants of the
 * erf-GELU epilogue (three floats and an int32; zero unless activation is GELU_ERF). */
export function packMatMulParams(
    batchA: number, batchB: number, m: number, n: number, k: number, transposeA: boolean,
    transposeB: boolean, activation: number, biasLen: number, preluLen: number,
    leakyreluAlpha = 0.2, gelu?: [number, number, number, boolean]): ArrayBuffer {
  const buf = new ArrayBuffer(64);
  const v = new DataView(buf);
  [batchA, batchB, m, n, k, transposeA ? 1 : 0, transposeB ? 1 : 0, activation, biasLen, preluLen]
      .forEach((x, i) => v.setInt32(4 * i, x, true));
  v.setFloat64(40, leakyreluAlpha, true);
  if (gelu) {
    v.setFloat32(48, gelu[0], true);
    v.setFloat32(52, gelu[1], true);
    v.setFloat32(56, gelu[2], true);
    v.setInt32(60, gelu[3] ? 1 : 0, true);
  }
  return buf;
}

export function i64(values: number[]): BigInt64Array {
  return BigInt64Array.from((values.length ? values : [0]).map(x => BigInt(x)));
}
