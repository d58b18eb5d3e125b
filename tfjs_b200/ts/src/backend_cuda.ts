/**
 * CudaBackend: the KernelBackend of `tfjs-backend-cuda`
 * (contract: tfjs-core/src/backends/backend.ts; reference semantics:
 * tfjs-backend-cpu/src/backend_cpu.ts).  One instance owns one GPU context.
 *
 * Python twin (executed by the tests): tfjs_b200/backend.py.
 */
import {backend_util, BackendTimingInfo, DataStorage, DataType, engine, KernelBackend,
        TensorInfo, TypedArray, util} from '@tensorflow/tfjs-core';

import {binding, Ctx} from './binding';
import {Desc, Pending, PendingConv, PendingDepthwise, PendingMatMul} from './pending';

interface Record {
  id: number;          // device buffer id; 0 = host-resident or not launched yet
  nbytes: number;
  dtype: DataType;
  refCount: number;
  host?: TypedArray;   // kept for small host-written tensors
  pending?: Pending;   // a deferred launch produces this tensor (pending.ts)
  held: number;        // how many of refCount belong to pending launches that read it
}

const HOST_RESIDENT_BYTES = 4096;

function bytesPerElement(dtype: DataType): number {
  if (dtype === 'float32' || dtype === 'int32') return 4;
  if (dtype === 'bool') return 1;
  throw new Error(`tfjs-backend-cuda: dtype ${dtype} is not supported`);
}

export class CudaBackend extends KernelBackend {
  readonly ctx: Ctx;
  private data: DataStorage<Record>;
  private hidden = 0;           // records kept alive only by pending launches
  private logDepth = 0;
  /** chain signature -> the library has a straight-line kernel for it */
  readonly ewCatalogue = new Map<string, boolean>();
  /** Deferred launches; TFJS_CUDA_NO_LAZY_FUSION=1 launches every kernel when called. */
  lazyFusion = !['1', 'true'].includes(process.env['TFJS_CUDA_NO_LAZY_FUSION'] ?? '0');
  /** A pending 3x3 depthwise convolution consumed by a 1x1 convolution runs inside that
   * convolution's launch (TFJS_CUDA_NO_DW_PROJECT=1 keeps the two launches). */
  fuseDepthwiseProject = !['1', 'true'].includes(process.env['TFJS_CUDA_NO_DW_PROJECT'] ?? '0');

  constructor(readonly deviceOrdinal = 0) {
    super();
    this.ctx = binding.create(deviceOrdinal);   // throws when there is no sm_100a GPU
    this.data = new DataStorage(this, engine());
  }

  override write(values: backend_util.BackendValues, shape: number[], dtype: DataType): object {
    const dataId = {};
    this.move(dataId, values, shape, dtype, 1);
    return dataId;
  }

  override move(dataId: object, values: backend_util.BackendValues, shape: number[],
                dtype: DataType, refCount: number): void {
    const nbytes = util.sizeFromShape(shape) * bytesPerElement(dtype);
    const typed = values as TypedArray;
    if (typed != null && nbytes <= HOST_RESIDENT_BYTES) {
      // The graph executor reads axis / shape / perm constants with dataSync() in its
      // node loop; host-resident small tensors keep those reads off the stream.
      this.data.set(dataId, {id: 0, nbytes, dtype, refCount, host: typed.slice(), held: 0});
      return;
    }
    const id = binding.alloc(this.ctx, nbytes);
    if (typed != null && nbytes > 0) binding.write(this.ctx, id, typed, nbytes);
    this.data.set(dataId, {id, nbytes, dtype, refCount, held: 0});
  }

  /** A tensor over a device buffer the library made (the weight loader's results). */
  adopt(id: number, shape: number[], dtype: DataType): TensorInfo {
    const dataId = {};
    const nbytes = util.sizeFromShape(shape) * bytesPerElement(dtype);
    this.data.set(dataId, {id, nbytes, dtype, refCount: 1, held: 0});
    return {dataId, shape, dtype};
  }

  /** Allocates an uninitialised device tensor for a kernel result. */
  makeOutput(shape: number[], dtype: DataType): TensorInfo {
    const nbytes = util.sizeFromShape(shape) * bytesPerElement(dtype);
    const dataId = {};
    this.data.set(dataId, {id: binding.alloc(this.ctx, nbytes), nbytes, dtype, refCount: 1, held: 0});
    return {dataId, shape, dtype};
  }

  // ------------------------------------------------------------ deferred launches --
  /** Changes a record's counts, tracking whether only pending launches keep it alive
   * (such records are not reported by numDataIds). */
  private adjust(r: Record, dRef: number, dHeld: number): void {
    const was = r.held > 0 && r.refCount <= r.held;
    r.refCount += dRef;
    r.held += dHeld;
    const now = r.held > 0 && r.refCount <= r.held;
    if (was !== now) this.hidden += now ? 1 : -1;
  }

  /** Output tensor of a kernel whose launch is deferred; its inputs stay alive until the
   * launch happened or the output was disposed. */
  defer(shape: number[], dtype: DataType, pending: Pending): TensorInfo {
    const nbytes = util.sizeFromShape(shape) * bytesPerElement(dtype);
    const dataId = {};
    for (const d of pending.deps()) this.adjust(this.data.get(d), 1, 1);
    this.data.set(dataId, {id: 0, nbytes, dtype, refCount: 1, pending, held: 0});
    if (pending instanceof PendingMatMul) this.noteMatMul(dataId, pending);
    return {dataId, shape, dtype};
  }

  pendingOf(t: TensorInfo): Pending|undefined { return this.data.get(t.dataId).pending; }
  pendingOfId(dataId: object): Pending|undefined { return this.data.get(dataId)?.pending; }

  /** The pending convolution behind `t` with `act` as the last step of its epilogue, as a
   * new pending tensor; `t` itself stays pending (another consumer launches it without). */
  withActivation(t: TensorInfo, act: 'relu'|'relu6', desc: Desc): TensorInfo {
    const p = this.data.get(t.dataId).pending as PendingConv|PendingDepthwise;
    return this.defer(t.shape, 'float32', p.withAct(act, desc));
  }

  private release(pending: Pending): void {
    for (const d of pending.deps()) {
      const r = this.data.get(d);
      this.adjust(r, -1, -1);
      if (r.refCount <= 0) this.drop(d, r);
    }
  }

  /** Products that share their first operand launch together (TFJS_CUDA_NO_MATMUL_GROUP=1
   * launches each on its own); dataId of `a` -> dataIds of the pending products on it. */
  groupMatMuls = !['1', 'true'].includes(process.env['TFJS_CUDA_NO_MATMUL_GROUP'] ?? '0');
  private matMulsOn = new Map<object, object[]>();

  private stillPendingMatMul(dataId: object): boolean {
    return this.data.has(dataId) && this.data.get(dataId).pending instanceof PendingMatMul;
  }

  private noteMatMul(dataId: object, pending: PendingMatMul): void {
    const ids = (this.matMulsOn.get(pending.a) ?? []).filter(d => this.stillPendingMatMul(d));
    this.matMulsOn.set(pending.a, [...ids, dataId]);
    if (this.matMulsOn.size > 64) {   // forget operands whose products are all gone
      for (const [a, list] of this.matMulsOn) {
        if (!list.some(d => this.stillPendingMatMul(d))) this.matMulsOn.delete(a);
      }
    }
  }

  /** Launches `pending` together with the other products pending on the same operand (same
   * dimensions, layout and bias kind).  False when there is none or the library does not
   * take the group; nothing has been launched then. */
  private resolveMatMulGroup(r: Record, pending: PendingMatMul): boolean {
    const mates = (this.matMulsOn.get(pending.a) ?? [])
                      .filter(d => this.stillPendingMatMul(d))
                      .map(d => this.data.get(d) as Record)
                      .filter(m => m !== r && (m.pending as PendingMatMul).key === pending.key)
                      .slice(0, 3);
    if (!this.groupMatMuls || mates.length === 0) return false;
    // operands that are pending launch first; the group is what is still pending then
    const of0 = (m: Record) => m.pending as PendingMatMul;
    this.deviceIdOf(pending.a);
    for (const m of [r, ...mates]) {
      if (m.pending instanceof PendingMatMul) {
        this.deviceIdOf(of0(m).b);
        if (of0(m).bias != null) this.deviceIdOf(of0(m).bias!);
      }
    }
    const ready = mates.filter(m => m.pending instanceof PendingMatMul);
    if (r.pending !== pending || ready.length === 0) return false;
    const members = [r, ...ready];
    const devs = members.map(m => binding.alloc(this.ctx, m.nbytes));
    let ok = false;
    try {
      const of = (m: Record) => m.pending as PendingMatMul;
      const heads = pending.heads ?? [0, 0, 0];
      ok = binding.fusedMatMulGroup(
          this.ctx, pending.params, this.deviceIdOf(pending.a),
          Int32Array.from(members.map(m => this.deviceIdOf(of(m).b))),
          Int32Array.from(members.map(m => of(m).bias != null ? this.deviceIdOf(of(m).bias!) : 0)),
          heads[0], heads[1], heads[2], Int32Array.from(devs));
    } finally {
      if (!ok) devs.forEach(d => binding.free(this.ctx, d));
    }
    if (!ok) return false;
    members.forEach((m, i) => {
      const done = m.pending!;
      m.pending = undefined;
      m.id = devs[i];
      this.release(done);
    });
    return true;
  }

  private resolve(r: Record): void {
    const pending = r.pending!;
    if (pending instanceof PendingMatMul && this.resolveMatMulGroup(r, pending)) return;
    if (r.pending !== pending) return;     // launched meanwhile, by an operand's own launch
    const dev = binding.alloc(this.ctx, r.nbytes);
    try {
      pending.launch(this, dev);
    } catch (e) {
      binding.free(this.ctx, dev);
      throw e;
    }
    r.id = dev;
    r.pending = undefined;
    this.release(pending);
  }

  /** Device buffer id behind a dataId: launches a pending producer or uploads a
   * host-resident tensor first. */
  deviceIdOf(dataId: object): number {
    const r = this.data.get(dataId);
    if (r.pending != null) {
      this.resolve(r);
    } else if (r.id === 0) {
      r.id = binding.alloc(this.ctx, r.nbytes);
      if (r.nbytes > 0) binding.write(this.ctx, r.id, r.host!, r.nbytes);
    }
    return r.id;
  }

  /** Device buffer id of a tensor (0 for an absent optional input). */
  deviceId(t?: TensorInfo): number { return t == null ? 0 : this.deviceIdOf(t.dataId); }

  hostValues(t: TensorInfo): TypedArray|undefined { return this.data.get(t.dataId).host; }

  // ------------------------------------------------------------------------ data --
  override readSync(dataId: object): backend_util.BackendValues {
    const r = this.data.get(dataId);
    if (r.pending != null) this.resolve(r);
    if (r.host != null) return r.host.slice();
    const out = util.getTypedArrayFromDType(r.dtype as 'float32', r.nbytes / bytesPerElement(r.dtype));
    binding.read(this.ctx, r.id, out, r.nbytes);
    return out;
  }

  /** The copy is queued behind the kernels launched so far; the promise resolves on a
   *  later turn of the event loop, so code between `data()` and `await` keeps launching. */
  override read(dataId: object): Promise<backend_util.BackendValues> {
    const r = this.data.get(dataId);
    if (r.pending != null) this.resolve(r);
    if (r.host != null) return Promise.resolve(r.host.slice());
    const out = util.getTypedArrayFromDType(r.dtype as 'float32', r.nbytes / bytesPerElement(r.dtype));
    const ticket = binding.readBegin(this.ctx, r.id, out, r.nbytes);
    return new Promise((resolve, reject) => setImmediate(() => {
      try { binding.readWait(this.ctx, ticket); resolve(out); } catch (e) { reject(e); }
    }));
  }

  override disposeData(dataId: object, force = false): boolean {
    if (!this.data.has(dataId)) return false;
    const r = this.data.get(dataId);
    this.adjust(r, -1, 0);
    if (r.refCount > 0 && (!force || r.held > 0)) return false;
    this.drop(dataId, r);
    return true;
  }

  private drop(dataId: object, r: Record): void {
    if (r.held > 0 && r.refCount <= r.held) this.hidden--;
    this.data.delete(dataId);
    if (r.id !== 0) binding.free(this.ctx, r.id);
    if (r.pending != null) {
      const p = r.pending;
      r.pending = undefined;
      this.release(p);
    }
  }

  override refCount(dataId: object): number {
    if (!this.data.has(dataId)) return 0;
    const r = this.data.get(dataId);
    return r.refCount - r.held;
  }
  override incRef(dataId: object): void { this.adjust(this.data.get(dataId), 1, 0); }
  decRef(dataId: object): void { if (this.data.has(dataId)) this.adjust(this.data.get(dataId), -1, 0); }
  override numDataIds(): number { return this.data.numDataIds() - this.hidden; }

  /** Zero-copy view: same dataId, one more reference. */
  view(t: TensorInfo, shape: number[], dtype = t.dtype): TensorInfo {
    this.incRef(t.dataId);
    return {dataId: t.dataId, shape, dtype};
  }

  override memory() { return {unreliable: false, ...binding.memory(this.ctx)}; }

  // ---------------------------------------------------------------------- timing --
  /** Turns the library's launch log on or off (calls nest). */
  launchLog(enable: boolean): void {
    this.logDepth += enable ? 1 : -1;
    if (enable && this.logDepth === 1) binding.launchLog(this.ctx, 1);
    if (!enable && this.logDepth === 0) binding.launchLog(this.ctx, 0);
  }

  /** BackendTimingInfo (tfjs-core/src/backends/backend.ts:26-30): kernelMs from CUDA events
   * on the stream; getExtraProfileInfo names the kernel instantiations launched inside f,
   * which tf.profile prints per kernel (tfjs-core/src/profiler.ts:74-76). */
  override async time(f: () => void): Promise<BackendTimingInfo> {
    const nested = this.logDepth > 0;
    this.launchLog(true);
    let kernelMs: number, info = '';
    try {
      binding.timeBegin(this.ctx);
      f();
      kernelMs = binding.timeEnd(this.ctx);
      if (!nested) info = binding.launchLogTake(this.ctx);
    } finally {
      this.launchLog(false);
    }
    return {kernelMs, getExtraProfileInfo: () => info};
  }
  override timerAvailable(): boolean { return true; }
  override floatPrecision(): 16|32 { return 32; }
  override epsilon(): number { return 1e-7; }
  mathMode: 'tf32'|'fp32' = 'tf32';
  setMathMode(mode: 'tf32'|'fp32'): void {
    binding.setMathMode(this.ctx, mode === 'tf32' ? 0 : 1);
    this.mathMode = mode;
  }
  override dispose(): void { /* the context is destroyed when the external is collected */ }
}
