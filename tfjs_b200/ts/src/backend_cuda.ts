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

interface Record {
  id: number;          // device buffer id; 0 = host-resident, not uploaded yet
  nbytes: number;
  dtype: DataType;
  refCount: number;
  host?: TypedArray;   // kept for small host-written tensors
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
      this.data.set(dataId, {id: 0, nbytes, dtype, refCount, host: typed.slice()});
      return;
    }
    const id = binding.alloc(this.ctx, nbytes);
    if (typed != null && nbytes > 0) binding.write(this.ctx, id, typed, nbytes);
    this.data.set(dataId, {id, nbytes, dtype, refCount});
  }

  /** Allocates an uninitialised device tensor for a kernel result. */
  makeOutput(shape: number[], dtype: DataType): TensorInfo {
    const nbytes = util.sizeFromShape(shape) * bytesPerElement(dtype);
    const dataId = {};
    this.data.set(dataId, {id: binding.alloc(this.ctx, nbytes), nbytes, dtype, refCount: 1});
    return {dataId, shape, dtype};
  }

  /** Device buffer id of a tensor (0 for an absent optional input). */
  deviceId(t?: TensorInfo): number {
    if (t == null) return 0;
    const r = this.data.get(t.dataId);
    if (r.id === 0) {
      r.id = binding.alloc(this.ctx, r.nbytes);
      if (r.nbytes > 0) binding.write(this.ctx, r.id, r.host, r.nbytes);
    }
    return r.id;
  }

  hostValues(t: TensorInfo): TypedArray|undefined { return this.data.get(t.dataId).host; }

  override readSync(dataId: object): backend_util.BackendValues {
    const r = this.data.get(dataId);
    if (r.host != null) return r.host.slice();
    const out = util.getTypedArrayFromDType(r.dtype as 'float32', r.nbytes / bytesPerElement(r.dtype));
    binding.read(this.ctx, r.id, out, r.nbytes);
    return out;
  }

  /** The copy is queued behind the kernels launched so far; the promise resolves on a
   *  later turn of the event loop, so code between `data()` and `await` keeps launching. */
  override read(dataId: object): Promise<backend_util.BackendValues> {
    const r = this.data.get(dataId);
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
    r.refCount--;
    if (!force && r.refCount > 0) return false;
    if (r.id !== 0) binding.free(this.ctx, r.id);
    this.data.delete(dataId);
    return true;
  }

  override refCount(dataId: object): number {
    return this.data.has(dataId) ? this.data.get(dataId).refCount : 0;
  }
  override incRef(dataId: object): void { this.data.get(dataId).refCount++; }
  decRef(dataId: object): void { if (this.data.has(dataId)) this.data.get(dataId).refCount--; }
  override numDataIds(): number { return this.data.numDataIds(); }

  /** Zero-copy view: same dataId, one more reference. */
  view(t: TensorInfo, shape: number[], dtype = t.dtype): TensorInfo {
    this.incRef(t.dataId);
    return {dataId: t.dataId, shape, dtype};
  }

  override memory() { return {unreliable: false, ...binding.memory(this.ctx)}; }

  override async time(f: () => void): Promise<BackendTimingInfo> {
    binding.timeBegin(this.ctx);
    f();
    return {kernelMs: binding.timeEnd(this.ctx)};
  }
  override timerAvailable(): boolean { return true; }
  override floatPrecision(): 16|32 { return 32; }
  override epsilon(): number { return 1e-7; }
  setMathMode(mode: 'tf32'|'fp32'): void { binding.setMathMode(this.ctx, mode === 'tf32' ? 0 : 1); }
  override dispose(): void { /* the context is destroyed when the external is collected */ }
}
