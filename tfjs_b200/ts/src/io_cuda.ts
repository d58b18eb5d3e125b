/**
 * An `io` namespace whose decodeWeights / decodeWeightsStream hand the weight bytes to the
 * library's loader (tfjs_cuda_weights_begin / push / end): pinned staging, one async copy
 * per piece, uint8 / uint16 affine-quantised and float16-stored entries decoded on the GPU
 * once, at load, so they cross PCIe at 1-2 bytes per value.  GraphModel takes the io
 * namespace as a constructor argument and calls `this.io.decodeWeights`
 * (tfjs-converter/src/executor/graph_model.ts:104-107, :177):
 *
 *     const model = await tf.loadGraphModel(url, {}, cudaIO);
 *
 * `loadWeightFiles` reads the shard files named by weightsManifest[].paths inside the
 * library (pread straight into the pinned ring).  Python twin: WeightsLoader in
 * tfjs_b200/io.py.
 */
import {DataType, engine, io, NamedTensorMap, Tensor, util} from '@tensorflow/tfjs-core';

import {CudaBackend} from './backend_cuda';
import {binding, DTYPE, packWeightSpecs, WEIGHT_STORAGE} from './binding';

const HOST_RESIDENT_BYTES = 4096;

interface Entry { n: number; storage: number; dtype: number; scale: number; min: number; skip: boolean;
                  offset: number; nbytes: number; }

/** Storage kind and stored bytes of a manifest entry, with the checks of decodeWeight
 * (tfjs-core/src/io/io_utils.ts:196-218, :269-272). */
function entryOf(spec: io.WeightsManifestEntry, offset: number): Entry {
  const n = util.sizeFromShape(spec.shape);
  const q = spec.quantization;
  let storage = WEIGHT_STORAGE.raw, nbytes: number;
  if (q != null) {
    if (q.dtype === 'uint8' || q.dtype === 'uint16') {
      if (q.min == null || q.scale == null) {
        throw new Error(`Weight ${spec.name} with quantization ${q.dtype} ` +
                        `doesn't have corresponding metadata min and scale.`);
      }
      if (spec.dtype !== 'float32' && spec.dtype !== 'int32') {
        throw new Error(`Unsupported dtype in weight '${spec.name}': ${spec.dtype}`);
      }
      storage = q.dtype === 'uint8' ? WEIGHT_STORAGE.uint8 : WEIGHT_STORAGE.uint16;
      nbytes = n * (q.dtype === 'uint8' ? 1 : 2);
    } else if (q.dtype === 'float16') {
      if (spec.dtype !== 'float32') {
        throw new Error(`Weight ${spec.name} is quantized with ${q.dtype} which only supports ` +
                        `weights of type float32 not ${spec.dtype}.`);
      }
      storage = WEIGHT_STORAGE.float16;
      nbytes = n * 2;
    } else {
      throw new Error(`Weight ${spec.name} has unknown quantization dtype ${q.dtype}. ` +
                      `Supported quantization dtypes are: 'uint8', 'uint16', and 'float16'.`);
    }
  } else {
    if (spec.dtype !== 'float32' && spec.dtype !== 'int32' && spec.dtype !== 'bool') {
      throw new Error(`Unsupported dtype in weight '${spec.name}': ${spec.dtype}`);
    }
    nbytes = n * (spec.dtype === 'bool' ? 1 : 4);
  }
  // small entries stored in their own dtype stay on the host (shape / axis constants)
  const skip = storage === WEIGHT_STORAGE.raw && nbytes <= HOST_RESIDENT_BYTES;
  return {n, storage, dtype: DTYPE[spec.dtype], scale: q?.scale ?? 1, min: q?.min ?? 0, skip, offset, nbytes};
}

class WeightsLoader {
  private entries: Entry[] = [];
  private host = new Map<number, Uint8Array>();
  private handle: number;
  private pushed = 0;
  private backend = engine().backend as CudaBackend;

  constructor(private specs: io.WeightsManifestEntry[]) {
    let offset = 0;
    specs.forEach((spec, i) => {
      const e = entryOf(spec, offset);
      this.entries.push(e);
      if (e.skip) this.host.set(i, new Uint8Array(e.nbytes));
      offset += e.nbytes;
    });
    this.handle = binding.weightsBegin(this.backend.ctx, packWeightSpecs(this.entries));
  }

  /** One piece of the concatenated weight bytes, cut anywhere. */
  push(chunk: ArrayBuffer|Uint8Array): void {
    const view = chunk instanceof Uint8Array ? chunk : new Uint8Array(chunk);
    if (view.length === 0) return;
    try {
      binding.weightsPush(this.backend.ctx, this.handle, view);
    } catch (e) {
      this.abandon();
      throw e;
    }
    const base = this.pushed, end = base + view.length;
    this.host.forEach((bytes, i) => {             // the parts that belong to host-resident entries
      const off = this.entries[i].offset, lo = Math.max(off, base), hi = Math.min(off + bytes.length, end);
      if (lo < hi) bytes.set(view.subarray(lo - base, hi - base), lo - off);
    });
    this.pushed = end;
  }

  abandon(): void {
    if (this.handle !== 0) {
      const h = this.handle;
      this.handle = 0;
      try { binding.weightsEnd(this.backend.ctx, h, null); } catch (_) { /* already released */ }
    }
  }

  finish(): NamedTensorMap {
    const ids = new Int32Array(Math.max(this.specs.length, 1));
    const h = this.handle;
    this.handle = 0;
    binding.weightsEnd(this.backend.ctx, h, ids);
    const out: NamedTensorMap = {};
    this.specs.forEach((spec, i) => {
      const bytes = this.host.get(i);
      if (bytes != null) {
        Object.assign(out, io.decodeWeights(bytes.buffer.slice(bytes.byteOffset, bytes.byteOffset + bytes.length),
                                            [spec]));
      } else {
        const info = this.backend.adopt(ids[i], spec.shape, spec.dtype as DataType);
        out[spec.name] = engine().makeTensorFromTensorInfo(info) as Tensor;
      }
    });
    return out;
  }
}

function decodeWeights(weightData: io.WeightData, specs: io.WeightsManifestEntry[]): NamedTensorMap {
  const loader = new WeightsLoader(specs);
  for (const shard of weightData instanceof ArrayBuffer ? [weightData] : weightData as ArrayBuffer[]) {
    loader.push(shard);
  }
  return loader.finish();
}

/** decodeWeightsStream (io_utils.ts:316-353): every chunk goes to the device loader as it
 * arrives. */
async function decodeWeightsStream(weightStream: ReadableStream<ArrayBuffer>,
                                   specs: io.WeightsManifestEntry[]): Promise<NamedTensorMap> {
  const loader = new WeightsLoader(specs);
  const reader = weightStream.getReader();
  try {
    for (;;) {
      const {done, value} = await reader.read();
      if (done) break;
      loader.push(value);
    }
  } catch (e) {
    loader.abandon();
    throw e;
  }
  return loader.finish();
}

/** The shards of a weights group read from disk by the library itself, in the order of
 * weightsManifest[].paths (weights_loader.ts:38-131 fetches and concatenates them).  Entries
 * kept on the host are read from the files here. */
export function loadWeightFiles(paths: string[], specs: io.WeightsManifestEntry[]): NamedTensorMap {
  // tslint:disable-next-line:no-require-imports
  const fs = require('fs');
  const loader = new WeightsLoader(specs);
  const backend = engine().backend as CudaBackend;
  const anyLoader = loader as unknown as {handle: number, pushed: number, host: Map<number, Uint8Array>,
                                          entries: Entry[]};
  for (const path of paths) {
    try {
      binding.weightsPushFile(backend.ctx, anyLoader.handle, path);
    } catch (e) {
      loader.abandon();
      throw e;
    }
    const size = fs.statSync(path).size as number, base = anyLoader.pushed, end = base + size;
    const fd = fs.openSync(path, 'r');
    anyLoader.host.forEach((bytes, i) => {
      const off = anyLoader.entries[i].offset, lo = Math.max(off, base), hi = Math.min(off + bytes.length, end);
      if (lo < hi) fs.readSync(fd, bytes, lo - off, hi - lo, lo - base);
    });
    fs.closeSync(fd);
    anyLoader.pushed = end;
  }
  return loader.finish();
}

export const cudaIO = {...io, decodeWeights, decodeWeightsStream};
