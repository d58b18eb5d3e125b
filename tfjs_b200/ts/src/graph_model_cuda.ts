/**
 * Opt-in wrapper around tf.GraphModel for the 'cuda' backend: plan rewrites at load and
 * whole-step replay at execute.  Both sit above the KernelBackend boundary; a model loaded
 * with the stock tf.loadGraphModel runs unchanged on the backend without them.
 *
 *   const model = await loadGraphModelCuda(tfconv, url);
 *   const y = model.execute(x) as tf.Tensor;
 *
 * Replay: GraphModel.execute launches the same kernels with the same shapes at every call
 * (tfjs-converter/src/executor/graph_executor.ts:228-310).  Per input signature the first
 * execute runs eagerly and measures the step's peak memory; the second runs the unmodified
 * executor between captureBegin(arena) and captureEnd, which records every kernel call into
 * a CUDA graph; later executes copy the inputs into the captured input tensors, launch the
 * graph and copy the outputs out.  A step the library cannot capture (a host read in the
 * middle, new weights to pack) stays eager; a graph that went stale (a weight it reads was
 * freed or rewritten) is captured again.
 *
 * Python twin (executed by the tests): GraphModel._execute_replayed / _capture in
 * tfjs_b200/graph_model.py.
 */
import * as tfc from '@tensorflow/tfjs-core';
import {io, NamedTensorMap, Tensor} from '@tensorflow/tfjs-core';

import {CudaBackend} from './backend_cuda';
import {binding} from './binding';
import {registerGraphOps, rewriteArtifacts} from './graph_rewrites';
import {cudaIO} from './io_cuda';

/** The part of tfjs-converter this module uses (passed in, so the package does not pin a
 * converter version): loadGraphModel and registerOp. */
export interface Converter {
  loadGraphModel(url: string|io.IOHandler, options?: {}, tfio?: typeof io): Promise<GraphModelLike>;
  registerOp(name: string, fn: (node: any) => Tensor|Tensor[]): void;
}
export interface GraphModelLike {
  execute(inputs: Tensor|Tensor[]|NamedTensorMap, outputs?: string|string[]): Tensor|Tensor[];
  inputs: Array<{name: string}>;
  dispose(): void;
}

interface Replay {
  state: 'warm'|'ready'|'eager';
  peak: number;
  graph?: number;
  fixed?: NamedTensorMap;
  outs?: Tensor[];
  why?: string;
  arenaRetries: number;
  recaptures: number;
}

let opsRegistered = false;

export async function loadGraphModelCuda(conv: Converter, url: string|io.IOHandler,
                                         options: {replay?: boolean} = {}): Promise<CudaGraphModel> {
  if (!opsRegistered) {
    registerGraphOps(conv.registerOp);
    opsRegistered = true;
  }
  const handler = typeof url === 'string' ? io.getLoadHandlers(url)[0] : url;
  // the handler's artifacts pass through the plan rewrites on their way to the converter
  const rewriting: io.IOHandler = {load: async () => rewriteArtifacts(await handler.load!())};
  const model = await conv.loadGraphModel(rewriting, {}, cudaIO as unknown as typeof io);
  return new CudaGraphModel(model, options.replay ?? true);
}

export class CudaGraphModel {
  private replays = new Map<string, Replay>();
  constructor(readonly model: GraphModelLike, readonly replay: boolean) {}

  private get backend(): CudaBackend { return tfc.engine().backend as CudaBackend; }

  execute(inputs: Tensor|Tensor[]|NamedTensorMap, outputs?: string|string[]): Tensor|Tensor[] {
    if (!this.replay) return this.model.execute(inputs, outputs);
    const named: NamedTensorMap = inputs instanceof Tensor ? {[this.model.inputs[0].name]: inputs} :
        Array.isArray(inputs) ? Object.fromEntries(inputs.map((t, i) => [this.model.inputs[i].name, t])) : inputs;
    const key = JSON.stringify([Object.keys(named).sort().map(n => [n, named[n].shape, named[n].dtype]), outputs]);
    const be = this.backend;
    let st = this.replays.get(key);
    if (st == null) {
      const res = this.eagerStep(named, outputs);
      this.replays.set(key, {state: 'warm', peak: res.peak, arenaRetries: 0, recaptures: 0});
      return res.out;
    }
    if (st.state === 'warm') {
      try {
        this.capture(st, named, outputs);
        st.state = 'ready';
      } catch (e) {
        const msg = String((e as Error).message);
        if (msg.includes('arena') && st.arenaRetries < 2) {
          st.arenaRetries++;
          st.peak = Math.floor(st.peak * 1.6) + (64 << 20);
        } else {
          st.state = 'eager';
        }
        st.why = msg;
      }
    }
    if (st.state !== 'ready') return this.model.execute(named, outputs);
    for (const name of Object.keys(named)) {
      binding.copy(be.ctx, be.deviceId(named[name]), be.deviceId(st.fixed![name]),
                   named[name].size * (named[name].dtype === 'bool' ? 1 : 4));
    }
    try {
      binding.graphLaunch(be.ctx, st.graph!);
    } catch (e) {
      if (!String((e as Error).message).includes('stale')) throw e;
      this.drop(st);
      const again = st.recaptures + 1;
      const res = this.eagerStep(named, outputs);
      Object.assign(st, {state: again <= 3 ? 'warm' : 'eager', peak: res.peak, recaptures: again,
                         graph: undefined, fixed: undefined, outs: undefined});
      return res.out;
    }
    const outs = st.outs!.map(o => {
      const fresh = be.makeOutput(o.shape, o.dtype);
      binding.copy(be.ctx, be.deviceId(o), be.deviceId(fresh), o.size * (o.dtype === 'bool' ? 1 : 4));
      return tfc.engine().makeTensorFromTensorInfo(fresh);
    });
    return Array.isArray(outputs) || outs.length > 1 ? outs : outs[0];
  }

  private eagerStep(named: NamedTensorMap, outputs?: string|string[]): {out: Tensor|Tensor[], peak: number} {
    const be = this.backend;
    binding.highWaterReset(be.ctx);
    const before = binding.memory(be.ctx).numBytesInGPU;
    const out = this.model.execute(named, outputs);
    for (const t of Array.isArray(out) ? out : [out]) be.deviceId(t);      // launch anything still pending
    return {out, peak: Math.max(binding.memory(be.ctx).poolHighWater - before, 0)};
  }

  private capture(st: Replay, named: NamedTensorMap, outputs?: string|string[]): void {
    const be = this.backend;
    const fixed: NamedTensorMap = {};
    for (const name of Object.keys(named)) {
      const info = be.makeOutput(named[name].shape, named[name].dtype);
      fixed[name] = tfc.engine().makeTensorFromTensorInfo(info);
      binding.copy(be.ctx, be.deviceId(named[name]), be.deviceId(info),
                   named[name].size * (named[name].dtype === 'bool' ? 1 : 4));
    }
    let outs: Tensor[]|null = null;
    binding.captureBegin(be.ctx, Math.floor(st.peak * 1.25) + (4 << 20));
    try {
      const res = this.model.execute(fixed, outputs);
      outs = Array.isArray(res) ? res : [res];
      for (const t of outs) be.deviceId(t);
      st.graph = binding.captureEnd(be.ctx, 0);
    } catch (e) {
      try { binding.captureEnd(be.ctx, 1); } catch (_) { /* already discarded */ }
      (outs ?? []).forEach(t => t.dispose());
      Object.values(fixed).forEach(t => t.dispose());
      throw e;
    }
    st.fixed = fixed;
    st.outs = outs;
  }

  private drop(st: Replay): void {
    if (st.state !== 'ready') return;
    st.outs!.forEach(t => t.dispose());
    Object.values(st.fixed!).forEach(t => t.dispose());
    binding.graphDestroy(this.backend.ctx, st.graph!);
  }

  dispose(): void {
    this.replays.forEach(st => this.drop(st));
    this.replays.clear();
    this.model.dispose();
  }
}
