/**
 * Deferred launches: kernels whose result exists as a tensor before anything ran.
 *
 * A FusedConv2D / depthwise convolution with a linear activation, the float32 unary and
 * binary elementwise kernels and Tile return a tensor whose record carries one of the
 * classes below instead of a device buffer.  The launch happens when the tensor is first
 * read or consumed by a kernel that cannot absorb it; until then a following Add / Relu /
 * clip folds into the convolution's epilogue, elementwise kernels chain into one pass, and
 * a batch normalisation indexes an untiled tensor.  Every fp32 rounding step of the
 * separate kernels is kept, so the results do not change.
 *
 * Python twin (executed by the tests): the Pending* classes of tfjs_b200/backend.py.
 */
import {util} from '@tensorflow/tfjs-core';

import type {CudaBackend} from './backend_cuda';
import {ACTIVATION, BINARY_OP, binding, DTYPE, EW, i64, packEwProgram, UNARY_OP} from './binding';

/** What tf.profile would have recorded for a kernel that was folded into a launch. */
export interface Desc {
  name: string;
  inputShapes: {[k: string]: number[]};
  outputShapes: number[][];
}

export interface Pending {
  desc: Desc[];
  /** dataIds that must stay alive until the launch happened or the tensor was dropped. */
  deps(): object[];
  launch(backend: CudaBackend, outDev: number): void;
}

function setActivation(params: ArrayBuffer, act: string): ArrayBuffer {
  const p = params.slice(0);
  new DataView(p).setInt32(60, ACTIVATION[act], true);   // tfjs_cuda_conv2d_params.activation
  return p;
}

export class PendingConv implements Pending {
  constructor(
      readonly params: ArrayBuffer, readonly x: object, readonly filter: object,
      readonly bias: object|null, readonly residual: object|null, readonly desc: Desc[],
      readonly act: 'linear'|'relu'|'relu6' = 'linear') {}

  deps(): object[] {
    return [this.x, this.filter, this.bias, this.residual].filter(d => d != null) as object[];
  }
  withAct(act: 'relu'|'relu6', desc: Desc): PendingConv {
    return new PendingConv(this.params, this.x, this.filter, this.bias, this.residual,
                           [...this.desc, desc], act);
  }
  withResidual(residual: object, desc: Desc): PendingConv {
    return new PendingConv(this.params, this.x, this.filter, this.bias, residual,
                           [...this.desc, desc], this.act);
  }
  /**
   * If the input is a depthwise convolution that is still pending and this is the 1x1
   * convolution behind it (the projection of an inverted-residual block), both run as one
   * launch and the depthwise result is never written.  False when the library does not
   * take the shapes.
   */
  private launchWithDepthwise(backend: CudaBackend, outDev: number): boolean {
    const dw = backend.pendingOfId(this.x);
    if (!backend.fuseDepthwiseProject || !(dw instanceof PendingDepthwise)) return false;
    // without a shortcut the trailing activation is the projection's own
    const pw = this.residual == null ? setActivation(this.params, this.act) : this.params;
    // Operands that are pending themselves launch now, and such a launch may, further down,
    // need this very depthwise result and materialise it (a block's output feeds both the
    // next block and that block's shortcut).  So the shortcut and the weights come first,
    // then the depthwise convolution is looked at again, and its input, which it keeps
    // alive, comes last.
    const ids = [dw.filter, dw.bias, this.filter, this.bias, this.residual]
                    .map(d => d != null ? backend.deviceIdOf(d) : 0);
    if (backend.pendingOfId(this.x) !== dw) return false;
    const ok = binding.fusedDepthwiseProject(
        backend.ctx, setActivation(dw.params, dw.act), pw, backend.deviceIdOf(dw.x), ids[0], ids[1],
        ids[2], ids[3], ids[4],
        this.residual != null ? ACTIVATION[this.act] : ACTIVATION['linear'], outDev);
    if (ok && !this.dwFolded) {
      // profile records: the depthwise kernels join this launch, and the convolution no
      // longer reads its input from memory
      const {x: _x, ...rest} = this.desc[0].inputShapes;
      this.desc.splice(0, 1, ...dw.desc, {...this.desc[0], inputShapes: rest});
      this.dwFolded = true;
    }
    return ok;
  }
  private dwFolded = false;

  launch(backend: CudaBackend, outDev: number): void {
    if (this.launchWithDepthwise(backend, outDev)) return;
    const bias = this.bias != null ? backend.deviceIdOf(this.bias) : 0;
    if (this.residual == null) {
      binding.fusedConv2d(backend.ctx, setActivation(this.params, this.act),
                          backend.deviceIdOf(this.x), backend.deviceIdOf(this.filter), bias, 0,
                          outDev);
    } else {
      binding.fusedConv2dResidual(backend.ctx, this.params, backend.deviceIdOf(this.x),
                                  backend.deviceIdOf(this.filter), bias, 0,
                                  backend.deviceIdOf(this.residual), ACTIVATION[this.act], outDev);
    }
  }
}

/** DepthwiseConv2dNative + the biasAdd and Relu / clip that tfjs-layers issues after it
 * (tfjs-layers/src/layers/convolutional_depthwise.ts:154-169). */
export class PendingDepthwise implements Pending {
  constructor(
      readonly params: ArrayBuffer, readonly x: object, readonly filter: object,
      readonly bias: object|null, readonly desc: Desc[],
      readonly act: 'linear'|'relu'|'relu6' = 'linear') {}

  deps(): object[] {
    return [this.x, this.filter, this.bias].filter(d => d != null) as object[];
  }
  withBias(bias: object, biasLen: number, desc: Desc): PendingDepthwise {
    const p = this.params.slice(0);
    new DataView(p).setInt32(64, biasLen, true);          // tfjs_cuda_conv2d_params.bias_len
    return new PendingDepthwise(p, this.x, this.filter, bias, [...this.desc, desc], this.act);
  }
  withAct(act: 'relu'|'relu6', desc: Desc): PendingDepthwise {
    return new PendingDepthwise(this.params, this.x, this.filter, this.bias,
                                [...this.desc, desc], act);
  }
  launch(backend: CudaBackend, outDev: number): void {
    binding.fusedDepthwiseConv2d(
        backend.ctx, setActivation(this.params, this.act), backend.deviceIdOf(this.x),
        backend.deviceIdOf(this.filter), this.bias != null ? backend.deviceIdOf(this.bias) : 0, 0,
        outDev);
  }
}

/**
 * A _FusedMatMul (or its heads-split form) with a fused bias, not launched yet.  When it is
 * launched, the other products still pending on the same `a` operand with the same
 * dimensions (the query, key and value projections of an attention layer) go with it in
 * one `fusedMatMulGroup` launch (CudaBackend.resolveMatMulGroup); each member's result is
 * the one its own launch would give.
 */
export class PendingMatMul implements Pending {
  readonly key: string;
  constructor(
      readonly params: ArrayBuffer, readonly a: object, readonly b: object,
      readonly bias: object|null,
      /** [layout, rowsOrHeads, headDim] of the permuted store, or null */
      readonly heads: [number, number, number]|null, readonly desc: Desc[]) {
    this.key = `${Array.from(new Uint8Array(params)).join(',')}|${heads}|${bias == null}`;
  }
  deps(): object[] { return [this.a, this.b, this.bias].filter(d => d != null) as object[]; }
  launch(backend: CudaBackend, outDev: number): void {
    const bias = this.bias != null ? backend.deviceIdOf(this.bias) : 0;
    if (this.heads == null) {
      binding.fusedMatMul(backend.ctx, this.params, backend.deviceIdOf(this.a),
                          backend.deviceIdOf(this.b), bias, 0, outDev);
    } else {
      binding.fusedMatMulHeads(backend.ctx, this.params, backend.deviceIdOf(this.a),
                               backend.deviceIdOf(this.b), bias, 0, this.heads[0], this.heads[1],
                               this.heads[2], outDev);
    }
  }
}

/** A Tile that a consumer able to index the untiled tensor never materialises (the
 * batch normalisation behind tfjs-layers' LayerNormalization). */
export class PendingTile implements Pending {
  constructor(
      readonly src: object, readonly srcShape: number[], readonly reps: number[],
      readonly shape: number[], readonly dtype: string, readonly desc: Desc[]) {}

  deps(): object[] { return [this.src]; }
  launch(backend: CudaBackend, outDev: number): void {
    const strides = (s: number[]) => s.map((_, i) => s.slice(i + 1).reduce((a, b) => a * b, 1));
    binding.copyStrided(backend.ctx, this.dtype === 'bool' ? 1 : 4, this.shape.length,
                        i64(this.shape), backend.deviceIdOf(this.src), 0, i64(strides(this.srcShape)),
                        i64(this.srcShape), outDev, 0, i64(strides(this.shape)));
  }
}

/** Operand reference inside a chain: leaf k, or the result of op j. */
export type Ref = ['in', number]|['op', number];
export type EwOp = [number, Ref, Ref];

const COMMUTATIVE = new Set([BINARY_OP.Add, BINARY_OP.Multiply, BINARY_OP.Maximum,
                             BINARY_OP.Minimum, BINARY_OP.SquaredDifference]);

/**
 * Canonical form of a chain: operands of commutative ops ordered by a structural key, ops
 * emitted in evaluation order from the result, leaves numbered by first use, a value used
 * twice emitted once.  The library's catalogue of straight-line chain kernels is written
 * in this form.
 */
export function canonicalProgram(ops: EwOp[], leafModes: number[]): {ops: EwOp[], leafOrder: number[]} {
  const keys = new Map<string, string>();
  const id = (r: Ref) => `${r[0]}${r[1]}`;
  const key = (r: Ref): string => {
    let k = keys.get(id(r));
    if (k == null) {
      if (r[0] === 'in') {
        k = `L${leafModes[r[1]]}`;
      } else {
        const [code, a, b] = ops[r[1]];
        if (code >= EW.UNARY) {
          k = `(${code} ${key(a)})`;
        } else {
          let ka = key(a), kb = key(b);
          if (COMMUTATIVE.has(code) && kb < ka) [ka, kb] = [kb, ka];
          k = `(${code} ${ka} ${kb})`;
        }
      }
      keys.set(id(r), k);
    }
    return k;
  };
  const out: EwOp[] = [];
  const leafOrder: number[] = [];
  const done = new Map<string, Ref>();
  const emit = (r: Ref): Ref => {
    let res = done.get(id(r));
    if (res == null) {
      if (r[0] === 'in') {
        leafOrder.push(r[1]);
        res = ['in', leafOrder.length - 1];
      } else {
        let [code, a, b] = ops[r[1]];
        let ra: Ref, rb: Ref;
        if (code >= EW.UNARY) {
          ra = rb = emit(a);
        } else {
          if (COMMUTATIVE.has(code) && key(b) < key(a)) [a, b] = [b, a];
          ra = emit(a);
          rb = emit(b);
        }
        out.push([code, ra, rb]);
        res = ['op', out.length - 1];
      }
      done.set(id(r), res);
    }
    return res;
  };
  emit(['op', ops.length - 1]);
  return {ops: out, leafOrder};
}

/** A chain of float32 elementwise kernels (PendingEw of tfjs_b200/backend.py). */
export class PendingEw implements Pending {
  consumed = 0;
  constructor(
      readonly leaves: object[], readonly leafShapes: number[][], readonly ops: EwOp[],
      readonly shape: number[], readonly desc: Desc[],
      /** the kernel call that made this tensor: opcode, operands and their shapes */
      readonly top: {code: number, a: object, aShape: number[], b: object|null, bShape: number[]|null},
      readonly depth = 1) {}

  deps(): object[] {
    const out = [...this.leaves];
    for (const d of [this.top.a, this.top.b]) if (d != null && !out.includes(d)) out.push(d);
    return out;
  }

  /** True when every leaf is smaller than the result: recomputing costs no memory pass. */
  cheap(): boolean {
    const n = util.sizeFromShape(this.shape);
    return this.ops.length <= 2 && this.leafShapes.every(s => util.sizeFromShape(s) < n);
  }

  /** [mode, period, aux] of a leaf relative to the result's flat index, or null. */
  private leafMode(shape: number[]): [number, number, number]|null {
    const out = this.shape, rank = out.length;
    const n = util.sizeFromShape(out), m = util.sizeFromShape(shape);
    if (shape.length > rank) return null;
    const sh = new Array(rank - shape.length).fill(1).concat(shape);
    const eq = (a: number[], b: number[]) => a.length === b.length && a.every((v, i) => v === b[i]);
    if (m === 1) return [EW.SCALAR, 1, 0];
    if (m === n) return [EW.FULL, 0, 0];
    let d = 0;
    while (d < rank && sh[d] === 1) ++d;
    if (eq(sh.slice(d), out.slice(d))) return [EW.PERIODIC, m, 0];
    if (rank >= 1 && sh[rank - 1] === 1 && eq(sh.slice(0, -1), out.slice(0, -1))) return [EW.ROW, 0, 0];
    let p = 0;
    while (p < rank && sh[p] === out[p]) ++p;
    let q = p;
    while (q < rank && sh[q] === 1) ++q;
    if (p > 0 && p < q && q < rank && eq(sh.slice(q), out.slice(q))) {
      const inner = util.sizeFromShape(out.slice(q));
      return [EW.BATCHED, inner, inner * util.sizeFromShape(out.slice(p, q))];
    }
    return null;
  }

  launch(backend: CudaBackend, outDev: number): void {
    const n = util.sizeFromShape(this.shape);
    const modes = this.leafShapes.map(s => this.leafMode(s));
    if (this.ops.length === 1 || n >= 2 ** 31 || modes.some(m => m == null)) {
      return this.launchTop(backend, outDev);
    }
    // Add (+ Relu / Relu6) of two full tensors has a kernel of its own
    const relu = EW.UNARY + UNARY_OP.Relu, relu6 = EW.UNARY + UNARY_OP.Relu6;
    if (this.leaves.length === 2 && modes.every(m => m![0] === EW.FULL) && this.ops.length === 2 &&
        this.ops[0][0] === BINARY_OP.Add && this.ops[0][1][0] === 'in' && this.ops[0][2][0] === 'in' &&
        this.ops[0][1][1] !== this.ops[0][2][1] && (this.ops[1][0] === relu || this.ops[1][0] === relu6)) {
      binding.addActivation(backend.ctx, ACTIVATION[this.ops[1][0] === relu ? 'relu' : 'relu6'],
                            backend.deviceIdOf(this.leaves[0]), backend.deviceIdOf(this.leaves[1]), n,
                            outDev);
      return;
    }
    const {ops, leafOrder} = canonicalProgram(this.ops, modes.map(m => m![0]));
    const slot = (r: Ref) => r[0] === 'in' ? r[1] : leafOrder.length + r[1];
    const packed = ops.map(([code, a, b]) => ({opcode: code, a: slot(a), b: slot(b)}));
    const signature = packed.map(o => `${o.opcode}:${o.a}:${o.b}`).join(',');
    let known = backend.ewCatalogue.get(signature);
    const cols = Math.max(this.shape.length ? this.shape[this.shape.length - 1] : 1, 1);
    if (known == null) {
      known = binding.fusedElementwiseCatalogued(
                  backend.ctx, packEwProgram({n, cols, inputs: [], ops: packed})) !== 0;
      backend.ewCatalogue.set(signature, known);
    }
    if (!known) return this.launchTop(backend, outDev);
    const inputs = leafOrder.map(leaf => ({
      id: backend.deviceIdOf(this.leaves[leaf]), mode: modes[leaf]![0], period: modes[leaf]![1],
      aux: modes[leaf]![2]
    }));
    binding.fusedElementwise(backend.ctx, packEwProgram({n, cols, inputs, ops: packed}), outDev);
  }

  /** The separate kernel of the call that made this tensor, on its operand tensors (whose
   * own pending launches happen first): nothing is ever computed twice. */
  private launchTop(backend: CudaBackend, outDev: number): void {
    const {code, a, aShape, b, bShape} = this.top;
    const last = this.desc[this.desc.length - 1];
    this.desc.length = 0;
    this.desc.push({...last, inputShapes: b != null ? {a: aShape, b: bShape!} : {x: aShape}});
    if (code >= EW.UNARY) {
      binding.unary(backend.ctx, code - EW.UNARY, 0, 0, backend.deviceIdOf(a),
                    util.sizeFromShape(this.shape), outDev);
      return;
    }
    const rank = this.shape.length;
    const pad = (s: number[]) => i64(new Array(rank - s.length).fill(1).concat(s));
    binding.binary(backend.ctx, code, DTYPE['float32'], rank, backend.deviceIdOf(a), pad(aShape),
                   backend.deviceIdOf(b!), pad(bShape!), outDev, i64(this.shape));
  }
}
