/**
 * Plan rewrites for converted graphs, applied to the model.json topology before the
 * unmodified tfjs-converter sees it, with the new node types executed through the
 * converter's public custom-op registry (registerOp,
 * tfjs-converter/src/operations/custom_op/register.ts:48).  The converter's own graph passes
 * produce _FusedConv2D / _FusedMatMul the same way, at conversion time.
 *
 *   fuseLayerNorms      Mean, SquaredDifference, Mean, AddV2(eps), Rsqrt, Sub, Mul, Mul, AddV2
 *                       (+ the AddV2 of the residual connection in front) -> _FusedLayerNorm
 *   fuseAttentionHeads  matMul + Reshape + Transpose([0,2,1,3]) and batchMatMul + Transpose +
 *                       Reshape -> _MatMulHeads
 *   fuseSoftmaxInputs   Softmax(AddV2(Mul(scores, c), mask)) -> _SoftmaxScaledMasked
 *   fuseGeluIntoMatMul  _FusedMatMul + the five nodes of the erf GELU -> _FusedMatMulGelu
 *   fuseAttention       _MatMulHeads(merge)(softmax(batchMatMul(q, k, adj_y) ...), v) -> _FusedAttention
 *   hoistSharedOperandMatMuls  products on one operand run next to each other, so that the
 *                       backend launches them as a group
 *
 * A subgraph is replaced only if its intermediates have no consumer outside it and are not
 * among the model's signature outputs; the new node keeps the name of the subgraph's last
 * node.  Every custom op falls back to the stored ops for shapes its kernel does not take.
 * These rewrites sit ABOVE the KernelBackend boundary: a user opts in by loading the model
 * through `loadGraphModelCuda` (graph_model_cuda.ts) instead of tf.loadGraphModel.
 *
 * Python twin (executed by the tests): fuse_layer_norms / fuse_attention_heads /
 * fuse_softmax_inputs / fuse_gelu_into_matmul / fuse_attention and the _exec_* functions of
 * tfjs_b200/graph_model.py.
 */
import * as tfc from '@tensorflow/tfjs-core';
import {io, Tensor} from '@tensorflow/tfjs-core';

import {layerNormSupported, softmaxMaskRows} from './kernels/fused_graph_ops';

interface NodeDef { name: string; op: string; input?: string[]; attr?: {[k: string]: any}; }
type Consts = Map<string, {shape: number[], values: () => number[]}>;

const b64 = (s: string) => Buffer.from(s).toString('base64');
const nodeName = (inp: string) => inp.split(':')[0];
const isFirstOutput = (inp: string) => !inp.includes(':') || inp.endsWith(':0');

/** Small constants of the graph (axes, perms, shapes, scalars), decoded on the host. */
export function smallConstants(artifacts: io.ModelArtifacts): Consts {
  const out: Consts = new Map();
  const data = artifacts.weightData instanceof ArrayBuffer ? artifacts.weightData :
      io.concatenateArrayBuffers(artifacts.weightData as ArrayBuffer[]);
  let offset = 0;
  for (const spec of artifacts.weightSpecs ?? []) {
    const n = spec.shape.reduce((a, b) => a * b, 1);
    const q = spec.quantization;
    const bytes = n * (q ? (q.dtype === 'uint8' ? 1 : 2) : spec.dtype === 'bool' ? 1 : 4);
    const start = offset;
    offset += bytes;
    if (q != null || n > 64 || (spec.dtype !== 'float32' && spec.dtype !== 'int32')) continue;
    out.set(spec.name, {
      shape: spec.shape,
      values: () => Array.from(spec.dtype === 'int32' ? new Int32Array(data.slice(start, start + bytes)) :
                                                        new Float32Array(data.slice(start, start + bytes)))
    });
  }
  return out;
}

class Graph {
  byName = new Map<string, NodeDef>();
  consumers = new Map<string, string[]>();
  constructor(readonly nodes: NodeDef[], readonly consts: Consts, readonly protectedNames: Set<string>) {
    for (const n of nodes) this.byName.set(n.name, n);
    for (const n of nodes) {
      for (const i of (n.input ?? []).filter(s => !s.startsWith('^'))) {
        const k = nodeName(i);
        this.consumers.set(k, [...(this.consumers.get(k) ?? []), n.name]);
      }
    }
  }
  node(inp: string, ops?: string[]): NodeDef|null {
    const n = this.byName.get(nodeName(inp));
    return n != null && isFirstOutput(inp) && (ops == null || ops.includes(n.op)) ? n : null;
  }
  isConst(inp: string): boolean {
    const n = this.node(inp, ['Const']);
    return n != null && this.consts.has(n.name);
  }
  values(inp: string): number[]|null { return this.isConst(inp) ? this.consts.get(nodeName(inp))!.values() : null; }
  scalar(inp: string): number|null {
    const v = this.values(inp);
    return v != null && v.length === 1 ? Math.fround(v[0]) : null;
  }
  only(n: NodeDef, users: NodeDef[]): boolean {
    const have = [...(this.consumers.get(n.name) ?? [])].sort();
    const want = users.map(u => u.name).sort();
    return !this.protectedNames.has(n.name) && have.length === want.length && have.every((v, i) => v === want[i]);
  }
  /** The two inputs of a commutative node as [a, b] with a and b matching the predicates. */
  split(n: NodeDef, wantA: (i: string) => boolean, wantB: (i: string) => boolean): [string, string]|null {
    const ins = n.input ?? [];
    if (ins.length !== 2) return null;
    for (const [a, b] of [[ins[0], ins[1]], [ins[1], ins[0]]]) if (wantA(a) && wantB(b)) return [a, b];
    return null;
  }
}

function apply(nodes: NodeDef[], removed: Set<string>, replaced: Map<string, NodeDef>): NodeDef[] {
  return nodes.filter(n => !removed.has(n.name)).map(n => replaced.get(n.name) ?? n);
}

export function fuseLayerNorms(nodes: NodeDef[], consts: Consts, prot: Set<string>): NodeDef[] {
  const g = new Graph(nodes, consts, prot);
  const ADD = ['Add', 'AddV2'];
  const lastAxisMean = (n: NodeDef|null) => {
    if (n == null || n.op !== 'Mean' || (n.input ?? []).length !== 2 || !n.attr?.['keep_dims']?.b) return false;
    const axes = g.values(n.input![1]);
    return axes != null && axes.length === 1 && axes[0] === -1;
  };
  const removed = new Set<string>(), replaced = new Map<string, NodeDef>();
  for (const out of nodes) {
    if (!ADD.includes(out.op)) continue;
    let ab = g.split(out, i => g.node(i, ['Mul']) != null, i => g.isConst(i));
    if (!ab) continue;
    const m2 = g.node(ab[0])!, beta = ab[1];
    ab = g.split(m2, i => g.node(i, ['Mul']) != null, i => g.isConst(i));
    if (!ab) continue;
    const norm = g.node(ab[0])!, gamma = ab[1];
    ab = g.split(norm, i => g.node(i, ['Sub']) != null, i => g.node(i, ['Rsqrt']) != null);
    if (!ab) continue;
    const sub = g.node(ab[0])!, rs = g.node(ab[1])!;
    if ((sub.input ?? []).length !== 2) continue;
    const xIn = sub.input![0], mean = g.node(sub.input![1]);
    if (!lastAxisMean(mean) || mean!.input![0] !== xIn) continue;
    const add = g.node(rs.input![0], ADD);
    if (add == null) continue;
    ab = g.split(add, i => lastAxisMean(g.node(i)), i => g.isConst(i));
    if (!ab) continue;
    const variance = g.node(ab[0])!, eps = g.scalar(ab[1]);
    const sq = g.node(variance.input![0], ['SquaredDifference']);
    if (sq == null || eps == null || [...sq.input!].sort().join() !== [xIn, mean!.name].sort().join()) continue;
    const gShape = consts.get(nodeName(gamma))!.shape, bShape = consts.get(nodeName(beta))?.shape;
    if (gShape.length !== 1 || bShape == null || bShape.length !== 1 || bShape[0] !== gShape[0]) continue;
    const inner = [mean!, sq, variance, add, rs, sub, norm, m2];
    if (new Set(inner.map(n => n.name)).size !== inner.length || inner.some(n => removed.has(n.name))) continue;
    if (!(g.only(mean!, [sq, sub]) && g.only(sq, [variance]) && g.only(variance, [add]) && g.only(add, [rs]) &&
          g.only(rs, [norm]) && g.only(sub, [norm]) && g.only(norm, [m2]) && g.only(m2, [out]))) continue;
    inner.forEach(n => removed.add(n.name));
    const attr: {[k: string]: any} = {epsilon: {f: eps}};
    let input = [xIn, gamma, beta];
    const xn = g.node(xIn, ADD);
    if (xn != null && (xn.input ?? []).length === 2 && !removed.has(xn.name) && g.only(xn, [mean!, sq, sub])) {
      removed.add(xn.name);
      input = [xn.input![0], xn.input![1], gamma, beta];
      attr['residual'] = {b: true};
    }
    replaced.set(out.name, {name: out.name, op: '_FusedLayerNorm', input, attr});
  }
  return apply(nodes, removed, replaced);
}

export function fuseAttentionHeads(nodes: NodeDef[], consts: Consts, prot: Set<string>): NodeDef[] {
  const g = new Graph(nodes, consts, prot);
  const MATMULS = ['_FusedMatMul', 'MatMul', 'BatchMatMul', 'BatchMatMulV2'];
  const isHeadsPerm = (inp: string) => (g.values(inp) ?? []).join() === '0,2,1,3';
  const removed = new Set<string>(), replaced = new Map<string, NodeDef>();
  for (const last of nodes) {
    let mm: NodeDef|null = null, mid: NodeDef|null = null, dims: number[]|null = null, layout = '';
    if (last.op === 'Transpose' && (last.input ?? []).length === 2 && isHeadsPerm(last.input![1])) {
      mid = g.node(last.input![0], ['Reshape']);                                    // heads split
      mm = mid != null ? g.node(mid.input![0], MATMULS) : null;
      dims = mid != null ? g.values(mid.input![1]) : null;
      layout = 'split';
    } else if (last.op === 'Reshape' && (last.input ?? []).length === 2) {
      mid = g.node(last.input![0], ['Transpose']);                                  // heads merge
      mm = mid != null && isHeadsPerm(mid.input![1]) ? g.node(mid.input![0], MATMULS) : null;
      dims = g.values(last.input![1]);
      layout = 'merge';
    }
    if (mm == null || mid == null || dims == null || dims.some(d => d <= 0) ||
        (layout === 'split' && dims.length !== 4) || removed.has(mm.name) || !g.only(mm, [mid]) ||
        !g.only(mid, [last])) {
      continue;
    }
    removed.add(mm.name);
    removed.add(mid.name);
    replaced.set(last.name, {
      name: last.name, op: '_MatMulHeads', input: [...(mm.input ?? [])],
      attr: {...(mm.attr ?? {}), _layout: {s: b64(layout)}, _op: {s: b64(mm.op)},
             _dims: {list: {i: dims.map(String)}}}
    });
  }
  return apply(nodes, removed, replaced);
}

export function fuseSoftmaxInputs(nodes: NodeDef[], consts: Consts, prot: Set<string>): NodeDef[] {
  const g = new Graph(nodes, consts, prot);
  const scaled = (inp: string): {scores: string, scale: number, mul: NodeDef}|null => {
    const m = g.node(inp, ['Mul']);
    if (m == null || (m.input ?? []).length !== 2) return null;
    for (const [a, b] of [[m.input![0], m.input![1]], [m.input![1], m.input![0]]]) {
      const c = g.scalar(b);
      if (c != null && g.scalar(a) == null) return {scores: a, scale: c, mul: m};
    }
    return null;
  };
  const removed = new Set<string>(), replaced = new Map<string, NodeDef>();
  for (const sm of nodes) {
    if (sm.op !== 'Softmax' || (sm.input ?? []).length !== 1) continue;
    let input: string[]|null = null, scale = 1, gone: NodeDef[] = [];
    const add = g.node(sm.input![0], ['Add', 'AddV2']);
    if (add != null && (add.input ?? []).length === 2 && g.only(add, [sm])) {
      for (const [a, b] of [[add.input![0], add.input![1]], [add.input![1], add.input![0]]]) {
        const sc = scaled(a);
        if (sc != null && g.only(sc.mul, [add])) { input = [sc.scores, b]; scale = sc.scale; gone = [add, sc.mul]; break; }
      }
    } else {
      const sc = scaled(sm.input![0]);
      if (sc != null && g.only(sc.mul, [sm])) { input = [sc.scores]; scale = sc.scale; gone = [sc.mul]; }
    }
    if (input == null) continue;
    gone.forEach(n => removed.add(n.name));
    replaced.set(sm.name, {name: sm.name, op: '_SoftmaxScaledMasked', input, attr: {_scale: {f: scale}}});
  }
  return apply(nodes, removed, replaced);
}

/**
 * h = _FusedMatMul(a, b, bias) (no activation) followed by the erf GELU a converted graph
 * spells as Mul(Mul(h, half), AddV2(Erf(Mul(h, scale)), one)) (or Erf(RealDiv(h, scale))), with
 * scalar constants and h consumed by those two products only, becomes that product with the
 * GELU as its epilogue (`_FusedMatMulGelu`, named like the final Mul).  The epilogue performs
 * the same fp32 operations on the same h, so the bits do not change.
 * Python twin: fuse_gelu_into_matmul (tfjs_b200/graph_model.py).
 */
export function fuseGeluIntoMatMul(nodes: NodeDef[], consts: Consts, prot: Set<string>): NodeDef[] {
  const g = new Graph(nodes, consts, prot);
  /** [other input, constant] of a two-input node one of whose inputs is a scalar constant. */
  const withConst = (n: NodeDef|null, commutative = true): [string, number]|null => {
    const ins = n?.input ?? [];
    if (n == null || ins.length !== 2) return null;
    const pairs = commutative ? [[ins[0], ins[1]], [ins[1], ins[0]]] : [[ins[0], ins[1]]];
    for (const [a, b] of pairs) {
      const c = g.scalar(b);
      if (c != null && g.scalar(a) == null) return [a, c];
    }
    return null;
  };
  const removed = new Set<string>(), replaced = new Map<string, NodeDef>();
  for (const out of nodes) {
    if (out.op !== 'Mul' || (out.input ?? []).length !== 2) continue;
    for (const [mi, ai] of [[out.input![0], out.input![1]], [out.input![1], out.input![0]]]) {
      const m2 = g.node(mi, ['Mul']), add = g.node(ai, ['Add', 'AddV2']);
      const hm = withConst(m2), ea = withConst(add);
      if (m2 == null || add == null || hm == null || ea == null) continue;
      const erf = g.node(ea[0], ['Erf']);
      if (erf == null) continue;
      const inner = g.node(erf.input![0], ['Mul', 'RealDiv', 'Div']);
      const hs = withConst(inner, inner != null && inner.op === 'Mul');
      if (inner == null || hs == null || hs[0] !== hm[0]) continue;
      const mm = g.node(hm[0], ['_FusedMatMul']);
      if (mm == null || removed.has(mm.name)) continue;
      const fused = ((mm.attr?.['fused_ops']?.list?.s ?? []) as string[])
                        .map(x => Buffer.from(x, 'base64').toString().toLowerCase());
      if (fused.join() !== 'biasadd' || Number(mm.attr?.['num_args']?.i ?? 0) !== 1) continue;
      if (!g.only(mm, [m2, inner]) || !g.only(m2, [out]) || !g.only(add, [out]) || !g.only(erf, [add]) ||
          !g.only(inner, [erf])) {
        continue;
      }
      [mm, m2, add, erf, inner].forEach(n => removed.add(n.name));
      replaced.set(out.name, {
        name: out.name, op: '_FusedMatMulGelu', input: [...(mm.input ?? [])],
        attr: {...(mm.attr ?? {}), _gelu: {list: {f: [hs[1], hm[1], ea[1], inner.op !== 'Mul' ? 1 : 0]}}}
      });
      break;
    }
  }
  return apply(nodes, removed, replaced);
}

/**
 * The heads-merging product of softmax(scores) and v, with scores = batchMatMul(q, k, adj_y)
 * (scaled and masked on the way into the softmax or not), becomes one
 * _FusedAttention(q, k, v[, mask]; _scale) node named like the merge.  Runs after
 * fuseAttentionHeads and fuseSoftmaxInputs, whose nodes it matches.
 * Python twin: fuse_attention (tfjs_b200/graph_model.py).
 */
export function fuseAttention(nodes: NodeDef[], consts: Consts, prot: Set<string>): NodeDef[] {
  const g = new Graph(nodes, consts, prot);
  const str = (n: NodeDef, key: string) => Buffer.from(n.attr?.[key]?.s ?? '', 'base64').toString();
  const flag = (n: NodeDef, key: string) => !!n.attr?.[key]?.b;
  const removed = new Set<string>(), replaced = new Map<string, NodeDef>();
  for (const last of nodes) {
    if (last.op !== '_MatMulHeads' || str(last, '_layout') !== 'merge' || (last.input ?? []).length !== 2 ||
        !str(last, '_op').startsWith('BatchMatMul') || flag(last, 'adj_x') || flag(last, 'adj_y')) {
      continue;
    }
    const sm = g.node(last.input![0], ['_SoftmaxScaledMasked', 'Softmax']);
    if (sm == null || !g.only(sm, [last]) || (sm.input ?? []).length < 1 || (sm.input ?? []).length > 2) continue;
    const sc = g.node(sm.input![0], ['BatchMatMul', 'BatchMatMulV2']);
    if (sc == null || (sc.input ?? []).length !== 2 || !g.only(sc, [sm]) || flag(sc, 'adj_x') || !flag(sc, 'adj_y')) {
      continue;
    }
    const attr: {[k: string]: any} = {_dims: last.attr!['_dims']};
    if (sm.op === '_SoftmaxScaledMasked' && sm.attr?.['_scale'] != null) attr['_scale'] = sm.attr['_scale'];
    removed.add(sc.name);
    removed.add(sm.name);
    replaced.set(last.name, {name: last.name, op: '_FusedAttention',
                             input: [sc.input![0], sc.input![1], last.input![1], ...sm.input!.slice(1)], attr});
  }
  return apply(nodes, removed, replaced);
}

/**
 * Scheduling only: products whose first operand is the same tensor and whose other operands
 * are constants are moved next to the first of them in the stored node list (with the
 * constants they read).  The backend launches the products pending on one operand as a
 * group (PendingMatMul); in the stored order of an attention layer the value projection
 * comes after the softmax and would miss the group of the query and key projections.  The
 * converter derives its execution order from this list (children are visited in list
 * order), so products that become ready together stay together; where its traversal
 * separates them anyway, only the ones pending at the same time form a group.
 * Python twin: hoist_shared_operand_matmuls (tfjs_b200/graph_model.py).
 */
export function hoistSharedOperandMatMuls(nodes: NodeDef[]): NodeDef[] {
  const MATMULS = new Set(['_FusedMatMul', 'MatMul', '_MatMulHeads']);
  const byName = new Map(nodes.map(n => [n.name, n] as [string, NodeDef]));
  const isConst = (inp: string) => byName.get(nodeName(inp))?.op === 'Const';
  const first = new Map<string, string>();
  const moved = new Map<string, NodeDef[]>();
  for (const n of nodes) {
    const inputs = n.input ?? [];
    if (!MATMULS.has(n.op) || inputs.length < 2 || !inputs.slice(1).every(isConst)) continue;
    const lead = first.get(inputs[0]);
    if (lead != null) moved.set(lead, [...(moved.get(lead) ?? []), n]);
    else first.set(inputs[0], n.name);
  }
  if (moved.size === 0) return nodes;
  const late = new Set([...moved.values()].flat().map(n => n.name));
  const out: NodeDef[] = [];
  const placed = new Set<string>();
  for (const n of nodes) {
    if (late.has(n.name) || placed.has(n.name)) continue;
    out.push(n);
    placed.add(n.name);
    for (const m of moved.get(n.name) ?? []) {
      for (const inp of (m.input ?? []).slice(1)) {      // its constants must precede it
        const c = byName.get(nodeName(inp));
        if (c != null && !placed.has(c.name)) {
          out.push(c);
          placed.add(c.name);
        }
      }
      out.push(m);
      placed.add(m.name);
    }
  }
  return out;
}

/** The three rewrites over a loaded model's topology (in place on a copy of the artifacts).
 * TFJS_CUDA_NO_GRAPH_FUSION = 1 | all switches them off; a comma-separated list of
 * layernorm, heads, gelu, softmax, attention, hoist switches single ones off. */
export function rewriteArtifacts(artifacts: io.ModelArtifacts): io.ModelArtifacts {
  const off = process.env['TFJS_CUDA_NO_GRAPH_FUSION'] ?? '0';
  if (off === '1' || off === 'all') return artifacts;
  const skip = new Set(off.split(','));
  const topology = JSON.parse(JSON.stringify(artifacts.modelTopology)) as {node: NodeDef[]};
  const consts = smallConstants(artifacts);
  const sig = (artifacts.signature ?? (artifacts.userDefinedMetadata as any)?.signature ?? {}) as any;
  const prot = new Set<string>([...Object.keys(sig.inputs ?? {}), ...Object.keys(sig.outputs ?? {})]
                                   .concat(Object.values(sig.outputs ?? {}).map((o: any) => nodeName(o.name ?? ''))));
  let nodes = topology.node;
  if (!skip.has('layernorm')) nodes = fuseLayerNorms(nodes, consts, prot);
  if (!skip.has('heads')) nodes = fuseAttentionHeads(nodes, consts, prot);
  if (!skip.has('gelu') && !['1', 'true'].includes(process.env['TFJS_CUDA_NO_FUSE_GELU'] ?? '')) {
    nodes = fuseGeluIntoMatMul(nodes, consts, prot);
  }
  if (!skip.has('softmax')) nodes = fuseSoftmaxInputs(nodes, consts, prot);
  if (!skip.has('attention')) nodes = fuseAttention(nodes, consts, prot);
  if (!skip.has('hoist')) nodes = hoistSharedOperandMatMuls(nodes);
  topology.node = nodes;
  return {...artifacts, modelTopology: topology};
}

// --------------------------------------------------------------- custom-op executors --
const kernel = (name: string, inputs: {[k: string]: Tensor|undefined}, attrs: {[k: string]: unknown}) =>
    tfc.engine().runKernel(name, inputs as {}, attrs as {}) as Tensor;

/** Registers the executors of the three node types with tfjs-converter (`registerOp` is
 * passed in so this module does not import the converter itself). */
export function registerGraphOps(
    registerOp: (name: string, fn: (node: {inputs: Tensor[], attrs: {[k: string]: any}}) => Tensor|Tensor[]) => void): void {
  registerOp('_FusedLayerNorm', node => tfc.tidy(() => {
    const eps = node.attrs['epsilon'] as number;
    const residual = !!node.attrs['residual'];
    let [x, gamma, beta] = residual ? [node.inputs[0], node.inputs[2], node.inputs[3]] : node.inputs;
    if (residual) {
      const b = node.inputs[1];
      if (x.dtype === 'float32' && b.dtype === 'float32' && util_sameShape(x.shape, b.shape) &&
          layerNormSupported(x.shape, gamma.shape, beta.shape)) {
        return kernel('_FusedLayerNorm', {x, gamma, beta, residual: b}, {epsilon: eps});
      }
      x = tfc.add(x, b);
    }
    if (x.dtype === 'float32' && layerNormSupported(x.shape, gamma.shape, beta.shape)) {
      return kernel('_FusedLayerNorm', {x, gamma, beta}, {epsilon: eps});
    }
    // shapes the one-launch kernel does not take: the matched subgraph, op by op
    const mean = tfc.mean(x, [-1], true);
    const variance = tfc.mean(tfc.squaredDifference(x, mean), [-1], true);
    const norm = tfc.mul(tfc.sub(x, mean), tfc.rsqrt(tfc.add(variance, tfc.scalar(eps))));
    return tfc.add(tfc.mul(norm, gamma), beta);
  }));

  registerOp('_SoftmaxScaledMasked', node => tfc.tidy(() => {
    const scale = node.attrs['_scale'] as number|undefined;
    const [x, mask] = node.inputs;
    if (x.dtype === 'float32' && x.rank >= 1 &&
        (mask == null || (mask.dtype === 'float32' && softmaxMaskRows(x.shape, mask.shape) != null))) {
      return kernel('_SoftmaxScaledMasked', {logits: x, mask}, {scale});
    }
    let y = scale != null ? tfc.mul(x, tfc.scalar(scale)) : x;
    if (mask != null) y = tfc.add(y, mask);
    return tfc.softmax(y);
  }));

  registerOp('_FusedMatMulGelu', node => tfc.tidy(() => {
    // _FusedMatMul(a, b, bias) whose epilogue is the erf GELU the five following nodes spelled out
    const [a, b, bias] = node.inputs;
    const [scale, half, one, divide] = node.attrs['_gelu'] as number[];
    const ta = !!node.attrs['transpose_a'], tb = !!node.attrs['transpose_b'];
    if (bias != null) {
      try {
        return kernel('_FusedMatMul', {a, b, bias},
                      {transposeA: ta, transposeB: tb, activation: 'gelu_erf',
                       geluParams: [scale, half, one, divide !== 0]});
      } catch (e) {
        // the fp32 math mode, a bias that does not fuse: the stored ops
      }
    }
    const h = tfc.fused.matMul({a, b, transposeA: ta, transposeB: tb, bias});
    const inner = divide !== 0 ? tfc.div(h, tfc.scalar(scale)) : tfc.mul(h, tfc.scalar(scale));
    return tfc.mul(tfc.mul(h, tfc.scalar(half)), tfc.add(tfc.erf(inner), tfc.scalar(one)));
  }));

  const refusedAttention = new Set<string>();   // operand shapes the library has declined once
  registerOp('_FusedAttention', node => tfc.tidy(() => {
    const scale = node.attrs['_scale'] as number|undefined;
    const dims = node.attrs['_dims'] as number[];
    const [q, k, v, mask] = node.inputs;
    const sig = [q.shape, k.shape, v.shape, mask?.shape].join(';');
    if (!refusedAttention.has(sig)) {
      try {
        return tfc.reshape(kernel('_FusedAttention', {q, k, v, mask}, {scale}), dims);
      } catch (e) {
        refusedAttention.add(sig);   // not 128 positions x 64 features, fp32 math mode: the stored ops
      }
    }
    let s = tfc.matMul(q, k, false, true);
    if (scale != null) s = tfc.mul(s, tfc.scalar(scale));
    if (mask != null) s = tfc.add(s, mask);
    const o = tfc.matMul(tfc.softmax(s), v);
    return tfc.reshape(tfc.transpose(o, [0, 2, 1, 3]), dims);
  }));

  const refused = new Set<string>();   // (layout, operand shapes) the library has declined once
  registerOp('_MatMulHeads', node => tfc.tidy(() => {
    const a = node.attrs;
    const layout = a['_layout'] as string, innerOp = a['_op'] as string, dims = a['_dims'] as number[];
    const [x, w, bias] = node.inputs;
    const fused = innerOp === '_FusedMatMul';
    const ta = !!(fused || innerOp === 'MatMul' ? a['transpose_a'] : a['adj_x']);
    const tb = !!(fused || innerOp === 'MatMul' ? a['transpose_b'] : a['adj_y']);
    let heads: number[]|null = null;
    if (layout === 'split') {
      heads = dims.length === 4 ? dims : null;
    } else if (x.rank === 4 && w.rank === 4) {
      heads = [x.shape[0], ta ? x.shape[3] : x.shape[2], x.shape[1], tb ? w.shape[2] : w.shape[3]];
    }
    const sig = [layout, x.shape, w.shape, ta, tb].join();
    if (heads != null && !refused.has(sig)) {
      try {
        const y = kernel('_MatMulHeads', {a: x, b: w, bias: fused ? bias : undefined},
                         {layout, heads, transposeA: ta, transposeB: tb, activation: 'linear'});
        return layout === 'split' ? y : tfc.reshape(y, dims);
      } catch (e) {
        refused.add(sig);     // S or D not a multiple of 32, fp32 math mode, ...: the stored ops
      }
    }
    const y = fused ? tfc.fused.matMul({a: x, b: w, transposeA: ta, transposeB: tb, bias}) :
                      tfc.matMul(x, w, ta, tb);
    return layout === 'split' ? tfc.transpose(tfc.reshape(y, dims), [0, 2, 1, 3]) :
                                tfc.reshape(tfc.transpose(y, [0, 2, 1, 3]), dims);
  }));
}

function util_sameShape(a: number[], b: number[]): boolean {
  return a.length === b.length && a.every((v, i) => v === b[i]);
}
