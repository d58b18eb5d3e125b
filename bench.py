"""Benchmark of the tfjs 'cuda' backend on B200: GraphModel.execute throughput.

    python bench.py --gpus N --steps K --warmup W [--model mobilenet_v2|resnet50|bert]
    python bench.py --impl reference ...        # the CPU path, timed on the host cores

One step = one GraphModel.execute over one batch per GPU (MobileNetV2-1.0 batch
256, ResNet-50 batch 128 with uint8-quantised weights dequantised on the device
at load, BERT-base encoder batch 64 x seq 128).  Weights are random-initialised
and inputs are seeded synthetic tensors of the published shapes.  With N > 1
every rank runs its own backend on its own GPU with its own batch (weak
scaling, no collective on the data path); rank 0 prints one JSON line.

Without --model the line's top-level keys describe MobileNetV2 batch 256 and the
same measurements of the other configurations (ResNet-50 b128, BERT b64,
MobileNetV2 b64 and b1) follow under "workloads", each with its own value, e2e,
roofline, sustained figure and clocks; --model X measures X alone.
--scaling strong splits the workload's batch over the ranks instead (contiguous
ceil(B/N) slices, outputs gathered on rank 0 inside the end-to-end region).

value      device-timed throughput with the input batch resident in HBM.  The timed
           steps are replays of the step captured during warm-up (GraphModel's
           whole-step replay; --no-replay launches every kernel from the host).
e2e        the same metric through the public API with HOST buffers: every step
           uploads the batch from pinned memory (copy stream) and downloads the
           logits with tensor.data(); batch i+1 is uploaded and launched before the
           result of batch i is awaited, every result is awaited in the timed region.
roofline   for the kernel kind that takes the most device time, from CUDA events
           recorded around every kernel on the launching stream during extra
           eagerly launched steps (tf.profile-style) right after the timed region;
           HBM-bound kinds also carry the fraction of the nominal 8 TB/s.
sustained  the same resident-input steps repeated back to back for at least two
           seconds (median ms per step over chunks of K steps, the SM clock sampled
           meanwhile, and ms x MHz), next to the K-step burst that `value` reports.
e2e_copy_ceiling  the end-to-end loop without the execute: the same uploads and result
           downloads alone, i.e. what the host side allows at this N.
cpu_baseline  the CPU oracle (a C restatement of tfjs-backend-cpu) on a bounded
           sample of the same workload: all host cores (OpenMP over independent
           outputs), one thread (JavaScript runs the reference on one), and a
           labelled stand-in for the XNNPACK-based wasm backend (PyTorch CPU, oneDNN,
           all cores), which cannot run here.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    "mobilenet_v2": dict(batch=256, unit="images/s", metric="images/sec", out="logits",
                         gflop=0.601548544, name="mobilenet_v2_1.0_224_b256_graphmodel"),
    "resnet50": dict(batch=128, unit="images/s", metric="images/sec", out="logits",
                     gflop=8.178368512, name="resnet50_v1.5_224_b128_uint8weights_graphmodel"),
    "bert": dict(batch=64, unit="sequences/s", metric="sequences/sec", out="sequence_output",
                 gflop=22.347251712, name="bert_base_encoder_seq128_b64_graph"),
}


def build_model(model, batch):
    from tfjs_b200 import model_zoo
    if model == "mobilenet_v2":
        return model_zoo.mobilenet_v2(batch)
    if model == "resnet50":
        return model_zoo.resnet50(batch)
    return model_zoo.bert_encoder(batch)


def make_feeds(model, batch, seed):
    r = np.random.default_rng(seed)
    if model == "mobilenet_v2":
        return {"input": r.uniform(-1, 1, (batch, 224, 224, 3)).astype(np.float32)}
    if model == "resnet50":
        return {"input": r.uniform(0, 1, (batch, 224, 224, 3)).astype(np.float32)}
    return {"input_ids": r.integers(0, 30522, (batch, 128)).astype(np.int32),
            "attention_mask": np.ones((batch, 128), np.float32)}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=float(p["hbm_gbs"]), bf16=float(p["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, bf16=1590.0, source="fallback")


class ClockSampler(object):
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.tmp = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(device), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=self.tmp, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.tmp.flush()
        rows = [l.strip().split(", ") for l in open(self.tmp.name) if l.strip()]
        os.unlink(self.tmp.name)
        sm, reasons, mx = [], set(), None
        for r in rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx = float(r[2])
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                "sw_power_cap"), r[5:9]):
                if v.strip().lower().startswith("active"):
                    reasons.add(name)
        if sm:
            busy = [s for s in sm if s > 0.5 * max(sm)] or sm
            out.update(sm_mhz=float(np.median(busy)), sm_max_mhz=mx, reasons=sorted(reasons),
                       samples=len(sm))
        return out


# ------------------------------------------------------------ work accounting --
def _prod(s):
    n = 1
    for v in s:
        n *= int(v)
    return n


def kernel_work(rec):
    """Algorithmic (flops, bytes) of one profiled kernel call: each input and
    output tensor is moved once; contractions count 2 flops per MAC."""
    outs = rec["outputShapes"]
    if rec.get("parts"):
        # one launch that covers several kernels (a convolution with the Add / Relu
        # that followed it folded in): the operands of each part are read once, the
        # final result is written once, intermediate results never reach memory
        flops = nbytes = 0
        for part in rec["parts"]:
            f, _ = kernel_work(dict(part, parts=None))
            flops += f
            nbytes += 4 * sum(_prod(s) for s in part["inputShapes"].values())
        return flops, nbytes + 4 * sum(_prod(s) for s in outs)
    ins = rec["inputShapes"]
    nbytes = 4 * (sum(_prod(s) for s in ins.values()) + sum(_prod(s) for s in outs))
    name, flops = rec["name"], 0
    if name in ("FusedConv2D", "Conv2D"):
        f = ins["filter"]
        flops = 2 * _prod(outs[0]) * f[0] * f[1] * f[2]
    elif name in ("FusedDepthwiseConv2D", "DepthwiseConv2dNative"):
        f = ins["filter"]
        flops = 2 * _prod(outs[0]) * f[0] * f[1]
    elif name in ("_FusedMatMul", "BatchMatMul", "_MatMulHeads"):
        a = ins["a"]
        k = a[-2] if rec["attrs"].get("transposeA") else a[-1]
        flops = 2 * _prod(outs[0]) * k
    elif name in ("Reshape", "Identity", "ExpandDims"):
        nbytes = 0
    return flops, nbytes


def summarise_profile(records, steps):
    kinds = {}
    for rec in records:
        if rec.get("deferred"):
            continue  # launched later, inside the record that lists it under `parts`
        flops, nbytes = kernel_work(rec)
        k = kinds.setdefault(rec["name"], dict(launches=0, ms=0.0, flops=0, bytes=0))
        k["launches"] += 1
        k["ms"] += rec["kernelTimeMs"]
        k["flops"] += flops
        k["bytes"] += nbytes
    total = sum(k["ms"] for k in kinds.values()) or 1.0
    out = {}
    for name, k in kinds.items():
        sec = k["ms"] / 1e3 or 1e-12
        out[name] = dict(launches_per_step=k["launches"] // steps,
                         ms_per_step=round(k["ms"] / steps, 4), share=round(k["ms"] / total, 4),
                         gbs=round(k["bytes"] / sec / 1e9, 1),
                         tflops=round(k["flops"] / sec / 1e12, 2),
                         flops_per_byte=round(k["flops"] / max(k["bytes"], 1), 1))
    return out


def measure_tf32_peak():
    """cuBLAS TF32 GEMM throughput (8192^3, best of 10), the tensor roofline
    denominator for a TF32 kernel; measured the way the bf16 figure in
    MEASURED_PEAKS.json was.  Measurement only; not on the product path."""
    try:
        import torch
        torch.backends.cuda.matmul.allow_tf32 = True
        n = 8192
        a = torch.randn(n, n, device="cuda")
        b = torch.randn(n, n, device="cuda")
        for _ in range(3):
            a @ b
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(True), torch.cuda.Event(True)
            e0.record()
            a @ b
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        del a, b
        torch.cuda.empty_cache()
        return 2 * n ** 3 / (best / 1e3) / 1e12
    except Exception:
        return None


# ------------------------------------------------------------------ reference --
def cpu_sample(model, sample_batch, threads=None, min_seconds=0.0):
    """Times the CPU oracle on batches of `sample_batch` units of the workload, repeated
    until `min_seconds` of CPU work have been done; returns (units/s, seconds, threads,
    units)."""
    from oracle import graph_oracle, oracle as orc
    if threads:
        orc.set_threads(threads)
    model_json, weights = build_model(model, sample_batch)
    feeds = make_feeds(model, sample_batch, 1)
    units, t0 = 0, time.perf_counter()
    while True:
        graph_oracle.run(model_json, weights, feeds)
        units += sample_batch
        dt = time.perf_counter() - t0
        if dt >= min_seconds:
            break
    return units / dt, dt, orc.max_threads(), units


def run_reference(args, rank, world):
    args.model = args.model or "mobilenet_v2"
    w = WORKLOADS[args.model]
    if rank != 0:
        return
    sample = args.cpu_sample or {"mobilenet_v2": 32, "resnet50": 4, "bert": 2}[args.model]
    # torchrun exports OMP_NUM_THREADS=1; the reference arm uses every host core
    threads = os.cpu_count() or 1
    for _ in range(max(args.warmup, 0) and 1):
        cpu_sample(args.model, 1, threads=threads)
    vals = []
    t_all = time.perf_counter()
    for _ in range(args.steps):
        v, dt, cores, _ = cpu_sample(args.model, sample, threads=threads)
        vals.append(v)
    total = time.perf_counter() - t_all
    value = float(np.mean(vals))
    sample_txt = ("%d %s per step through the C restatement of tfjs-backend-cpu (same graph, "
                  "same layer shapes), OpenMP over independent outputs" %
                  (sample, "images" if "image" in w["unit"] else "sequences"))
    line = {"impl": "reference", "metric": w["metric"], "value": round(value, 3),
            "unit": w["unit"], "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(total / args.steps * 1e3, 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f64-math/f32-store",
            "data": "synthetic",
            "config": {"workload": w["name"], "batch_per_gpu": w["batch"],
                       "sample_batch": sample},
            "cpu_baseline": {"value": round(value, 3), "unit": w["unit"], "cores": cores,
                             "kind": "port", "sample": sample_txt},
            "e2e": {"value": round(value, 3), "unit": w["unit"], "h2d_bytes_per_step": 0,
                    "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


# ----------------------------------------------------------- CPU stand-in (oneDNN) --
def torch_cpu_sample(model, sample_batch, min_seconds):
    """Labelled stand-in for the reference's wasm backend (XNNPACK, SIMD + threads), which
    needs Node and the built .wasm: the same graph through PyTorch's CPU kernels (oneDNN)
    on all host cores.  Returns (units/s, seconds, threads, units) or None.  Measurement
    only; never on the product path."""
    try:
        import torch
        import torch.nn.functional as F
        from oracle import graph_oracle
    except Exception:
        return None
    torch.set_num_threads(os.cpu_count() or 1)
    model_json, weight_bytes = build_model(model, sample_batch)
    specs = model_json["weightsManifest"][0]["weights"]
    vals = {k: torch.from_numpy(np.ascontiguousarray(v))
            for k, v in graph_oracle.decode_weights(weight_bytes, specs).items()}
    nodes = model_json["modelTopology"]["node"]
    import base64
    att_s = lambda a, n: base64.b64decode(a[n]["s"]).decode().lower() if n in a else None
    att_i = lambda a, n: [int(v) for v in a[n]["list"]["i"]]
    fused = lambda a: [base64.b64decode(v).decode().lower() for v in a["fused_ops"]["list"]["s"]]
    act = {"relu": F.relu, "relu6": F.relu6}
    # filters to OIHW once, outside the timed loop
    prepared = {}
    for n in nodes:
        if n["op"] == "_FusedConv2D":
            prepared[n["input"][1]] = vals[n["input"][1]].permute(3, 2, 0, 1).contiguous(
                memory_format=torch.channels_last)
        elif n["op"] == "FusedDepthwiseConv2dNative":
            w = vals[n["input"][1]]
            prepared[n["input"][1]] = w.permute(2, 3, 0, 1).contiguous()

    def same_pad(x, k, s):
        h, w = x.shape[2], x.shape[3]
        ph = max((-(-h // s) - 1) * s + k - h, 0)
        pw = max((-(-w // s) - 1) * s + k - w, 0)
        return F.pad(x, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2)) if ph or pw else x

    def run(feeds):
        v = dict(vals)
        for k, a in feeds.items():
            t = torch.from_numpy(a)
            v[k] = t.permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last) \
                if t.dim() == 4 else t
        nchw = set(k for k, a in feeds.items() if a.ndim == 4)
        for n in nodes:
            op, a = n["op"], n.get("attr", {})
            if op in ("Const", "Placeholder"):
                continue
            x = [v[i.split(":")[0]] for i in n["input"]]
            src0 = n["input"][0].split(":")[0]
            if op in ("_FusedConv2D", "FusedDepthwiseConv2dNative"):
                w = prepared[n["input"][1]]
                st = att_i(a, "strides")[1]
                xin = same_pad(x[0], w.shape[2], st)
                y = F.conv2d(xin, w, x[2], st, 0, 1, w.shape[0] if op[0] == "F" else 1)
                for f in fused(a)[1:]:
                    y = act[f](y)
                nchw.add(n["name"])
            elif op == "_FusedMatMul":
                y = torch.addmm(x[2], x[0], x[1])
                for f in fused(a)[1:]:
                    y = act[f](y)
            elif op == "BatchMatMulV2":
                xa = x[0].transpose(-1, -2) if a.get("adj_x", {}).get("b") else x[0]
                xb = x[1].transpose(-1, -2) if a.get("adj_y", {}).get("b") else x[1]
                y = torch.matmul(xa, xb)
            elif op == "MaxPool":
                k, st = att_i(a, "ksize")[1], att_i(a, "strides")[1]
                y = F.max_pool2d(F.pad(x[0], (0, 1, 0, 1), value=float("-inf")), k, st)
                nchw.add(n["name"])
            elif op == "Mean":
                axes = [int(t) for t in x[1].reshape(-1)]
                if src0 in nchw:
                    axes = [{1: 2, 2: 3, 3: 1}.get(t, t) for t in axes]
                y = x[0].mean(axes, keepdim=bool(a.get("keep_dims", {}).get("b")))
            elif op in ("AddV2", "Sub", "Mul", "SquaredDifference"):
                y = {"AddV2": torch.add, "Sub": torch.sub, "Mul": torch.mul,
                     "SquaredDifference": lambda p, q: (p - q) ** 2}[op](x[0], x[1])
                if src0 in nchw:
                    nchw.add(n["name"])
            elif op in ("Relu", "Relu6", "Rsqrt", "Erf"):
                y = {"Relu": F.relu, "Relu6": F.relu6, "Rsqrt": torch.rsqrt,
                     "Erf": torch.erf}[op](x[0])
                if src0 in nchw:
                    nchw.add(n["name"])
            elif op == "Softmax":
                y = torch.softmax(x[0], -1)
            elif op == "GatherV2":
                y = x[0][x[1].long()]
            elif op == "Reshape":
                y = x[0].reshape([int(t) for t in x[1].reshape(-1)])
            elif op == "Transpose":
                y = x[0].permute([int(t) for t in x[1].reshape(-1)])
            else:
                raise NotImplementedError(op)
            v[n["name"]] = y
        return v

    feeds = make_feeds(model, sample_batch, 1)
    try:
        with torch.no_grad():
            run(feeds)
            units, t0 = 0, time.perf_counter()
            while True:
                run(feeds)
                units += sample_batch
                dt = time.perf_counter() - t0
                if dt >= min_seconds:
                    break
    except Exception:
        return None
    return units / dt, dt, torch.get_num_threads(), units


def cpu_baselines(model, unit, headline):
    """The CPU figures beside the GPU number (rank 0, N = 1 only)."""
    sample = {"mobilenet_v2": 64, "resnet50": 8, "bert": 4}[model]
    what = "the same graph through the C restatement of tfjs-backend-cpu"
    v, dt, cores, units = cpu_sample(model, sample, min_seconds=10.0 if headline else 4.0)
    out = {"value": round(v, 3), "unit": unit, "cores": cores, "kind": "port",
           "sample": "%d units (batches of %d) of %s in %.1f s" % (units, sample, what, dt)}
    one = {"mobilenet_v2": 4, "resnet50": 1, "bert": 1}[model]
    v1, dt1, _, units1 = cpu_sample(model, one, threads=1, min_seconds=6.0 if headline else 3.0)
    out["single_thread"] = {
        "value": round(v1, 3), "unit": unit, "cores": 1, "kind": "port",
        "sample": "%d units (batches of %d) of %s on one thread, as JavaScript runs the "
                  "reference, in %.1f s" % (units1, one, what, dt1)}
    from oracle import oracle as orc
    orc.set_threads(os.cpu_count() or 1)
    t = torch_cpu_sample(model, sample, 4.0 if headline else 2.0)
    if t is not None:
        out["xnnpack_stand_in"] = {
            "value": round(t[0], 3), "unit": unit, "cores": t[2], "kind": "stand-in",
            "sample": "NOT the reference: tfjs-backend-wasm (XNNPACK) is unavailable on this box "
                      "(no Node, no .wasm); PyTorch CPU fp32 (oneDNN) ran %d units of the same "
                      "graph in %.1f s" % (t[3], t[1])}
    return out


# ----------------------------------------------------------------------- cuda --
# DRAM traffic of each workload's dominant kernel kind: dram__bytes_read.sum +
# dram__bytes_write.sum summed over that kind's launches in ONE step of the workload, from
# an ncu pass over an eagerly launched step at the bench batch (so every launch sees the L2
# state it sees in the benchmark); the commands and the per-launch rows are in the
# profile summary named here.  bench.py reports the mean per launch and the ratio to the
# algorithmic bytes it computes itself.
NCU_TRAFFIC = {
    # "<workload>/<kind>": (profile summary, launches per step, dram bytes per step)
    "mobilenet_v2_1.0_224_b256_graphmodel/FusedConv2D":
        ("profiles/bench_dram_traffic_mobilenet_v2_b256.md", 19, 4604911104),
    "mobilenet_v2_1.0_224_b256_graphmodel/FusedDepthwiseConv2D":
        ("profiles/bench_dram_traffic_mobilenet_v2_b256.md", 2, 1780078080),
    "mobilenet_v2_1.0_224_b256_graphmodel/FusedDepthwiseConv2D+FusedConv2D":
        ("profiles/bench_dram_traffic_mobilenet_v2_b256.md", 6, 2263849472),
    "mobilenet_v2_1.0_224_b256_graphmodel/FusedDepthwiseConv2D+FusedConv2D+Add":
        ("profiles/bench_dram_traffic_mobilenet_v2_b256.md", 9, 1038357760),
    "resnet50_v1.5_224_b128_uint8weights_graphmodel/FusedConv2D":
        ("profiles/bench_dram_traffic_resnet50_b128.md", 37, 6562264832),
    "resnet50_v1.5_224_b128_uint8weights_graphmodel/FusedConv2D+Add+Relu":
        ("profiles/bench_dram_traffic_resnet50_b128.md", 16, 6475964416),
    "bert_base_encoder_seq128_b64_graph/_FusedMatMul":
        ("profiles/bench_dram_traffic_bert_base_b64.md", 36, 3146692096),
    "bert_base_encoder_seq128_b64_graph/_MatMulHeads+_MatMulHeads+_MatMulHeads":
        ("profiles/bench_dram_traffic_bert_base_b64.md", 12, 909686784),
    "bert_base_encoder_seq128_b64_graph/_FusedAttention":
        ("profiles/bench_dram_traffic_bert_base_b64.md", 12, 750211584),
}


def run_workload(args, model, batch, eng, group, rank, world, local_rank, headline, near_cpus,
                 tf32_peak):
    """All measurements of one workload on this rank; rank 0 gets the JSON dict."""
    import tfjs_b200
    from tfjs_b200.graph_model import GraphModel
    from tfjs_b200.replicas import shard_range
    be = eng.backend
    w = WORKLOADS[model]
    barrier, max_over_ranks = group.barrier, group.max_over_ranks
    strong = args.scaling == "strong"
    if strong:
        lo, hi = shard_range(batch, world, rank)
        local_batch, global_units = hi - lo, batch
    else:
        lo, local_batch, global_units = 0, batch, batch * world
    if local_batch == 0:
        raise SystemExit("rank %d has no units: use --gpus <= the batch" % rank)

    model_json, weights = build_model(model, local_batch)
    # whole-step replay: the second warm-up step is captured into a CUDA graph and every
    # later step is one graph launch (the per-kernel profile below runs eagerly)
    t_load = time.perf_counter()
    gm = GraphModel(model_json, weights, eng, replay=not args.no_replay)
    be.sync()
    load_ms = (time.perf_counter() - t_load) * 1e3
    if strong:
        full = make_feeds(model, batch, 1000)
        feeds = {k: np.ascontiguousarray(v[lo:lo + local_batch]) for k, v in full.items()}
    else:
        feeds = make_feeds(model, local_batch, 1000 + rank)
    pinned, dtypes = {}, {}
    for k, v in feeds.items():
        dt = "int32" if v.dtype == np.int32 else "float32"
        p = be.pinned_empty(v.shape, dt)
        p[...] = v
        pinned[k], dtypes[k] = p, dt

    def upload_inputs():
        return {k: eng.make_tensor_from_info(
            tfjs_b200.TensorInfo(be.write_from(pinned[k], pinned[k].shape, dtypes[k]),
                                 pinned[k].shape, dtypes[k])) for k in pinned}

    resident = upload_inputs()
    out_name = w["out"]

    def step_resident():
        y = gm.execute(resident, [out_name])[0]
        be.device_id(y.dataId)     # a result whose launch is still pending is launched (no sync)
        y.dispose()

    out_probe = gm.execute(resident, [out_name])[0]
    out_shape = out_probe.shape
    out_probe.dispose()
    out_hosts = [be.pinned_empty(out_shape, "float32"), be.pinned_empty(out_shape, "float32")]
    h2d = int(sum(p.nbytes for p in pinned.values()))
    d2h = int(out_hosts[0].nbytes)

    def run_e2e(steps, execute=True):
        """Each step uploads its batch from pinned host memory (copy stream), executes,
        and downloads the result with tensor.data() into pinned memory.  The loop is the
        one an application writes with promises: the upload and the launches of batch
        i+1 are issued before the result of batch i is awaited, so the GPU never waits
        for the host to enqueue a step.  Every result is awaited inside the timed
        region.  execute=False keeps the transfers and drops the model (the copy-only
        ceiling): the download then reads a resident tensor of the output's size."""
        nxt = upload_inputs()
        prev = None
        gathered = None
        for i in range(steps):
            ins = nxt
            if execute:
                y = gm.execute(ins, [out_name])[0]
            else:
                y = ceiling_src     # (disposing an unused upload orders the stream behind it)
            for t in ins.values():
                t.dispose()                      # stream-ordered: after the step's kernels
            pending = y.data(into=out_hosts[i & 1])      # D2H queued behind the step
            if execute:
                y.dispose()
            nxt = upload_inputs() if i + 1 < steps else None
            if prev is not None:
                prev.wait()
                if strong and execute:
                    gathered = group.gather_to_root(out_hosts[(i - 1) & 1])
            prev = pending
        prev.wait()
        if strong and execute:
            gathered = group.gather_to_root(out_hosts[(steps - 1) & 1])
        return gathered

    for _ in range(max(args.warmup, 3)):
        step_resident()
    be.sync()

    from ctypes import byref, c_float

    def timed_steps(n):
        be.check(be.lib.tfjs_cuda_time_begin(be.ctx))
        for _ in range(n):
            step_resident()
        ms = c_float()
        be.check(be.lib.tfjs_cuda_time_end(be.ctx, byref(ms)))   # records + syncs
        return float(ms.value)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    # ---- timed region: device time (CUDA events on the launching stream) ----
    barrier()
    be.sync()
    launches0 = be.launch_count()
    t_host0 = time.perf_counter()
    ms = timed_steps(args.steps)
    be.sync()
    host_ms = (time.perf_counter() - t_host0) * 1e3
    barrier()
    launches = be.launch_count() - launches0
    dev_ms = max_over_ranks(ms)

    # ---- end to end through the public API with host buffers -----------------
    run_e2e(2)
    barrier()
    be.sync()
    t0 = time.perf_counter()
    gathered = run_e2e(args.steps)
    be.sync()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    clocks = sampler.stop() if sampler is not None else None

    # ---- the same loop without the model: what the host side allows at this N ----
    ceiling_src = eng.make_tensor_from_info(be.make_output(out_shape, "float32"))
    run_e2e(2, execute=False)
    barrier()
    be.sync()
    t0 = time.perf_counter()
    run_e2e(args.steps, execute=False)
    be.sync()
    copy_s = max_over_ranks(time.perf_counter() - t0)
    ceiling_src.dispose()
    barrier()

    # ---- sustained: back-to-back steps for >= 2 s ------------------------------
    sampler2 = ClockSampler(local_rank) if rank == 0 else None
    chunks, t0 = [], time.perf_counter()
    barrier()
    while True:
        chunks.append(timed_steps(args.steps) / args.steps)
        # every rank runs the same number of chunks: the decision is rank 0's
        more = group.max_over_ranks(1.0 if (time.perf_counter() - t0 < args.sustain_seconds
                                            and rank == 0) else 0.0)
        if not more:
            break
    sus_ms = max_over_ranks(float(np.median(chunks)))
    sus_clocks = sampler2.stop() if sampler2 is not None else None

    line = None
    if rank == 0:
        # three profiled steps (launched eagerly); per kernel call the fastest of the three
        # is kept, which drops one-off host stalls between the two events of a call
        step_resident()
        runs = [eng.profile(step_resident)["kernels"] for _ in range(3)]
        records = runs[0]
        if all(len(r) == len(records) for r in runs):
            for i, rec in enumerate(records):
                rec["kernelTimeMs"] = min(r[i]["kernelTimeMs"] for r in runs)
        kinds = summarise_profile(records, 1)
        top = max(kinds, key=lambda k: kinds[k]["ms_per_step"])
        pk = peaks()
        tk = kinds[top]
        tensor_bound = tk["flops_per_byte"] >= 100.0
        roof = {"kernel": top, "launches_per_step": tk["launches_per_step"],
                "share_of_device_time": tk["share"], "traffic": None}
        alg_step = tk["gbs"] * 1e9 * tk["ms_per_step"] / 1e3     # algorithmic bytes per step
        roof["algorithmic_bytes_per_launch"] = int(alg_step / max(tk["launches_per_step"], 1))
        known = NCU_TRAFFIC.get("%s/%s" % (w["name"] if batch == w["batch"] else "-", top))
        if known is not None and known[1] == tk["launches_per_step"]:
            roof["traffic"] = int(known[2] / known[1])
            roof["traffic_over_algorithmic"] = round(known[2] / alg_step, 3)
            roof["traffic_source"] = ("dram__bytes_read.sum + dram__bytes_write.sum over this "
                                      "kind's launches in one step under ncu, per launch (%s)"
                                      % known[0])
        if tensor_bound:
            peak = tf32_peak or pk["bf16"] / 2.0
            roof.update(bound="tensor", achieved=tk["tflops"], peak=round(peak, 1),
                        unit="TFLOP/s", frac=round(tk["tflops"] / peak, 4),
                        peak_source=("measured in this run: torch.matmul TF32 8192^3 best of 10"
                                     if tf32_peak else "half of the %s bf16 figure" % pk["source"]))
        else:
            roof.update(bound="hbm", achieved=tk["gbs"], peak=pk["hbm"], unit="GB/s",
                        frac=round(tk["gbs"] / pk["hbm"], 4),
                        peak_source="%s copy bandwidth" % pk["source"],
                        frac_of_nominal_8tbs=round(tk["gbs"] / 8000.0, 4))
        units = global_units
        value = units * args.steps / (dev_ms / 1e3)
        e2e_v = units * args.steps / e2e_s
        ceil_v = units * args.steps / copy_s
        sus_mhz = (sus_clocks or {}).get("sm_mhz")
        line = {"metric": w["metric"], "value": round(value, 2), "unit": w["unit"],
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True,
                "scaling": args.scaling, "vs_baseline": None, "dtype": "tf32",
                "data": "synthetic",
                "config": {"workload": w["name"] if batch == w["batch"] else
                           w["name"].replace("_b%d" % w["batch"], "_b%d" % batch),
                           "batch_per_gpu": local_batch,
                           "global_batch": units, "parallelism": "replicas x%d" % world,
                           "l2": "activations per step are far larger than L2" if batch > 1 else
                                 "batch 1: the step's tensors fit in L2, as they do in use",
                           "step_replay": bool(gm.replay),
                           "cpu_binding": ("GPU-local cores" if near_cpus else "none"),
                           "weights": "random init"},
                "host_ms_per_step": round(host_ms / args.steps, 4),
                "tflops": round(units * w["gflop"] / 1e3 / (dev_ms / args.steps / 1e3), 2),
                "clocks": clocks,
                "e2e": {"value": round(e2e_v, 2), "unit": w["unit"],
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "frac_of_copy_ceiling": round(e2e_v / ceil_v, 4)},
                "e2e_copy_ceiling": {"value": round(ceil_v, 2), "unit": w["unit"],
                                     "h2d_gbs_per_gpu": round(h2d * args.steps / copy_s / 1e9, 2),
                                     "what": "the e2e loop's uploads and downloads without the "
                                             "execute, max over ranks"},
                "sustained": {"ms_per_step": round(sus_ms, 4),
                              "value": round(units / (sus_ms / 1e3), 2), "unit": w["unit"],
                              "seconds": round(float(np.sum(chunks)) * args.steps / 1e3, 2),
                              "sm_mhz_median": sus_mhz,
                              "ms_x_mhz": round(sus_ms * sus_mhz, 1) if sus_mhz else None,
                              "burst_ms_x_mhz": (round(dev_ms / args.steps * clocks["sm_mhz"], 1)
                                                 if clocks and clocks.get("sm_mhz") else None),
                              "reasons": (sus_clocks or {}).get("reasons"),
                              "burst_over_sustained": round(dev_ms / args.steps / sus_ms, 4)},
                "gpu_launches": int(launches),
                "load_ms": round(load_ms, 1),
                "roofline": roof,
                "kernels": kinds}
        if strong and gathered is not None:
            line["config"]["gathered_output_shape"] = list(gathered.shape)
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baselines(model, w["unit"], headline)
    for t in resident.values():
        t.dispose()
    gm.dispose()
    be.check(be.lib.tfjs_cuda_trim(be.ctx))
    return line


def run_cuda(args, rank, world, local_rank):
    os.environ["TFJS_CUDA_DEVICE_ORDINAL"] = str(local_rank)
    from tfjs_b200.replicas import ReplicaGroup, bind_to_gpu_cpus
    near_cpus = bind_to_gpu_cpus(local_rank) if world > 1 else None
    import tfjs_b200
    eng = tfjs_b200.ENGINE
    eng.set_backend("cuda")          # raises if the CUDA library or a GPU is missing
    group = ReplicaGroup(rank, world)
    if args.model:
        todo = [(args.model, args.batch or WORKLOADS[args.model]["batch"])]
    else:
        todo = [("mobilenet_v2", 256), ("resnet50", 128), ("bert", 64), ("mobilenet_v2", 64),
                ("mobilenet_v2", 1)]
    tf32_peak = measure_tf32_peak() if rank == 0 else None
    line = None
    for i, (model, batch) in enumerate(todo):
        res = run_workload(args, model, batch, eng, group, rank, world, local_rank, i == 0,
                           near_cpus, tf32_peak)
        if rank != 0:
            continue
        if i == 0:
            line = res
            if len(todo) > 1:
                line["workloads"] = {}
        else:
            res.pop("kernels", None)
            line["workloads"][res["config"]["workload"]] = res
    if rank == 0:
        print(json.dumps(line))
    group.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--model", default=None, choices=sorted(WORKLOADS),
                    help="measure this workload alone (default: MobileNetV2 b256 as the "
                         "headline, the other configurations under 'workloads')")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every GPU runs the workload's batch; strong: the batch is "
                         "split over the GPUs and the outputs are gathered on rank 0")
    ap.add_argument("--sustain-seconds", type=float, default=2.0)
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the workload's)")
    ap.add_argument("--cpu-sample", type=int, default=0)
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-replay", action="store_true",
                    help="launch every kernel from the host at every step")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_cuda(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
