"""Benchmark of the tfjs 'cuda' backend on B200: GraphModel.execute throughput.

    python bench.py --gpus N --steps K --warmup W [--model mobilenet_v2|resnet50|bert]
    python bench.py --impl reference ...        # the CPU path, timed on the host cores

One step = one GraphModel.execute over one batch per GPU (MobileNetV2-1.0 batch
256, ResNet-50 batch 128 with uint8-quantised weights dequantised on the device
at load, BERT-base encoder batch 64 x seq 128).  Weights are random-initialised
and inputs are seeded synthetic tensors of the published shapes.  With N > 1
every rank runs its own backend on its own GPU with its own batch (weak
scaling, no collective on the data path); rank 0 prints one JSON line.

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
cpu_baseline  the CPU oracle (a C restatement of tfjs-backend-cpu) on a bounded
           sample of the same workload.
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


# ----------------------------------------------------------------------- cuda --
def run_cuda(args, rank, world, local_rank):
    os.environ["TFJS_CUDA_DEVICE_ORDINAL"] = str(local_rank)
    from tfjs_b200.replicas import bind_to_gpu_cpus
    near_cpus = bind_to_gpu_cpus(local_rank) if world > 1 else None
    import tfjs_b200
    from tfjs_b200.graph_model import GraphModel
    eng = tfjs_b200.ENGINE
    eng.set_backend("cuda")          # raises if the CUDA library or a GPU is missing
    be = eng.backend
    w = WORKLOADS[args.model]
    batch = args.batch or w["batch"]

    from tfjs_b200.replicas import ReplicaGroup
    group = ReplicaGroup(rank, world)
    barrier = group.barrier
    max_over_ranks = group.max_over_ranks

    model_json, weights = build_model(args.model, batch)
    # whole-step replay: the second warm-up step is captured into a CUDA graph and every
    # later step is one graph launch (the per-kernel profile below runs eagerly)
    gm = GraphModel(model_json, weights, eng, replay=not args.no_replay)
    feeds = make_feeds(args.model, batch, 1000 + rank)
    pinned, dtypes = {}, {}
    for k, v in feeds.items():
        dt = "int32" if v.dtype == np.int32 else "float32"
        p = be.pinned_empty(v.shape, dt)
        p[...] = v
        pinned[k], dtypes[k] = p, dt
    resident = {k: eng.make_tensor_from_info(
        tfjs_b200.TensorInfo(be.write_from(pinned[k], pinned[k].shape, dtypes[k]),
                             pinned[k].shape, dtypes[k])) for k in pinned}
    out_name = w["out"]

    def step_resident():
        y = gm.execute(resident, [out_name])[0]
        y.dispose()

    out_probe = gm.execute(resident, [out_name])[0]
    out_shape = out_probe.shape
    out_probe.dispose()
    out_host = be.pinned_empty(out_shape, "float32")
    h2d = int(sum(p.nbytes for p in pinned.values()))
    d2h = int(out_host.nbytes)

    def upload_inputs():
        return {k: eng.make_tensor_from_info(
            tfjs_b200.TensorInfo(be.write_from(pinned[k], pinned[k].shape, dtypes[k]),
                                 pinned[k].shape, dtypes[k])) for k in pinned}

    out_hosts = [out_host, be.pinned_empty(out_shape, "float32")]

    def run_e2e(steps):
        """Each step uploads its batch from pinned host memory (copy stream), executes,
        and downloads the result with tensor.data() into pinned memory.  The loop is the
        one an application writes with promises: the upload and the launches of batch
        i+1 are issued before the result of batch i is awaited, so the GPU never waits
        for the host to enqueue a step.  Every result is awaited inside the timed
        region."""
        nxt = upload_inputs()
        prev = None
        for i in range(steps):
            ins = nxt
            y = gm.execute(ins, [out_name])[0]
            for t in ins.values():
                t.dispose()                      # stream-ordered: after the step's kernels
            pending = y.data(into=out_hosts[i & 1])      # D2H queued behind the step
            y.dispose()
            nxt = upload_inputs() if i + 1 < steps else None
            if prev is not None:
                prev.wait()
            prev = pending
        prev.wait()

    for _ in range(max(args.warmup, 3)):
        step_resident()
    be.sync()

    sampler = ClockSampler(local_rank) if rank == 0 else None
    # ---- timed region: device time (CUDA events on the launching stream) ----
    barrier()
    be.sync()
    launches0 = be.launch_count()
    t_host0 = time.perf_counter()
    be.check(be.lib.tfjs_cuda_time_begin(be.ctx))
    for _ in range(args.steps):
        step_resident()
    from ctypes import byref, c_float
    ms = c_float()
    be.check(be.lib.tfjs_cuda_time_end(be.ctx, byref(ms)))   # records + syncs
    be.sync()
    host_ms = (time.perf_counter() - t_host0) * 1e3
    barrier()
    launches = be.launch_count() - launches0
    dev_ms = max_over_ranks(float(ms.value))

    # ---- end to end through the public API with host buffers -----------------
    run_e2e(2)
    barrier()
    be.sync()
    t0 = time.perf_counter()
    run_e2e(args.steps)
    be.sync()
    e2e_s = max_over_ranks(time.perf_counter() - t0)
    barrier()
    clocks = sampler.stop() if sampler is not None else None

    # ---- per-kernel profile (rank 0) -------------------------------------------
    line = None
    if rank == 0:
        # three profiled steps (launched eagerly); per kernel call the fastest of the three
        # is kept, which drops one-off host stalls between the two events of a call
        step_resident()
        runs = [eng.profile(step_resident)["kernels"] for _ in range(3)]
        prof_steps = 1
        records = runs[0]
        if all(len(r) == len(records) for r in runs):
            for i, rec in enumerate(records):
                rec["kernelTimeMs"] = min(r[i]["kernelTimeMs"] for r in runs)
        kinds = summarise_profile(records, prof_steps)
        top = max(kinds, key=lambda k: kinds[k]["ms_per_step"])
        pk = peaks()
        tk = kinds[top]
        tensor_bound = tk["flops_per_byte"] >= 100.0
        roof = {"kernel": top, "launches_per_step": tk["launches_per_step"],
                "share_of_device_time": tk["share"], "traffic": None}
        if tensor_bound:
            tf32_peak = measure_tf32_peak()
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
        units = batch * world
        value = units * args.steps / (dev_ms / 1e3)
        line = {"metric": w["metric"], "value": round(value, 2), "unit": w["unit"],
                "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
                "ms_per_step": round(dev_ms / args.steps, 4), "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "tf32", "data": "synthetic",
                "config": {"workload": w["name"], "batch_per_gpu": batch,
                           "global_batch": units, "parallelism": "replicas x%d" % world,
                           "l2": "activations per step are far larger than L2",
                           "step_replay": bool(gm.replay),
                           "cpu_binding": ("GPU-local cores" if near_cpus else "none"),
                           "weights": "random init"},
                "host_ms_per_step": round(host_ms / args.steps, 4),
                "tflops": round(units * w["gflop"] / 1e3 / (dev_ms / args.steps / 1e3), 2),
                "clocks": clocks,
                "e2e": {"value": round(units * args.steps / e2e_s, 2), "unit": w["unit"],
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
                "gpu_launches": int(launches),
                "roofline": roof,
                "kernels": kinds}
        if world == 1 and not args.no_cpu:
            sample = args.cpu_sample or {"mobilenet_v2": 64, "resnet50": 8, "bert": 4}[args.model]
            v, dt, cores, units = cpu_sample(args.model, sample, min_seconds=10.0)
            line["cpu_baseline"] = {
                "value": round(v, 3), "unit": w["unit"], "cores": cores, "kind": "port",
                "sample": "%d units (batches of %d) of the same graph through the C restatement "
                          "of tfjs-backend-cpu in %.1f s" % (units, sample, dt)}
    for t in resident.values():
        t.dispose()
    gm.dispose()
    if rank == 0:
        print(json.dumps(line))
    group.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="cuda", choices=["cuda", "reference"])
    ap.add_argument("--model", default="mobilenet_v2", choices=sorted(WORKLOADS))
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
