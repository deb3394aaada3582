#!/usr/bin/env python3
"""Headline benchmark: sage's BERT-base encoder forward (models::Bert, BertConfig::base(), f32,
seq 128, batch 32 per GPU) on the B200 CUDA backend, in sequences per second.

  python bench.py --gpus N --steps K --warmup W            this backend
  python bench.py --impl reference --gpus N --steps K ...   the CPU restatement of the reference's
                                                            path (its own code cannot be built: nightly
                                                            Rust + OpenCL), timed on the host cores

A step is one forward pass over one batch of synthetic token ids (uniform in [0, 30522), mask all
ones) with random N(0, 0.02) weights.  `value` times K steps with the inputs already in HBM
(CUDA events on the context's stream); `e2e` times the same K steps through the public API with
the ids/mask copied from pinned host memory and the logits read back every step.  With N > 1 each
rank holds a full weight replica and its own batch of 32 (weak scaling); the only cross-GPU step
is the copy of each rank's logits into rank 0's memory.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BATCH, SEQ = 32, 128
CFG = dict(embed_dim=768, num_vocabs=30522, max_num_tokens=512, hidden_dim=3072, num_layers=12, num_heads=12, num_classes=2)
METRIC, UNIT = "bert_base_fwd_seq_per_s", "seq/s"


WORKLOAD = ("sage models::Bert BertConfig::base() forward (12 layers, hidden 768, 12 heads, FFN 3072, ReLU, "
            "LayerNorm eps 1e-5, vocab 30522), seq 128, f32, random N(0,0.02) weights")


def gemm_flops(batch, seq, c=CFG):
    """Logical 2*M*N*K of every contraction in one forward pass."""
    t, e, f, h = batch * seq, c["embed_dim"], c["hidden_dim"], c["num_heads"]
    d = e // h
    per_layer = 4 * 2 * t * e * e + 2 * 2 * t * e * f + 2 * 2 * batch * h * seq * seq * d
    return c["num_layers"] * per_layer + 2 * batch * e * c["num_classes"]


# DRAM traffic of the dominant kernel per launch, from the ncu capture summarised in
# profiles/bench_bert_base_gemm_traffic.md (5800 MB over the 72 tensor-core GEMM launches of one step).
GEMM_DRAM_BYTES_PER_LAUNCH = 80.56e6


def tf32_library_peak(device):
    """TF32 GEMM rate of the vendor library on this GPU (torch.matmul, 8192^3, best of 3 bursts of 10):
    the same method as the bf16 figure of MEASURED_PEAKS.json.  Only a denominator; nothing on the
    benchmarked path uses it."""
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    n = 8192
    x, y = torch.randn(n, n, device=device), torch.randn(n, n, device=device)
    for _ in range(3):
        x @ y
    torch.cuda.synchronize(device)
    best = 0.0
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(10):
            x @ y
        e1.record()
        torch.cuda.synchronize(device)
        best = max(best, 2.0 * n ** 3 * 10 / (e0.elapsed_time(e1) * 1e-3) / 1e12)
    return best


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        m = json.load(open(p))
        return dict(hbm_gbs=m["hbm_gbs"], bf16=m["bf16_tflops"], bf16_sustained=m["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi in the background during the timed region (read-only queries)."""
    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, gpu):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(gpu), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()  # the exact child started above
        self.thread.join(timeout=2)
        sm = [float(r[0]) for r in self.rows if len(r) >= 7 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 7 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 7 and r[3 + i].lower().startswith("active") for r in self.rows)]
        busy = [s for s in sm if s > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": float(np.median(busy)) if busy else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def make_weights(shapes, seed):
    rng = np.random.default_rng(seed)
    return [(rng.standard_normal(s, dtype=np.float32) * np.float32(0.02)) for s in shapes]


# ------------------------------------------------------------------------------ CPU arm (oracle)
class CpuBert:
    """The CPU restatement of the reference's path (oracle/): one loop nest per reference kernel,
    OpenMP over the reference's work-items.  Used only as the timed baseline."""

    def __init__(self, seed=3001):
        from oracle import sage_ref as R
        self.R = R
        self.model = R.Bert(R.BertConfig(**{k: CFG[k] for k in ("embed_dim", "num_vocabs", "max_num_tokens", "hidden_dim", "num_layers", "num_classes")},
                                         num_heads=CFG["num_heads"]))
        params = self.model.params()
        for p, v in zip(params, make_weights([p.extents for p in params], seed)):
            p.set(v)
        self.cores = R.num_threads()

    def forward(self, ids, mask):
        R = self.R
        return self.model(R.Var.new(R.Tensor.new(ids, R.UINT)), R.Var.new(R.Tensor.new(mask))).eval().numpy()


def cpu_sample(cpu, sample_batch, min_seconds, rng):
    """Runs forward passes of `sample_batch` sequences until `min_seconds` have passed; seq/s."""
    ids = rng.integers(0, CFG["num_vocabs"], (sample_batch, SEQ)).astype(np.uint32)
    mask = np.ones((sample_batch, SEQ), np.float32)
    n, t0 = 0, time.perf_counter()
    while True:
        cpu.forward(ids, mask)
        n += 1
        el = time.perf_counter() - t0
        if el >= min_seconds:
            return n * sample_batch / el, n, el


def run_reference(args, rank, world):
    """--impl reference: the reference's path on the host cores (all OpenMP threads), same metric and
    config; each step is a bounded sample of the batch so the run ends within minutes."""
    if rank != 0:
        return
    sample_batch = 2
    cpu = CpuBert()
    rng = np.random.default_rng(7)
    ids = rng.integers(0, CFG["num_vocabs"], (sample_batch, SEQ)).astype(np.uint32)
    mask = np.ones((sample_batch, SEQ), np.float32)
    for _ in range(args.warmup):
        cpu.forward(ids, mask)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu.forward(ids, mask)
    el = time.perf_counter() - t0
    value = args.steps * sample_batch / el
    sample = "%d sequences of %d tokens per step (full 12-layer model); CPU oracle, no GPU" % (sample_batch, SEQ)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * el / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "batch_per_gpu": BATCH, "global_batch": BATCH, "seq_len": SEQ,
                   "sample_batch_per_step": sample_batch},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cpu.cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


# ------------------------------------------------------------------------------ GPU arm
def run_ours(args, rank, local_rank, world, dist):
    import sage_b200 as S  # raises if libsagecuda.so is missing: there is no fallback
    from sage_b200.shard import OutputGather, max_over_ranks

    if S.device_count() <= local_rank:
        raise RuntimeError("bench.py needs CUDA device %d; there is no CPU fallback" % local_rank)
    ctx = S.Context(local_rank)
    model = S.Bert(**CFG)
    params = model.params()
    for p, v in zip(params, make_weights([p.extents for p in params], 3001)):
        ctx.set(p, v)
    rng = np.random.default_rng(100 + rank)
    n_pool = 4  # distinct host batches cycled through the steps
    ids_host = [ctx.pinned((BATCH, SEQ), np.uint32) for _ in range(n_pool)]
    mask_host = ctx.pinned((BATCH, SEQ), np.float32)
    mask_host[...] = 1.0
    for a in ids_host:
        a[...] = rng.integers(0, CFG["num_vocabs"], (BATCH, SEQ)).astype(np.uint32)
    out_host = ctx.pinned((BATCH, CFG["num_classes"]), np.float32)
    ids, mask = ctx.var(ids_host[0]), ctx.var(mask_host)
    logits = model.pass_(ids, mask)
    gather = OutputGather(ctx, dist, rank, world, BATCH * world, CFG["num_classes"] * 4)

    def barrier():
        ctx.sync()
        if world > 1:
            dist.barrier()

    def step_resident():
        ctx.clear()
        ctx.eval(logits)
        gather.write(logits)

    def step_e2e(i):
        ctx.set(ids, None, pinned_ptr=ids_host[i % n_pool].ctypes.data)
        ctx.set(mask, None, pinned_ptr=mask_host.ctypes.data)
        ctx.clear()
        ctx.eval(logits)
        gather.write(logits)
        ctx.read_into(logits, out_host.ctypes.data, out_host.nbytes)  # blocking device-to-host read

    for _ in range(max(args.warmup, 3)):
        step_resident()
    barrier()

    # ---- value: K steps, inputs resident in HBM, CUDA events on the launching stream
    k0 = ctx.launch_count()[0]
    sampler = ClockSampler(local_rank)
    ctx.timer_start()
    for _ in range(args.steps):
        step_resident()
    ms = ctx.timer_stop()
    barrier()
    clocks = sampler.stop()
    launches = ctx.launch_count()[0] - k0

    # ---- roofline: the same K steps again with an event in front of every launch
    ctx.profile_begin()
    for _ in range(args.steps):
        step_resident()
    prof = ctx.profile_end()
    barrier()

    # ---- e2e: host buffers in, host logits out, every step
    for i in range(2):
        step_e2e(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(args.steps):
        step_e2e(i)
    ctx.sync()
    e2e_s = time.perf_counter() - t0
    barrier()

    ms, e2e_s = max_over_ranks(dist, world, [ms, e2e_s], device="cuda:%d" % local_rank)
    gathered_ok = None
    if rank == 0:
        g = gather.read((BATCH * world, CFG["num_classes"]))
        gathered_ok = bool(np.isfinite(g).all() and np.abs(g).max() > 0)
    status = ctx.status_word()
    tf32_live = None
    if rank == 0:
        try:
            tf32_live = tf32_library_peak("cuda:%d" % local_rank)
        except Exception as e:  # the denominator is optional; the benchmark is not
            tf32_live = "unavailable: %s" % e
    return dict(tf32_live=tf32_live, ms=ms, e2e_s=e2e_s, clocks=clocks, launches=launches, prof=prof, gathered_ok=gathered_ok, status=status,
                mem=ctx.mem_stats())


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod
        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=torch.device("cuda:%d" % local_rank))
        dist = dist_mod
    r = run_ours(args, rank, local_rank, world, dist)
    if rank != 0:
        if dist:
            dist.barrier()
            dist.destroy_process_group()
        return

    pk = peaks()
    seqs = BATCH * world * args.steps
    value = seqs / (r["ms"] / 1e3)
    flops = gemm_flops(BATCH, SEQ)
    gemm_ms = sum(ms for name, (n, ms) in r["prof"].items() if name.startswith("gemm"))
    gemm_n = sum(n for name, (n, ms) in r["prof"].items() if name.startswith("gemm"))
    total_ms = sum(ms for n, ms in r["prof"].values()) or 1.0
    tc = any(name.startswith("gemm_tc") for name in r["prof"])
    # The GEMMs run 3xTF32: every logical product is three tensor-core MMAs on the TF32 pipe, whose
    # dense rate is half the bf16 rate.  achieved = tensor-pipe work (6*M*N*K per GEMM) / time; peak =
    # the measured bf16 figure / 2.  The f32-equivalent rate (2*M*N*K / time) is reported beside it.
    f32_eq = (flops * args.steps / (gemm_ms / 1e3) / 1e12) if gemm_ms else None
    tf32_peak = pk["bf16_sustained"] / 2
    roofline = {
        "bound": "tensor", "kernel": "gemm_tcgen05_3xtf32" if tc else "gemm_simt",
        "achieved": 3 * f32_eq if f32_eq else None, "peak": tf32_peak, "unit": "TFLOP/s",
        "frac": (3 * f32_eq / tf32_peak) if f32_eq else None, "traffic": GEMM_DRAM_BYTES_PER_LAUNCH,
        "peak_source": "%s bf16 dense sustained (MEASURED_PEAKS.json) / 2: the TF32 pipe runs at half the bf16 rate" % pk["source"],
        "f32_equivalent_tflops": f32_eq, "tf32_library_peak_live": r.get("tf32_live"),
        "algorithmic_flops_per_step": flops, "tensor_pipe_flops_per_step": 3 * flops,
        "launches_per_step": gemm_n / args.steps if args.steps else None,
        "avg_launch_us": 1e3 * gemm_ms / gemm_n if gemm_n else None, "share_of_device_time": gemm_ms / total_ms,
        "timed": "second pass of the same K steps with a CUDA event in front of every launch",
        "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum over the 72 GEMM launches of one step / 72 "
                          "(profiles/bench_bert_base_gemm_traffic.md)",
    }
    out = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": r["ms"] / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD,
                   "batch_per_gpu": BATCH, "global_batch": BATCH * world, "seq_len": SEQ, "parallelism": "batch-sharded x%d, weight replicas" % world,
                   "l2": "weights (436 MB) + activations exceed the 126 MB L2; no explicit flush"},
        "clocks": r["clocks"],
        "e2e": {"value": seqs / r["e2e_s"], "unit": UNIT, "h2d_bytes_per_step": BATCH * SEQ * 8, "d2h_bytes_per_step": BATCH * CFG["num_classes"] * 4,
                "timed": "host wall clock, synchronised at both ends"},
        "gpu_launches": r["launches"],
        "roofline": roofline,
        "kernels": {k: {"launches": n, "ms": round(ms, 4)} for k, (n, ms) in r["prof"].items()},
        "gathered_ok": r["gathered_ok"], "status_word": r["status"], "mem_peak_bytes": r["mem"]["mem_peak"],
    }
    if world == 1 and not args.no_cpu_baseline:
        cpu = CpuBert()
        v, n, el = cpu_sample(cpu, 2, 10.0, np.random.default_rng(7))
        out["cpu_baseline"] = {"value": v, "unit": UNIT, "cores": cpu.cores, "kind": "port",
                               "sample": "%d forward passes of 2 sequences x 128 tokens (full 12-layer model) in %.1f s" % (n, el)}
    print(json.dumps(out))
    if dist:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
