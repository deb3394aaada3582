"""Kernel-level micro-benchmarks of the B200 backend: achieved HBM GB/s of the fused map / reduce /
row kernels and f32-equivalent TFLOP/s of the tensor-core GEMM, each as one JSON line.

  python -m sage_b200.microbench --case gemm --m 4096 --n 768 --k 768 [--batch 1] [--reps 20]
  python -m sage_b200.microbench --case map --rows 16384 --cols 4096      # z = x*y + x*3.14 (one fused kernel)
  python -m sage_b200.microbench --case reduce|softmax|layernorm|lse --rows 16384 --cols 4096
  python -m sage_b200.microbench --case config1 --rows 16384 --cols 4096  # whole forward + grad graph
  python -m sage_b200.microbench --case all
  python -m sage_b200.microbench --case train_resnet --batch 128             # examples/train.rs: one Adam step of ResNet-18
  python -m sage_b200.microbench --case train_bert                           # one Adam step of Bert base, batch 32 x 128 tokens
  python -m sage_b200.microbench --case attention --batch 32 --heads 12 --seq 128 --d 64   # fused attention block
  python -m sage_b200.microbench --case conv --batch 32 --h 56 --c 64 --oc 64 --ker 3 --stride 1 --pad 1   # conv_2d, NHWC
  python -m sage_b200.microbench --case tf32_peak                          # library TF32 GEMM: the tensor-pipe denominator

Times are device times from CUDA events recorded on the context's stream in front of every launch
(Context.profile_begin / profile_end).  Algorithmic bytes: every distinct input once + the output once.
"""
import argparse
import ctypes
import json
import os

import numpy as np

import sage_b200 as S

L = ctypes.c_int64


def peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        m = json.load(open(p))
        return m["hbm_gbs"], m["bf16_tflops"], "measured"
    return 6650.0, 1590.0, "fallback"


def timed(ctx, fn, reps, names):
    for _ in range(3):
        fn()
    ctx.sync()
    ctx.profile_begin()
    for _ in range(reps):
        fn()
    prof = ctx.profile_end()
    ms = sum(t for k, (n, t) in prof.items() if any(k.startswith(p) for p in names))
    return ms / reps, prof


def case_gemm(ctx, a):
    m, n, k, b = a.m, a.n, a.k, a.batch
    ta, tb = int(getattr(a, "ta", 0)), int(getattr(a, "tb", 0))  # 1: the operand is stored transposed ([k, m] / [n, k])
    A = ctx.tensor(np.random.default_rng(0).uniform(-1, 1, (b, k, m) if ta else (b, m, k)).astype(np.float32))
    B = ctx.tensor(np.random.default_rng(1).uniform(-1, 1, (b, n, k) if tb else (b, k, n)).astype(np.float32))
    C = ctx.empty((b, m, n))

    def go():
        ctx._ck(S.lib.sage_gemm_strided_batched(ctx.h, ta, tb, L(m), L(n), L(k), A.buf, L(0), L(m if ta else k), L(m * k), B.buf, L(0), L(k if tb else n), L(k * n),
                                                C.buf, L(0), L(n), L(m * n), L(b)))
    ms, prof = timed(ctx, go, a.reps, ["gemm", "reduce"])  # "reduce": the sum over K slices when the product is split over K
    split_ms = prof.get("split_tf32", (0, 0.0))[1] / a.reps
    hbm, bf16, src = peaks()
    tf = 2.0 * m * n * k * b / (ms * 1e-3) / 1e12
    return {"case": "gemm", "m": m, "n": n, "k": k, "batch": b, "ta": ta, "tb": tb, "us": 1e3 * ms, "split_us": 1e3 * split_ms, "tflops_f32_equivalent": tf,
            "tensor_pipe_tflops": 3 * tf, "peak_bf16_tflops": bf16, "frac_of_bf16_peak": 3 * tf / bf16,
            "note": "3xTF32: 3 tensor-core MMAs per logical product; TF32 runs at half the bf16 rate, so 1.0 here would be frac 0.5",
            "peak_source": src, "kernel": [k_ for k_ in prof if k_.startswith("gemm")][0]}


def case_gemm_trace(ctx, a):
    """Where the cycles of one tensor-core GEMM launch go, counted inside the kernel (SAGE_GEMM_TRACE: the launch runs
    the instrumented build and the host reads 16 words per CTA; see TcParams::trace).  Cycles become microseconds with
    the launch's own clock: cycles of the longest CTA / its global-timer duration."""
    import struct
    import tempfile
    m, n, k, b = a.m, a.n, a.k, a.batch
    A = ctx.tensor(np.random.default_rng(0).uniform(-1, 1, (b, m, k)).astype(np.float32))
    B = ctx.tensor(np.random.default_rng(1).uniform(-1, 1, (b, k, n)).astype(np.float32))
    C = ctx.empty((b, m, n))

    def go():
        ctx._ck(S.lib.sage_gemm_strided_batched(ctx.h, 0, 0, L(m), L(n), L(k), A.buf, L(0), L(k), L(m * k), B.buf, L(0), L(n), L(k * n),
                                                C.buf, L(0), L(n), L(m * n), L(b)))
    for _ in range(3):
        go()
    ctx.sync()
    path = tempfile.mktemp(suffix=".gemm_trace")
    os.environ["SAGE_GEMM_TRACE"] = path
    try:
        for _ in range(3):
            go()
        ctx.sync()
    finally:
        del os.environ["SAGE_GEMM_TRACE"]
    raw = open(path, "rb").read()
    os.unlink(path)
    recs, at = [], 0
    while at < len(raw):
        hdr = struct.unpack("8i", raw[at:at + 32])
        at += 32
        grid = hdr[6]
        recs.append((hdr, np.frombuffer(raw[at:at + grid * 128], dtype=np.uint64).reshape(grid, 16).astype(np.int64)))
        at += grid * 128
    hdr, t = recs[-1]
    ctas = hdr[5]
    lead = t[::ctas]                      # the CTAs that issue the MMAs
    ns = (t[:, 1].max() - t[:, 0].min())  # the launch, by the global timer
    cyc_per_us = float((t[:, 15] / np.maximum(t[:, 1] - t[:, 0], 1)).mean() * 1e3)

    def us(c):
        return float(np.mean(c)) / cyc_per_us
    kb = lead[:, 9]
    span = lead[:, 8] - lead[:, 7]
    return {"case": "gemm_trace", "m": m, "n": n, "k": k, "batch": b, "bn": hdr[4], "ctas_per_tile": ctas, "grid": hdr[6], "stages": hdr[7],
            "launch_us": ns / 1e3, "sm_mhz_during_launch": cyc_per_us,
            "k_blocks_per_leader": [int(kb.min()), int(kb.max())],
            "cycles_per_k_block": float(span.mean() / max(kb.mean(), 1)),
            "mma_cycles_per_k_block_at_the_nominal_rate": 3 * 4 * (128 * hdr[4] * 8) // 2048,
            "issue_cycles_of_12_mmas": {"first_k_block": float(lead[:, 10].mean()), "k_block_41": float(lead[:, 11][lead[:, 11] > 0].mean()) if (lead[:, 11] > 0).any() else None},
            "us": {"barriers_and_tmem_ready": us(t[:, 2]), "first_load_issued": us(t[:, 4]), "first_mma": us(lead[:, 7]),
                   "last_commit": us(lead[:, 8]), "cta_end_mean": us(t[:, 15]), "cta_end_max": float(t[:, 15].max()) / cyc_per_us,
                   "mma_warp_waited_for_operands": us(lead[:, 5]), "mma_warp_waited_for_tmem": us(lead[:, 6]),
                   "tma_waited_for_a_free_stage": us(t[:, 3]), "epilogue_waited_for_accumulators": us(t[:, 12]),
                   "epilogue_stores": us(t[:, 13]), "store_per_tile": float(t[:, 13].sum()) / max(float(t[:, 14].sum()), 1.0) / cyc_per_us}}


def row_case(ctx, a, kind):
    rows, cols = a.rows, a.cols
    x = ctx.var(np.random.default_rng(2).standard_normal((rows, cols), dtype=np.float32))
    if kind == "map":
        y = ctx.var(np.random.default_rng(3).standard_normal((rows, cols), dtype=np.float32))
        out, bytes_, names = x * y + x * 3.14, 3 * rows * cols * 4, ["sage_map"]
    elif kind == "reduce":
        out, bytes_, names = x.sum([1], True), rows * cols * 4 + rows * 4, ["reduce"]
    elif kind == "softmax":
        out, bytes_, names = S.softmax(x, [1]), 2 * rows * cols * 4, ["softmax"]
    elif kind == "lse":
        out, bytes_, names = S.log_sum_exp(x, [1]), rows * cols * 4 + rows * 4, ["lse"]
    else:
        g, b = ctx.var(np.float32([1.0])), ctx.var(np.float32([0.0]))
        out, bytes_, names = S.layer_norm(x, [1], g, b, 1e-5), 2 * rows * cols * 4, ["layernorm"]

    def go():
        ctx.clear()
        ctx.eval(out)
    ms, prof = timed(ctx, go, a.reps, [""])  # every kernel of the evaluation (one, whichever way it is lowered)
    hbm, _, src = peaks()
    gbs = bytes_ / (ms * 1e-3) / 1e9
    return {"case": kind, "rows": rows, "cols": cols, "us": 1e3 * ms, "algorithmic_bytes": bytes_, "gb_per_s": gbs, "peak_hbm_gb_per_s": hbm,
            "frac": gbs / hbm, "peak_source": src, "kernels": {k: v for k, v in prof.items()}}


def case_config1(ctx, a):
    rows, cols = a.rows, a.cols
    rng = np.random.default_rng(1001)
    x, y = ctx.var(rng.standard_normal((rows, cols), dtype=np.float32)), ctx.var(rng.standard_normal((rows, cols), dtype=np.float32))
    lab = ctx.var(rng.integers(0, cols, (rows, 1)).astype(np.uint32))
    loss = S.softmax_cross_entropy(x * y + x * 3.14, lab)
    gx = x.grad(loss)

    def go():
        ctx.clear()
        ctx.eval(loss, gx)
    ms, prof = timed(ctx, go, a.reps, [""])
    hbm, _, src = peaks()
    bytes_ = 3 * rows * cols * 4 + rows * 8  # x, y read once, gx written once, labels + loss
    gbs = bytes_ / (ms * 1e-3) / 1e9
    return {"case": "config1_fwd_grad", "rows": rows, "cols": cols, "us": 1e3 * ms, "compulsory_bytes": bytes_, "gb_per_s": gbs,
            "peak_hbm_gb_per_s": hbm, "frac": gbs / hbm, "peak_source": src, "kernels": {k: v for k, v in prof.items()}}


def case_train_resnet(ctx, a):
    """The reference's training example (examples/train.rs): ResNet d18(1, 10) on 28 x 28 x 1 images, batch
    128, Adam(1e-4).  One step = upload of the batch from pinned memory, evaluation of loss + accuracy +
    all gradients (Program::exec), Optimizer::update, read-back of loss and accuracy, Context::data.clear().
    Device time per step from events around the whole loop; the kernel table is from a separate profiled step."""
    batch = a.batch if a.batch > 1 else 128
    rng = np.random.default_rng(6001)
    model = S.ResNet18(1, 10)
    for p in model.params():
        e = p.extents
        ctx.set(p, (rng.standard_normal(e) * (np.sqrt(2.0 / (e[0] * e[1] * e[2])) if len(e) == 4 else 0.05)).astype(np.float32))
    xin, lin = S.Var.empty([batch, 28, 28, 1]), S.Var.empty([batch, 1], S.U32)
    logits = model.pass_(xin)
    loss = S.softmax_cross_entropy(logits, lin).mean([0], False)
    acc = S.accuracy(logits, lin)
    grads = S.grad_param(loss, model)
    opt = S.Adam(1e-4)
    opt.init(ctx)
    hx, hl = ctx.pinned((batch, 28, 28, 1), np.float32), ctx.pinned((batch, 1), np.uint32)
    hx[...] = rng.standard_normal(hx.shape).astype(np.float32)
    hl[...] = rng.integers(0, 10, hl.shape).astype(np.uint32)
    targets = list(grads.values()) + [loss, acc]
    last = {}

    def step():
        ctx.set(xin, None, pinned_ptr=hx.ctypes.data)
        ctx.set(lin, None, pinned_ptr=hl.ctypes.data)
        ctx.eval(*targets)
        opt.update(grads, ctx)
        last["loss"], last["acc"] = float(ctx.read(loss)[0]), float(ctx.read(acc)[0])
        ctx.clear()
    for _ in range(3):
        step()
    first_loss = last["loss"]
    ctx.sync()
    ctx.timer_start()
    for _ in range(a.reps):
        step()
    ms = ctx.timer_stop() / a.reps
    ctx.profile_begin()
    step()
    prof = ctx.profile_end()
    total = sum(t for n, t in prof.values())
    top = sorted(prof.items(), key=lambda kv: -kv[1][1])[:a.top]
    return {"case": "train_resnet18_mnist_shape", "batch": batch, "ms_per_step": ms, "images_per_s": batch / (ms * 1e-3),
            "launches_per_step": sum(n for n, t in prof.values()), "loss_after_3_steps": first_loss, "loss_now": last["loss"],
            "kernel_ms": {k: [n, round(t, 4)] for k, (n, t) in top}, "profiled_step_ms": total}


def case_train_bert(ctx, a):
    """One Adam step of sage's Bert (BertConfig::base(), batch 32, 128 tokens, 2 classes): loss = mean softmax
    cross entropy of the logits, gradients of all parameters, Optimizer::update.  Token ids / mask / labels are
    uploaded and the loss read back every step."""
    batch, seq = (a.batch if a.batch > 1 else 32), 128
    rng = np.random.default_rng(6002)
    model = S.Bert()
    for p in model.params():
        ctx.set(p, (rng.standard_normal(p.extents) * 0.02).astype(np.float32))
    ids, mask, lab = S.Var.empty([batch, seq], S.U32), S.Var.empty([batch, seq]), S.Var.empty([batch, 1], S.U32)
    logits = model.pass_(ids, mask)
    loss = S.softmax_cross_entropy(logits, lab).mean([0], False)
    grads = S.grad_param(loss, model)
    opt = S.Adam(1e-4)
    opt.init(ctx)
    h_ids, h_mask, h_lab = ctx.pinned((batch, seq), np.uint32), ctx.pinned((batch, seq), np.float32), ctx.pinned((batch, 1), np.uint32)
    h_ids[...] = rng.integers(0, 30522, h_ids.shape)
    h_mask[...] = 1.0
    h_lab[...] = rng.integers(0, 2, h_lab.shape)
    targets = list(grads.values()) + [loss]
    last = {}

    def step():
        ctx.set(ids, None, pinned_ptr=h_ids.ctypes.data)
        ctx.set(mask, None, pinned_ptr=h_mask.ctypes.data)
        ctx.set(lab, None, pinned_ptr=h_lab.ctypes.data)
        ctx.eval(*targets)
        opt.update(grads, ctx)
        last["loss"] = float(ctx.read(loss)[0])
        ctx.clear()
    for _ in range(3):
        step()
    first_loss = last["loss"]
    ctx.sync()
    ctx.timer_start()
    for _ in range(a.reps):
        step()
    ms = ctx.timer_stop() / a.reps
    ctx.profile_begin()
    step()
    prof = ctx.profile_end()
    top = sorted(prof.items(), key=lambda kv: -kv[1][1])[:a.top]
    return {"case": "train_bert_base", "batch": batch, "seq": seq, "ms_per_step": ms, "sequences_per_s": batch / (ms * 1e-3),
            "launches_per_step": sum(n for n, t in prof.values()), "loss_after_3_steps": first_loss, "loss_now": last["loss"],
            "kernel_ms": {k: [n, round(t, 4)] for k, (n, t) in top}, "profiled_step_ms": sum(t for n, t in prof.values()),
            "mem_peak_gb": ctx.mem_stats()["mem_peak"] / 1e9}


def case_conv(ctx, a):
    """conv_2d (src/ops/conv.rs:61-96) on [batch, h, h, c] with a [ker, ker, c, oc] filter through sage_conv2d_nhwc.
    FLOPs: 2 * N * OH * OW * OC * KH * KW * C; three times that on the tensor pipe."""
    n, h, c, oc, ker, stride, pad = a.batch, a.h, a.c, a.oc, a.ker, a.stride, a.pad
    rng = np.random.default_rng(0)
    oh = (h + 2 * pad - (ker - 1) - 1) // stride + 1
    X = ctx.tensor(rng.standard_normal((n, h, h, c), dtype=np.float32))
    F = ctx.tensor(rng.standard_normal((ker, ker, c, oc), dtype=np.float32) * np.float32(0.05))
    Y = ctx.empty((n, oh, oh, oc))
    cx, cf, cy, win = X.c(), F.c(), Y.c(), S.window(1, stride, pad, 1)

    def go():
        ctx._ck(S.lib.sage_conv2d_nhwc(ctx.h, ctypes.byref(cx), ctypes.byref(cf), ctypes.byref(win), ctypes.byref(cy)))
    ms_all, prof = timed(ctx, go, a.reps, [""])
    ms = sum(t for k_, (cnt, t) in prof.items() if k_.startswith("gemm")) / a.reps
    flops = 2.0 * n * oh * oh * oc * ker * ker * c
    _, bf16, src = peaks()
    return {"case": "conv", "batch": n, "h": h, "c": c, "oc": oc, "ker": ker, "stride": stride, "pad": pad, "gemm_us": 1e3 * ms, "all_kernels_us": 1e3 * ms_all,
            "tflops_f32_equivalent": flops / (ms * 1e-3) / 1e12, "tensor_pipe_tflops": 3 * flops / (ms * 1e-3) / 1e12,
            "frac_of_bf16_burst_half": 3 * flops / (ms * 1e-3) / 1e12 / (bf16 / 2), "peak_source": src,
            "kernels": {k_: [cnt, t / a.reps * 1e3] for k_, (cnt, t) in prof.items()}}


def case_attention(ctx, a):
    """softmax(Q K^T / sqrt(d) + mask) V for [batch, heads, seq, d] as the model builds it (src/models/bert.rs:250-280):
    one fused launch.  FLOPs: 2 * 2 * seq^2 * d per (batch, head); three times that on the tensor pipe (3xTF32)."""
    n, h, l, d = a.batch, a.heads, a.seq, a.d
    rng = np.random.default_rng(0)
    q, k, v = (ctx.var(rng.standard_normal((n, l, h * d)).astype(np.float32)) for _ in range(3))
    mask = ctx.var(np.ones((n, l), np.float32))

    def split(t):
        return S.transpose(S.view(t, [n, l, h, d]), 2, 1)
    # the operands are results of kernels, as in the model, so that their producers write the tf32 planes
    qv, kv, vv = q * 1.0, k * 1.0, v * 1.0
    ctx.eval(qv, kv, vv)
    scores = S.matmul_batched(split(qv), S.transpose(split(kv), -1, -2)) / float(np.sqrt(np.float32(d)))
    p = S.softmax(scores + (-(S.view(mask, [n, 1, 1, l])) + 1.0) * -1e5, [3])
    y = S.view(S.transpose(S.matmul_batched(p, split(vv)), 2, 1), [n, l, h * d])

    ms, prof = timed_graph(ctx, y, [qv, kv, vv], a.reps, ["attention", "gemm", "softmax"])
    flops = 4.0 * n * h * l * l * d
    _, bf16, src = peaks()
    return {"case": "attention", "batch": n, "heads": h, "seq": l, "d": d, "us": 1e3 * ms, "tflops_f32_equivalent": flops / (ms * 1e-3) / 1e12,
            "tensor_pipe_tflops": 3 * flops / (ms * 1e-3) / 1e12, "frac_of_bf16_burst_half": 3 * flops / (ms * 1e-3) / 1e12 / (bf16 / 2),
            "peak_source": src, "kernels": {k_: [c, t / a.reps * 1e3] for k_, (c, t) in prof.items()}}


def timed_graph(ctx, y, keep, reps, names):
    """Evaluates `y` `reps` times with `keep` held evaluated; device time of the kernels whose names start with `names`."""
    def once():
        ctx.clear()
        ctx.eval(*keep)
        ctx.eval(y)
    for _ in range(3):
        once()
    ctx.sync()
    ctx.profile_begin()
    for _ in range(reps):
        once()
    prof = ctx.profile_end()
    ms = sum(t for k, (n, t) in prof.items() if any(k.startswith(p) for p in names))
    return ms / reps, prof


def case_tf32_peak(a):
    """The tensor-pipe denominator for 3xTF32: the library TF32 GEMM (torch.matmul with TF32 allowed) at
    8192^3, measured like the bf16 figure of MEASURED_PEAKS.json — a burst of 10 and a loop of ~3 s."""
    import time
    import torch
    torch.backends.cuda.matmul.allow_tf32 = True
    dev = "cuda:%d" % a.device
    n = 8192
    x, y = torch.randn(n, n, device=dev), torch.randn(n, n, device=dev)
    for _ in range(3):
        x @ y
    torch.cuda.synchronize()

    def run(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            x @ y
        e1.record()
        torch.cuda.synchronize()
        return 2.0 * n ** 3 * iters / (e0.elapsed_time(e1) * 1e-3) / 1e12
    burst = max(run(10) for _ in range(3))
    t0 = time.time()
    sustained = []
    while time.time() - t0 < 3.0:
        sustained.append(run(50))
    return {"case": "tf32_peak", "n": n, "tf32_tflops_burst": burst, "tf32_tflops_sustained": sustained[-1],
            "f32_equivalent_ceiling_3xtf32_burst": burst / 3, "f32_equivalent_ceiling_3xtf32_sustained": sustained[-1] / 3,
            "method": "torch.matmul fp32 inputs, allow_tf32=True (library kernel; used only as the roofline denominator)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", default="all")
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=768)
    ap.add_argument("--k", type=int, default=768)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--ta", type=int, default=0, help="gemm: operand A is stored as [k, m]")
    ap.add_argument("--tb", type=int, default=0, help="gemm: operand B is stored as [n, k]")
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--h", type=int, default=56)
    ap.add_argument("--c", type=int, default=64)
    ap.add_argument("--oc", type=int, default=64)
    ap.add_argument("--ker", type=int, default=3)
    ap.add_argument("--stride", type=int, default=1)
    ap.add_argument("--pad", type=int, default=1)
    ap.add_argument("--heads", type=int, default=12)
    ap.add_argument("--seq", type=int, default=128)
    ap.add_argument("--d", type=int, default=64)
    ap.add_argument("--top", type=int, default=10, help="training cases: how many kernels of the profiled step to list "
                    "(SAGE_VERBOSE_NAMES=1 gives one name per GEMM shape and map expression)")
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    if a.case == "tf32_peak":
        print(json.dumps(case_tf32_peak(a)), flush=True)
        return
    ctx = S.Context(a.device)
    cases = ["gemm", "map", "reduce", "softmax", "lse", "layernorm", "config1"] if a.case == "all" else [a.case]
    for c in cases:
        if c == "gemm":
            r = case_gemm(ctx, a)
        elif c == "gemm_trace":
            r = case_gemm_trace(ctx, a)
        elif c == "config1":
            r = case_config1(ctx, a)
        elif c == "train_resnet":
            r = case_train_resnet(ctx, a)
        elif c == "conv":
            r = case_conv(ctx, a)
        elif c == "attention":
            r = case_attention(ctx, a)
        elif c == "train_bert":
            r = case_train_bert(ctx, a)
        else:
            r = row_case(ctx, a, c)
        print(json.dumps(r), flush=True)
    ctx.close()


if __name__ == "__main__":
    main()
