"""BASELINE configs 3, 4 and 5 at their full sizes.  The CPU oracle cannot evaluate them in reasonable
time, so the full batch is checked through properties that do not depend on size:

  * a forward pass is independent per sample: the first rows of the full-batch result must equal the
    result of evaluating those samples alone — bit for bit where the batch size does not change how a
    product is tiled (ResNet, 64 of 256 images), to fp32 rounding where it does (small batches cut long-K
    products into K slices);
  * shuffling the batch shuffles the outputs (again bit for bit);
  * the small batch itself is compared with the oracle (rel <= 1e-3 on logits).

Config 3 is sage's Bert base graph at batch 32 x 128 tokens (the benchmarked workload: at this batch the
projections take other tile widths, the grouped Q / K / V launch and the fused attention kernel's full grid).
Config 4 is the BERT-large-shaped graph (24 layers, width 1024, 16 heads, FFN 4096, L 512, batch 256,
ragged padding 0-128 per sequence); config 5 is sage's ResNet-18 graph on [256, 224, 224, 3].
Weights and inputs are seeded synthetic tensors with the distributions BASELINE.json states.
"""
import time

import numpy as np
import pytest

import sage_b200 as S
from oracle import sage_ref as R

pytestmark = pytest.mark.gpu


def rel_err(a, b, floor):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    scale = np.maximum(np.abs(b), floor * max(np.abs(b).max(), 1e-30))
    return float((np.abs(a - b) / scale).max())


def RV(a, dtype=None):
    return R.Var.new(R.Tensor.new(a, dtype))


LARGE = dict(embed_dim=1024, num_vocabs=30522, max_num_tokens=512, hidden_dim=4096, num_layers=24, num_heads=16, num_classes=2)


@pytest.mark.parametrize("pad", [False, True])
def test_config3_bert_base_full_batch(pad):
    """pad=False is BASELINE config 3 as stated (mask all ones); pad=True adds ragged padding so that the additive
    mask is exercised at the benchmarked batch too."""
    rng = np.random.default_rng(3001)
    batch, seq = 32, 128
    ctx = S.Context(0)
    try:
        model = S.Bert()
        params = model.params()
        values = [(rng.standard_normal(p.extents) * 0.02).astype(np.float32) for p in params]
        for p, v in zip(params, values):
            ctx.set(p, v)
        ids = rng.integers(0, 30522, (batch, seq)).astype(np.uint32)
        mask = np.ones((batch, seq), np.float32)
        if pad:
            for i, n in enumerate(rng.integers(0, 33, batch)):
                mask[i, seq - n:] = 0

        def run(rows):
            return model.pass_(ctx.var(ids[rows]), ctx.var(mask[rows])).eval(ctx)
        full = run(np.arange(batch))
        assert full.shape == (batch, 2) and np.isfinite(full).all() and np.array_equal(full, run(np.arange(batch)))
        small = run(np.arange(2))
        # per-sample independence, to fp32 rounding: at 2 sequences the projections are cut into K slices
        rms = float(np.sqrt((full.astype(np.float64) ** 2).mean()))
        assert float(np.abs(small - full[:2]).max()) / rms <= 1e-5
        perm = rng.permutation(batch)
        assert np.array_equal(run(perm), full[perm])                # batch order does not matter, bit for bit
        assert ctx.status_word() == 0
        rm = R.Bert(R.BertConfig())
        for p, v in zip(rm.params(), values):
            p.set(v)
        ref = rm(RV(ids[:2], R.UINT), RV(mask[:2])).eval().numpy()
        assert rel_err(small, ref, floor=1e-3) <= 1e-3
        assert rel_err(full[:2], ref, floor=1e-3) <= 1e-3          # the batch-32 rows themselves against the oracle
    finally:
        ctx.close()


def test_config4_bert_large_full_batch():
    rng = np.random.default_rng(4001)
    batch, seq = 256, 512
    ctx = S.Context(0)
    try:
        model = S.Bert(**LARGE)
        params = model.params()
        values = [(rng.standard_normal(p.extents) * 0.02).astype(np.float32) for p in params]
        for p, v in zip(params, values):
            ctx.set(p, v)
        ids = rng.integers(0, 30522, (batch, seq)).astype(np.uint32)
        mask = np.ones((batch, seq), np.float32)
        for i, pad in enumerate(rng.integers(0, 129, batch)):
            mask[i, seq - pad:] = 0

        def run(rows):
            t0 = time.perf_counter()
            out = model.pass_(ctx.var(ids[rows]), ctx.var(mask[rows])).eval(ctx)
            ctx.sync()
            return out, time.perf_counter() - t0
        full, _ = run(np.arange(batch))
        full2, dt = run(np.arange(batch))  # second pass: weights split, kernels compiled
        print("\nconfig 4: %d sequences in %.3f s = %.1f seq/s, peak memory %.1f GB" %
              (batch, dt, batch / dt, ctx.mem_stats()["mem_peak"] / 1e9))
        assert full.shape == (batch, 2) and np.isfinite(full).all() and np.array_equal(full, full2)
        small, _ = run(np.arange(2))
        # per-sample independence.  Not bit for bit: at 2 sequences the projections have so few output tiles that
        # they are cut into K slices (another summation order than at 256 sequences); a contraction's error is
        # measured against the rms of its outputs
        assert float(np.abs(small - full[:2]).max() / np.sqrt((full[:2].astype(np.float64) ** 2).mean())) <= 1e-5
        perm = rng.permutation(batch)
        shuffled, _ = run(perm)
        assert np.array_equal(shuffled, full[perm])                 # batch order does not matter
        assert ctx.status_word() == 0
        # the two-sequence batch against the oracle (one layer stack of 24 on the host cores)
        rm = R.Bert(R.BertConfig(embed_dim=1024, num_vocabs=30522, max_num_tokens=512, hidden_dim=4096, num_layers=24,
                                 num_heads=16, num_classes=2))
        for p, v in zip(rm.params(), values):
            p.set(v)
        ref = rm(RV(ids[:2], R.UINT), RV(mask[:2])).eval().numpy()
        assert rel_err(small, ref, floor=1e-3) <= 1e-3
    finally:
        ctx.close()


def test_config5_resnet18_full_batch():
    rng = np.random.default_rng(5001)
    batch = 256
    ctx = S.Context(0)
    try:
        model = S.ResNet18(3, 1000)
        params = model.params()
        values = []
        for p in params:
            e = p.extents
            if len(e) == 4:    # conv filter [KH, KW, C, OC]: He-normal
                values.append((rng.standard_normal(e) * np.sqrt(2.0 / (e[0] * e[1] * e[2]))).astype(np.float32))
            elif len(e) == 2:  # classifier
                values.append((rng.standard_normal(e) * np.sqrt(1.0 / e[0])).astype(np.float32))
            else:
                values.append(np.zeros(e, np.float32))
        for p, v in zip(params, values):
            ctx.set(p, v)
        x = rng.standard_normal((batch, 224, 224, 3)).astype(np.float32)

        def run(rows):
            t0 = time.perf_counter()
            out = model.pass_(ctx.var(x[rows])).eval(ctx)
            ctx.sync()
            return out, time.perf_counter() - t0
        full, _ = run(np.arange(batch))
        full2, dt = run(np.arange(batch))
        print("\nconfig 5: %d images in %.3f s = %.1f img/s, peak memory %.1f GB" %
              (batch, dt, batch / dt, ctx.mem_stats()["mem_peak"] / 1e9))
        assert full.shape == (batch, 1000) and np.isfinite(full).all() and np.array_equal(full, full2)
        # 64 samples keep every contraction on the tensor-core kernel (the classifier has M = batch), so
        # the arithmetic per element is the same as in the full batch
        part, _ = run(np.arange(64))
        assert np.array_equal(full[:64], part)
        perm = rng.permutation(batch)
        shuffled, _ = run(perm)
        assert np.array_equal(shuffled, full[perm])
        assert ctx.status_word() == 0
        small, _ = run(np.arange(2))
        # batch 2 sends the classifier (M = batch) to the SIMT kernel: other summation order, same values
        # (a contraction's error is measured against the rms of its outputs)
        assert float(np.abs(small - full[:2]).max() / np.sqrt((full[:2].astype(np.float64) ** 2).mean())) <= 1e-5
        rm = R.resnet18(3, 1000)
        for p, v in zip(rm.params(), values):
            p.set(v)
        ref = rm(RV(x[:2])).eval().numpy()
        assert rel_err(small, ref, floor=1e-3) <= 1e-3
    finally:
        ctx.close()
