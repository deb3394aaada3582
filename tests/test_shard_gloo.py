"""Host side of the multi-GPU path, run as two gloo ranks on the CPU: how the batch is cut, the
rendezvous that carries rank 0's IPC handle to the others, the max-over-ranks timing, and that
each rank plans the same launch list for its own slice (weight replicas, no data-path collective).
"""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np

from sage_b200.shard import batch_slice, row_offsets

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys, json
    sys.path.insert(0, %r)
    import torch.distributed as dist
    import sage_b200 as S
    from sage_b200.shard import batch_slice, row_offsets, share_from_rank0, max_over_ranks

    dist.init_process_group(backend="gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    GLOBAL = 9                                   # ragged on purpose: 5 + 4
    lo, hi = batch_slice(GLOBAL, rank, world)
    # rank 0 "exports" a 64-byte handle and an offset; every rank must end up with the same bytes
    payload = (bytes(range(64)), 4096) if rank == 0 else None
    got = share_from_rank0(dist, world, payload)
    assert got == (bytes(range(64)), 4096), got
    # slowest rank sets the time
    t = max_over_ranks(dist, world, [10.0 + rank, 5.0 - rank])
    assert t == [10.0 + world - 1, 5.0], t
    # each rank plans its slice on a planning context: same kernels, batch-dependent shapes only
    ctx = S.Context(-1)
    model = S.Bert(num_vocabs=64, embed_dim=64, num_heads=2, seq_len=16, ffn_dim=128, num_layers=2, num_classes=3)
    import numpy as np
    for p in model.params():
        ctx.set(p, np.zeros(p.extents, np.float32))
    ids = ctx.var(np.zeros((hi - lo, 16), np.uint32))
    mask = ctx.var(np.ones((hi - lo, 16), np.float32))
    logits = model.pass_(ids, mask)
    ctx.trace_begin()
    ctx.eval(logits)
    names = [n for n in ctx.trace()]
    rows = [None] * world
    dist.all_gather_object(rows, dict(rank=rank, lo=lo, hi=hi, shape=list(logits.extents), n=len(names),
                                      kinds=sorted(set(x.split("<")[0].split("(")[0] for x in names))))
    dist.barrier()
    if rank == 0:
        print("RESULT " + json.dumps(rows))
    ctx.close()
    dist.destroy_process_group()
""")


def test_batch_slice_tiles_the_batch():
    for g in (0, 1, 7, 32, 255, 256):
        for w in (1, 2, 3, 4, 8):
            cuts = [batch_slice(g, r, w) for r in range(w)]
            assert cuts[0][0] == 0 and cuts[-1][1] == g
            assert all(cuts[i][1] == cuts[i + 1][0] for i in range(w - 1))
            sizes = [b - a for a, b in cuts]
            assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)
            assert row_offsets(g, w, 12) == [a * 12 for a, _ in cuts]


def test_two_ranks_gloo(tmp_path):
    import json
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=240)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outs.append(out)
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    line = [l for l in outs[0].splitlines() if l.startswith("RESULT ")][0]
    rows = json.loads(line[len("RESULT "):])
    assert [(r["lo"], r["hi"]) for r in rows] == [(0, 5), (5, 9)]
    assert [r["shape"] for r in rows] == [[5, 3], [4, 3]]
    assert rows[0]["n"] == rows[1]["n"] and rows[0]["kinds"] == rows[1]["kinds"]
    assert np.all([r["n"] > 0 for r in rows])
