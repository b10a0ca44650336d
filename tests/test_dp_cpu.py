"""The data-parallel arithmetic on CPU ranks (gloo, world size 2, no GPU): a shard's gradient,
computed with its own weight sum and rescaled to the whole batch's, summed over the ranks, is the
gradient one device computes on the whole batch; shards of the synthetic batch are slices of the
global batch; and the sharded dropout mask is a slice of the global mask."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
WORKER = '''
import os, sys
sys.path.insert(0, %(root)r); sys.path.insert(0, %(here)r)
import numpy as np, torch, torch.distributed as dist
import oracle_lib
from modelspec_b200 import models, synthetic
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo")
batch, seq, vocab = 2, 8, 50
kw = dict(name="T", layers=1, hidden=16, heads=2, ffn=32, vocab=vocab, seq=seq, dropout=0.0, lr=1e-3, warmup_steps=1, steps=2)
rows = batch * seq
full = synthetic.mlm_batch(0, vocab=vocab, seq=seq, batch=batch * world, selection_rate=0.4, mask_id=4)
mine = {k: v[rank * rows:(rank + 1) * rows] for k, v in full.items()}
again = synthetic.mlm_batch(0, vocab=vocab, seq=seq, batch=batch, selection_rate=0.4, mask_id=4, row_offset=rank * rows)
# The token draw of a shard addressed by row offset is the slice of the global draw.
assert np.array_equal(again["labels"], mine["labels"]) and np.array_equal(again["ids"], mine["ids"])
local = oracle_lib.Trainer(models.bert(batch=batch, **kw))
for name, value in mine.items():
    local.set_input(name, value)
local.step(0, 2)
den_local, den_global = float(mine["weights"].sum()), float(full["weights"].sum())
assert den_local > 0 and den_global > den_local
ok = True
whole = oracle_lib.Trainer(models.bert(batch=batch * world, **kw))
for name, value in full.items():
    whole.set_input(name, value)
whole.step(0, 2)
for i, path in enumerate(local.param_paths()):
    g = torch.from_numpy(local.read("grad", i).astype(np.float64) * (den_local / den_global))
    dist.all_reduce(g)
    want = whole.read("grad", i).astype(np.float64)
    if not np.allclose(g.numpy(), want, rtol=1e-4, atol=1e-6):
        ok = False
        print("MISMATCH", path, np.abs(g.numpy() - want).max(), flush=True)
dist.barrier()
dist.destroy_process_group()
print("DP_CPU_OK" if ok else "DP_CPU_FAILED", flush=True)
sys.exit(0 if ok else 1)
'''


def test_summed_shard_gradients_equal_the_whole_batch_gradient(tmp_path):
    import subprocess
    script = tmp_path / "worker.py"
    script.write_text(WORKER % {"root": os.path.dirname(HERE), "here": HERE})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29741", str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and r.stdout.count("DP_CPU_OK") == 2, r.stdout[-2000:] + r.stderr[-2000:]


def test_a_sharded_dropout_mask_is_a_slice_of_the_global_mask():
    import ctypes as C
    import oracle_lib
    L = oracle_lib.lib()
    draw = L.orc_dropout_id(b"M.forward.dropout#0", 3)
    width, rows_per_rank = 8, 4
    whole = [L.orc_dropout_keeps(42, draw, i, C.c_float(0.3)) for i in range(2 * rows_per_rank * width)]
    for rank in range(2):
        base = rank * rows_per_rank * width  # what msx_set_shard adds to every element index
        shard = [L.orc_dropout_keeps(42, draw, base + i, C.c_float(0.3)) for i in range(rows_per_rank * width)]
        assert shard == whole[base:base + rows_per_rank * width]
