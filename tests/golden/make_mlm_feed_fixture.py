"""Writes tests/golden/mlm_feed.npz: batches and epoch orders of a small packed directory as the
reference's own Python copy of its feed draws them (opponents/bert_tiny/bert_tiny.py, `Packed`:
`epoch_order` and `batch`, which the reference keeps bit-identical to dataset/mlm.rs `epoch_order`
and `mlm_batch`). The fixture holds the packed ids too, so the test rebuilds the directory.

    python tests/golden/make_mlm_feed_fixture.py <reference checkout>
"""
import importlib.util
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import packed_dir  # noqa: E402

if len(sys.argv) != 2:
    raise SystemExit(__doc__)
spec = importlib.util.spec_from_file_location("bert_tiny_opponent", os.path.join(sys.argv[1], "opponents/bert_tiny/bert_tiny.py"))
opponent = importlib.util.module_from_spec(spec)
spec.loader.exec_module(opponent)

SEQ, VOCAB, BATCH, SEED = 16, 61, 4, 42
rng = np.random.default_rng(20240607)
train = rng.integers(0, VOCAB, 37 * SEQ).astype(np.int32)   # 37 sequences: 9 whole batches of 4 an epoch
heldout = rng.integers(0, VOCAB, 9 * SEQ).astype(np.int32)  # 2 whole batches
out = {"train": train, "heldout": heldout, "seq": SEQ, "vocab": VOCAB, "batch": BATCH, "seed": SEED}
with tempfile.TemporaryDirectory() as d:
    packed_dir.write(d, train, heldout, SEQ, VOCAB)
    packed = opponent.Packed(d)
    for epoch in (0, 1, 7):
        out["order_%d" % epoch] = np.array(packed.epoch_order(SEED, epoch), dtype=np.uint32)
    for role, steps in (("Train", (0, 1, 8, 9, 10, 30)), ("HeldOut", (0, 1, 2))):
        for step in steps:
            ids, labels, weights = packed.batch(role, SEED, step, BATCH)
            out["%s_%d_ids" % (role, step)] = np.array(ids, dtype=np.int32)
            out["%s_%d_labels" % (role, step)] = np.array(labels, dtype=np.int32)
            out["%s_%d_weights" % (role, step)] = np.array(weights, dtype=np.float32)
np.savez_compressed(os.path.join(HERE, "mlm_feed.npz"), **out)
print("wrote", os.path.join(HERE, "mlm_feed.npz"))
