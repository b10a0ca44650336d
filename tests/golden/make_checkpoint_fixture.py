"""Writes tests/golden/two_tensors.msckpt with this repository's checkpoint writer and has the
reference's own Python reader of the format accept it: `read_checkpoint` of
opponents/transformer_block/transformer_block.py, which verifies the header, the header checksum,
the manifest's file_size and the payload hash as the reference's Rust reader does, and reads the
records at their offsets. The script fails unless that reader returns the tensors' bits.

    python tests/golden/make_checkpoint_fixture.py <reference checkout>
"""
import importlib.util
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
import modelspec_b200 as M  # noqa: E402

if len(sys.argv) != 2:
    raise SystemExit(__doc__)
spec = importlib.util.spec_from_file_location("block_opponent", os.path.join(sys.argv[1], "opponents/transformer_block/transformer_block.py"))
opponent = importlib.util.module_from_spec(spec)
spec.loader.exec_module(opponent)


def tensors():
    rng = np.random.default_rng(11)
    return {"w1": rng.standard_normal((4, 8)).astype(np.float32), "w2": rng.standard_normal((8, 1)).astype(np.float32)}


def build(step=3):
    ckpt = M.Checkpoint(step=step, seed=42, schema_hash="ab" * 32)
    ckpt.set_optimizer(M.OPTIMIZER_SGD, float(np.float32(0.1)))
    for name, value in tensors().items():
        ckpt.add("TwoLayer." + name, value)
    return ckpt


if __name__ == "__main__":
    path = os.path.join(HERE, "two_tensors.msckpt")
    ckpt = build()
    ckpt.write(path)
    ckpt.destroy()
    # The reference's reader looks the records up by its own model's names: give it this file's.
    opponent.MODEL = "TwoLayer"
    opponent.shapes = lambda: [(name, value.shape) for name, value in tensors().items()]
    params, step = opponent.read_checkpoint(path, "cpu")
    assert step == 3
    for name, value in tensors().items():
        assert np.array_equal(params[name].detach().numpy().view(np.uint32), value.view(np.uint32)), name
    print("the reference's reader accepts", path, os.path.getsize(path), "bytes")
