"""`train --backend cuda --data <packed directory>`: a run fed from a packed directory through the
C ABI gives the bits of the same run fed the same batches by hand, its held-out split is the
directory's, and the declarations a packed directory cannot feed are refused with the
reference's diagnostics (crates/modelspec-runtime/src/train/data.rs:1588-1840,
train/eval.rs:167-199)."""
import os

import numpy as np
import pytest

import modelspec_b200 as M
import packed_dir
from modelspec_b200 import models

pytestmark = pytest.mark.gpu

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "mlm_feed.npz"))
SEQ, VOCAB, BATCH, SEED = (int(GOLDEN[k]) for k in ("seq", "vocab", "batch", "seed"))
SHAPE = dict(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=VOCAB, seq=SEQ, batch=BATCH, warmup_steps=1, seed=SEED)


@pytest.fixture()
def packed(tmp_path):
    packed_dir.write(str(tmp_path), GOLDEN["train"], GOLDEN["heldout"], SEQ, VOCAB)
    p = M.Packed(str(tmp_path))
    yield p
    p.close()


def test_a_run_on_a_packed_directory_is_the_run_on_its_batches(device, packed):
    steps = 12  # past the 9 batches of epoch 0
    source = models.bert(steps=steps, **SHAPE)
    runs = []
    for by_hand in (False, True):
        gpu = M.Training(device, source, 16)
        try:
            if by_hand:
                gpu.heldout_begin(2, "labels", "weights")
                for b in range(2):
                    for name, value in packed.batch(M.SPLIT_HELDOUT, SEED, b, BATCH).items():
                        gpu.heldout_set(b, name, value)
            else:
                gpu.bind_packed(packed)
                assert gpu.heldout_packed() == 2
            seen = [gpu.heldout_evaluate()]
            for k in range(steps):
                if by_hand:
                    for name, value in packed.batch(M.SPLIT_TRAIN, SEED, k, BATCH).items():
                        gpu.set_input(name, value)
                else:
                    gpu.feed_packed(k)
                gpu.step(k, steps)
                seen.append(gpu.loss())
            seen.append(gpu.heldout_evaluate())
            runs.append(np.array([np.ravel(x) for x in seen[1:-1]], dtype=np.float32).tobytes() + np.array(seen[0] + seen[-1], dtype=np.float32).tobytes())
            assert seen[-1][0] < seen[0][0], "twelve steps lower the held-out loss"
        finally:
            gpu.destroy()
    assert runs[0] == runs[1]


def refused(device, source, packed, code, text):
    gpu = M.Training(device, source, 0)
    try:
        with pytest.raises(M.MsxError) as e:
            gpu.bind_packed(packed)
        assert e.value.status == M.BAD_INPUT and code in str(e.value) and text in str(e.value), str(e.value)
    finally:
        gpu.destroy()


def test_declarations_a_packed_directory_cannot_feed_are_refused(device, packed):
    refused(device, models.linear_regression(steps=2), packed, "E-DATA-005", "the input `x` names no tensor of the masked-language-model batch")
    # 4 x 8 ids are two sequences of 16, so `ids` gives B = 2 and the [4, 8] key mask does not fit; 4 x 5 ids give no B at all.
    refused(device, models.bert(steps=2, **{**SHAPE, "seq": 8}), packed, "E-DATA-006",
            "the input `key_mask` is not of the type of the batch tensor `key_mask`: it is Tensor<f32, [4, 8]>, expected Tensor<f32, [2, 16]> or Tensor<f32, [32]>")
    refused(device, models.bert(steps=2, **{**SHAPE, "seq": 5}), packed, "E-DATA-006",
            "the input `ids` is not of the type of the batch tensor `ids`: it is Tensor<i32, [20]>, expected Tensor<i32, [B, 16]> or Tensor<i32, [B·16]>")
    refused(device, models.bert(steps=2, **{**SHAPE, "vocab": VOCAB + 3}), packed, "E-DATA-006",
            "the table `BertTiny.tok_table` of the `embedding` that reads `ids` has 64 rows, not the 61 tokens of the packed vocabulary")
    refused(device, models.bert(steps=2, **{**SHAPE, "batch": 40}), packed, "", "a batch of 40 sequences, more than the 37 of the Train split")


def test_a_held_out_split_smaller_than_a_batch_is_refused(device, tmp_path):
    packed_dir.write(str(tmp_path), GOLDEN["train"], GOLDEN["heldout"][:3 * SEQ], SEQ, VOCAB)
    packed = M.Packed(str(tmp_path))
    gpu = M.Training(device, models.bert(steps=2, **SHAPE), 0)
    try:
        gpu.bind_packed(packed)
        with pytest.raises(M.MsxError) as e:
            gpu.heldout_packed()
        assert "holds 3 sequences, fewer than the batch of 4 that --eval-every evaluates" in str(e.value)
        gpu.feed_packed(0)
        gpu.step(0, 2)
        assert np.isfinite(gpu.loss())
    finally:
        gpu.destroy()
        packed.close()
