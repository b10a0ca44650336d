"""The packed masked-language-model feed against the batches and epoch orders the reference's own
Python copy of `mlm_batch` drew (tests/golden/mlm_feed.npz, written by
tests/golden/make_mlm_feed_fixture.py), bit for bit, and the refusals of a directory that
disagrees with its record (dataset/mlm.rs:583-660, train/data.rs:1443-1483 of the reference).
Host code: no GPU needed."""
import json
import os

import numpy as np
import pytest

import modelspec_b200 as M
import packed_dir

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "mlm_feed.npz"))
SEQ, VOCAB, BATCH, SEED = (int(GOLDEN[k]) for k in ("seq", "vocab", "batch", "seed"))


@pytest.fixture()
def directory(tmp_path):
    packed_dir.write(str(tmp_path), GOLDEN["train"], GOLDEN["heldout"], SEQ, VOCAB)
    return str(tmp_path)


def test_the_directory_opens_with_its_record(directory):
    packed = M.Packed(directory)
    try:
        assert (packed.seq_len, packed.vocabulary) == (SEQ, VOCAB)
        assert packed.sequences(M.SPLIT_TRAIN) == 37 and packed.sequences(M.SPLIT_HELDOUT) == 9
        assert packed.binding_id == packed_dir.binding_id(packed_dir.DATASET_ID, packed_dir.TOKENIZER_ID, SEQ, packed_dir.BERT_POLICY)
    finally:
        packed.close()


def test_the_uuid_marks_version_8_and_the_rfc_variant():
    # dataset/mod.rs:234-239 of the reference.
    assert packed_dir.uuid_of(b"\xff" * 32) == "ffffffff-ffff-8fff-bfff-ffffffffffff"
    assert packed_dir.uuid_of(b"\x00" * 32) == "00000000-0000-8000-8000-000000000000"


def test_epoch_orders_are_the_reference_copy_s(directory):
    packed = M.Packed(directory)
    try:
        for epoch in (0, 1, 7):
            order = packed.epoch_order(SEED, epoch)
            assert np.array_equal(order, GOLDEN["order_%d" % epoch])
            assert sorted(order.tolist()) == list(range(37))
    finally:
        packed.close()


@pytest.mark.parametrize("role,split,steps", [("Train", M.SPLIT_TRAIN, (0, 1, 8, 9, 10, 30)), ("HeldOut", M.SPLIT_HELDOUT, (0, 1, 2))])
def test_batches_are_the_reference_copy_s(directory, role, split, steps):
    packed = M.Packed(directory)
    try:
        for step in steps:
            batch = packed.batch(split, SEED, step, BATCH)
            for key in ("ids", "labels", "weights"):
                assert np.array_equal(batch[key], GOLDEN["%s_%d_%s" % (role, step, key)]), (role, step, key)
            assert np.array_equal(batch["positions"], np.tile(np.arange(SEQ, dtype=np.int32), BATCH))
            assert np.array_equal(batch["key_mask"], np.ones(BATCH * SEQ, dtype=np.float32))
            # Special tokens are never selected; a selected row keeps its label.
            assert not batch["weights"][batch["labels"] < 5].any()
    finally:
        packed.close()


def test_a_held_out_batch_is_in_stored_order_and_a_train_batch_in_epoch_order(directory):
    packed = M.Packed(directory)
    try:
        held = packed.batch(M.SPLIT_HELDOUT, SEED, 1, BATCH)
        assert np.array_equal(held["labels"], GOLDEN["heldout"][BATCH * SEQ:2 * BATCH * SEQ])
        assert np.array_equal(packed.batch(M.SPLIT_HELDOUT, SEED, 3, BATCH)["labels"], held["labels"]), "2 whole batches: step 3 is batch 1"
        order = packed.epoch_order(SEED, 1)
        train = packed.batch(M.SPLIT_TRAIN, SEED, 9 + 2, BATCH)  # 9 batches an epoch: batch 2 of epoch 1
        rows = np.concatenate([GOLDEN["train"][s * SEQ:(s + 1) * SEQ] for s in order[2 * BATCH:3 * BATCH]])
        assert np.array_equal(train["labels"], rows)
    finally:
        packed.close()


def test_batch_sizes_the_split_cannot_fill_are_refused(directory):
    packed = M.Packed(directory)
    try:
        for size, text in ((0, "a batch of 0 sequences"), (10, "a batch of 10 sequences, more than the 9 of the split")):
            with pytest.raises(M.MsxError) as e:
                packed.batch(M.SPLIT_HELDOUT, SEED, 0, size)
            assert e.value.status == M.BAD_INPUT and text in str(e.value)
    finally:
        packed.close()


def rewrite(directory, name, change):
    path = os.path.join(directory, name)
    record = json.load(open(path))
    change(record)
    json.dump(record, open(path, "w"))


def test_a_directory_that_disagrees_with_its_record_is_refused(directory):
    def refused(text):
        with pytest.raises(M.MsxError) as e:
            M.Packed(directory)
        assert e.value.status == M.BAD_INPUT and text in str(e.value), str(e.value)

    tokens = os.path.join(directory, "train.tokens")
    good = open(tokens, "rb").read()
    open(tokens, "wb").write(good[:-4])
    refused("bytes, not 37 sequences of 16 ids")
    flipped = bytearray(good)
    flipped[0] ^= 1
    open(tokens, "wb").write(bytes(flipped))
    refused("blake3 differs from the content_hash of packed.json")
    open(tokens, "wb").write(good)
    M.Packed(directory).close()
    rewrite(directory, "packed.json", lambda r: r.update(vocabulary_size=5))
    refused("vocabulary_size 5 is not between 6 and 2^31")
    rewrite(directory, "packed.json", lambda r: r.update(vocabulary_size=VOCAB - 30))
    refused("outside a vocabulary of 31")
    rewrite(directory, "packed.json", lambda r: r.update(vocabulary_size=VOCAB, splits=r["splits"][::-1]))
    refused("not a record of a Train and a HeldOut split")
    rewrite(directory, "packed.json", lambda r: r.update(splits=r["splits"][::-1], binding_id=packed_dir.uuid_of(b"\x01" * 32)))
    refused("are not those of binding.json")
    rewrite(directory, "binding.json", lambda r: r.update(seq_len=32))
    refused("is not the id of its dataset, tokenizer, seq_len and masking policy")
    os.remove(os.path.join(directory, "binding.json"))
    refused("binding.json")
