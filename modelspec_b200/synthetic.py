"""Seeded synthetic batches that stand in for the datasets the reference measures on (MNIST,
packed WikiText-103), which are not available offline. Every draw is a Philox4x32-10 block
addressed as the reference addresses its draws (key = seed, counter = [index, stream, id lo, id
hi]); generators the reference does not have use stream tags from 16 up. The masking rule is the
reference's `mlm_batch` (crates/modelspec-runtime/src/dataset/mlm.rs:766-786) with the mask id and
the count of special ids as parameters.
"""
import numpy as np

M0, M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
W0, W1 = np.uint64(0x9E3779B9), np.uint64(0xBB67AE85)
MASK32 = np.uint64(0xFFFFFFFF)

STREAM_MASKING = 3
STREAM_TOKENS = 16
STREAM_LABELS = 17
STREAM_FEATURES = 18


def philox(index, stream, draw_id, seed):
    """Blocks [n, 4] (uint32) of elements `index` (array) of draw `draw_id` on `stream`."""
    c0 = np.asarray(index, dtype=np.uint64) & MASK32
    n = c0.shape[0]
    c1 = np.full(n, stream, dtype=np.uint64)
    c2 = np.full(n, draw_id & 0xFFFFFFFF, dtype=np.uint64)
    c3 = np.full(n, (draw_id >> 32) & 0xFFFFFFFF, dtype=np.uint64)
    k0 = np.uint64(seed & 0xFFFFFFFF)
    k1 = np.uint64((seed >> 32) & 0xFFFFFFFF)
    for r in range(10):
        if r > 0:
            k0 = (k0 + W0) & MASK32
            k1 = (k1 + W1) & MASK32
        p0 = M0 * c0
        p1 = M1 * c2
        n0 = ((p1 >> np.uint64(32)) ^ c1 ^ k0) & MASK32
        n1 = p1 & MASK32
        n2 = ((p0 >> np.uint64(32)) ^ c3 ^ k1) & MASK32
        n3 = p0 & MASK32
        c0, c1, c2, c3 = n0, n1, n2, n3
    return np.stack([c0, c1, c2, c3], axis=1).astype(np.uint32)


def uniform(words):
    return (words.astype(np.float64) + 0.5) / 4294967296.0


def zipf_cdf(n, s=1.1):
    w = 1.0 / np.arange(1, n + 1, dtype=np.float64) ** s
    c = np.cumsum(w)
    return c / c[-1]


def mlm_batch(step, seed=42, batch=32, seq=128, vocab=30522, mask_id=103, specials=5,
              selection_rate=0.15, mask_fraction=0.8, random_fraction=0.1, zipf_s=1.1,
              row_offset=0):
    """One MLM batch: Zipf(s) token ids over the non-special vocabulary, positions 0..seq-1 per
    sequence, an all-ones key mask, and the reference's masking of the rows drawn for `step`.
    `row_offset` shifts the row index of the draws (a shard of a larger global batch)."""
    rows = batch * seq
    index = np.arange(rows, dtype=np.uint64) + np.uint64(row_offset)
    tok = philox(index, STREAM_TOKENS, step, seed)
    cdf = zipf_cdf(vocab - specials, zipf_s)
    rank = np.searchsorted(cdf, uniform(tok[:, 0]), side="left")
    labels = (specials + np.minimum(rank, vocab - specials - 1)).astype(np.int32)
    blk = philox(index, STREAM_MASKING, step, seed)
    u0, u1 = uniform(blk[:, 0]), uniform(blk[:, 1])
    selected = (labels >= specials) & (u0 < selection_rate)
    random_id = (specials + ((blk[:, 2].astype(np.uint64) * np.uint64(vocab - specials)) >> np.uint64(32))).astype(np.int32)
    ids = labels.copy()
    to_mask = selected & (u1 < mask_fraction)
    to_random = selected & ~to_mask & (u1 < mask_fraction + random_fraction)
    ids[to_mask] = mask_id
    ids[to_random] = random_id[to_random]
    positions = np.tile(np.arange(seq, dtype=np.int32), batch)
    return {
        "ids": ids,
        "positions": positions,
        "key_mask": np.ones(rows, dtype=np.float32),
        "labels": labels,
        "weights": selected.astype(np.float32),
    }


def classifier_batch(seed=42, batch=64, inputs=784, classes=10):
    """Features uniform in [0, 1), labels uniform in 0..classes-1, unit weights."""
    x = uniform(philox(np.arange(batch * inputs, dtype=np.uint64), STREAM_FEATURES, 0, seed)[:, 0]).astype(np.float32)
    x = np.minimum(x, np.float32(1.0) - np.float32(2.0 ** -24))
    u = uniform(philox(np.arange(batch, dtype=np.uint64), STREAM_LABELS, 0, seed)[:, 0])
    labels = np.minimum((u * classes).astype(np.int32), classes - 1)
    return {"x": x, "labels": labels, "weights": np.ones(batch, dtype=np.float32)}


def normal_batch(name_seed, count, seed=42, stream=STREAM_FEATURES):
    """`count` standard normal values by Box-Muller over words 0 and 1."""
    blk = philox(np.arange(count, dtype=np.uint64), stream, name_seed, seed)
    return (np.sqrt(-2.0 * np.log(uniform(blk[:, 0]))) * np.cos(2.0 * np.pi * uniform(blk[:, 1]))).astype(np.float32)
