"""Writes a packed masked-language-model directory in the layout the reference's `pack` writes
(crates/modelspec-runtime/src/dataset/mlm.rs:25-120, :161-184): binding.json, packed.json,
train.tokens and heldout.tokens. Test infrastructure: the digests come from the oracle's BLAKE3."""
import ctypes as C
import json
import os
import struct

import numpy as np

import oracle_lib

BERT_POLICY = {"selection_rate": 0.15, "mask_fraction": 0.8, "random_fraction": 0.1, "keep_fraction": 0.1}
DATASET_ID = "00112233-4455-8677-8899-aabbccddeeff"
TOKENIZER_ID = "ffeeddcc-bbaa-8988-b766-554433221100"


def blake3(data):
    out = (C.c_uint8 * 32)()
    oracle_lib.lib().orc_blake3(bytes(data), len(data), out)
    return bytes(out)


def uuid_of(digest):
    b = bytearray(digest[:16])
    b[6] = (b[6] & 0x0F) | 0x80
    b[8] = (b[8] & 0x3F) | 0x80
    h = b.hex()
    return "-".join((h[0:8], h[8:12], h[12:16], h[16:20], h[20:32]))


def binding_id(dataset_id, tokenizer_id, seq_len, policy):
    data = bytes.fromhex(dataset_id.replace("-", "")) + bytes.fromhex(tokenizer_id.replace("-", "")) + struct.pack("<Q", seq_len)
    for key in ("selection_rate", "mask_fraction", "random_fraction", "keep_fraction"):
        data += struct.pack("<d", policy[key])
    return uuid_of(blake3(data))


def write(directory, train, heldout, seq_len, vocabulary, policy=BERT_POLICY):
    """`train` and `heldout`: int32 arrays of whole sequences. Returns the binding id."""
    os.makedirs(directory, exist_ok=True)
    bid = binding_id(DATASET_ID, TOKENIZER_ID, seq_len, policy)
    binding = {"binding_id": bid, "dataset_id": DATASET_ID, "tokenizer_id": TOKENIZER_ID, "seq_len": seq_len, "masking_policy": policy,
               "state": "Recorded"}
    splits, digests = [], b""
    for role, name, ids in (("Train", "train.tokens", train), ("HeldOut", "heldout.tokens", heldout)):
        data = np.ascontiguousarray(ids, dtype="<i4").tobytes()
        with open(os.path.join(directory, name), "wb") as f:
            f.write(data)
        digest = blake3(data)
        digests += digest
        splits.append({"role": role, "sequence_count": len(ids) // seq_len, "content_hash": digest.hex()})
    record = {"packed_id": uuid_of(blake3(digests)), "binding_id": bid, "seq_len": seq_len, "vocabulary_size": vocabulary, "splits": splits,
              "heldout_unigram_baseline_nats": 3.5, "state": "Recorded"}
    with open(os.path.join(directory, "binding.json"), "w") as f:
        json.dump(binding, f)
    with open(os.path.join(directory, "packed.json"), "w") as f:
        json.dump(record, f)
    return bid
