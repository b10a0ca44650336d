"""The `.msckpt` writer and reader: the byte layout the reference's tests state
(crates/modelspec-runtime/tests/checkpoint.rs:47-123), a file the reference's own Python reader
accepted (tests/golden/two_tensors.msckpt, made and checked by
tests/golden/make_checkpoint_fixture.py), round trips, and the refusals of the reference's reader
with their codes (train/checkpoint.rs:640-921). Host code: no GPU needed."""
import ctypes as C
import json
import os
import struct

import numpy as np
import pytest

import modelspec_b200 as M
import oracle_lib

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "two_tensors.msckpt")


def blake3(data):
    out = (C.c_uint8 * 32)()
    oracle_lib.lib().orc_blake3(bytes(data), len(data), out)
    return bytes(out)


def tensors():
    rng = np.random.default_rng(11)
    return {"w1": rng.standard_normal((4, 8)).astype(np.float32), "w2": rng.standard_normal((8, 1)).astype(np.float32)}


def build(step=3, adamw=False, order=("w1", "w2")):
    ckpt = M.Checkpoint(step=step, seed=42, schema_hash="ab" * 32)
    if adamw:
        ckpt.set_optimizer(M.OPTIMIZER_ADAMW, float(np.float32(1e-4)), float(np.float32(0.01)), float(np.float32(0.9)), float(np.float32(0.999)),
                           float(np.float32(1e-6)), 10)
    else:
        ckpt.set_optimizer(M.OPTIMIZER_SGD, float(np.float32(0.1)))
    values = tensors()
    for name in order:
        ckpt.add("TwoLayer." + name, values[name])
        if adamw:
            ckpt.add("TwoLayer." + name, values[name] * 0.5, slot="v")
            ckpt.add("TwoLayer." + name, values[name] * 0.25, slot="m")
    return ckpt


def manifest_of(data):
    size = struct.unpack_from("<Q", data, 16)[0]
    return json.loads(data[56:56 + size]), size


def test_the_writer_gives_the_file_the_reference_reader_accepted():
    ckpt = build()
    try:
        assert ckpt.encode() == open(GOLDEN, "rb").read()
    finally:
        ckpt.destroy()


def test_the_header_has_the_documented_byte_layout():
    ckpt = build()
    data = ckpt.encode()
    ckpt.destroy()
    assert data[0:4] == b"MSCK" and struct.unpack_from("<I", data, 4)[0] == 1 and data[8:12] == bytes([4, 3, 2, 1])
    assert struct.unpack_from("<I", data, 12)[0] == 0
    manifest, size = manifest_of(data)
    signed = bytearray(data[:56 + size])
    signed[24:56] = bytes(32)
    assert data[24:56] == blake3(signed)
    assert manifest["file_size"] == len(data) and manifest["alignment"] == 64 and manifest["step"] == 3
    assert manifest["optimizer_slots"] == [] and manifest["optimizer"] == {"kind": "Sgd", "learning_rate": float(np.float32(0.1))}
    assert manifest["rng"] == {"algorithm": "Philox4x32x10", "seed": 42, "counter": 0}
    assert list(manifest) == ["checkpoint_id", "file_size", "alignment", "schema_hash", "step", "payload_hash", "optimizer", "optimizer_slots",
                              "rng", "parameters"]
    # The id is a version-8 UUID of the manifest with the nil UUID in its place.
    text = data[56:56 + size].decode()
    unnamed = text.replace(manifest["checkpoint_id"], "00000000-0000-0000-0000-000000000000")
    digest = bytearray(blake3(b"modelspec-checkpoint-id/1\n" + unnamed.encode())[:16])
    digest[6] = (digest[6] & 0x0F) | 0x80
    digest[8] = (digest[8] & 0x3F) | 0x80
    assert manifest["checkpoint_id"].replace("-", "") == digest.hex()


def test_the_payload_is_64_byte_aligned_and_hashed():
    ckpt = build(order=("w2", "w1"))  # added out of order: written in path order
    data = ckpt.encode()
    ckpt.destroy()
    manifest, size = manifest_of(data)
    start = -(-(56 + size) // 64) * 64
    records = manifest["parameters"]
    assert [r["path"] for r in records] == ["TwoLayer.w1", "TwoLayer.w2"] and records[0]["offset"] == start
    end = 0
    for r in records:
        assert r["offset"] % 64 == 0 and r["offset"] >= end and not any(data[end:r["offset"]][56 + size - end if end == 0 else 0:])
        end = r["offset"] + r["length"]
    assert records[0]["length"] == 4 * 8 * 4 and records[0]["shape"] == [4, 8] and records[0]["dtype"] == "F32" and end == len(data)
    assert manifest["payload_hash"] == blake3(data[start:]).hex()
    assert data[records[0]["offset"]:records[0]["offset"] + 4] == tensors()["w1"].tobytes()[:4]


def test_a_written_checkpoint_reads_back_to_the_same_state(tmp_path):
    for adamw in (False, True):
        ckpt = build(step=5, adamw=adamw)
        path = str(tmp_path / "round_trip.msckpt")
        ckpt.write(path)
        assert not os.path.exists(path + ".tmp")
        read = M.Checkpoint.read(path)
        try:
            assert (read.step, read.seed, read.schema_hash, read.id) == (5, 42, "ab" * 32, ckpt.id)
            assert read.optimizer_json() == ckpt.optimizer_json()
            values = tensors()
            assert [(p, s) for p, s, _ in read.tensors()] == [("TwoLayer.w1", ""), ("TwoLayer.w2", "")]
            for path_, _, value in read.tensors():
                assert value.tobytes() == values[path_.split(".")[1]].tobytes() and value.shape == values[path_.split(".")[1]].shape
            slots = read.tensors(slots=True)
            assert [(p, s) for p, s, _ in slots] == ([("TwoLayer.w1", "m"), ("TwoLayer.w1", "v"), ("TwoLayer.w2", "m"), ("TwoLayer.w2", "v")] if adamw else [])
            for path_, slot, value in slots:
                assert value.tobytes() == (values[path_.split(".")[1]] * (0.25 if slot == "m" else 0.5)).tobytes()
            assert read.encode() == ckpt.encode()
        finally:
            read.destroy()
            ckpt.destroy()


def test_the_same_state_encodes_to_the_same_bytes():
    a, b, other = build(4), build(4), build(5)
    try:
        assert a.encode() == b.encode() and a.encode() != other.encode() and a.id != other.id
        adamw = build(4, adamw=True)
        assert adamw.id != a.id, "two checkpoints that differ only in their optimizer have different ids"
        adamw.destroy()
    finally:
        for c in (a, b, other):
            c.destroy()


def test_numbers_are_written_as_serde_json_writes_them():
    cases = [(float(np.float32(0.1)), "0.10000000149011612"), (float(np.float32(1e-4)), "0.00009999999747378752"), (1e-5, "0.00001"),
             (1e-6, "1e-6"), (float(np.float32(1e-6)), "9.999999974752427e-7"), (0.001, "0.001"), (100.0, "100.0"), (1e16, "1e16"),
             (1234000000000000.0, "1234000000000000.0"), (1.5e300, "1.5e300"), (0.3, "0.3"), (2.718281828459045, "2.718281828459045"),
             (0.0, "0.0"), (12.5, "12.5")]
    for value, text in cases:
        ckpt = M.Checkpoint(step=0, seed=1, schema_hash="")
        ckpt.set_optimizer(M.OPTIMIZER_SGD, value)
        got = ckpt.optimizer_json()
        ckpt.destroy()
        assert got == '{"kind":"Sgd","learning_rate":%s}' % text and json.loads(got)["learning_rate"] == value
    adamw = build(adamw=True)
    assert adamw.optimizer_json() == ('{"kind":"AdamW","learning_rate":0.00009999999747378752,"weight_decay":0.009999999776482582,"beta1":0.8999999761581421,'
                                      '"beta2":0.9990000128746033,"epsilon":9.999999974752427e-7,"schedule":{"warmup_steps":10}}')
    adamw.destroy()


def resealed(data, edit):
    """The file with its manifest edited and its header checksum made right again."""
    manifest, size = manifest_of(data)
    edit(manifest)
    text = json.dumps(manifest, separators=(",", ":")).encode()
    head = bytearray(data[:16] + struct.pack("<Q", len(text)) + bytes(32) + text)
    head[24:56] = blake3(head)
    start, old_start = -(-len(head) // 64) * 64, -(-(56 + size) // 64) * 64
    return bytes(head) + bytes(start - len(head)) + data[old_start:]


def refusals():
    good = open(GOLDEN, "rb").read()
    manifest, size = manifest_of(good)
    first = manifest["parameters"][0]["offset"]
    flip = lambda at: good[:at] + bytes([good[at] ^ 1]) + good[at + 1:]
    yield "E-CKPT-002", "fewer than the 56-byte header", good[:40]
    yield "E-CKPT-001", "the magic is not MSCK", b"MSCX" + good[4:]
    yield "E-CKPT-001", "format version 2 is not 1", good[:4] + struct.pack("<I", 2) + good[8:]
    yield "E-CKPT-001", "the endian marker is big-endian", good[:8] + bytes([1, 2, 3, 4]) + good[12:]
    yield "E-CKPT-001", "the reserved header field is not zero", good[:12] + struct.pack("<I", 7) + good[16:]
    yield "E-CKPT-002", "does not fit the 800-byte file after its header", good[:16] + struct.pack("<Q", 10 ** 6) + good[24:]
    yield "E-CKPT-001", "the checksum differs from the header and manifest", flip(60)
    yield "E-CKPT-004", "the payload hash differs from the payload", flip(first + 5)
    yield "E-CKPT-002", "lies between tensors and is not zero", flip(56 + size + 1)
    yield "E-CKPT-002", "is not the file's 804 bytes", good + bytes(4)
    yield "E-CKPT-001", "is not a UUID", resealed(good, lambda m: m.update(checkpoint_id="not-a-uuid"))
    yield "E-CKPT-001", "the optimizer's fields do not fit its kind", resealed(good, lambda m: m["optimizer"].update(beta1=0.9))
    yield "E-CKPT-001", "an SGD checkpoint has optimizer slots", resealed(good, lambda m: m.update(optimizer_slots=[dict(m["parameters"][0], slot="m")]))
    yield "E-CKPT-001", "the manifest has no parameter", resealed(good, lambda m: m.update(parameters=[]))
    yield "E-CKPT-001", "is recorded twice", resealed(good, lambda m: m.update(parameters=[m["parameters"][0]] * 2))
    yield "E-CKPT-001", "has a slot name", resealed(good, lambda m: m["parameters"][0].update(slot="m"))
    yield "E-CKPT-001", "unknown field `extra`", resealed(good, lambda m: m.update(extra=1))
    yield "E-CKPT-001", "more than 8 dimensions", resealed(good, lambda m: m["parameters"][0].update(shape=[1] * 9))
    yield "E-CKPT-001", "has a zero dimension", resealed(good, lambda m: m["parameters"][0].update(shape=[0, 8]))
    yield "E-CKPT-002", "the alignment 32 is not 64", resealed(good, lambda m: m.update(alignment=32))
    yield "E-CKPT-002", "is not a multiple of 64", resealed(good, lambda m: m["parameters"][0].update(offset=m["parameters"][0]["offset"] + 4))
    yield "E-CKPT-002", "lies inside the header or manifest", resealed(good, lambda m: m["parameters"][0].update(offset=64))
    yield "E-CKPT-002", "end past the 800-byte file", resealed(good, lambda m: m["parameters"][1].update(offset=1 << 40))
    yield "E-CKPT-002", "is not the shape [4, 4] times 4 bytes", resealed(good, lambda m: m["parameters"][0].update(shape=[4, 4]))
    yield "E-CKPT-002", "overlap", resealed(good, lambda m: m["parameters"][1].update(offset=m["parameters"][0]["offset"] + 64))


@pytest.mark.parametrize("code,text,data", list(refusals()), ids=[t for _, t, _ in refusals()])
def test_what_the_reference_reader_refuses_is_refused_with_its_code(tmp_path, code, text, data):
    path = str(tmp_path / "bad.msckpt")
    open(path, "wb").write(data)
    with pytest.raises(M.MsxError) as e:
        M.Checkpoint.read(path)
    assert e.value.status == M.BAD_INPUT and code in str(e.value) and text in str(e.value), str(e.value)


def test_a_resealed_file_that_changes_nothing_reads(tmp_path):
    path = str(tmp_path / "same.msckpt")
    open(path, "wb").write(resealed(open(GOLDEN, "rb").read(), lambda m: None))
    M.Checkpoint.read(path).destroy()
    with pytest.raises(M.MsxError) as e:
        M.Checkpoint.read(str(tmp_path / "absent.msckpt"))
    assert "E-CKPT-001" in str(e.value)
