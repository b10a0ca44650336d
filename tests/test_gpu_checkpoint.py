"""Checkpoints of a device run: a run resumed from its checkpoint equals the run that never
stopped (crates/modelspec-runtime/tests/checkpoint.rs:152-189 of the reference), for SGD and, with
the moments in the file, for AdamW with dropout; and the checkpoints that do not match the compiled
file are refused with E-CKPT-003, the first difference named (train/checkpoint.rs:519-609)."""
import ctypes as C
import json
import struct

import numpy as np
import pytest

import modelspec_b200 as M
import oracle_lib
from modelspec_b200 import models, synthetic

pytestmark = pytest.mark.gpu


def blake3(data):
    out = (C.c_uint8 * 32)()
    oracle_lib.lib().orc_blake3(bytes(data), len(data), out)
    return bytes(out)


def test_the_schema_hash_covers_paths_dtypes_and_shapes_in_declaration_order(device):
    # artifact.rs:170-194 of the reference, restated.
    gpu = M.Training(device, models.two_layer_relu(steps=2), 0)
    try:
        data = b"modelspec-schema/1\n"
        for path, shape in (("TwoLayer.w1", (4, 8)), ("TwoLayer.w2", (8, 1))):
            data += struct.pack("<Q", len(path)) + path.encode() + b"f32" + struct.pack("<Q", len(shape))
            for n in shape:
                data += b"\x00" + struct.pack("<Q", n)
        assert gpu.schema_hash() == blake3(data).hex()
    finally:
        gpu.destroy()


def run_linear(device, steps, total, start_from=None):
    """`steps` steps of linear regression ending at `total`, from a checkpoint file or from step 0;
    returns (losses by step, encoded checkpoint at the end)."""
    source = models.linear_regression(steps=total)
    gpu = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    try:
        gpu.synthetic()
        start = 0
        if start_from is not None:
            loaded = M.Checkpoint.read(start_from)
            start = gpu.resume(loaded)
            loaded.destroy()
        losses = {}
        for k in range(start, start + steps):
            gpu.step(k, total)
            losses[k] = gpu.loss()
        ckpt = gpu.checkpoint(start + steps)
        data = ckpt.encode()
        return losses, data, ckpt
    finally:
        gpu.destroy()


def test_a_resumed_sgd_run_equals_one_that_never_stopped(device, tmp_path):
    whole_losses, whole, c = run_linear(device, 6, 6)
    c.destroy()
    _, _, half = run_linear(device, 2, 6)
    path = str(tmp_path / "half.msckpt")
    half.write(path)
    half.destroy()
    rest_losses, rest, c = run_linear(device, 4, 6, start_from=path)
    c.destroy()
    assert sorted(rest_losses) == [2, 3, 4, 5]
    assert all(rest_losses[k].tobytes() == whole_losses[k].tobytes() for k in rest_losses)
    assert rest == whole, "the same bytes, checkpoint id included"
    manifest = json.loads(whole[56:56 + struct.unpack_from("<Q", whole, 16)[0]])
    assert manifest["step"] == 6 and manifest["optimizer"] == {"kind": "Sgd", "learning_rate": float(np.float32(0.1))}
    assert [r["path"] for r in manifest["parameters"]] == ["LinearReg.w"] and manifest["optimizer_slots"] == []


BERT = dict(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=304, seq=16, batch=8, warmup_steps=2)


def run_bert(device, first, count, total, flags, start_from=None):
    gpu = M.Training(device, models.bert(steps=total, **BERT), 64, flags)
    try:
        if start_from is not None:
            assert gpu.resume(start_from) == first
        losses = []
        for k in range(first, first + count):
            for name, value in synthetic.mlm_batch(k, vocab=304, seq=16, batch=8).items():
                gpu.set_input(name, value)
            gpu.step(k, total)
            losses.append(gpu.loss())
        return np.array(losses, dtype=np.float32), gpu.checkpoint(first + count)
    finally:
        gpu.destroy()


@pytest.mark.parametrize("flags", [M.PLAN_DEFAULT, M.PLAN_BF16])
def test_a_resumed_adamw_run_with_dropout_equals_one_that_never_stopped(device, tmp_path, flags):
    whole_losses, whole = run_bert(device, 0, 6, 6, flags)
    _, half = run_bert(device, 0, 2, 6, flags)
    path = str(tmp_path / "half.msckpt")
    half.write(path)
    half.destroy()
    loaded = M.Checkpoint.read(path)
    paths = [p for p, _, _ in loaded.tensors()]
    assert paths == sorted(paths) and len(loaded.tensors(slots=True)) == 2 * len(paths)
    rest_losses, rest = run_bert(device, 2, 4, 6, flags, start_from=loaded)
    try:
        assert rest_losses.tobytes() == whole_losses[2:].tobytes()
        assert rest.encode() == whole.encode()
    finally:
        for c in (loaded, rest, whole):
            c.destroy()


def test_an_adamw_checkpoint_without_moments_resumes_only_from_step_0(device):
    source = models.bert(steps=4, **BERT)
    gpu = M.Training(device, source, 64)
    try:
        full = gpu.checkpoint(0)
        for step in (0, 3):
            bare = M.Checkpoint(step=step, seed=42, schema_hash=gpu.schema_hash())
            bare.set_optimizer(M.OPTIMIZER_ADAMW, float(np.float32(1e-4)), float(np.float32(0.01)), float(np.float32(0.9)), float(np.float32(0.999)),
                               float(np.float32(1e-6)), 2)
            for path, _, value in full.tensors():
                bare.add(path, value)
            if step == 0:
                assert gpu.resume(bare) == 0
            else:
                with pytest.raises(M.MsxError) as e:
                    gpu.resume(bare)
                assert "holds no first and second moments" in str(e.value)
            bare.destroy()
        full.destroy()
    finally:
        gpu.destroy()


def test_a_checkpoint_that_does_not_match_the_compiled_file_is_refused(device):
    linear = M.Training(device, models.linear_regression(steps=3), 0)
    two = M.Training(device, models.two_layer_relu(steps=3), 0)
    try:
        def refused(run, ckpt, text):
            with pytest.raises(M.MsxError) as e:
                run.resume(ckpt)
            assert e.value.status == M.BAD_INPUT and "E-CKPT-003" in str(e.value) and text in str(e.value), str(e.value)

        of_two, of_linear = two.checkpoint(1), linear.checkpoint(1)
        refused(linear, of_two, "a parameter path differs (checkpoint `TwoLayer.w1`, compiled file `LinearReg.w`)")
        refused(two, of_linear, "a parameter path differs (checkpoint `LinearReg.w`, compiled file `TwoLayer.w1`)")
        w = of_linear.tensors()[0][2]
        for shape, schema, lr, text in (((2, 2), linear.schema_hash(), 0.1, "parameter `LinearReg.w` has another shape (checkpoint [2, 2]"),
                                        ((4, 1), "cd" * 32, 0.1, "the schema hash differs"),
                                        ((4, 1), linear.schema_hash(), 0.2, "the optimizer differs")):
            other = M.Checkpoint(step=1, seed=42, schema_hash=schema)
            other.set_optimizer(M.OPTIMIZER_SGD, float(np.float32(lr)))
            other.add("LinearReg.w", w.reshape(shape))
            refused(linear, other, text)
            other.destroy()
        extra = M.Checkpoint(step=1, seed=42, schema_hash=linear.schema_hash())
        extra.set_optimizer(M.OPTIMIZER_SGD, float(np.float32(0.1)))
        extra.add("LinearReg.w", w)
        extra.add("LinearReg.z", w)
        refused(linear, extra, "a parameter path differs (checkpoint `LinearReg.z`, compiled file none)")
        extra.destroy()
        assert linear.resume(of_linear) == 1
        of_two.destroy()
        of_linear.destroy()
    finally:
        linear.destroy()
        two.destroy()
