"""The CPU oracle against everything the reference records for this path: known answers of its
RNG, the training logs of two recorded CPU runs bit for bit, the first loss of its transformer
block, and hand-computed exact cases of single ops. No GPU."""
import ctypes as C
import json
import os

import numpy as np
import pytest

import oracle_lib
from modelspec_b200 import models
from helpers import ProgramText

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_philox_matches_the_random123_known_answers():
    """The three vectors of crates/modelspec-runtime/src/train/init.rs:425-441."""
    vectors = [
        ([0, 0, 0, 0], [0, 0], [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]),
        ([0xffffffff] * 4, [0xffffffff] * 2, [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]),
        ([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0],
         [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]),
    ]
    for counter, key, expected in vectors:
        c = np.array(counter, dtype=np.uint32); k = np.array(key, dtype=np.uint32); out = np.zeros(4, dtype=np.uint32)
        oracle_lib.lib().orc_philox(c.ctypes.data, k.ctypes.data, out.ctypes.data)
        assert out.tolist() == expected
    from modelspec_b200 import synthetic
    assert synthetic.philox(np.array([0x243f6a88]), 0x85a308d3, 0x0370734413198a2e, 0x299f31d0a4093822)[0].tolist() == vectors[2][2]


def test_blake3_matches_the_reference_known_answer_and_the_package_digests():
    L = oracle_lib.lib()
    assert L.orc_canonical_id(b"") == 0xa6a1f9f5b94913af  # init.rs:453-456
    cases = json.load(open(os.path.join(GOLDEN, "blake3.json")))
    for key, digest in cases.items():
        data = b"LinearReg.w" if key.startswith("path:") else bytes((i * 7 + 3) % 251 for i in range(int(key)))
        out = C.create_string_buffer(32)
        L.orc_blake3(data, len(data), out)
        assert out.raw.hex() == digest, key
    assert L.orc_canonical_id(b"LinearReg.w") != L.orc_canonical_id(b"LinearReg.b")


def test_a_dropout_draw_is_addressed_by_site_step_and_index():
    L = oracle_lib.lib()
    a, b = L.orc_dropout_id(b"M.forward.dropout#0", 5), L.orc_dropout_id(b"M.forward.dropout#0", 6)
    assert a != b
    import struct
    out = C.create_string_buffer(32)
    data = b"M.forward.dropout#0" + struct.pack("<Q", 5)
    L.orc_blake3(data, len(data), out)
    assert a == struct.unpack("<Q", out.raw[:8])[0]
    kept = sum(L.orc_dropout_keeps(42, a, i, C.c_float(0.3)) for i in range(20000))
    assert abs(kept / 20000 - 0.7) < 0.02
    assert all(L.orc_dropout_keeps(42, a, i, C.c_float(0.0)) for i in range(100))


def run_synthetic(source, steps):
    t = oracle_lib.Trainer(source)
    t.synthetic()
    losses = [t.step(k, steps) for k in range(steps)]
    losses.append(t.final_loss())
    return t, np.array(losses, dtype=np.float32)


def test_linear_regression_log_is_reproduced_bit_for_bit():
    """Initial parameters, 501 losses and final parameters of the reference's CPU run
    (tests/golden/linear_regression.train.stdout, tests/fixtures/linear_regression.run.jsonl):
    pins BLAKE3 ids, Philox, xavier_uniform, the teacher batch, matmul, mse and SGD end to end."""
    golden = json.load(open(os.path.join(GOLDEN, "linear_regression.losses.json")))
    t = oracle_lib.Trainer(models.linear_regression())
    assert t.read("param", 0).tolist() == np.array(golden["initial_param"], dtype=np.float32).tolist()
    t, losses = run_synthetic(models.linear_regression(), 500)
    assert losses.tolist() == np.array(golden["losses"], dtype=np.float32).tolist()
    assert t.read("param", 0).tolist() == np.array(golden["final_param"], dtype=np.float32).tolist()


def test_two_layer_relu_losses_are_reproduced_bit_for_bit():
    golden = json.load(open(os.path.join(GOLDEN, "two_layer_relu.losses.json")))
    _, losses = run_synthetic(models.two_layer_relu(), 200)
    assert losses.tolist() == np.array(golden["losses"], dtype=np.float32).tolist()


def test_transformer_block_first_loss_is_the_recorded_one():
    """`step 0 loss 0.74829835` of `train examples/transformer_block.mspec --backend cpu --steps 0`
    (benchmarks/raw/2026-10-27-transformer-block/loss-cpu.txt): pins attention, layer_norm, gelu,
    add_rows and the f64 mse on 1024 x 128 activations."""
    t = oracle_lib.Trainer(models.transformer_block())
    t.synthetic()
    assert t.final_loss() == np.float32(0.74829835)


def evaluate(text, inputs, outputs, wide=False, seed=None):
    s = oracle_lib.Session(text, wide=wide)
    for name, value in inputs.items():
        s.set_input(name, value)
    if seed is not None:
        s.set_seed(seed)
    s.run()
    return [s.value(v, n) for v, n in outputs]


@pytest.mark.parametrize("wide", [False, True])
def test_exact_cases_of_single_ops(wide):
    """Exactly representable expectations, the same in f32 and f64, in the style of the
    reference's crates/modelspec-runtime/tests/cpu_golden.rs."""
    p = ProgramText()
    a = p.input("a", "f32", [2, 3]); b = p.input("b", "f32", [3, 2]); bias = p.input("bias", "f32", [2])
    ids = p.input("ids", "i32", [3])
    mm = p.op("MatMul", [2, 2], [a, b])
    ar = p.op("AddRows", [2, 2], [mm, bias])
    sr = p.op("SumRows", [2], [ar])
    tr = p.op("Transpose", [3, 2], [a])
    relu = p.op("Relu", [2, 3], [a])
    total = p.op("ReduceSum", [], [a]); mean = p.op("ReduceMean", [], [a])
    emb = p.op("Embedding", [3, 2], [b, ids])
    eg = p.op("EmbeddingGrad", [3, 2], [ids, emb], attr="[3]")
    outs = [(mm, 4), (ar, 4), (sr, 2), (tr, 6), (relu, 6), (total, 1), (mean, 1), (emb, 6), (eg, 6)]
    for v, _ in outs:
        p.output(v)
    av = np.array([[1, -2, 3], [0.5, 0, -4]], dtype=np.float32)
    bv = np.array([[2, 0], [1, -1], [0.25, 4]], dtype=np.float32)
    got = evaluate(p.text(), {"a": av, "b": bv, "bias": np.array([10, -10], np.float32), "ids": np.array([2, 0, 2], np.int32)}, outs, wide)
    assert got[0].tolist() == [0.75, 14, 0, -16]
    assert got[1].tolist() == [10.75, 4, 10, -26]
    assert got[2].tolist() == [20.75, -22]
    assert got[3].tolist() == [1, 0.5, -2, 0, 3, -4]
    assert got[4].tolist() == [1, 0, 3, 0.5, 0, 0]
    assert got[5].tolist() == [-1.5] and got[6].tolist() == [-0.25]
    assert got[7].tolist() == [0.25, 4, 2, 0, 0.25, 4]
    assert got[8].tolist() == [2, 0, 0, 0, 0.5, 8]


def test_softmax_layer_norm_and_cross_entropy_on_symmetric_rows():
    p = ProgramText()
    x = p.input("x", "f32", [2, 4]); g = p.input("gamma", "f32", [4]); b = p.input("beta", "f32", [4])
    labels = p.input("labels", "i32", [2]); w = p.input("w", "f32", [2])
    sm = p.op("Softmax", [2, 4], [x]); ln = p.op("LayerNorm", [2, 4], [x, g, b]); ce = p.op("CrossEntropy", [], [x, labels, w])
    for v in (sm, ln, ce):
        p.output(v)
    xv = np.array([[3, 3, 3, 3], [-1, 1, -1, 1]], dtype=np.float32)
    got = evaluate(p.text(), {"x": xv, "gamma": np.ones(4, np.float32) * 2, "beta": np.ones(4, np.float32),
                              "labels": np.array([1, 3], np.int32), "w": np.array([1, 0], np.float32)},
                   [(sm, 8), (ln, 8), (ce, 1)])
    assert got[0][:4].tolist() == [0.25] * 4
    assert got[1][:4].tolist() == [1.0] * 4          # a constant row normalises to 0, times gamma plus beta
    assert np.allclose(got[1][4:], [-1, 3, -1, 3], atol=1e-5)
    assert got[2][0] == np.float32(np.log(np.float32(4.0)))  # only the first row has weight


def test_dropout_keeps_scale_and_zero_in_the_oracle():
    p = ProgramText()
    x = p.input("x", "f32", [1000]); token = p.input("S.forward.dropout#0", "i32", [2])
    y = p.op("Dropout", [1000], [x, token], attr="[p = 0.25, site = S.forward.dropout#0]")
    p.output(y)
    [out] = evaluate(p.text(), {"x": np.ones(1000, np.float32), "S.forward.dropout#0": np.array([7, 9], np.int32)}, [(y, 1000)], seed=42)
    scale = np.float32(1.0) / (np.float32(1.0) - np.float32(0.25))
    assert set(np.unique(out.astype(np.float32)).tolist()) == {0.0, float(scale)}
    L = oracle_lib.lib()
    draw = 7 | (9 << 32)
    for i in range(50):
        assert (out[i] != 0) == bool(L.orc_dropout_keeps(42, draw, i, C.c_float(0.25)))


def test_gradients_agree_with_f64_central_differences():
    """Autodiff plus the gradient ops against central differences of the f64 interpreter, the
    reference's gate for every op (crates/modelspec-runtime/tests/common/finite_difference.rs),
    on the hidden-32 BERT twin's step with dropout off."""
    import modelspec_b200 as M
    source = models.bert(name="T", layers=1, hidden=8, heads=2, ffn=16, vocab=11, seq=4, batch=2, dropout=0.0,
                         lr=1e-3, warmup_steps=1, steps=4)
    step_ir = M.compile_mspec(source, "step")
    forward_ir = M.compile_mspec(source, "forward")
    r = np.random.default_rng(0)
    rows = 8
    feed = {"ids": r.integers(0, 11, rows).astype(np.int32), "positions": np.tile(np.arange(4, dtype=np.int32), 2),
            "key_mask": np.array([1, 1, 0, 1, 1, 1, 1, 1], np.float32), "labels": r.integers(0, 11, rows).astype(np.int32),
            "weights": np.array([1, 0, 1, 1, 0, 1, 1, 1], np.float32)}
    param_lines = [l for l in step_ir.splitlines() if l.startswith("param ")]
    shapes = [[int(d) for d in l.split("[")[1].split("]")[0].split(",")] for l in param_lines]
    values = [r.standard_normal(int(np.prod(s))).astype(np.float32) * 0.5 for s in shapes]
    grads = {}
    for line in step_ir.splitlines():
        if line.startswith("output ") and " gradient @" in line:
            grads[line.split("@")[1]] = int(line.split()[1][1:])
    names = [l.split("@")[1].split(":")[0] for l in param_lines]
    s = oracle_lib.Session(step_ir, wide=True)
    for name, v in feed.items():
        s.set_input(name, v)
    for name in names:
        s.set_input("optimizer.m@" + name, np.zeros(int(np.prod(shapes[names.index(name)])), np.float32))
        s.set_input("optimizer.v@" + name, np.zeros(int(np.prod(shapes[names.index(name)])), np.float32))
    for scalar in ("optimizer.lr_t", "optimizer.c1", "optimizer.c2"):
        s.set_input(scalar, np.ones(1, np.float32))
    for i, v in enumerate(values):
        s.set_param(i, v)
    s.run()
    loss_id = int([l for l in forward_ir.splitlines() if l.startswith("output ")][0].split()[1][1:])

    def loss_at(index, element, delta):
        f = oracle_lib.Session(forward_ir, wide=True)
        for name, v in feed.items():
            f.set_input(name, v)
        for i, v in enumerate(values):
            if i == index:
                v = v.copy()
                v[element] += delta
            f.set_param(i, v)
        f.run()
        return f.value(loss_id, 1)[0]

    checked = 0
    for index, name in enumerate(names):
        if name not in grads:
            continue
        analytic = s.value(grads[name], values[index].size)
        for element in {0, values[index].size // 2, values[index].size - 1}:
            h = 1.0 / 1024  # exactly representable, so the perturbed f32 parameter is exact
            numeric = (loss_at(index, element, h) - loss_at(index, element, -h)) / (2 * h)
            assert abs(numeric - analytic[element]) <= 2e-5 + 1e-3 * abs(numeric), (name, element, numeric, analytic[element])
            checked += 1
    assert checked >= 40
