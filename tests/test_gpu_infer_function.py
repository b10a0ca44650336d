"""`infer --data <dir> --function <name> --out <path>` on the device
(crates/modelspec-cli/src/infer.rs:306-470 and train/data.rs:676-815 of the reference): a model
function run over every block of a dense directory with a checkpoint's parameters, its results
written one row per sample; and what is refused before anything is written."""
import os
import subprocess
import sys

import numpy as np
import pytest

import modelspec_b200 as M

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))

SEVERAL = """model Several {
    param w: Tensor<f32, [3, 2]> = xavier_uniform();
    param b: Tensor<f32, [2]> = zeros();

    fn forward(x: Tensor<f32, [4, 3]>) -> Tensor<f32, [4, 2]> {
        return add_rows(matmul(x, w), add(b, unused_head()));
    }

    fn unused_head() -> Tensor<f32, [2]> {
        return b;
    }

    fn scores(x: Tensor<f32, [4, 3]>) -> Tensor<f32, [4, 2]> {
        return gelu(matmul(x, w));
    }

    fn picked(table: Tensor<f32, [6, 3]>, ids: Tensor<i32, [4]>) -> Tensor<f32, [4, 3]> {
        return embedding(table, ids);
    }

    fn turned(x: Tensor<f32, [4, 3]>) -> Tensor<f32, [3, 4]> {
        return transpose(x);
    }
}
train Fit {
    model = Several;
    input x: Tensor<f32, [4, 3]>;
    target y: Tensor<f32, [4, 2]>;
    loss = mse(model.forward(x), y);
    optimizer = adamw(lr = 0.05, weight_decay = 0.01, beta1 = 0.9, beta2 = 0.999, eps = 1e-8, warmup_steps = 1);
    steps = 3;
    seed = 5;
    device = cpu;
}
"""


def gelu(v):
    u = 0.7978845608028654 * (v + 0.044715 * v ** 3)
    return v / (1.0 + np.exp(-2.0 * u))


@pytest.fixture
def trained(device, tmp_path):
    """A directory of 12 samples, and the checkpoint of three adamw steps on it."""
    r = np.random.default_rng(3)
    x = r.standard_normal((12, 3)).astype(np.float32)
    y = r.standard_normal((12, 2)).astype(np.float32)
    data = tmp_path / "data"
    data.mkdir()
    x.tofile(str(data / "x.f32"))
    y.tofile(str(data / "y.f32"))
    run = M.Training(device, SEVERAL, 0, M.PLAN_EXACT_MATMUL)
    try:
        run.bind_dense(str(data))
        run.run()
        done = run.checkpoint(run.steps)
        done.write(str(tmp_path / "fit.msckpt"))
        params = {path: value for path, _, value in done.tensors()}
        done.destroy()
    finally:
        run.destroy()
    return data, tmp_path / "fit.msckpt", x, params


def function_run(device, name, checkpoint=None):
    run = M.Training(device, SEVERAL, 0, M.PLAN_EXACT_MATMUL, function=name)
    if checkpoint is not None:
        loaded = M.Checkpoint.read(str(checkpoint))
        try:
            assert run.load_parameters(loaded) == 3  # an adamw checkpoint into an sgd entry: the optimizer is not compared
        finally:
            loaded.destroy()
    return run


def test_a_function_runs_on_every_block_with_the_checkpoints_parameters(device, trained, tmp_path):
    data, checkpoint, x, params = trained
    out = tmp_path / "scores.f32"
    out.write_bytes(b"old")
    run = function_run(device, "scores", checkpoint)
    try:
        run.refuse_out_reading(data, out, tmp_path / "several.mspec", checkpoint)
        assert run.infer_dense(data, out) == (3, 12)
    finally:
        run.destroy()
    got = np.fromfile(str(out), dtype=np.float32)
    want = gelu(x.astype(np.float64) @ params["Several.w"].astype(np.float64))  # `b` is a parameter this entry does not read
    assert got.shape == (24,)
    np.testing.assert_allclose(got.reshape(12, 2), want, rtol=1e-5, atol=1e-6)
    assert not [f for f in os.listdir(str(tmp_path)) if f.endswith(".tmp")]


def test_a_function_without_parameters_gathers_its_rows_bit_for_bit(device, tmp_path):
    r = np.random.default_rng(4)
    # B is 1: the two arguments share no leading dimension, so a sample is a whole table and its ids.
    table = r.standard_normal((2, 6, 3)).astype(np.float32)
    ids = r.integers(0, 6, size=(2, 4)).astype(np.int32)
    table.tofile(str(tmp_path / "table.f32"))
    ids.tofile(str(tmp_path / "ids.i32"))
    run = function_run(device, "picked")
    try:
        assert run.infer_dense(tmp_path, tmp_path / "rows.f32") == (2, 2)
        got = np.fromfile(str(tmp_path / "rows.f32"), dtype=np.float32).reshape(2, 4, 3)
        assert np.array_equal(got, np.stack([table[s][ids[s]] for s in range(2)]))
        # An id outside the table that reads it (E-DATA-011), the argument named.
        ids[1, 2] = 6
        ids.tofile(str(tmp_path / "ids.i32"))
        with pytest.raises(M.MsxError) as e:
            run.infer_dense(tmp_path, tmp_path / "rows.f32")
        assert "E-DATA-011: the data file of the argument `ids` holds 6, outside the 6 rows of the `embedding` table" in str(e.value)
    finally:
        run.destroy()


def test_what_is_refused_leaves_the_output_file_as_it_was(device, trained, tmp_path):
    data, checkpoint, x, _ = trained
    out = tmp_path / "kept.f32"
    out.write_bytes(b"kept")
    with pytest.raises(M.MsxError) as e:
        M.Training(device, SEVERAL, 0, function="logits")
    assert e.value.status == M.BAD_INPUT and "E-DATA-010: the model declares no function `logits`" in str(e.value)
    assert "functions: forward, unused_head, scores, picked, turned" in str(e.value)

    def refused(name, directory, code, text):
        run = function_run(device, name)
        try:
            with pytest.raises(M.MsxError) as e:
                run.infer_dense(directory, out)
            assert e.value.status == M.BAD_INPUT and code in str(e.value) and text in str(e.value), str(e.value)
        finally:
            run.destroy()
        assert out.read_bytes() == b"kept"

    refused("unused_head", data, "E-DATA-010", "the function `unused_head` takes no argument a data file could bind")
    refused("turned", data, "E-DATA-010", "the result of the function `turned` is not one row per sample")
    empty = tmp_path / "empty"
    empty.mkdir()
    refused("scores", empty, "E-DATA-007", "cannot read the data file of the argument `x`")
    ragged = tmp_path / "ragged"
    ragged.mkdir()
    x[:10].tofile(str(ragged / "x.f32"))
    refused("scores", ragged, "E-DATA-009", "the data is not a whole number of blocks")

    # `--out` that names a file the run reads, by its path, through a symbolic link and a hard link.
    run = function_run(device, "scores")
    try:
        os.symlink(str(data / "x.f32"), str(tmp_path / "alias.f32"))
        os.link(str(checkpoint), str(tmp_path / "same.msckpt"))
        for target, what in ((data / "x.f32", "argument `x`"), (tmp_path / "alias.f32", "argument `x`"), (tmp_path / "same.msckpt", "checkpoint"),
                             (tmp_path / "several.mspec", "model")):
            with pytest.raises(M.MsxError) as e:
                run.refuse_out_reading(data, target, tmp_path / "several.mspec", checkpoint)
            assert "E-DATA-010: `--out` names a file the run reads" in str(e.value) and what in str(e.value)
        run.refuse_out_reading(data, out, tmp_path / "several.mspec", checkpoint)
        # A checkpoint of another model is refused as `infer` refuses it.
        other = M.Checkpoint(step=1, seed=5, schema_hash="0" * 64)
        other.set_optimizer(M.OPTIMIZER_SGD, 0.1)
        other.add("Other.w", np.zeros((3, 2), dtype=np.float32))
        with pytest.raises(M.MsxError) as e:
            run.load_parameters(other)
        other.destroy()
        assert "E-CKPT-003" in str(e.value) and "a parameter path differs" in str(e.value)
    finally:
        run.destroy()


def test_the_command_line_runs_a_function_over_a_directory(trained, tmp_path):
    data, checkpoint, x, params = trained
    spec = tmp_path / "several.mspec"
    spec.write_text(SEVERAL)
    out = tmp_path / "cli.f32"
    env = dict(os.environ, PYTHONPATH=os.path.dirname(HERE))
    base = [sys.executable, "-m", "modelspec_b200", "infer", str(spec), "--resume", str(checkpoint)]
    done = subprocess.run(base + ["--data", str(data), "--function", "scores", "--out", str(out)], capture_output=True, text=True, env=env)
    assert done.returncode == 0, done.stderr
    assert done.stdout == "function scores blocks 3 rows 12 out %s\n" % out
    assert np.fromfile(str(out), dtype=np.float32).shape == (24,)
    done = subprocess.run(base + ["--data", str(data), "--function", "scores", "--out", str(data / "x.f32")], capture_output=True, text=True, env=env)
    assert done.returncode == 1 and "E-DATA-010" in done.stderr
    done = subprocess.run(base + ["--function", "scores"], capture_output=True, text=True, env=env)
    assert done.returncode == 2


CORNERS = """model Base {
    param w: Tensor<f32, [3, 2]> = xavier_uniform();
    fn forward(x: Tensor<f32, [4, 3]>) -> Tensor<f32, [4, 2]> {
        return matmul(x, w);
    }
    fn same(x: Tensor<f32, [4, 3]>) -> Tensor<f32, [4, 3]> {
        return x;
    }
    fn half_read(x: Tensor<f32, [4, 3]>, ids: Tensor<i32, [4]>) -> Tensor<f32, [4, 2]> {
        return matmul(x, w);
    }
    fn scaled(x: Tensor<f32, [4, 3]>, y: Tensor<f32, []>) -> Tensor<f32, []> {
        return mul(mean(x), y);
    }
}
train Fit {
    model = Base;
    input x: Tensor<f32, [4, 3]>;
    target y: Tensor<f32, [4, 2]>;
    loss = mse(model.forward(x), y);
    optimizer = sgd(lr = 0.1);
    steps = 3;
    seed = 5;
    device = cpu;
}
"""


def test_corner_functions_write_one_row_per_sample(device, tmp_path):
    """Three of the reference's corner cases (crates/modelspec-cli/tests/adversary_infer_data.rs):
    a function that returns its argument writes it back byte for byte; an argument the function
    does not read is still bound by its file and shifts no row; arguments without a shared
    leading dimension make a sample a whole block, and a rank-0 result is its one value."""
    r = np.random.default_rng(9)
    x = (r.integers(-8, 9, size=(8, 3)) / 4.0).astype(np.float32)   # multiples of 1/4: sums and products are exact
    x.tofile(str(tmp_path / "x.f32"))
    r.integers(-50, 50, size=8).astype(np.int32).tofile(str(tmp_path / "ids.i32"))   # unread: no bound holds it
    run = M.Training(device, CORNERS, 0, M.PLAN_EXACT_MATMUL, function="same")
    try:
        assert run.infer_dense(tmp_path, tmp_path / "same.f32") == (2, 8)
        assert (tmp_path / "same.f32").read_bytes() == x.tobytes()
    finally:
        run.destroy()
    run = M.Training(device, CORNERS, 0, M.PLAN_EXACT_MATMUL, function="half_read")
    try:
        w = run.forward_plan.param_download(0).reshape(3, 2)
        assert run.infer_dense(tmp_path, tmp_path / "half.f32") == (2, 8)
        got = np.fromfile(str(tmp_path / "half.f32"), dtype=np.float32).reshape(8, 2)
        np.testing.assert_allclose(got, x.astype(np.float64) @ w.astype(np.float64), rtol=1e-5, atol=1e-6)
        os.remove(str(tmp_path / "ids.i32"))
        with pytest.raises(M.MsxError) as e:
            run.infer_dense(tmp_path, tmp_path / "half.f32")
        assert "E-DATA-007: cannot read the data file of the argument `ids`" in str(e.value)
    finally:
        run.destroy()
    y = np.array([0.5, -2.0], dtype=np.float32)
    y.tofile(str(tmp_path / "y.f32"))
    run = M.Training(device, CORNERS, 0, M.PLAN_EXACT_MATMUL, function="scaled")
    try:
        assert run.infer_dense(tmp_path, tmp_path / "scaled.f32") == (2, 2)   # B = 1: a sample is a block of 4 rows of x and one y
        got = np.fromfile(str(tmp_path / "scaled.f32"), dtype=np.float32)
        want = [np.float32(x[4 * s:4 * s + 4].astype(np.float64).mean()) * y[s] for s in range(2)]
        np.testing.assert_allclose(got, want, rtol=1e-6, atol=1e-7)
    finally:
        run.destroy()
