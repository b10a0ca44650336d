"""A run fed from a dense `--data` directory (crates/modelspec-runtime/src/train/data.rs:513-577):
the whole run through msx_training_run equals the same batches set by hand, with and without an
order file; an id outside the table that reads it is refused before the first step; and the
command line takes a dense directory where it finds no binding file."""
import os
import subprocess
import sys

import numpy as np
import pytest

import modelspec_b200 as M
from modelspec_b200 import models

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))


def regression_directory(path, samples=40, order=None):
    r = np.random.default_rng(11)
    x = r.standard_normal((samples, 4)).astype(np.float32)
    y = (x @ np.array([[1.0], [-2.0], [0.5], [3.0]], dtype=np.float32) + 0.01 * r.standard_normal((samples, 1))).astype(np.float32)
    x.tofile(os.path.join(path, "x.f32"))
    y.tofile(os.path.join(path, "y.f32"))
    if order is not None:
        np.asarray(order, dtype=np.uint32).tofile(os.path.join(path, "order.u32"))
    return x, y


@pytest.mark.parametrize("ordered", [False, True])
def test_a_dense_run_is_the_run_on_the_same_batches_set_by_hand(device, tmp_path, ordered):
    steps, batch = 12, 8
    order = np.random.default_rng(3).permutation(40).astype(np.uint32)
    order = np.concatenate([order, order, order])[: steps * batch]
    x, y = regression_directory(str(tmp_path), order=order if ordered else None)
    source = models.linear_regression(steps=steps)
    whole = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    by_hand = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    try:
        whole.bind_dense(str(tmp_path))
        lines = whole.run().splitlines()

        def rows(k):
            at = [k * batch + i for i in range(batch)]
            return [int(order[p % len(order)]) for p in at] if ordered else [p % 40 for p in at]

        losses = []
        for k in range(steps):
            by_hand.set_input("x", x[rows(k)])
            by_hand.set_input("y", y[rows(k)])
            by_hand.step(k, steps)
            losses.append(by_hand.loss_of(k))
        by_hand.set_input("x", x[rows(steps)])
        by_hand.set_input("y", y[rows(steps)])
        losses.append(by_hand.final_loss())
        got = {int(l.split()[1]): np.float32(l.split()[3]) for l in lines if l.startswith("step ")}
        assert sorted(got) == [0, steps]                      # the first and the last loss have lines (12 steps, none at a multiple of 50)
        for k, value in got.items():
            assert value == losses[k], (k, value, losses[k])   # the printed text reads back to the f32 it shows
        assert lines[0].startswith("init @LinearReg.w") and lines[-1].startswith("param @LinearReg.w")
        assert got[steps] < got[0]
    finally:
        whole.destroy()
        by_hand.destroy()


def test_an_id_outside_its_table_is_refused_before_the_first_step(device, tmp_path):
    vocab, seq, batch = 300, 16, 4
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=vocab, seq=seq, batch=batch, steps=3, warmup_steps=1)
    rows, samples = batch * seq, 3
    r = np.random.default_rng(2)
    ids = r.integers(5, vocab, size=(samples * batch, seq)).astype(np.int32)
    files = {"ids.i32": ids.reshape(-1), "positions.i32": np.tile(np.arange(seq, dtype=np.int32), samples * batch),
             "key_mask.f32": np.ones((samples * batch, seq), dtype=np.float32), "labels.i32": ids.reshape(-1),
             "weights.f32": (r.random(samples * rows) < 0.15).astype(np.float32)}
    for name, values in files.items():
        values.tofile(os.path.join(str(tmp_path), name))
    run = M.Training(device, source, 16)
    try:
        run.bind_dense(str(tmp_path))
        text = run.run()
        assert text.count("\nstep ") + text.startswith("step ") >= 2 and "NaN" not in text
        bad = ids.copy().reshape(-1)
        bad[37] = vocab
        bad.tofile(os.path.join(str(tmp_path), "ids.i32"))
        with pytest.raises(M.MsxError) as e:
            run.bind_dense(str(tmp_path))
        message = str(e.value)
        assert e.value.status == M.BAD_INPUT and "E-DATA-011" in message and "holds 300, outside the 300 rows of the `embedding` table" in message
        assert "position 37" in message
    finally:
        run.destroy()


def test_the_command_line_takes_a_dense_directory(tmp_path):
    regression_directory(str(tmp_path))
    spec = tmp_path / "fit.mspec"
    spec.write_text(models.linear_regression(steps=10))
    done = subprocess.run([sys.executable, "-m", "modelspec_b200", "train", str(spec), "--data", str(tmp_path)], capture_output=True, text=True,
                          cwd=os.path.dirname(HERE))
    assert done.returncode == 0, done.stderr
    lines = done.stdout.splitlines()
    assert lines[0].startswith("init @LinearReg.w") and lines[1].startswith("step 0 loss ") and lines[-1].startswith("param @LinearReg.w")
    os.remove(os.path.join(str(tmp_path), "y.f32"))
    done = subprocess.run([sys.executable, "-m", "modelspec_b200", "train", str(spec), "--data", str(tmp_path)], capture_output=True, text=True,
                          cwd=os.path.dirname(HERE))
    assert done.returncode == 1 and "E-DATA-007" in done.stderr and "the target `y`" in done.stderr


WIDE_REGRESSION = """model LinearReg {
    param w: Tensor<f32, [4, 3]> = xavier_uniform();
    fn forward(x: Tensor<f32, [8, 4]>) -> Tensor<f32, [8, 3]> {
        return matmul(x, w);
    }
}
train Fit {
    model = LinearReg;
    input x: Tensor<f32, [8, 4]>;
    target y: Tensor<f32, [8, 3]>;
    loss = mse(model.forward(x), y);
    optimizer = sgd(lr = 0.1);
    steps = 6;
    seed = 42;
    device = cpu;
}
"""


def test_an_eval_directory_gives_the_mean_batch_loss_and_the_accuracy(device, tmp_path):
    """`--eval <dir>` (train/runner.rs:571-624): the mean of the batch losses summed in f64 and
    the fraction of target rows whose prediction has its first maximum where the target has its."""
    r = np.random.default_rng(8)
    x = r.standard_normal((24, 4)).astype(np.float32)
    y = r.standard_normal((24, 3)).astype(np.float32)
    x.tofile(os.path.join(str(tmp_path), "x.f32"))
    y.tofile(os.path.join(str(tmp_path), "y.f32"))
    run = M.Training(device, WIDE_REGRESSION, 0, M.PLAN_EXACT_MATMUL)
    try:
        run.bind_dense(str(tmp_path))
        run.run()
        loss, accuracy = run.eval_dense(str(tmp_path))
        total, correct = 0.0, 0
        for b in range(3):
            run.set_input("x", x[8 * b:8 * b + 8])
            run.set_input("y", y[8 * b:8 * b + 8])
            prediction, batch_loss = run.infer()
            total += float(batch_loss)
            correct += int((prediction.reshape(8, 3).argmax(axis=1) == y[8 * b:8 * b + 8].argmax(axis=1)).sum())
        assert loss == total / 3 and accuracy == correct / 24
        assert M.eval_line(loss, accuracy).startswith("eval loss=") and " accuracy=" in M.eval_line(loss, accuracy)
        # A directory that is not a whole number of batches is refused.
        x[:20].tofile(os.path.join(str(tmp_path), "x.f32"))
        y[:20].tofile(os.path.join(str(tmp_path), "y.f32"))
        with pytest.raises(M.MsxError) as e:
            run.eval_dense(str(tmp_path))
        assert "E-DATA-009" in str(e.value)
    finally:
        run.destroy()
    # Labels that a cross_entropy reads are no compared target: no accuracy (data.rs:640-655).
    vocab, seq, batch = 300, 16, 4
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=vocab, seq=seq, batch=batch, steps=2, warmup_steps=1)
    ids = r.integers(5, vocab, size=(2 * batch, seq)).astype(np.int32)
    files = {"ids.i32": ids.reshape(-1), "positions.i32": np.tile(np.arange(seq, dtype=np.int32), 2 * batch),
             "key_mask.f32": np.ones((2 * batch, seq), dtype=np.float32), "labels.i32": ids.reshape(-1),
             "weights.f32": (r.random(2 * batch * seq) < 0.15).astype(np.float32)}
    where = tmp_path / "mlm"
    where.mkdir()
    for name, values in files.items():
        values.tofile(os.path.join(str(where), name))
    run = M.Training(device, source, 16)
    try:
        run.bind_dense(str(where))
        run.run()
        loss, accuracy = run.eval_dense(str(where))
        assert accuracy is None and np.isfinite(loss) and loss > 0
    finally:
        run.destroy()


WEIGHTED_CLASSES = """model Classes {
    param w: Tensor<f32, [3, 5]> = xavier_uniform();
    fn forward(x: Tensor<f32, [6, 3]>) -> Tensor<f32, [6, 5]> {
        return matmul(x, w);
    }
}
train Fit {
    model = Classes;
    input x: Tensor<f32, [6, 3]>;
    input labels: Tensor<i32, [6]>;
    target weights: Tensor<f32, [6]>;
    loss = cross_entropy(model.forward(x), labels, weights);
    optimizer = sgd(lr = 0.1);
    steps = 2;
    seed = 7;
    device = cpu;
}
"""


def test_the_one_compared_target_is_held_to_the_model_output_type(device, tmp_path):
    """read_dense (train/data.rs:640-662): a block's single target that is no cross_entropy's
    labels has the type of the model output, else E-DATA-002 with both types, before any file
    is opened (the directory here is empty); the same target as labels is accepted."""
    run = M.Training(device, WEIGHTED_CLASSES, 0)
    try:
        for bind in (run.bind_dense, run.eval_dense):
            with pytest.raises(M.MsxError) as e:
                bind(str(tmp_path))
            message = str(e.value)
            assert e.value.status == M.BAD_INPUT and "E-DATA-002: the target is not of the model output type" in message
            assert "target: Tensor<f32, [6]>" in message and "model output: Tensor<f32, [6, 5]>" in message
    finally:
        run.destroy()
    labelled = WEIGHTED_CLASSES.replace("input labels", "target labels").replace("target weights", "input weights")
    r = np.random.default_rng(2)
    r.standard_normal((12, 3)).astype(np.float32).tofile(os.path.join(str(tmp_path), "x.f32"))
    r.integers(0, 5, size=12).astype(np.int32).tofile(os.path.join(str(tmp_path), "labels.i32"))
    np.ones(12, dtype=np.float32).tofile(os.path.join(str(tmp_path), "weights.f32"))
    run = M.Training(device, labelled, 0)
    try:
        run.bind_dense(str(tmp_path))
        run.run()
        loss, accuracy = run.eval_dense(str(tmp_path))
        assert accuracy is None and np.isfinite(loss)
    finally:
        run.destroy()
