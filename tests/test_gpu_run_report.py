"""The whole run as one call and the text it prints: the reference's `train` standard output
(crates/modelspec-cli/src/train.rs:7-17, :1494-1560) for a recorded linear-regression run
(crates/modelspec-cli/tests/golden/linear_regression.train.stdout), for a run on a packed directory
with held-out evaluation, for a run that stops at a loss that is not finite, and through the
command line."""
import json
import os
import re
import subprocess
import sys

import numpy as np
import pytest

import modelspec_b200 as M
import packed_dir
from helpers import assert_run_close
from modelspec_b200 import models

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
GOLDEN = json.load(open(os.path.join(HERE, "golden", "linear_regression.losses.json")))
FEED = np.load(os.path.join(HERE, "golden", "mlm_feed.npz"))
SEQ, VOCAB, BATCH, SEED = (int(FEED[k]) for k in ("seq", "vocab", "batch", "seed"))


def vector(line):
    return np.array([np.float32(x) for x in line.rsplit("[", 1)[1].rstrip("]").split(", ")], dtype=np.float32)


def test_a_linear_regression_run_prints_the_recorded_log(device):
    gpu = M.Training(device, models.linear_regression(), 0, M.PLAN_EXACT_MATMUL)
    try:
        gpu.synthetic()
        got, want = gpu.run().splitlines(), GOLDEN["log"]
        assert len(got) == len(want) == 13
        assert got[0] == want[0], "the initial parameters are drawn on the host: the same text"
        for mine, theirs in zip(got[1:-1], want[1:-1]):
            a, b = mine.split(), theirs.split()
            assert a[:2] == b[:2] and a[2] == "loss" and len(a) == 4
            assert_run_close(np.float32(a[3]), np.float32(b[3]), mine, atol=1e-9)
        assert got[-1].split(" = ")[0] == want[-1].split(" = ")[0] == "param @LinearReg.w: Tensor<f32, [4, 1]>"
        assert_run_close(vector(got[-1]), vector(want[-1]), "final parameter")
        # Every number is the shortest text that reads back to its f32.
        for line in got[1:-1]:
            text = line.split()[3]
            assert "e" not in text and np.float32(text) == np.float32(float(text))
    finally:
        gpu.destroy()


def test_a_packed_run_with_held_out_evaluation(device, tmp_path):
    packed_dir.write(str(tmp_path), FEED["train"], FEED["heldout"], SEQ, VOCAB)
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=VOCAB, seq=SEQ, batch=BATCH, warmup_steps=1, seed=SEED, steps=12)
    packed = M.Packed(str(tmp_path))
    whole = M.Training(device, source, 16)
    by_hand = M.Training(device, source, 16)
    try:
        for run in (whole, by_hand):
            run.bind_packed(packed)
            assert run.heldout_packed() == 2
        lines = whole.run(0, 5).splitlines()
        assert lines[0] == packed.data_line().rstrip("\n")
        assert re.fullmatch(r"data dataset %s tokenizer %s seq_len 16 masking 0.15/0.8/0.1/0.1 binding [0-9a-f-]{36}" %
                            (packed_dir.DATASET_ID, packed_dir.TOKENIZER_ID), lines[0])
        inits = [l for l in lines if l.startswith("init @")]
        params = [l for l in lines if l.startswith("param @")]
        paths = [l.split(":")[0][6:] for l in inits]
        assert len(inits) == len(params) == 41 and paths == sorted(paths) and [l.split(":")[0][7:] for l in params] == paths
        body = lines[1 + len(inits):len(lines) - len(params)]
        assert [l.split()[:2] for l in body] == [["step", "0"], ["eval", "0"], ["step", "5"], ["eval", "5"], ["step", "10"], ["eval", "10"],
                                                 ["step", "12"], ["eval", "12"]]
        # The same numbers as the calls made one by one.
        expect = {}
        for k in range(12):
            if k % 5 == 0:
                expect["eval %d" % k] = by_hand.heldout_evaluate()
            by_hand.feed_packed(k)
            by_hand.step(k, 12)
            expect["step %d" % k] = by_hand.loss()
        by_hand.feed_packed(12)
        expect["eval 12"] = by_hand.heldout_evaluate()
        expect["step 12"] = by_hand.final_loss()
        for line in body:
            words = line.split()
            value = expect[" ".join(words[:2])]
            if words[0] == "step":
                assert np.float32(words[3]).tobytes() == np.float32(value).tobytes(), line
            else:
                assert words[2] == "loss" and words[4] == "accuracy"
                assert (np.float32(words[3]), np.float32(words[5])) == tuple(value), line
        final = {l.split(":")[0][7:]: vector(l) for l in params}
        for i, path in enumerate(sorted(paths)):
            pass
        ckpt = by_hand.checkpoint(12)
        for path, _, value in ckpt.tensors():
            assert final[path].tobytes() == value.reshape(-1).tobytes(), path
        ckpt.destroy()
    finally:
        whole.destroy()
        by_hand.destroy()
        packed.close()


def test_a_run_that_diverges_stops_at_its_step_without_param_lines(device):
    source = models.linear_regression(steps=12).replace("lr = 0.1", "lr = 3e12")
    gpu = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    try:
        gpu.synthetic()
        with pytest.raises(M.MsxError) as e:
            gpu.run()
        assert e.value.status == M.NON_FINITE and "E-TRAIN-001" in str(e.value)
        lines = gpu.report().splitlines()
        assert lines[0].startswith("init @") and not any(l.startswith("param @") for l in lines)
        last = lines[-1].split()
        assert last[0] == "step" and last[2] == "loss" and last[3] in ("inf", "NaN", "-inf")
    finally:
        gpu.destroy()


def test_the_command_line_prints_the_run(device, tmp_path):
    source = models.linear_regression(steps=100)
    path = tmp_path / "fit.mspec"
    path.write_text(source)
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.dirname(HERE), os.environ.get("PYTHONPATH", "")]))
    done = subprocess.run([sys.executable, "-m", "modelspec_b200", "train", str(path), "--stats", "--checkpoint", str(tmp_path / "out.msckpt")],
                          env=env, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    lines = done.stdout.splitlines()
    assert lines[0].startswith("init @LinearReg.w") and [l.split()[1] for l in lines if l.startswith("step ")] == ["0", "50", "100"]
    assert any(l.startswith("param @LinearReg.w") for l in lines) and "steps: 100" in lines
    saved = M.Checkpoint.read(str(tmp_path / "out.msckpt"))
    assert saved.step == 100
    saved.destroy()
    again = subprocess.run([sys.executable, "-m", "modelspec_b200", "infer", str(path), "--resume", str(tmp_path / "out.msckpt")],
                           env=env, capture_output=True, text=True, timeout=600)
    assert again.returncode == 0 and again.stdout.startswith("prediction: Tensor<f32, [8, 1]> = [") and "\nloss " in again.stdout
    missing = subprocess.run([sys.executable, "-m", "modelspec_b200", "train", str(tmp_path / "none.mspec")], env=env, capture_output=True, text=True)
    assert missing.returncode == 1 and missing.stderr.startswith("error: ") and missing.stdout == ""
