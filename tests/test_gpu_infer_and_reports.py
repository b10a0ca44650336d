"""`infer --backend cuda` and the `--stats` / `--profile` report lines: the forward program on a
run's parameters through the C ABI against the oracle, and the text the reference's CLI prints
for a device run (crates/modelspec-cli/src/infer.rs:251-262, crates/modelspec-runtime/src/vulkan/
runner.rs:143-163, vulkan/profile.rs:237-338), line for line in shape."""
import re

import numpy as np
import pytest

import modelspec_b200 as M
import oracle_lib
from modelspec_b200 import models, synthetic

pytestmark = pytest.mark.gpu


def test_infer_gives_the_prediction_and_the_loss_of_the_trained_parameters(device):
    source = models.linear_regression(steps=5)
    gpu = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    cpu = oracle_lib.Trainer(source)
    try:
        cpu.synthetic()
        for name, nbytes, _ in gpu.forward_plan.inputs():
            gpu.set_input(name, cpu.get_input(name, nbytes // 4))
        for k in range(5):
            gpu.step(k, 5)
            cpu.step(k, 5)
        prediction, loss = gpu.infer()
        assert prediction.shape == (8,)
        # The loss `infer` prints for a run's last parameters is that run's final loss line.
        assert loss == gpu.final_loss()
        assert abs(float(loss) - float(cpu.final_loss())) <= 1e-4 + 1e-3 * abs(float(cpu.final_loss()))
        # prediction = x w with the trained w: checked against the host's own product.
        x = cpu.get_input("x", 32).reshape(8, 4).astype(np.float64)
        w = gpu.step_plan.param_download(0).astype(np.float64)
        assert np.abs(prediction - (x @ w)).max() <= 1e-5
        lines = gpu.infer_report().splitlines()
        assert len(lines) == 2
        assert lines[0].startswith("prediction: Tensor<f32, [8, 1]> = [") and lines[0].endswith("]")
        printed = np.array([np.float32(v) for v in lines[0].split("= [", 1)[1][:-1].split(", ")], dtype=np.float32)
        assert np.array_equal(printed, prediction), "every printed number reads back as the same f32"
        assert lines[1].startswith("loss ") and np.float32(lines[1][5:]) == loss
    finally:
        gpu.destroy()


def test_infer_on_a_bert_twin_in_both_precisions(device):
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=304, seq=16, batch=8, steps=3, warmup_steps=1)
    batch = synthetic.mlm_batch(0, vocab=304, seq=16, batch=8)
    results = []
    for flags in (M.PLAN_DEFAULT, M.PLAN_BF16):
        gpu = M.Training(device, source, 64, flags)
        try:
            for name, value in batch.items():
                gpu.set_input(name, value)
            for k in range(3):
                gpu.step(k, 3)
            prediction, loss = gpu.infer()
            assert prediction.shape == (8 * 16 * 304,) and np.isfinite(prediction).all()
            # The plan that keeps the prediction adds the decoder bias in its own launch, the
            # final-loss plan in the product's epilogue: the same loss within the run tolerance.
            final = float(gpu.final_loss())
            assert abs(float(loss) - final) <= 1e-4 + (2e-2 if flags & M.PLAN_BF16 else 1e-3) * abs(final)
            results.append((prediction, float(loss)))
        finally:
            gpu.destroy()
    assert abs(results[0][1] - results[1][1]) <= 2e-2 * abs(results[0][1])


def test_the_stats_and_profile_lines_have_the_reference_shape(device):
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=304, seq=16, batch=8, steps=4, warmup_steps=1)
    gpu = M.Training(device, source, 64)
    try:
        for name, value in synthetic.mlm_batch(0, vocab=304, seq=16, batch=8).items():
            gpu.set_input(name, value)
        for k in range(4):
            gpu.step(k, 4)
        gpu.loss()
        plan = gpu.step_plan
        launches = plan.stats()["launches_per_step"]
        stats = dict(line.split(": ", 1) for line in plan.stats_report().splitlines())
        assert list(stats) == ["steps", "host waits", "submits", "dispatches", "dispatches per step", "barriers per step", "bytes uploaded",
                               "bytes downloaded", "device allocations", "peak device bytes", "numerics class", "us per step", "pipelines",
                               "pipeline creation us"]
        assert stats["steps"] == "4" and stats["submits"] == "4" and stats["dispatches"] == str(4 * launches)
        assert stats["dispatches per step"] == str(launches) and stats["numerics class"] == "tolerance"
        assert int(stats["bytes uploaded"]) >= 4 * plan.stats()["upload_bytes_per_step"] and int(stats["peak device bytes"]) > 0
        assert re.fullmatch(r"\d+\.\d{3}", stats["us per step"])
        gpu.final_loss()
        report = plan.profile_report(gpu.forward_plan, repeats=2).splitlines()
        dispatch = [l for l in report if l.startswith("profile dispatch ")]
        shape = re.compile(r"profile dispatch (step|final) (\d+) (\d+) (\w+) calls 1 total_us \d+\.\d{3} mean_us \d+\.\d{3} "
                           r"flop \d+ bytes \d+ gflop_per_s (\d+\.\d{3}|unavailable) gb_per_s (\d+\.\d{3}|unavailable)")
        assert all(shape.fullmatch(l) for l in dispatch), [l for l in dispatch if not shape.fullmatch(l)][:3]
        assert sum(l.startswith("profile dispatch step ") for l in dispatch) == launches
        assert any(l.startswith("profile dispatch final ") for l in dispatch)
        rest = [l.split()[1] for l in report if not l.startswith("profile dispatch ")]
        assert rest == ["pipeline", "dispatches", "submits", "host_waits", "barriers_per_step", "bytes_uploaded", "bytes_downloaded",
                        "device_allocations", "peak_device_bytes", "pipeline_creation_us", "compile_us", "steady_us_per_step", "step_total"]
        assert re.fullmatch(r"profile step_total flop \d+ bytes \d+ gflop_per_s \d+\.\d{3} gb_per_s \d+\.\d{3} uncounted_sites 0", report[-1])
    finally:
        gpu.destroy()
