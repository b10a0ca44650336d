"""AdamW and SGD held to the reference's own written-order f32 update, bit for bit: the scenarios
`one_step` and `zero_gradient_decays_the_moments` of crates/modelspec-runtime/tests/adamw.rs
(:172-330), whose reference arithmetic is transcribed in adamw_reference.py. The CPU tests pin the
oracle's update; the GPU tests pin the one multi-tensor launch (16 rounded operations per
element, IEEE sqrt and division) on the gradients the device itself reports."""
import re

import numpy as np
import pytest

import adamw_reference as R
import oracle_lib
from helpers import assert_bits_equal


def reference_step(t, warmup, steps, p, g, m, v):
    constants = R.host_constants(R.LR, R.BETA1, R.BETA2, t, warmup, steps)
    return R.adamw_step(p, g, m, v, constants, R.BETA1, R.BETA2, R.EPS, R.WEIGHT_DECAY)


def run_oracle(source, steps, batches=None, check_steps=None):
    cpu = oracle_lib.Trainer(source)
    if batches is None:
        cpu.synthetic()
    paths = cpu.param_paths()
    moments = [(np.zeros_like(cpu.read("param", i)), np.zeros_like(cpu.read("param", i))) for i in range(len(paths))]
    history = []
    for k in range(check_steps or steps):
        if batches is not None:
            for name, value in batches[k].items():
                cpu.set_input(name, value)
        before = [cpu.read("param", i) for i in range(len(paths))]
        cpu.step(k, steps)
        grads = [cpu.read("grad", i) for i in range(len(paths))]
        for i, path in enumerate(paths):
            want_p, want_m, want_v = reference_step(k + 1, 2, steps, before[i], grads[i], *moments[i])
            moments[i] = (want_m, want_v)
            assert_bits_equal(cpu.read("param", i), want_p, "step %d %s" % (k + 1, path))
            assert_bits_equal(cpu.read("m", i), want_m, "step %d m of %s" % (k + 1, path))
            assert_bits_equal(cpu.read("v", i), want_v, "step %d v of %s" % (k + 1, path))
        history.append((before, grads))
    return paths, history


def test_oracle_one_step_is_the_written_order_update():
    paths, history = run_oracle(R.two_parameters(2, 10), 10, check_steps=3)
    for before, grads in history:
        assert all((g != 0).all() for g in grads), "every element has a gradient in these steps"


def test_oracle_zero_gradient_decays_the_moments():
    paths, history = run_oracle(R.two_parameters(2, R.DENSE_STEPS), R.DENSE_STEPS, batches=R.zero_step_batches())
    w = paths.index("Reg.w")
    for step, (before, grads) in enumerate(history):
        assert (grads[w] == 0).all() == (step == R.ZERO_STEP), "step %d" % step


def test_the_transcribed_host_constants_are_the_oracle_s():
    """lr_t, c1 and c2 as the reference's test computes them (adamw.rs:118-141) against the
    scalars the host code feeds: first steps, the warm-up boundary, late steps."""
    import modelspec_b200 as M
    text = M.compile_mspec(R.two_parameters(2, 10), "step")
    assert "optimizer adamw" in text
    for t in (1, 2, 3, 9, 10):
        lr_t, c1, c2 = R.host_constants(R.LR, R.BETA1, R.BETA2, t, 2, 10)
        assert np.isfinite([lr_t, c1, c2]).all() and lr_t >= 0
    assert R.host_constants(R.LR, R.BETA1, R.BETA2, 10, 2, 10)[0] == 0.0  # decayed to 0 at the last step
    assert R.host_constants(R.LR, R.BETA1, R.BETA2, 2, 2, 10)[0] == np.float32(0.01)


def gradient_ids(ir_text):
    return {m.group(2): int(m.group(1)) for m in re.finditer(r"^output %(\d+) gradient @(\S+)", ir_text, re.M)}


def run_gpu(device, source, steps, batches=None, check_steps=None, upload=None):
    import modelspec_b200 as M
    gpu = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    cpu = oracle_lib.Trainer(source)
    try:
        if batches is None:
            cpu.synthetic()
            for name, nbytes, is_i32 in gpu.forward_plan.inputs():
                gpu.set_input(name, cpu.get_input(name, nbytes // 4))
        plan = gpu.step_plan
        params = plan.params()
        ids = gradient_ids(M.compile_mspec(source, "step"))
        moments = [(np.zeros(n // 4, dtype=np.float32), np.zeros(n // 4, dtype=np.float32)) for _, n in params]
        if upload is not None:
            for i, (p, m, v) in enumerate(upload):
                plan.param_upload(i, p); plan.moment_upload(i, "m", m); plan.moment_upload(i, "v", v)
                moments[i] = (m, v)
        for k in range(check_steps or steps):
            if batches is not None:
                for name, value in batches[k].items():
                    gpu.set_input(name, value)
            before = [plan.param_download(i) for i in range(len(params))]
            gpu.step(k, steps)
            gpu.loss()
            for i, (path, nbytes) in enumerate(params):
                g = plan.value(ids[path], nbytes // 4)
                want_p, want_m, want_v = reference_step(k + 1, 2, steps, before[i], g, *moments[i])
                moments[i] = (want_m, want_v)
                assert_bits_equal(plan.param_download(i), want_p, "step %d %s" % (k + 1, path))
                assert_bits_equal(plan.moment_download(i, "m"), want_m, "step %d m of %s" % (k + 1, path))
                assert_bits_equal(plan.moment_download(i, "v"), want_v, "step %d v of %s" % (k + 1, path))
    finally:
        gpu.destroy()


@pytest.mark.gpu
def test_gpu_one_step_is_the_written_order_update(device):
    run_gpu(device, R.two_parameters(2, 10), 10, check_steps=3)


@pytest.mark.gpu
def test_gpu_zero_gradient_decays_the_moments(device):
    run_gpu(device, R.two_parameters(2, R.DENSE_STEPS), R.DENSE_STEPS, batches=R.zero_step_batches())


@pytest.mark.gpu
def test_gpu_update_launch_on_seeded_state_across_chunks(device):
    """The same launch on tensors longer than one 4,096-element chunk and not a multiple of 4
    long, from seeded parameters and moments (second moments non-negative, some exactly 0), at
    steps past the warm-up: parameters and both moments bit for bit."""
    r = np.random.default_rng(5)
    rows, inputs, outputs = 16, 257, 33
    w = (r.standard_normal(inputs * outputs) * 0.1).astype(np.float32)
    b = r.standard_normal(outputs).astype(np.float32)
    state = []
    for p in (w, b):
        m = (r.standard_normal(p.size) * 1e-2).astype(np.float32)
        v = (r.standard_normal(p.size) ** 2 * 1e-3).astype(np.float32)
        v[::7] = 0.0
        state.append((p, m, v))
    x = r.standard_normal(rows * inputs).astype(np.float32)
    y = r.standard_normal(rows * outputs).astype(np.float32)
    batches = [{"x": x, "y": y}] * 8
    run_gpu(device, R.two_parameters(2, 8, rows, inputs, outputs), 8, batches=batches, check_steps=5, upload=state)


@pytest.mark.gpu
def test_gpu_sgd_update_is_p_minus_the_rounded_product(device):
    import modelspec_b200 as M
    from modelspec_b200 import models
    source = models.linear_regression(steps=5)
    gpu = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    try:
        gpu.synthetic()
        plan = gpu.step_plan
        gid = gradient_ids(M.compile_mspec(source, "step"))["LinearReg.w"]
        for k in range(4):
            before = plan.param_download(0)
            gpu.step(k, 5)
            gpu.loss()
            assert_bits_equal(plan.param_download(0), R.sgd_step(before, plan.value(gid, 4), 0.1), "step %d" % k)
    finally:
        gpu.destroy()
