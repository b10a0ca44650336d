"""Shared pieces of the parity tests: IR text for one-op programs, the two-sided run of a
training program, and the tolerances."""
import numpy as np

import oracle_lib
import modelspec_b200 as M

# The reference's device tolerances (its design notes, section 9, and tests/common/mod.rs:19-43):
# per kernel |g - c| <= 1e-5 + 1e-4 * r with r the magnitude of the terms summed, per run
# |g - c| <= 1e-4 + 1e-3 * |c| for every loss and parameter element.
KERNEL_ATOL, KERNEL_RTOL = 1e-5, 1e-4
RUN_ATOL, RUN_RTOL = 1e-4, 1e-3


def tensor(dtype, shape):
    return "Tensor<%s, [%s]>" % (dtype, ", ".join(str(d) for d in shape))


class ProgramText:
    """Builds the text of a small Tensor IR program node by node."""

    def __init__(self):
        self.params, self.lines, self.outputs, self.next = [], [], [], 0

    def param(self, path, shape):
        self.params.append("param @%s: %s = zeros" % (path, tensor("f32", shape)))
        return self.node(tensor("f32", shape), "ParamRead @%s" % path)

    def node(self, ty, rest):
        self.lines.append("%%%d: %s = %s" % (self.next, ty, rest))
        self.next += 1
        return self.next - 1

    def input(self, name, dtype, shape):
        return self.node(tensor(dtype, shape), 'Input "%s"' % name)

    def op(self, name, shape, operands, attr="", dtype="f32", tag=""):
        rest = name + (" " + attr if attr else "") + " " + ", ".join("%%%d" % o for o in operands)
        at = self.node(tensor(dtype, shape), rest)
        if tag:  # a training program's subgraph tag: "forward", "loss", "gradient", "optimizer"
            self.lines[-1] = tag + " " + self.lines[-1]
        return at

    def output(self, value):
        self.outputs.append("output %%%d" % value)

    def text(self):
        return "\n".join(self.params + self.lines + self.outputs) + "\n"


def run_both(device, text, inputs, params=(), outputs=(), seed=None, flags=M.PLAN_NO_GRAPH | M.PLAN_EXACT_MATMUL):
    """Evaluates `text` on the oracle and on the GPU; returns [(oracle, gpu)] per output id,
    `outputs` being (value id, element count) pairs."""
    session = oracle_lib.Session(text)
    # Every op-level run keeps guard words after each value and checks them afterwards.
    plan = M.Plan(device, text, seed=seed or 0, flags=flags | M.PLAN_GUARD)
    try:
        for name, value in inputs.items():
            session.set_input(name, value)
            plan.set_input(name, value)
        for index, value in enumerate(params):
            session.set_param(index, value)
            plan.param_upload(index, value)
        if seed is not None:
            session.set_seed(seed)
        session.run()
        plan.run()
        plan.sync()
        plan.check_guards()
        return [(session.value(v, n).astype(np.float32), plan.value(v, n)) for v, n in outputs]
    finally:
        plan.destroy()


def assert_kernel_close(gpu, cpu, scale=None, what=""):
    cpu = np.asarray(cpu, dtype=np.float64)
    gpu = np.asarray(gpu, dtype=np.float64)
    r = np.maximum(np.abs(cpu), scale if scale is not None else 0.0)
    bad = np.abs(gpu - cpu) > KERNEL_ATOL + KERNEL_RTOL * r
    assert not bad.any(), "%s: %d of %d elements outside 1e-5 + 1e-4 r; worst |g-c| = %g at %d (c = %g)" % (
        what, bad.sum(), bad.size, np.abs(gpu - cpu).max(), int(np.abs(gpu - cpu).argmax()),
        cpu.flat[int(np.abs(gpu - cpu).argmax())])


def assert_bits_equal(gpu, cpu, what=""):
    g = np.ascontiguousarray(gpu, dtype=np.float32).view(np.uint32)
    c = np.ascontiguousarray(cpu, dtype=np.float32).view(np.uint32)
    diff = g != c
    assert not diff.any(), "%s: %d of %d elements differ in bits; first at %d: gpu %r cpu %r" % (
        what, diff.sum(), diff.size, int(diff.argmax()), gpu.flat[int(diff.argmax())], cpu.flat[int(diff.argmax())])


def assert_run_close(gpu, cpu, what="", atol=RUN_ATOL):
    cpu = np.asarray(cpu, dtype=np.float64)
    gpu = np.asarray(gpu, dtype=np.float64)
    bad = ~(np.abs(gpu - cpu) <= atol + RUN_RTOL * np.abs(cpu))
    assert not bad.any(), "%s: %d of %d outside %g + 1e-3 |c|; worst |g-c| = %g" % (
        what, bad.sum(), bad.size, atol, np.nanmax(np.abs(gpu - cpu)))


def train_both(device, source, steps, masked_rows=0, feed=None, synthetic=False, flags=M.PLAN_DEFAULT):
    """Runs `steps` steps of `source` on the oracle and on the GPU from the same initial
    parameters and the same batches. `feed(k)` gives the declared inputs of step k as a dict;
    `synthetic` uses the reference's synthetic batch instead. Returns a dict with both sides'
    losses (steps + the final loss), parameters, gradients of the last step and moments."""
    cpu = oracle_lib.Trainer(source, masked_rows)
    gpu = M.Training(device, source, masked_rows, flags)
    try:
        if synthetic:
            # The oracle draws the reference's synthetic batch; the GPU trains on the same bytes.
            cpu.synthetic()
            for name, nbytes, is_i32 in gpu.forward_plan.inputs():
                if not is_i32:
                    gpu.set_input(name, cpu.get_input(name, nbytes // 4))
        cpu_losses, gpu_losses = [], []
        for k in range(steps):
            if feed is not None:
                for name, value in feed(k).items():
                    cpu.set_input(name, value)
                    gpu.set_input(name, value)
            cpu_losses.append(cpu.step(k, steps))
            gpu.step(k, steps)
            gpu_losses.append(gpu.loss())
        if feed is not None:
            for name, value in feed(steps).items():
                cpu.set_input(name, value)
                gpu.set_input(name, value)
        cpu_losses.append(cpu.final_loss())
        gpu_losses.append(gpu.final_loss())
        paths = cpu.param_paths()
        if flags & M.PLAN_GUARD:
            gpu.step_plan.check_guards()
            gpu.forward_plan.check_guards()
        out = {"paths": paths, "cpu_losses": np.array(cpu_losses, dtype=np.float32),
               "gpu_losses": np.array(gpu_losses, dtype=np.float32), "cpu_params": [], "gpu_params": [],
               "stats": gpu.step_plan.stats()}
        for i in range(len(paths)):
            out["cpu_params"].append(cpu.read("param", i))
            try:
                out["gpu_params"].append(gpu.step_plan.param_download(i))
            except M.MsxError:
                out["gpu_params"].append(gpu.forward_plan.param_download(i))
        return out
    finally:
        gpu.destroy()
