"""The BERT-shaped ops pinned to something the reference wrote: 10 AdamW steps of the hidden-32
twin as the reference's own PyTorch restatement of the program computes them in float64
(tests/golden/bert_twin_torch.npz, written by tests/golden/make_bert_twin_fixture.py from
opponents/bert_tiny_pretrain/bert_tiny_pretrain.py). Embedding and its scatter, attention with
masked keys, layer norm, gelu, the tied decoder, weighted cross-entropy, every backward op and
AdamW with its warm-up schedule are all inside these numbers. The oracle (CPU test) and the CUDA
backend (GPU tests, with and without the masked-row gather, exact and tensor-core matmuls) are
each held to the run tolerance |x - c| <= 1e-4 + 1e-3 |c| on every loss and every final parameter
element, and the first step's gradients to 1e-3 of their tensor's largest magnitude."""
import os

import numpy as np
import pytest

import oracle_lib
from helpers import assert_run_close
from modelspec_b200 import models

FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bert_twin_torch.npz")


def load():
    z = np.load(FIXTURE)
    batch, seq, hidden, heads, ffn, vocab, layers = (int(x) for x in z["shape"])
    lr, wd, b1, b2, eps, warmup, steps = (float(x) for x in z["hyper"])
    source = models.bert(name="BertTiny", layers=layers, hidden=hidden, heads=heads, ffn=ffn, vocab=vocab, seq=seq,
                         batch=batch, dropout=0.0, lr=lr, weight_decay=wd, beta1=b1, beta2=b2, eps=eps,
                         warmup_steps=int(warmup), steps=int(steps))
    feed = {k[len("batch."):]: z[k] for k in z.files if k.startswith("batch.")}
    return z, source, feed, int(steps)


def check(z, paths, losses, final, gradients):
    assert_run_close(np.array(losses), z["losses"], "losses against the PyTorch restatement")
    for i, path in enumerate(paths):
        name = path.split(".", 1)[1]
        # A key bias has gradient exactly 0 in exact arithmetic; what AdamW makes of rounding noise
        # is bounded by the steps taken (the reference's own allowance, tests/common/mod.rs:33-43).
        atol = 1e-4 + 10 * 3e-3 * 1e-3 if name.endswith("_bk") else 1e-4
        assert_run_close(final[i], z["final." + name].reshape(-1), "final " + name, atol=atol)
        want = z["gradient0." + name].reshape(-1).astype(np.float64)
        scale = max(float(np.abs(want).max()), 1e-6)
        worst = float(np.abs(gradients[i].astype(np.float64) - want).max())
        if not name.endswith("_bk"):
            assert worst <= 1e-3 * scale, "first gradient of %s: worst |x - c| = %g, largest |c| = %g" % (name, worst, scale)
        else:
            assert worst <= 1e-6, "a key bias's gradient is rounding noise around 0"


def test_oracle_follows_the_pytorch_restatement():
    z, source, feed, steps = load()
    cpu = oracle_lib.Trainer(source)
    paths = cpu.param_paths()
    for i, path in enumerate(paths):
        cpu.write_param(i, z["initial." + path.split(".", 1)[1]].reshape(-1))
    for name, value in feed.items():
        cpu.set_input(name, value)
    losses, gradients = [], None
    for k in range(steps):
        losses.append(cpu.step(k, steps))
        if k == 0:
            gradients = [cpu.read("grad", i) for i in range(len(paths))]
    losses.append(cpu.final_loss())
    check(z, paths, losses, [cpu.read("param", i) for i in range(len(paths))], gradients)


@pytest.mark.gpu
@pytest.mark.parametrize("masked_rows,exact", [(0, False), (64, False), (64, True)])
def test_gpu_follows_the_pytorch_restatement(device, masked_rows, exact):
    import re
    import modelspec_b200 as M
    z, source, feed, steps = load()
    gpu = M.Training(device, source, masked_rows, M.PLAN_EXACT_MATMUL if exact else M.PLAN_DEFAULT)
    try:
        plan = gpu.step_plan
        params = plan.params()
        paths = [p for p, _ in params]
        for i, path in enumerate(paths):
            plan.param_upload(i, z["initial." + path.split(".", 1)[1]].reshape(-1))
        for name, value in feed.items():
            gpu.set_input(name, value)
        ids = {m.group(2): int(m.group(1))
               for m in re.finditer(r"^output %(\d+) gradient @(\S+)", M.compile_mspec(source, "step", masked_rows), re.M)}
        losses, gradients = [], None
        for k in range(steps):
            gpu.step(k, steps)
            losses.append(gpu.loss())
            if k == 0:
                gradients = [plan.value(ids[path], nbytes // 4) for path, nbytes in params]
        losses.append(gpu.final_loss())
        check(z, paths, losses, [plan.param_download(i) for i in range(len(paths))], gradients)
    finally:
        gpu.destroy()
