"""Restore and replay: a run rewound to a step is, bit for bit, the run that stopped after that
step, as the reference's device runner leaves the state of a diverged segment
(crates/modelspec-runtime/src/vulkan/stepwise.rs:84-92, :1024-1082). The divergence here is an
overflowing learning rate: arithmetic, no device fault."""
import numpy as np
import pytest

import modelspec_b200 as M
from modelspec_b200 import models, synthetic

pytestmark = pytest.mark.gpu

BERT = dict(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=304, seq=16, batch=8, warmup_steps=2)


def feed(gpu, k):
    for name, value in synthetic.mlm_batch(k, vocab=304, seq=16, batch=8).items():
        gpu.set_input(name, value)


@pytest.mark.parametrize("flags", [M.PLAN_DEFAULT, M.PLAN_BF16, M.PLAN_NO_GRAPH])
def test_a_rewound_run_is_the_run_that_stopped_there(device, flags):
    source = models.bert(steps=9, **BERT)
    stopped = M.Training(device, source, 64, flags)
    rewound = M.Training(device, source, 64, flags)
    try:
        for k in range(6):
            feed(stopped, k)
            stopped.step(k, 9)
        expected = stopped.checkpoint(6)
        rewound.set_replay_window(4)  # snapshots before steps 0 and 4
        for k in range(8):
            feed(rewound, k)
            rewound.step(k, 9)
        with pytest.raises(M.MsxError):
            rewound.rewind(2)  # before the last snapshot
        rewound.rewind(5)
        got = rewound.checkpoint(6)
        assert got.encode() == expected.encode(), "parameters and both moments after step 5"
        # Both go on from there alike.
        losses = []
        for run in (stopped, rewound):
            for k in range(6, 9):
                feed(run, k)
                run.step(k, 9)
                losses.append(run.loss())
            losses.append(run.final_loss())
        assert np.array(losses[:4]).tobytes() == np.array(losses[4:]).tobytes()
        got.destroy()
        expected.destroy()
    finally:
        stopped.destroy()
        rewound.destroy()


def test_a_diverged_run_is_left_as_one_step_per_submission_leaves_it(device):
    source = models.linear_regression(steps=12).replace("lr = 0.1", "lr = 3e12")
    assert "3e12" in source
    one_by_one = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    queued = M.Training(device, source, 0, M.PLAN_EXACT_MATMUL)
    try:
        one_by_one.synthetic()
        queued.synthetic()
        # One step per submission, each loss read before the next step: stops at the first bad one.
        failed = None
        for k in range(12):
            one_by_one.step(k, 12)
            try:
                one_by_one.loss()
            except M.MsxError as e:
                assert e.status == M.NON_FINITE
                failed = k
                break
        assert failed is not None and failed >= 1, "the learning rate overflows the loss within a few steps"
        expected = one_by_one.checkpoint(failed + 1)
        # Eight steps queued without a host wait, then the losses are read.
        queued.set_replay_window(8)
        for k in range(8):
            queued.step(k, 12)
        seen = None
        for k in range(8):
            try:
                queued.loss_of(k)
            except M.MsxError as e:
                assert e.status == M.NON_FINITE
                seen = k
                break
        assert seen == failed
        queued.rewind(seen)
        got = queued.checkpoint(seen + 1)
        assert got.encode() == expected.encode()
        got.destroy()
        expected.destroy()
    finally:
        one_by_one.destroy()
        queued.destroy()
