"""Run-level parity on the GPU: whole training runs through the C ABI against the CPU oracle on
the same seed and the same batches, held to the reference's run tolerance
|g - c| <= 1e-4 + 1e-3 |c| for every loss and every parameter element
(crates/modelspec-cli/tests/common/mod.rs:24-43 of the reference), and against the reference's
recorded outputs where it has some."""
import json
import os

import numpy as np
import pytest

import modelspec_b200 as M
from modelspec_b200 import models, synthetic
from helpers import assert_run_close, train_both

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def check_run(out, what, key_bias_atol=None):
    assert np.isfinite(out["gpu_losses"]).all()
    assert_run_close(out["gpu_losses"], out["cpu_losses"], what + " losses")
    for path, g, c in zip(out["paths"], out["gpu_params"], out["cpu_params"]):
        # The exact gradient of an attention key bias is 0; what is left is rounding, so the
        # reference bounds it by the steps taken (tests/common/mod.rs:33-43).
        atol = key_bias_atol if key_bias_atol and path.endswith("_bk") else 1e-4
        assert_run_close(g, c, "%s parameter %s" % (what, path), atol=atol)


def test_linear_regression_run_matches_the_recorded_log(device):
    golden = json.load(open(os.path.join(GOLDEN, "linear_regression.losses.json")))
    out = train_both(device, models.linear_regression(), 500, synthetic=True, flags=M.PLAN_EXACT_MATMUL)
    recorded = np.array(golden["losses"], dtype=np.float32)
    assert_run_close(out["gpu_losses"], recorded, "recorded losses")
    # The matmuls are the same fused chains and SGD the same two roundings: only the f64 tree of
    # the mse can move a last bit.
    assert np.abs(out["gpu_losses"][:50] - recorded[:50]).max() <= 1e-6 * recorded[:50].max()
    assert_run_close(out["gpu_params"][0], np.array(golden["final_param"], dtype=np.float32), "final parameter")
    check_run(out, "linear regression")


def test_two_layer_relu_run_matches_the_recorded_losses(device):
    golden = json.load(open(os.path.join(GOLDEN, "two_layer_relu.losses.json")))
    out = train_both(device, models.two_layer_relu(), 200, synthetic=True, flags=M.PLAN_EXACT_MATMUL)
    assert_run_close(out["gpu_losses"], np.array(golden["losses"], dtype=np.float32), "recorded losses")
    check_run(out, "two layer relu")


def test_the_device_draws_the_same_synthetic_batch_as_the_cpu(device):
    import oracle_lib
    source = models.transformer_block(batch=2, seq=16, hidden=32, heads=2, ffn=64, layers=1)
    cpu = oracle_lib.Trainer(source)
    cpu.synthetic()
    gpu = M.Training(device, source)
    try:
        gpu.synthetic()
        n = 2 * 16 * 32
        assert np.array_equal(gpu.get_input("x", n), cpu.get_input("x", n)), "the drawn input is the same bits"
        assert np.array_equal(gpu.get_input("key_mask", 32), np.ones(32, dtype=np.float32))
        assert_run_close(gpu.get_input("y", n), cpu.get_input("y", n), "teacher target")
    finally:
        gpu.destroy()


def test_transformer_block_first_loss_is_the_recorded_one(device):
    """The reference records `step 0 loss 0.74829835` for its transformer-block example on the
    CPU (benchmarks/raw/2026-10-27-transformer-block/loss-cpu.txt)."""
    out = train_both(device, models.transformer_block(), 3, synthetic=True)
    assert abs(float(out["gpu_losses"][0]) - 0.74829835) <= 1e-4 + 1e-3 * 0.74829835
    check_run(out, "transformer block")


def test_mlp_classifier_run_with_exact_matmuls(device):
    batch = synthetic.classifier_batch()
    out = train_both(device, models.mlp_classifier(steps=60), 60, feed=lambda k: batch, flags=M.PLAN_EXACT_MATMUL)
    check_run(out, "mlp classifier")
    # Everything in this model but expf is single-rounding arithmetic in the CPU's order.
    assert np.abs(out["gpu_losses"] - out["cpu_losses"]).max() <= 5e-7
    assert out["gpu_losses"][-1] < out["gpu_losses"][0]


def test_mlp_classifier_run_on_the_tensor_cores(device):
    """SGD at lr 0.1 makes this run's loss oscillate, so the 2^-21 differences of 3xTF32 grow
    along the trajectory: the first steps are held to the run tolerance, the whole run to the
    looser bound stated for the tensor-core path, 5e-3 + 1e-2 |c|."""
    batch = synthetic.classifier_batch()
    out = train_both(device, models.mlp_classifier(steps=60), 60, feed=lambda k: batch)
    assert_run_close(out["gpu_losses"][:10], out["cpu_losses"][:10], "first losses")
    diff = np.abs(out["gpu_losses"].astype(np.float64) - out["cpu_losses"])
    assert (diff <= 5e-3 + 1e-2 * np.abs(out["cpu_losses"])).all(), diff.max()
    assert out["gpu_losses"][-1] < out["gpu_losses"][0]


def test_encoder_block_with_dropout_and_adamw_over_100_steps(device):
    """The small twin of the encoder-block configuration: dropout, attention, layer norm, gelu,
    mse and AdamW over 100 steps, the length the tolerance is stated for."""
    source = models.CONFIGS["encoder_block"]["source"](batch=2, seq=16, hidden=32, heads=2, ffn=64, steps=100)
    n = 2 * 16 * 32
    x = synthetic.normal_batch(1, n)
    y = synthetic.normal_batch(2, n)
    feed = {"x": x, "y": y, "key_mask": np.ones(32, dtype=np.float32)}
    out = train_both(device, source, 100, feed=lambda k: feed)
    check_run(out, "encoder block twin", key_bias_atol=1e-4 + 100 * 1e-3 * 1e-3)


def test_encoder_block_at_full_size(device):
    source = models.CONFIGS["encoder_block"]["source"](steps=3)
    n = 4096 * 128
    feed = {"x": synthetic.normal_batch(1, n), "y": synthetic.normal_batch(2, n), "key_mask": np.ones(4096, dtype=np.float32)}
    out = train_both(device, source, 3, feed=lambda k: feed)
    check_run(out, "encoder block", key_bias_atol=1e-4 + 3 * 1e-3 * 1e-3)


def bert_feed(vocab, seq, batch):
    return lambda k: synthetic.mlm_batch(k, vocab=vocab, seq=seq, batch=batch, mask_id=min(103, vocab - 1))


@pytest.mark.parametrize("masked_rows", [0, 64])
def test_bert_twin_over_100_steps(device, masked_rows):
    """The hidden-32 twin of BERT-tiny (the reference trains the same twin on its CPU,
    crates/modelspec-cli/tests/fixtures/bert_cpu.mspec): embeddings, tied decoder, dropout,
    weighted cross-entropy, AdamW with warm-up, with and without the masked-row gather."""
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=8, lr=3e-3,
                         warmup_steps=10, steps=100)
    out = train_both(device, source, 100, masked_rows=masked_rows, feed=bert_feed(300, 16, 8))
    check_run(out, "bert twin", key_bias_atol=1e-4 + 100 * 3e-3 * 1e-3)
    assert out["gpu_losses"][-1] < out["gpu_losses"][0]


def test_bert_tiny_at_full_size_with_the_masked_row_gather(device):
    """BERT-tiny at vocabulary 30,522 with the default gather capacity (832 rows of 4,096): the
    benchmark's workload, two steps and the final loss."""
    source = models.bert(steps=2, warmup_steps=1)
    out = train_both(device, source, 2, masked_rows=models.default_masked_rows(4096), feed=bert_feed(30522, 128, 32))
    check_run(out, "bert tiny", key_bias_atol=1e-4 + 2 * 1e-4 * 1e-3)
    stats = out["stats"]
    assert stats["arena_bytes"] < stats["unshared_bytes"], "values share storage by liveness"
    assert stats["launches_per_step"] < 200


def test_bert_mini_at_full_size(device):
    """BERT-mini (4 layers, hidden 256, 4 heads, feed-forward 1024, vocabulary 30,522, 32 x 128
    tokens, 832 gathered rows): the data-parallel configuration's per-GPU step, two steps and the
    final loss through the default tensor-core plan."""
    cfg = models.CONFIGS["bert_mini"]
    source = cfg["source"](steps=2, warmup_steps=1)
    out = train_both(device, source, 2, masked_rows=models.default_masked_rows(cfg["rows"]),
                     feed=bert_feed(cfg["vocab"], cfg["seq"], cfg["batch"]))
    check_run(out, "bert mini", key_bias_atol=1e-4 + 2 * 1e-4 * 1e-3)


def test_bert_base_shaped_twin(device):
    """The shapes of the BERT-base configuration that no smaller test meets: hidden 768 in 12
    heads of 64, feed-forward 3072, 512 keys per sequence, vocabulary 30,522 behind the gather;
    one layer and two sequences keep the CPU side to seconds."""
    source = models.bert(name="BertBase", layers=1, hidden=768, heads=12, ffn=3072, vocab=30522, seq=512, batch=2,
                         steps=2, warmup_steps=1)
    out = train_both(device, source, 2, masked_rows=models.default_masked_rows(1024), feed=bert_feed(30522, 512, 2))
    check_run(out, "bert base twin", key_bias_atol=1e-4 + 2 * 1e-4 * 1e-3)


@pytest.mark.parametrize("source,steps,kwargs", [
    (models.linear_regression(), 60, dict(synthetic=True)),
    (models.two_layer_relu(), 60, dict(synthetic=True)),
])
def test_recorded_models_on_the_tensor_cores(device, source, steps, kwargs):
    """The same runs with 3xTF32 matmuls: inside the run tolerance of the exact CPU run."""
    check_run(train_both(device, source, steps, **kwargs), "tensor-core run")


def test_exact_matmul_mode_tracks_the_cpu_more_closely(device):
    """With the exact matmul kernel the BERT twin's first-step gradients differ from the CPU's
    only through the tolerance-class row reductions and expf."""
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=8, steps=3, warmup_steps=1)
    exact = train_both(device, source, 3, masked_rows=64, feed=bert_feed(300, 16, 8), flags=M.PLAN_EXACT_MATMUL)
    check_run(exact, "exact-matmul bert twin")
    assert np.abs(exact["gpu_losses"] - exact["cpu_losses"]).max() <= 2e-6 * np.abs(exact["cpu_losses"]).max()


@pytest.mark.parametrize("flags", [M.PLAN_GUARD, M.PLAN_GUARD | M.PLAN_BF16])
def test_no_kernel_of_a_bert_step_writes_past_its_values(device, flags):
    """The BERT twin with every intermediate in storage of its own and 16 guard words behind it
    (as the reference's device tests keep after every output): five steps and the final loss,
    f32 and mixed precision, then every guard is still intact."""
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=8, steps=5, warmup_steps=1)
    out = train_both(device, source, 5, masked_rows=64, feed=bert_feed(300, 16, 8), flags=flags)
    assert np.isfinite(out["gpu_losses"]).all()
    if not flags & M.PLAN_BF16:
        check_run(out, "guarded bert twin", key_bias_atol=1e-4 + 5 * 1e-4 * 1e-3)


def test_graph_and_direct_launches_agree_in_bits(device):
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=8, steps=5, warmup_steps=1)
    runs = [train_both(device, source, 5, masked_rows=64, feed=bert_feed(300, 16, 8), flags=flags)
            for flags in (M.PLAN_DEFAULT, M.PLAN_NO_GRAPH)]
    assert np.array_equal(runs[0]["gpu_losses"], runs[1]["gpu_losses"])
    for a, b in zip(runs[0]["gpu_params"], runs[1]["gpu_params"]):
        assert np.array_equal(a, b)


def test_more_selected_rows_than_the_gather_holds_is_refused(device):
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=8, steps=5, warmup_steps=1)
    t = M.Training(device, source, masked_rows=8)
    try:
        for name, value in bert_feed(300, 16, 8)(0).items():
            t.set_input(name, value)
        with pytest.raises(M.MsxError) as err:
            t.step(0, 5)
        assert err.value.status == M.BAD_INPUT and "E-DATA-012" in str(err.value)
    finally:
        t.destroy()


def test_a_non_finite_loss_is_reported_not_trained_through(device):
    """E-TRAIN-001 without any device fault: a NaN arrives through an input, the loss and then
    the parameters turn non-finite, and the host loop says so."""
    t = M.Training(device, models.linear_regression(steps=3))
    try:
        x = np.ones(32, dtype=np.float32)
        x[5] = np.nan
        t.set_input("x", x)
        t.set_input("y", np.zeros(8, dtype=np.float32))
        t.step(0, 3)
        with pytest.raises(M.MsxError) as err:
            t.loss()
        assert err.value.status == M.NON_FINITE and "E-TRAIN-001" in str(err.value)
        with pytest.raises(M.MsxError) as err:
            t.check_finite()
        assert err.value.status == M.NON_FINITE and "LinearReg.w" in str(err.value)
    finally:
        t.destroy()


def test_stored_dropout_decisions_give_the_bits_of_drawing_them_again(device):
    """MSX_FUSE bit 64: the backward launches read the keep decisions the forward launches stored
    instead of drawing them again. Same decisions, same arithmetic: every loss and every parameter
    and moment after four steps has the same bits with the bit on and off, in both precisions."""
    import json
    import os
    import subprocess
    import sys
    here = os.path.dirname(os.path.abspath(__file__))
    results = []
    for mask in ("63", "127"):
        env = dict(os.environ, MSX_FUSE=mask, PYTHONPATH=os.pathsep.join([os.path.dirname(here), here, os.environ.get("PYTHONPATH", "")]))
        done = subprocess.run([sys.executable, os.path.join(here, "fuse_worker.py")], env=env, capture_output=True, text=True, timeout=600)
        assert done.returncode == 0, done.stderr[-2000:]
        results.append(json.loads(done.stdout.strip().splitlines()[-1]))
    for precision in ("f32", "bf16"):
        assert results[0][precision]["losses"] == results[1][precision]["losses"], precision
        assert results[0][precision]["state"] == results[1][precision]["state"], precision
