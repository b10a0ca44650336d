"""The `.mspec` front door, autodiff and optimizer attachment against the reference's printed
IR, and the scheduler's launch list. No GPU."""
import os

import pytest

import modelspec_b200 as M
from modelspec_b200 import models

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def golden(name):
    return open(os.path.join(GOLDEN, name)).read()


def test_linear_regression_ir_is_the_reference_text():
    assert M.compile_mspec(models.linear_regression(), "tensor") == golden("linear_regression.tensor.ir")
    assert M.compile_mspec(models.linear_regression(), "step") == golden("linear_regression.training.ir")


def test_mnist_mlp_training_ir_is_the_reference_text():
    """Autodiff order, subgraph tags, folded constants and SGD effects of a two-layer relu net."""
    assert M.compile_mspec(models.mnist_mlp(), "step") == golden("mnist_mlp.training.ir")


def test_bert_tiny_lowers_to_the_documented_program():
    """All 104 nodes of the reference's BERT-tiny example at vocabulary 8,192, dropout sites and
    tied decoder included (website/docs/examples/bert-tiny.md of the reference)."""
    source = models.bert(vocab=8192, warmup_steps=1000, steps=10000)
    assert M.compile_mspec(source, "tensor") == golden("bert_tiny.tensor.ir")


def test_adamw_step_has_the_documented_shape():
    text = M.compile_mspec(models.bert(hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=2), "step")
    lines = text.splitlines()
    assert ("optimizer adamw lr = 0.0001 weight_decay = 0.01 beta1 = 0.9 beta2 = 0.999 eps = 1e-6 warmup_steps = 10") in lines
    for name in ("lr_t", "c1", "c2"):
        assert any(': Tensor<f32, []> = Input "optimizer.%s"' % name in l for l in lines)
    assert any('= Input "optimizer.m@BertTiny.tok_table" {' in l and " read m@BertTiny.tok_table v0}" in l for l in lines)
    assert sum(l.startswith("output ") and " moment " in l for l in lines) == 2 * 41
    ops = [l.split(" = ")[1].split()[0] for l in lines if l.startswith("optimizer %")]
    per_param = ["Input", "Input", "Mul", "Mul", "Add", "Mul", "Mul", "Mul", "Add", "Mul", "Mul", "Sqrt", "Add", "Div",
                 "Mul", "Add", "Mul", "Sub"]
    assert ops[9:9 + len(per_param)] == per_param


def test_the_masked_row_gather_reads_the_frontier_through_an_embedding():
    text = M.compile_mspec(models.bert(), "step", masked_rows=832)
    assert 'Tensor<i32, [832]> = Input "masked.rows"' in text
    assert 'Input "masked.labels.labels"' in text and 'Input "masked.weights.weights"' in text
    assert "Tensor<f32, [832, 30522]> = CrossEntropyGrad" in text
    assert "EmbeddingGrad [4096]" in text
    assert M.compile_mspec(models.bert(), "step", masked_rows=4096) == M.compile_mspec(models.bert(), "step")
    assert models.default_masked_rows(4096) == 832


def test_the_forward_program_has_no_dropout_and_no_gather():
    text = M.compile_mspec(models.bert(), "forward", masked_rows=832)
    assert "Dropout" not in text and "masked." not in text and "dropout#" not in text


def test_a_step_is_read_back_from_its_own_text():
    import oracle_lib
    text = M.compile_mspec(models.bert(hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=2), "step", 8)
    # The oracle parses and reprints through the same reader the backend uses.
    t = oracle_lib.Trainer(models.bert(hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=2), 8)
    assert t.ir("step") == text


def test_bad_source_is_refused_with_a_message():
    with pytest.raises(M.MsxError) as err:
        M.compile_mspec("model M { param w: Tensor<f32, [2]> = xavier_uniform(); }")
    assert "rank 2" in str(err.value)
    with pytest.raises(M.MsxError) as err:
        M.compile_mspec(models.linear_regression().replace("matmul(x, w)", "sigreg(x, slices = 2)"))
    assert "sigreg" in str(err.value)


def test_bert_tiny_step_schedule():
    """What the backend launches for BERT-tiny with the gather: the ungathered head is not run,
    every transpose is folded into a matmul, the three attention gradients share a launch pair,
    the query/key/value projections of a layer (and their input gradients) share a matmul launch,
    all weight gradients are jobs of one launch at the end of the backward pass, the tail of a sublayer (dropout, residual add, layer norm) is one launch, the
    sums of the projections' input gradients are formed inside the layer-norm backward that reads
    them, the bias gradients share one first-stage launch, the second stages of every column sum
    and split-k weight gradient are one launch, and the 41 AdamW updates are one launch."""
    listing = M.schedule_describe(M.compile_mspec(models.bert(), "step", masked_rows=832))
    kernels = [l.split()[1] for l in listing.strip().splitlines()[:-1]]
    assert kernels.count("adamw_multi_tensor") == 1 and kernels[-1] == "adamw_multi_tensor"
    assert "transpose" not in kernels
    assert kernels.count("attention_forward") == 2 and kernels.count("attention_backward") == 2
    # 42 products: 13 weight gradients as jobs of one launch, 4 groups of 3 (2 layers x
    # {projections, input gradients}) and 17 launches of one product.
    assert kernels.count("matmul") == 21 and kernels.count("matmul_jobs") == 1
    matmuls = [l for l in listing.strip().splitlines() if l.split()[1] == "matmul"]
    assert sum(1 for l in matmuls if l.split("writes")[1].count("%") + l.split("writes")[1].count("scratch") >= 3) == 4
    jobs = [l for l in listing.strip().splitlines() if l.split()[1] == "matmul_jobs"][0]
    assert len(jobs.split("reads")[1].split("writes")[0].split()) == 26
    # ... issued as soon as the last partial sums exist, beside the embedding gradients that follow.
    assert kernels.count("finalize_sums") == 1 and kernels[-4:] == ["finalize_sums", "embedding_grad", "embedding_grad", "adamw_multi_tensor"]
    assert "layer_norm_grad_x" not in kernels and kernels.count("layer_norm_backward") == 6
    assert kernels.count("cross_entropy_with_grad") == 1 and "cross_entropy_grad" not in kernels
    assert kernels.count("dropout_add_layer_norm") == 3 and kernels.count("sum_rows_batched") == 1
    # Only the 30,522-wide bias gradient keeps a column-sum launch of its own.
    assert kernels.count("sum_rows") == 1 and "binary" not in kernels
    # The embedding sum, its layer norm and the dropout after it are one launch; so is the last
    # sublayer's residual + dropout, which no layer norm follows (the gather does).
    assert kernels.count("add_layer_norm_dropout") == 1 and kernels.count("dropout_add") == 1
    # The head's transform: gelu and the layer norm behind it are one launch, and the gelu
    # gradient is applied to the dx of that layer norm by the backward launch that forms it.
    assert kernels.count("gelu_layer_norm") == 1 and kernels.count("gelu") == 2 and kernels.count("gelu_grad") == 2
    assert kernels.count("layer_norm") == 1
    # The dropout gradients of the backward pass are drawn inside the layer-norm backward launches:
    # on the dx that three of them write, and on the summed adjoint that the embedding's reads.
    assert kernels.count("dropout") == 1
    backward = [l for l in listing.strip().splitlines() if l.split()[1] == "layer_norm_backward"]
    assert max(len(l.split("reads")[1].split("writes")[0].split()) for l in backward) == 8  # x, four addends, gamma, token, the site's stored keep decisions
    assert sum(1 for l in backward if l.split("writes")[1].count("%") == 2) == 3
    assert sum(1 for l in backward if l.split("writes")[1].count("%") == 1) == 3  # one of them the gelu gradient alone
    assert "[4096, 30522]" not in listing
    # Launches that do not have to hold up the ones after them run beside them: the orders of the
    # three embedding gradients (from the step's first launches on), the 30,522-wide bias gradient,
    # the weight gradient of the tied table, and the two launches that carry every other weight
    # and bias gradient (issued as soon as the last adjoint they read exists), the launch that
    # finishes the deferred sums, and the position table's scatter (beside the token table's).
    beside = [l.split()[1] for l in listing.strip().splitlines() if " beside " in l]
    assert sorted(beside) == ["embedding_grad"] + ["embedding_order"] * 3 + ["finalize_sums", "matmul", "matmul_jobs", "sum_rows", "sum_rows_batched"]
    assert len(kernels) <= 58
    totals = listing.strip().splitlines()[-1]
    arena, unshared = int(totals.split()[1]), int(totals.split()[4])
    assert arena < unshared


def test_the_forward_program_schedule():
    """The dropout-free forward program (held-out loss): every residual sum shares a launch with its
    layer norm, the head's gelu with its layer norm, and nothing runs beside the main stream."""
    listing = M.schedule_describe(M.compile_mspec(models.bert(), "forward", masked_rows=832))
    kernels = [l.split()[1] for l in listing.strip().splitlines()[:-1]]
    assert kernels.count("add_layer_norm") == 5 and "binary" not in kernels and "dropout" not in kernels
    assert kernels.count("gelu_layer_norm") == 1 and "layer_norm" not in kernels and len(kernels) == 23
    assert kernels.count("cross_entropy") == 1 and "cross_entropy_with_grad" not in kernels
    assert " beside " not in listing


def test_a_dense_gradient_is_stored_where_its_scatter_adds_to_it():
    """The tied table of BERT-tiny: the head's weight-gradient product writes the slot of the
    parameter's gradient (the sum), and the token table's scatter reads and writes that slot."""
    lines = M.schedule_describe(M.compile_mspec(models.bert(), "step", masked_rows=832)).strip().splitlines()
    scatter = [l for l in lines if l.split()[1] == "embedding_grad"][-1]
    target = scatter.split("writes")[1].split()[0]
    assert target in scatter.split("reads")[1].split("writes")[0].split()
    product = [l for l in lines if l.split()[1] == "matmul" and l.split("writes")[1].split()[0] == target]
    assert len(product) == 1 and " beside " in product[0]
    # The launch the product is waited for at is that scatter.
    assert product[0].split(" beside ")[1].strip() == scatter.split(":")[0]


def test_unschedulable_programs_are_refused():
    with pytest.raises(M.MsxError) as err:
        M.schedule_describe('%0: Tensor<f32, [4, 3]> = Input "p"\n%1: Tensor<f32, [3]> = SigregColumns %0\noutput %1\n')
    assert "SigregColumns" in str(err.value)
    with pytest.raises(M.MsxError):
        M.schedule_describe("optimizer muon lr = 0.1 momentum = 0.9\n")
