"""The mixed-precision path on the GPU: the bf16 tensor-core matmul (TMA-fed tcgen05.mma kind::f16,
f32 accumulation) through the C ABI against the CPU oracle's f32 matmul of the same bf16-valued
operands. A product of two bf16 values is exact in f32, so what differs is the order and the
rounding of the f32 accumulation: held to the kernel tolerance |g - c| <= 1e-5 + 1e-4 r with
r = sum |a||b|, and for a bf16 result to one more rounding to 8 significant bits."""
import ctypes as C

import numpy as np
import pytest

import modelspec_b200 as M
import oracle_lib
from helpers import ProgramText

pytestmark = pytest.mark.gpu


def bf16_values(torch, r, *shape):
    x = torch.from_numpy(r.standard_normal(shape).astype(np.float32)).to(torch.bfloat16)
    flat = x.reshape(-1)
    flat[::7] = 0.0
    return x


def oracle_matmul(a, b):
    m, k = a.shape
    n = b.shape[1]
    p = ProgramText()
    ia = p.input("a", "f32", [m, k]); ib = p.input("b", "f32", [k, n])
    out = p.op("MatMul", [m, n], [ia, ib])
    p.output(out)
    s = oracle_lib.Session(p.text())
    s.set_input("a", a); s.set_input("b", b)
    s.run()
    return s.value(out, m * n).reshape(m, n)


SHAPES = [(128, 64, 128), (256, 512, 256), (136, 200, 72), (16, 8, 8), (1000, 264, 520), (768, 4096, 768), (832, 128, 3000),
          (64, 72, 1048), (2048, 768, 3072)]


@pytest.mark.parametrize("m,k,n", SHAPES)
@pytest.mark.parametrize("form", ["nn", "tn", "nt", "tt"])
@pytest.mark.parametrize("half_out", [False, True])
def test_bf16_matmul_against_the_oracle(device, m, k, n, form, half_out):
    import torch
    if half_out and form in ("tn", "tt") and (m, k, n) != (136, 200, 72):
        pytest.skip("the result type does not depend on the operand form: one shape covers it")
    r = np.random.default_rng(m * 7 + k * 3 + n)
    a = bf16_values(torch, r, m, k)
    b = bf16_values(torch, r, k, n)
    a_t, b_t = form[0] == "t", form[1] == "t"
    d_a = (a.t().contiguous() if a_t else a).cuda()
    d_b = (b.t().contiguous() if b_t else b).cuda()
    d_c = torch.full((m, n), float("nan"), dtype=torch.bfloat16 if half_out else torch.float32, device="cuda")
    L = M.lib()
    need = L.msx_op_matmul_bf16_workspace(m, n, k)
    ws = torch.empty(max(need, 1), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    rc = L.msx_op_matmul_bf16(C.c_void_p(d_a.data_ptr()), int(a_t), C.c_void_p(d_b.data_ptr()), int(b_t), C.c_void_p(d_c.data_ptr()),
                              int(half_out), m, n, k, C.c_void_p(ws.data_ptr()), need, C.c_void_p(status.data_ptr()), None)
    assert rc == M.OK, L.msx_last_error(None).decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside the kernel ran out"
    got = d_c.float().cpu().numpy().astype(np.float64)
    af, bf = a.float().numpy(), b.float().numpy()
    want = oracle_matmul(af, bf)
    terms = np.abs(af.astype(np.float64)) @ np.abs(bf.astype(np.float64))
    bound = 1e-5 + 1e-4 * terms
    if half_out:
        bound = bound + np.abs(want) * 2.0 ** -8
    bad = np.abs(got - want) > bound
    assert not bad.any(), "%s %dx%dx%d: %d of %d outside the tolerance; worst %g at %s" % (
        form, m, k, n, bad.sum(), bad.size, np.abs(got - want).max(), np.unravel_index(np.abs(got - want).argmax(), got.shape))
    if not half_out:
        assert np.abs(got - want).max() <= 1e-5 * max(terms.max(), 1e-30)


def test_bf16_matmul_refuses_operands_that_tma_cannot_read(device):
    import torch
    L = M.lib()
    a = torch.zeros((16, 12), dtype=torch.bfloat16, device="cuda")   # rows of 24 bytes
    b = torch.zeros((12, 16), dtype=torch.bfloat16, device="cuda")
    c = torch.zeros((16, 16), dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = L.msx_op_matmul_bf16(C.c_void_p(a.data_ptr()), 0, C.c_void_p(b.data_ptr()), 0, C.c_void_p(c.data_ptr()), 0, 16, 16, 12,
                              None, 0, C.c_void_p(status.data_ptr()), None)
    assert rc == M.BAD_ARGUMENT and "TMA" in L.msx_last_error(None).decode()


def bert_feed(vocab, seq, batch):
    from modelspec_b200 import synthetic
    return lambda k: synthetic.mlm_batch(k, vocab=vocab, seq=seq, batch=batch, mask_id=min(103, vocab - 1))


def relative_loss_gap(out):
    g, c = out["gpu_losses"].astype(np.float64), out["cpu_losses"].astype(np.float64)
    return float(np.max(np.abs(g - c) / np.abs(c)))


# The stated bound of the mixed-precision path against the f32 CPU run: every loss within 2 % over
# 100 steps of the BERT twin (activations carry 8 significant bits; the reference's f32 run
# tolerance 1e-4 + 1e-3 |c| does not apply to a 16-bit storage type).
BF16_LOSS_RTOL = 2e-2


@pytest.mark.parametrize("masked_rows", [0, 64])
def test_bf16_bert_twin_over_100_steps_tracks_the_f32_cpu_run(device, masked_rows):
    from helpers import train_both
    from modelspec_b200 import models
    source = models.bert(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=300, seq=16, batch=8, lr=3e-3, warmup_steps=10, steps=100)
    out = train_both(device, source, 100, masked_rows=masked_rows, feed=bert_feed(300, 16, 8), flags=M.PLAN_BF16)
    assert np.isfinite(out["gpu_losses"]).all()
    gap = relative_loss_gap(out)
    assert gap <= BF16_LOSS_RTOL, "worst relative loss difference %g" % gap
    assert out["gpu_losses"][-1] < 0.8 * out["gpu_losses"][0], "the bf16 run trains"
    # Parameters are f32 masters: after 100 steps they sit near the CPU's (a loose, stated bound).
    for path, g, c in zip(out["paths"], out["gpu_params"], out["cpu_params"]):
        scale = max(float(np.abs(c).max()), 1e-3)
        assert float(np.abs(g - c).max()) <= 0.15 * scale + 0.05, path


def test_bf16_bert_base_shaped_twin(device):
    """Hidden 768 in 12 heads of 64, feed-forward 3072, 512 keys, vocabulary 30,522 behind the
    gather (logits rows padded from 30,522 to 30,528 bf16 elements): the shapes of the
    configuration the mixed-precision path exists for, two steps and the final loss."""
    from helpers import train_both
    from modelspec_b200 import models
    source = models.bert(name="BertBase", layers=1, hidden=768, heads=12, ffn=3072, vocab=30522, seq=512, batch=2, steps=2, warmup_steps=1)
    out = train_both(device, source, 2, masked_rows=models.default_masked_rows(1024), feed=bert_feed(30522, 512, 2), flags=M.PLAN_BF16)
    assert np.isfinite(out["gpu_losses"]).all()
    assert relative_loss_gap(out) <= BF16_LOSS_RTOL


def test_bf16_plan_refuses_what_it_has_no_kernel_for(device):
    """An op without a bf16 kernel is a plan-creation error, as an op without any kernel is."""
    p = ProgramText()
    a = p.input("a", "f32", [16, 8]); b = p.input("b", "f32", [16, 8])
    c = p.op("Add", [16, 8], [a, b])
    d = p.op("Softmax", [16, 8], [c])
    p.output(p.op("ReduceSum", [], [d]))
    with pytest.raises(M.MsxError) as err:
        M.Plan(device, p.text(), flags=M.PLAN_BF16)
    assert err.value.status == M.UNSUPPORTED and "bf16" in str(err.value)
    with pytest.raises(M.MsxError) as err:
        M.Plan(device, p.text(), flags=M.PLAN_BF16 | M.PLAN_EXACT_MATMUL)
    assert err.value.status == M.BAD_ARGUMENT


@pytest.mark.parametrize("batch,seq,heads,d", [(2, 128, 2, 64), (1, 512, 3, 64), (2, 200, 2, 32), (3, 16, 2, 16), (1, 384, 1, 64)])
def test_fused_attention_and_its_gradients_against_the_oracle(device, batch, seq, heads, d):
    """Attention and AttentionGradQ/K/V as the two fused kernels, on bf16-valued q, k, v, g with a
    few keys masked out, against the oracle's f32 ops on the same values. Probabilities and score
    gradients pass through bf16 (8 significant bits) on their way to the tensor core and the
    results are stored as bf16: every element within 2 % of its tensor's largest magnitude."""
    import torch
    r = np.random.default_rng(batch * 1000 + seq + heads + d)
    h, rows = heads * d, batch * seq
    t = {name: torch.from_numpy(r.standard_normal((rows, h)).astype(np.float32)).to(torch.bfloat16) for name in "qkvg"}
    mask = np.ones((batch, seq), dtype=np.float32)
    mask[0, seq - 3:] = 0.0
    if seq > 130:
        mask[batch - 1, 125:131] = 0.0
    p = ProgramText()
    ids = {name: p.input(name, "f32", [rows, h]) for name in "qkvg"}
    im = p.input("mask", "f32", [batch, seq])
    attr = "[heads = %d]" % heads
    out = p.op("Attention", [rows, h], [ids["q"], ids["k"], ids["v"], im], attr)
    grads = [p.op(op, [rows, h], [ids["q"], ids["k"], ids["v"], im, ids["g"]], attr) for op in ("AttentionGradQ", "AttentionGradK", "AttentionGradV")]
    for value in [out] + grads:
        p.output(value)
    session = oracle_lib.Session(p.text())
    for name in "qkvg":
        session.set_input(name, t[name].float().numpy())
    session.set_input("mask", mask)
    session.run()
    want = [session.value(v, rows * h).reshape(rows, h) for v in [out] + grads]

    d_in = {name: t[name].cuda() for name in "qkvg"}
    d_mask = torch.from_numpy(mask).cuda()
    d_out = [torch.full((rows, h), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(4)]
    stats = torch.zeros(rows * heads * 2, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ptr = lambda x: C.c_void_p(x.data_ptr())
    rc = M.lib().msx_op_attention_bf16(ptr(d_in["q"]), ptr(d_in["k"]), ptr(d_in["v"]), ptr(d_mask), ptr(d_in["g"]), ptr(d_out[0]), ptr(d_out[1]),
                                       ptr(d_out[2]), ptr(d_out[3]), ptr(stats), batch, seq, seq, heads, d, ptr(status), None)
    assert rc == M.OK, M.lib().msx_last_error(None).decode()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "a bounded wait inside a kernel ran out"
    for name, got, c in zip(("out", "dq", "dk", "dv"), d_out, want):
        got = got.float().cpu().numpy().astype(np.float64)
        assert np.isfinite(got).all(), name
        worst = float(np.abs(got - c).max())
        assert worst <= 2e-2 * float(np.abs(c).max()), "%s: worst |g - c| = %g, largest |c| = %g" % (name, worst, np.abs(c).max())
    # A masked key takes no part: its dK and dV rows are zeros.
    dk = d_out[2].float().cpu().numpy()
    assert not dk[seq - 3:seq].any()
