"""Op-level parity on the GPU: each Tensor IR op as a one-node program through the C ABI,
against the CPU oracle on the same seeded inputs. Integer-addressed work (gathers, ordered
scatter-adds, dropout masks) and single-rounding arithmetic must match in bits; reductions and
transcendental ops within the reference's kernel tolerance 1e-5 + 1e-4 r."""
import numpy as np
import pytest

import modelspec_b200 as M
from helpers import ProgramText, assert_bits_equal, assert_kernel_close, run_both

pytestmark = pytest.mark.gpu


def rng(seed):
    return np.random.default_rng(seed)


def values(r, *shape):
    """Seeded f32 values with a signed zero every 7th element, as the reference's device tests
    draw them (tests/common/mod.rs:124-161)."""
    x = r.standard_normal(shape).astype(np.float32)
    flat = x.reshape(-1)
    flat[::7] = 0.0
    flat[::14] = -0.0
    return x


@pytest.mark.parametrize("m,k,n", [(8, 4, 1), (64, 784, 128), (100, 37, 10), (130, 129, 67), (1, 1, 1), (5, 300, 3)])
@pytest.mark.parametrize("form", ["nn", "tn", "nt"])
def test_matmul_is_the_ascending_k_fma_chain_bit_for_bit(device, m, k, n, form):
    r = rng(m * 1000 + k * 10 + n)
    p = ProgramText()
    if form == "nn":
        a = p.input("a", "f32", [m, k]); b = p.input("b", "f32", [k, n])
        out = p.op("MatMul", [m, n], [a, b])
        feed = {"a": values(r, m, k), "b": values(r, k, n)}
    elif form == "tn":  # X^T x G: the weight gradient
        a = p.input("a", "f32", [k, m]); b = p.input("b", "f32", [k, n])
        at = p.op("Transpose", [m, k], [a])
        out = p.op("MatMul", [m, n], [at, b])
        feed = {"a": values(r, k, m), "b": values(r, k, n)}
    else:  # G x W^T: the input adjoint
        a = p.input("a", "f32", [m, k]); b = p.input("b", "f32", [n, k])
        bt = p.op("Transpose", [k, n], [b])
        out = p.op("MatMul", [m, n], [a, bt])
        feed = {"a": values(r, m, k), "b": values(r, n, k)}
    p.output(out)
    [(cpu, gpu)] = run_both(device, p.text(), feed, outputs=[(out, m * n)])
    assert_bits_equal(gpu, cpu, "matmul %s %dx%dx%d" % (form, m, k, n))


def matmul_program(form, m, k, n, r):
    p = ProgramText()
    if form == "nn":
        a = p.input("a", "f32", [m, k]); b = p.input("b", "f32", [k, n])
        out = p.op("MatMul", [m, n], [a, b])
        feed = {"a": values(r, m, k), "b": values(r, k, n)}
        am, bm = feed["a"], feed["b"]
    elif form == "tn":
        a = p.input("a", "f32", [k, m]); b = p.input("b", "f32", [k, n])
        at = p.op("Transpose", [m, k], [a])
        out = p.op("MatMul", [m, n], [at, b])
        feed = {"a": values(r, k, m), "b": values(r, k, n)}
        am, bm = feed["a"].T, feed["b"]
    elif form == "nt":
        a = p.input("a", "f32", [m, k]); b = p.input("b", "f32", [n, k])
        bt = p.op("Transpose", [k, n], [b])
        out = p.op("MatMul", [m, n], [a, bt])
        feed = {"a": values(r, m, k), "b": values(r, n, k)}
        am, bm = feed["a"], feed["b"].T
    else:  # tt
        a = p.input("a", "f32", [k, m]); b = p.input("b", "f32", [n, k])
        at = p.op("Transpose", [m, k], [a]); bt = p.op("Transpose", [k, n], [b])
        out = p.op("MatMul", [m, n], [at, bt])
        feed = {"a": values(r, k, m), "b": values(r, n, k)}
        am, bm = feed["a"].T, feed["b"].T
    p.output(out)
    return p.text(), feed, out, am, bm


@pytest.mark.parametrize("m,k,n", [(128, 32, 128), (128, 64, 64), (8, 4, 1), (64, 784, 128), (130, 129, 67), (300, 1000, 40),
                                   (832, 128, 1002), (256, 4096, 128), (70, 3003, 130), (1, 1, 1), (1300, 100, 4001), (2100, 330, 2500)])
@pytest.mark.parametrize("form", ["nn", "tn", "nt", "tt"])
def test_tensor_core_matmul_within_the_kernel_tolerance(device, m, k, n, form):
    """3xTF32 on tcgen05: every storage form, tile tails in m, n and k, unaligned rows (no
    16-byte loads), k split across CTAs, and more 128 x 128 tiles than SMs (a CTA of the persistent
    kernel then walks several, the drain of one under the k loop of the next);
    |g - c| <= 1e-5 + 1e-4 r with r = sum |a||b|."""
    r = rng(m * 7 + k * 3 + n)
    text, feed, out, am, bm = matmul_program(form, m, k, n, r)
    [(cpu, gpu)] = run_both(device, text, feed, outputs=[(out, m * n)], flags=M.PLAN_NO_GRAPH)
    terms = (np.abs(am.astype(np.float64)) @ np.abs(bm.astype(np.float64))).reshape(-1)
    assert_kernel_close(gpu, cpu, scale=terms, what="matmul_tc %s %dx%dx%d" % (form, m, k, n))
    # 3xTF32 keeps about 21 bits of every product: far inside the tolerance.
    assert np.abs(gpu.astype(np.float64) - cpu).max() <= 4e-6 * max(terms.max(), 1e-30)


@pytest.mark.parametrize("rows,h,v", [(64, 32, 50), (130, 64, 1002), (96, 128, 4099), (333, 32, 1002), (400, 16, 40001), (96, 16, 30522)])
def test_a_vocabulary_head_of_odd_width_through_padded_rows(device, rows, h, v):
    """logits = x W^T + b, cross entropy and its gradient, the bias gradient (column sums of the
    logits gradient) and both matmuls that read it, with a width that is not a multiple of 4: on
    the tensor-core path the logits and their gradient are stored with padded rows, which no
    result may show. 40,001 logits do not fit the registers of the one-read kernel and take the
    general one."""
    r = rng(rows + v)
    p = ProgramText()
    x = p.input("x", "f32", [rows, h]); w = p.input("w", "f32", [v, h]); b = p.input("b", "f32", [v])
    labels = p.input("labels", "i32", [rows]); weights = p.input("weights", "f32", [rows]); seed = p.input("seed", "f32", [])
    wt = p.op("Transpose", [h, v], [w])
    raw = p.op("MatMul", [rows, v], [x, wt])
    logits = p.op("AddRows", [rows, v], [raw, b])
    loss = p.op("CrossEntropy", [], [logits, labels, weights])
    dlogits = p.op("CrossEntropyGrad", [rows, v], [logits, labels, weights, seed])
    db = p.op("SumRows", [v], [dlogits])
    dx = p.op("MatMul", [rows, h], [dlogits, w])
    dlt = p.op("Transpose", [v, rows], [dlogits])
    dw = p.op("MatMul", [v, h], [dlt, x])
    for value in (loss, db, dx, dw):
        p.output(value)
    feed = {"x": values(r, rows, h), "w": values(r, v, h) * 0.2, "b": values(r, v) * 0.1,
            "labels": r.integers(0, v, size=rows).astype(np.int32), "weights": (r.random(rows) < 0.8).astype(np.float32),
            "seed": np.float32(1.0)}
    res = run_both(device, p.text(), feed, outputs=[(loss, 1), (db, v), (dx, rows * h), (dw, v * h)], flags=M.PLAN_NO_GRAPH)
    for (cpu, gpu), what in zip(res, ("loss", "bias gradient", "input gradient", "weight gradient")):
        assert_kernel_close(gpu, cpu, scale=np.full(cpu.shape, max(1.0, float(np.abs(cpu).max()))), what=what)


def test_weight_gradients_of_different_shapes_share_one_launch(device):
    """Matmuls tagged `gradient` whose results nothing on the device reads (weight gradients) are
    jobs of one launch: different shapes, tails in every dimension, split and unsplit k, the partial
    tiles added by the finalize launch."""
    r = rng(41)
    shapes = [(4096, 128, 128), (4096, 128, 512), (1000, 100, 40), (300, 70, 130), (64, 33, 20), (8200, 64, 64)]
    p = ProgramText()
    feed, outs, refs = {}, [], []
    for j, (k, m, n) in enumerate(shapes):
        x = p.input("x%d" % j, "f32", [k, m]); g = p.input("g%d" % j, "f32", [k, n])
        xt = p.op("Transpose", [m, k], [x], tag="gradient")
        w = p.op("MatMul", [m, n], [xt, g], tag="gradient")
        feed["x%d" % j] = values(r, k, m); feed["g%d" % j] = values(r, k, n)
        outs.append((w, m * n)); p.output(w)
        refs.append(np.abs(feed["x%d" % j].T.astype(np.float64)) @ np.abs(feed["g%d" % j].astype(np.float64)))
    listing = M.schedule_describe(p.text())
    kernels = [l.split()[1] for l in listing.strip().splitlines()[:-1]]
    assert kernels.count("matmul_jobs") == 1 and "matmul" not in kernels and kernels[-1] == "finalize_sums"
    res = run_both(device, p.text(), feed, outputs=outs, flags=M.PLAN_NO_GRAPH)
    for (cpu, gpu), terms, shape in zip(res, refs, shapes):
        assert_kernel_close(gpu, cpu, scale=terms.reshape(-1), what="weight gradient k, m, n = %r" % (shape,))


def test_transposed_matmul_result_is_the_swapped_matmul(device):
    """Transpose(MatMul(A^T, G)) is scheduled as one matmul with its operands swapped."""
    r = rng(5)
    p = ProgramText()
    a = p.input("a", "f32", [50, 12]); g = p.input("g", "f32", [50, 33])
    at = p.op("Transpose", [12, 50], [a])
    mm = p.op("MatMul", [12, 33], [at, g])
    out = p.op("Transpose", [33, 12], [mm])
    p.output(out)
    text = p.text()
    assert "transpose" not in M.schedule_describe(text)
    [(cpu, gpu)] = run_both(device, text, {"a": values(r, 50, 12), "g": values(r, 50, 33)}, outputs=[(out, 33 * 12)])
    assert_bits_equal(gpu, cpu)


@pytest.mark.parametrize("op", ["Add", "Sub", "Mul", "Div"])
@pytest.mark.parametrize("form", ["same", "scalar_right", "scalar_left"])
def test_elementwise_ops_round_once_like_the_cpu(device, op, form):
    r = rng(11)
    n = 1003
    p = ProgramText()
    a = p.input("a", "f32", [] if form == "scalar_left" else [n])
    b = p.input("b", "f32", [] if form == "scalar_right" else [n])
    out = p.op(op, [n], [a, b])
    p.output(out)
    av = r.standard_normal(1 if form == "scalar_left" else n).astype(np.float32)
    bv = (r.standard_normal(1 if form == "scalar_right" else n).astype(np.float32) + np.float32(3.0))
    [(cpu, gpu)] = run_both(device, p.text(), {"a": av, "b": bv}, outputs=[(out, n)])
    assert_bits_equal(gpu, cpu, op)


def test_relu_and_its_gradient_are_exact_and_zero_at_zero(device):
    r = rng(2)
    p = ProgramText()
    a = p.input("a", "f32", [777]); g = p.input("g", "f32", [777])
    y = p.op("Relu", [777], [a]); d = p.op("ReluGrad", [777], [a, g]); s = p.op("Sqrt", [777], [y])
    for v in (y, d, s):
        p.output(v)
    res = run_both(device, p.text(), {"a": values(r, 777), "g": values(r, 777)}, outputs=[(y, 777), (d, 777), (s, 777)])
    for cpu, gpu in res:
        assert_bits_equal(gpu, cpu)


def test_gelu_and_its_gradient_within_tolerance(device):
    r = rng(3)
    n = 4096
    p = ProgramText()
    a = p.input("a", "f32", [n]); g = p.input("g", "f32", [n])
    y = p.op("Gelu", [n], [a]); d = p.op("GeluGrad", [n], [a, g])
    p.output(y); p.output(d)
    x = (r.standard_normal(n) * 3).astype(np.float32)
    x[:8] = [-20, -10, -3, -0.0, 0.0, 3, 10, 20]
    res = run_both(device, p.text(), {"a": x, "g": values(r, n)}, outputs=[(y, n), (d, n)])
    for cpu, gpu in res:
        assert_kernel_close(gpu, cpu, what="gelu")
        assert np.abs(gpu - cpu).max() <= 4e-6 * max(1.0, np.abs(cpu).max())


def test_add_rows_transpose_and_broadcast_are_exact(device):
    r = rng(4)
    p = ProgramText()
    x = p.input("x", "f32", [37, 130]); b = p.input("b", "f32", [130]); s = p.input("s", "f32", [])
    y = p.op("AddRows", [37, 130], [x, b]); t = p.op("Transpose", [130, 37], [x])
    f = p.op("BroadcastScalar", [5, 9], [s], attr="[5, 9]")
    for v in (y, t, f):
        p.output(v)
    res = run_both(device, p.text(), {"x": values(r, 37, 130), "b": values(r, 130), "s": np.float32([2.5])},
                   outputs=[(y, 37 * 130), (t, 37 * 130), (f, 45)])
    for cpu, gpu in res:
        assert_bits_equal(gpu, cpu)


@pytest.mark.parametrize("rows,h", [(1, 5), (64, 128), (4096, 128), (833, 30), (300, 513)])
def test_sum_rows_within_tolerance(device, rows, h):
    r = rng(rows + h)
    p = ProgramText()
    g = p.input("g", "f32", [rows, h])
    out = p.op("SumRows", [h], [g])
    p.output(out)
    gv = values(r, rows, h)
    [(cpu, gpu)] = run_both(device, p.text(), {"g": gv}, outputs=[(out, h)])
    assert_kernel_close(gpu, cpu, scale=np.abs(gv).sum(axis=0), what="sum_rows")


def test_whole_tensor_sums_round_once_from_f64(device):
    r = rng(6)
    n = 70001
    p = ProgramText()
    a = p.input("a", "f32", [n]); b = p.input("b", "f32", [n])
    s = p.op("ReduceSum", [], [a]); m = p.op("ReduceMean", [], [a]); e = p.op("Mse", [], [a, b])
    for v in (s, m, e):
        p.output(v)
    res = run_both(device, p.text(), {"a": values(r, n), "b": values(r, n)}, outputs=[(s, 1), (m, 1), (e, 1)])
    for cpu, gpu in res:
        # f64 partial sums in another order: at most the last f32 bit moves.
        assert abs(float(gpu[0]) - float(cpu[0])) <= 1.2e-7 * abs(float(cpu[0])) + 1e-30


def test_embedding_gathers_rows_exactly_and_its_gradient_adds_in_ascending_order(device):
    r = rng(7)
    rows, h, n = 50, 24, 400
    ids = r.integers(0, rows, size=n).astype(np.int32)
    ids[:40] = 3  # one row hit many times: the order of the adds shows
    ids[ids == 17] = 18  # a row never read stays exactly zero
    p = ProgramText()
    table = p.input("table", "f32", [rows, h]); i = p.input("ids", "i32", [n]); g = p.input("g", "f32", [n, h])
    e = p.op("Embedding", [n, h], [table, i])
    d = p.op("EmbeddingGrad", [rows, h], [i, g], attr="[%d]" % rows)
    p.output(e); p.output(d)
    res = run_both(device, p.text(), {"table": values(r, rows, h), "ids": ids, "g": values(r, n, h)},
                   outputs=[(e, n * h), (d, rows * h)])
    for cpu, gpu in res:
        assert_bits_equal(gpu, cpu)
    assert not res[1][1].reshape(rows, h)[17].any()


@pytest.mark.parametrize("rows,h,n,hot", [(300, 128, 2000, 700), (90, 33, 900, 150), (1000, 256, 3000, 65), (64, 20, 50, 0)])
def test_embedding_gradient_of_hot_rows_and_with_a_dense_addend(device, rows, h, n, hot):
    """A row read hundreds of times (the mask token of an MLM batch) goes through the block-wide
    path; the sum stays the sequential one, bit for bit, alone and with the dense gradient of a
    tied weight added by the same launch."""
    r = rng(rows + h + n)
    ids = r.integers(0, rows, size=n).astype(np.int32)
    ids[r.permutation(n)[:hot]] = 5
    p = ProgramText()
    i = p.input("ids", "i32", [n]); g = p.input("g", "f32", [n, h]); dense = p.input("dense", "f32", [rows, h])
    d = p.op("EmbeddingGrad", [rows, h], [i, g], attr="[%d]" % rows)
    d2 = p.op("EmbeddingGrad", [rows, h], [i, g], attr="[%d]" % rows)
    tied = p.op("Add", [rows, h], [dense, d2])
    # A dense addend that a launch made and nothing else reads is stored where the sum goes: the
    # scatter then adds in place and leaves the rows no id names alone.
    made = p.op("Mul", [rows, h], [dense, dense])
    d3 = p.op("EmbeddingGrad", [rows, h], [i, g], attr="[%d]" % rows)
    in_place = p.op("Add", [rows, h], [made, d3])
    p.output(d); p.output(tied); p.output(in_place)
    listing = M.schedule_describe(p.text()).strip().splitlines()
    product = [l for l in listing if l.split()[1] == "binary"][0]
    assert product.split("writes")[1].split()[0] == "%%%d" % in_place, listing
    res = run_both(device, p.text(), {"ids": ids, "g": values(r, n, h), "dense": values(r, rows, h)},
                   outputs=[(d, rows * h), (tied, rows * h), (in_place, rows * h)])
    for cpu, gpu in res:
        assert_bits_equal(gpu, cpu)


@pytest.mark.parametrize("rows,h", [(4, 8), (37, 128), (512, 768), (65, 33)])
def test_layer_norm_and_its_gradients(device, rows, h):
    r = rng(rows * h)
    p = ProgramText()
    x = p.input("x", "f32", [rows, h]); gamma = p.input("gamma", "f32", [h]); beta = p.input("beta", "f32", [h])
    g = p.input("g", "f32", [rows, h])
    y = p.op("LayerNorm", [rows, h], [x, gamma, beta])
    dx = p.op("LayerNormGradX", [rows, h], [x, gamma, g])
    dg = p.op("LayerNormGradGamma", [h], [x, g])
    db = p.op("SumRows", [h], [g])
    for v in (y, dx, dg, db):
        p.output(v)
    feed = {"x": values(r, rows, h) * 2 + 0.5, "gamma": values(r, h) + 1, "beta": values(r, h), "g": values(r, rows, h)}
    text = p.text()
    assert M.schedule_describe(text).count("sum_rows") == 0, "the beta gradient rides with the gamma gradient"
    res = run_both(device, text, feed, outputs=[(y, rows * h), (dx, rows * h), (dg, h), (db, h)])
    assert_kernel_close(res[0][1], res[0][0], what="layer_norm")
    assert_kernel_close(res[1][1], res[1][0], scale=np.abs(res[1][0]).max(), what="layer_norm_grad_x")
    scale = np.abs(feed["g"]).sum(axis=0) * 3
    assert_kernel_close(res[2][1], res[2][0], scale=scale, what="layer_norm_grad_gamma")
    assert_kernel_close(res[3][1], res[3][0], scale=scale, what="beta gradient")


def test_softmax_and_its_gradient(device):
    r = rng(9)
    rows, k = 19, 301
    p = ProgramText()
    x = p.input("x", "f32", [rows, k]); g = p.input("g", "f32", [rows, k])
    y = p.op("Softmax", [rows, k], [x]); d = p.op("SoftmaxGrad", [rows, k], [y, g])
    p.output(y); p.output(d)
    res = run_both(device, p.text(), {"x": values(r, rows, k) * 4, "g": values(r, rows, k)}, outputs=[(y, rows * k), (d, rows * k)])
    for cpu, gpu in res:
        assert_kernel_close(gpu, cpu, scale=1.0 / k, what="softmax")


@pytest.mark.parametrize("tensor_cores", [False, True])
@pytest.mark.parametrize("batch,q_len,k_len,heads,d", [(3, 40, 40, 2, 16), (2, 128, 128, 2, 64), (2, 7, 33, 1, 8), (1, 512, 512, 1, 64)])
def test_attention_and_its_three_gradients(device, batch, q_len, k_len, heads, d, tensor_cores):
    r = rng(batch * q_len + d)
    h = heads * d
    p = ProgramText()
    q = p.input("q", "f32", [batch * q_len, h]); k = p.input("k", "f32", [batch * k_len, h])
    v = p.input("v", "f32", [batch * k_len, h]); mask = p.input("mask", "f32", [batch, k_len])
    g = p.input("g", "f32", [batch * q_len, h])
    attr = "[heads = %d]" % heads
    out = p.op("Attention", [batch * q_len, h], [q, k, v, mask], attr=attr)
    dq = p.op("AttentionGradQ", [batch * q_len, h], [q, k, v, mask, g], attr=attr)
    dk = p.op("AttentionGradK", [batch * k_len, h], [q, k, v, mask, g], attr=attr)
    dv = p.op("AttentionGradV", [batch * k_len, h], [q, k, v, mask, g], attr=attr)
    for val in (out, dq, dk, dv):
        p.output(val)
    m = np.ones((batch, k_len), dtype=np.float32)
    m[:, 1::3] = 0.0  # masked keys: exact zero rows in dK and dV
    m[0, :] = 0.0
    m[0, k_len - 1] = 1.0  # a sequence with one unmasked key
    feed = {"q": values(r, batch * q_len, h), "k": values(r, batch * k_len, h), "v": values(r, batch * k_len, h),
            "mask": m, "g": values(r, batch * q_len, h)}
    text = p.text()
    listing = M.schedule_describe(text)
    assert listing.count("attention_forward") == 1 and listing.count("attention_backward") == 1
    flags = M.PLAN_NO_GRAPH | (0 if tensor_cores else M.PLAN_EXACT_MATMUL)
    res = run_both(device, text, feed, outputs=[(out, batch * q_len * h), (dq, batch * q_len * h),
                                                 (dk, batch * k_len * h), (dv, batch * k_len * h)], flags=flags)
    for (cpu, gpu), name in zip(res, ["attention", "grad_q", "grad_k", "grad_v"]):
        assert_kernel_close(gpu, cpu, scale=np.abs(cpu).max(), what=name)
    masked_rows = np.repeat(m.reshape(-1) == 0.0, h).reshape(-1)
    for cpu, gpu in res[2:]:
        assert not gpu[masked_rows].any() and not np.signbit(gpu[masked_rows]).any(), "a masked key's row is +0"


@pytest.mark.parametrize("rows,v", [(5, 11), (64, 1000), (33, 30522), (33, 30524), (9, 16388), (7, 32768), (300, 20000)])
def test_cross_entropy_and_its_gradient(device, rows, v):
    """Rows of 16-byte pitch and more than 16,384 logits take the kernel that runs two blocks per SM
    (part of the row in shared memory); 32,768 is the longest row it holds."""
    r = rng(rows + v)
    p = ProgramText()
    x = p.input("x", "f32", [rows, v]); labels = p.input("labels", "i32", [rows]); w = p.input("w", "f32", [rows])
    one = p.node("Tensor<f32, []>", "Scalar 1.0")
    loss = p.op("CrossEntropy", [], [x, labels, w]); d = p.op("CrossEntropyGrad", [rows, v], [x, labels, w, one])
    p.output(loss); p.output(d)
    wv = (r.random(rows) < 0.6).astype(np.float32)
    wv[0] = 1.0
    feed = {"x": values(r, rows, v) * 3, "labels": r.integers(0, v, size=rows).astype(np.int32), "w": wv}
    res = run_both(device, p.text(), feed, outputs=[(loss, 1), (d, rows * v)])
    assert_kernel_close(res[0][1], res[0][0], what="cross_entropy")
    assert_kernel_close(res[1][1], res[1][0], scale=1.0 / wv.sum(), what="cross_entropy_grad")
    zero_rows = np.repeat(wv == 0.0, v)
    assert not res[1][1][zero_rows].any()


def test_cross_entropy_with_no_weight_is_zero_loss_and_zero_gradient(device):
    p = ProgramText()
    x = p.input("x", "f32", [4, 9]); labels = p.input("labels", "i32", [4]); w = p.input("w", "f32", [4])
    one = p.node("Tensor<f32, []>", "Scalar 1.0")
    loss = p.op("CrossEntropy", [], [x, labels, w]); d = p.op("CrossEntropyGrad", [4, 9], [x, labels, w, one])
    p.output(loss); p.output(d)
    res = run_both(device, p.text(), {"x": values(rng(1), 4, 9), "labels": np.zeros(4, np.int32), "w": np.zeros(4, np.float32)},
                   outputs=[(loss, 1), (d, 36)])
    assert res[0][1][0] == 0.0 and not res[1][1].any()


@pytest.mark.parametrize("p_drop", [0.1, 0.5, 0.999])
def test_dropout_mask_and_values_match_the_cpu_in_bits(device, p_drop):
    r = rng(13)
    n = 128 * 1031
    p = ProgramText()
    x = p.input("x", "f32", [128, 1031]); token = p.input("M.forward.dropout#0", "i32", [2]); g = p.input("g", "f32", [128, 1031])
    y = p.op("Dropout", [128, 1031], [x, token], attr="[p = %r, site = M.forward.dropout#0]" % p_drop)
    d = p.op("DropoutGrad", [128, 1031], [token, g], attr="[p = %r, site = M.forward.dropout#0]" % p_drop)
    p.output(y); p.output(d)
    tok = np.array([0x12345678, -5], dtype=np.int32)
    feed = {"x": values(r, 128, 1031) + 1, "M.forward.dropout#0": tok, "g": values(r, 128, 1031) + 1}
    res = run_both(device, p.text(), feed, outputs=[(y, n), (d, n)], seed=0x0123456789abcdef)
    for cpu, gpu in res:
        assert_bits_equal(gpu, cpu, "dropout p=%r" % p_drop)
    kept = (res[0][1] != 0).mean()
    assert abs(kept - (1 - p_drop)) < 0.01


@pytest.mark.parametrize("rows,h", [(64, 128), (37, 96), (130, 768), (9, 33)])
def test_a_sublayer_tail_and_the_summed_adjoint_of_its_layer_norm(device, rows, h):
    """residual + dropout(x) with the layer norm of the sum is one launch, and a chain of Adds
    that only the three gradients of a layer norm read is added inside their launch: the stored
    sum is the separate kernels' bit for bit, the layer norm and its gradients stay inside the
    kernel tolerance, and the listing shows the fused launches."""
    r = rng(rows * 3 + h)
    p = ProgramText()
    x = p.input("x", "f32", [rows, h]); res = p.input("res", "f32", [rows, h]); token = p.input("M.forward.dropout#0", "i32", [2])
    gamma = p.input("gamma", "f32", [h]); beta = p.input("beta", "f32", [h])
    ga = p.input("ga", "f32", [rows, h]); gb = p.input("gb", "f32", [rows, h]); gc = p.input("gc", "f32", [rows, h]); gd = p.input("gd", "f32", [rows, h])
    dropped = p.op("Dropout", [rows, h], [x, token], attr="[p = 0.1, site = M.forward.dropout#0]")
    total = p.op("Add", [rows, h], [res, dropped])
    y = p.op("LayerNorm", [rows, h], [total, gamma, beta])
    s1 = p.op("Add", [rows, h], [ga, gb])
    s2 = p.op("Add", [rows, h], [s1, gc])
    s3 = p.op("Add", [rows, h], [s2, gd])
    dx = p.op("LayerNormGradX", [rows, h], [total, gamma, s3])
    dg = p.op("LayerNormGradGamma", [h], [total, s3])
    db = p.op("SumRows", [h], [s3])
    for value in (total, y, dx, dg, db):
        p.output(value)
    feed = {"x": values(r, rows, h), "res": values(r, rows, h), "M.forward.dropout#0": np.array([77, -3], dtype=np.int32),
            "gamma": values(r, h) + 1, "beta": values(r, h), "ga": values(r, rows, h), "gb": values(r, rows, h),
            "gc": values(r, rows, h), "gd": values(r, rows, h)}
    listing = M.schedule_describe(p.text())
    kernels = [l.split()[1] for l in listing.strip().splitlines()[:-1]]
    assert "dropout_add_layer_norm" in kernels and "dropout" not in kernels and "binary" not in kernels
    res_ = run_both(device, p.text(), feed, outputs=[(total, rows * h), (y, rows * h), (dx, rows * h), (dg, h), (db, h)], seed=99)
    assert_bits_equal(res_[0][1], res_[0][0], "residual + dropout")
    for (cpu, gpu), what in zip(res_[1:], ("layer norm", "dx", "dgamma", "dbeta")):
        assert_kernel_close(gpu, cpu, scale=np.full(cpu.shape, max(1.0, float(np.abs(cpu).max()))), what=what)


@pytest.mark.parametrize("rows,h", [(64, 128), (37, 96), (130, 768), (9, 33)])
def test_dropout_gradients_on_either_side_of_a_layer_norm_backward(device, rows, h):
    """dropout_grad of a sum that only a layer norm's three gradients read is drawn while the
    backward launch loads the sum, and dropout_grad of the dx it writes is a second output of the
    same launch: no dropout or add launch is left, the masked dx has exactly the zeros of the
    separate kernel's (the draw is the same) and the values of dx times the scale."""
    r = rng(rows * 5 + h)
    p = ProgramText()
    x = p.input("x", "f32", [rows, h]); gamma = p.input("gamma", "f32", [h])
    t_in = p.input("M.forward.dropout#0", "i32", [2]); t_out = p.input("M.forward.dropout#1", "i32", [2])
    ga = p.input("ga", "f32", [rows, h]); gb = p.input("gb", "f32", [rows, h]); gc = p.input("gc", "f32", [rows, h])
    s1 = p.op("Add", [rows, h], [ga, gb])
    s2 = p.op("Add", [rows, h], [s1, gc])
    g = p.op("DropoutGrad", [rows, h], [t_in, s2], attr="[p = 0.1, site = M.forward.dropout#0]")
    dx = p.op("LayerNormGradX", [rows, h], [x, gamma, g])
    dg = p.op("LayerNormGradGamma", [h], [x, g])
    db = p.op("SumRows", [h], [g])
    masked = p.op("DropoutGrad", [rows, h], [t_out, dx], attr="[p = 0.25, site = M.forward.dropout#1]")
    for value in (dx, dg, db, masked):
        p.output(value)
    feed = {"x": values(r, rows, h), "gamma": values(r, h) + 1, "M.forward.dropout#0": np.array([5, 0], dtype=np.int32),
            "M.forward.dropout#1": np.array([-9, 2], dtype=np.int32), "ga": values(r, rows, h), "gb": values(r, rows, h),
            "gc": values(r, rows, h)}
    listing = M.schedule_describe(p.text())
    kernels = [l.split()[1] for l in listing.strip().splitlines()[:-1]]
    assert kernels == ["layer_norm_backward", "finalize_sums"], listing
    res = run_both(device, p.text(), feed, outputs=[(dx, rows * h), (dg, h), (db, h), (masked, rows * h)], seed=4242)
    for (cpu, gpu), what in zip(res[:3], ("dx", "dgamma", "dbeta")):
        assert_kernel_close(gpu, cpu, scale=np.full(cpu.shape, max(1.0, float(np.abs(cpu).max()))), what=what)
    cpu_masked, gpu_masked = res[3]
    gpu_dx = res[0][1]
    assert np.array_equal(cpu_masked == 0, gpu_masked == 0) or np.array_equal((cpu_masked == 0) | (res[0][0] == 0), (gpu_masked == 0) | (gpu_dx == 0))
    assert_bits_equal(gpu_masked, np.where(gpu_masked != 0, gpu_dx * np.float32(1.0 / (1.0 - 0.25)), np.float32(0)).astype(np.float32), "masked dx")
    assert abs((gpu_masked != 0).mean() - 0.75) < 0.08


@pytest.mark.parametrize("rows,h", [(64, 128), (37, 96), (130, 768), (9, 33)])
def test_sums_with_their_layer_norm_and_dropout_in_one_launch(device, rows, h):
    """a + b with the layer norm of the sum and the dropout that alone reads it (an encoder's
    embedding sum), a + b with a layer norm that something else reads too, and residual +
    dropout(x) that no layer norm follows: one launch each, sums and dropout zeros bit for bit."""
    r = rng(rows * 7 + h)
    p = ProgramText()
    a = p.input("a", "f32", [rows, h]); b = p.input("b", "f32", [rows, h]); c = p.input("c", "f32", [rows, h])
    gamma = p.input("gamma", "f32", [h]); beta = p.input("beta", "f32", [h])
    t0 = p.input("M.forward.dropout#0", "i32", [2]); t1 = p.input("M.forward.dropout#1", "i32", [2])
    s1 = p.op("Add", [rows, h], [a, b])
    n1 = p.op("LayerNorm", [rows, h], [s1, gamma, beta])
    d1 = p.op("Dropout", [rows, h], [n1, t0], attr="[p = 0.1, site = M.forward.dropout#0]")
    s2 = p.op("Add", [rows, h], [d1, c])
    n2 = p.op("LayerNorm", [rows, h], [s2, gamma, beta])
    d2 = p.op("Dropout", [rows, h], [n2, t1], attr="[p = 0.5, site = M.forward.dropout#1]")
    s3 = p.op("Add", [rows, h], [s2, d2])
    for value in (s1, d1, s2, n2, s3):
        p.output(value)
    feed = {"a": values(r, rows, h), "b": values(r, rows, h), "c": values(r, rows, h), "gamma": values(r, h) + 1, "beta": values(r, h),
            "M.forward.dropout#0": np.array([3, 1], dtype=np.int32), "M.forward.dropout#1": np.array([-2, 8], dtype=np.int32)}
    listing = M.schedule_describe(p.text())
    kernels = [l.split()[1] for l in listing.strip().splitlines()[:-1]]
    assert kernels == ["add_layer_norm_dropout", "add_layer_norm", "dropout_add"], listing
    res = run_both(device, p.text(), feed, outputs=[(s1, rows * h), (d1, rows * h), (s2, rows * h), (n2, rows * h), (s3, rows * h)], seed=31337)
    assert_bits_equal(res[0][1], res[0][0], "a + b")
    for (cpu, gpu), what in zip(res[1:], ("dropout of the layer norm", "second sum", "second layer norm", "residual + dropout")):
        assert np.array_equal(cpu == 0, gpu == 0), what
        assert_kernel_close(gpu, cpu, scale=np.full(cpu.shape, max(1.0, float(np.abs(cpu).max()))), what=what)


@pytest.mark.parametrize("world,count", [(2, 1), (2, 4099), (3, 10), (4, 100003), (8, 5), (8, 262144 + 7)])
def test_the_peer_memory_all_reduce_sums_every_slice_in_rank_order(device, world, count):
    """Every rank's launch of the gradient exchange, one after the other on one device with the
    flag words already set: each copy ends as scale x (((c0 + c1) + c2) + ...), bit for bit, ragged
    ends and slices shorter than a 16-byte group included."""
    r = rng(world * 1000 + count)
    copies = [values(r, count) for _ in range(world)]
    scale = np.float32(1.0 / world)
    after, status = device.peer_reduce_check(copies, scale=float(scale), peers_present=True)
    assert status == 0
    want = copies[0].copy()
    for c in copies[1:]:
        want = want + c
    want = want * scale
    for q in range(world):
        assert_bits_equal(after[q], want, "copy of rank %d" % q)


@pytest.mark.parametrize("count", [4096, 40000])
def test_the_peer_memory_all_reduce_gives_up_when_no_peer_arrives(device, count):
    """Rank 0's launch with no other rank running (one block, and ten blocks that all give up
    side by side): its wait ends after the limit, the copies are left alone, the status word says
    so, and the next launch on the channel returns at once."""
    import time
    r = rng(77)
    copies = [values(r, count) for _ in range(2)]
    start = time.monotonic()
    after, status = device.peer_reduce_check(copies, peers_present=False, wait_ms=200)
    elapsed = time.monotonic() - start
    assert status & 2
    assert 0.19 < elapsed < 5.0  # one wait of 200 ms, not two
    for q in range(2):
        assert_bits_equal(after[q], copies[q], "copy of rank %d" % q)


@pytest.mark.parametrize("rows,h,keep_dx", [(64, 128, False), (37, 96, True), (130, 768, False), (9, 33, True)])
def test_a_gelu_on_either_side_of_a_layer_norm(device, rows, h, keep_dx):
    """dense -> gelu -> layer norm (a masked-LM head's transform): gelu and the layer norm are one
    launch that stores both, and in the backward pass gelu_grad is applied to the layer norm's dx by
    the launch that forms it; dx itself is stored only if something else reads it."""
    r = rng(rows * 11 + h)
    p = ProgramText()
    pre = p.input("pre", "f32", [rows, h]); gamma = p.input("gamma", "f32", [h]); beta = p.input("beta", "f32", [h])
    g = p.input("g", "f32", [rows, h])
    act = p.op("Gelu", [rows, h], [pre])
    y = p.op("LayerNorm", [rows, h], [act, gamma, beta])
    dx = p.op("LayerNormGradX", [rows, h], [act, gamma, g])
    dg = p.op("LayerNormGradGamma", [h], [act, g])
    db = p.op("SumRows", [h], [g])
    dpre = p.op("GeluGrad", [rows, h], [pre, dx])
    outputs = [act, y, dg, db, dpre] + ([dx] if keep_dx else [])
    for value in outputs:
        p.output(value)
    feed = {"pre": values(r, rows, h) * 2, "gamma": values(r, h) + 1, "beta": values(r, h), "g": values(r, rows, h)}
    listing = M.schedule_describe(p.text())
    kernels = [l.split()[1] for l in listing.strip().splitlines()[:-1]]
    assert kernels == ["gelu_layer_norm", "layer_norm_backward", "finalize_sums"], listing
    backward = listing.strip().splitlines()[1]
    assert ("%%%d" % dx in backward.split("writes")[1].split()) == keep_dx, listing
    sizes = {act: rows * h, y: rows * h, dg: h, db: h, dpre: rows * h, dx: rows * h}
    res = run_both(device, p.text(), feed, outputs=[(v, sizes[v]) for v in outputs], seed=1)
    for (cpu, gpu), value in zip(res, outputs):
        assert_kernel_close(gpu, cpu, scale=np.full(cpu.shape, max(1.0, float(np.abs(cpu).max()))), what="value %d" % value)


def test_bad_inputs_are_refused_like_the_interpreter_refuses_them(device):
    p = ProgramText()
    table = p.input("table", "f32", [5, 4]); ids = p.input("ids", "i32", [3])
    e = p.op("Embedding", [3, 4], [table, ids])
    p.output(e)
    plan = M.Plan(device, p.text())
    try:
        with pytest.raises(M.MsxError) as err:
            plan.set_input("ids", np.array([0, 5, 1], dtype=np.int32))
        assert err.value.status == M.BAD_INPUT and "[1] = 5" in str(err.value)
        with pytest.raises(M.MsxError) as err:
            plan.set_input("nope", np.zeros(3, dtype=np.int32))
        assert err.value.status == M.BAD_ARGUMENT
        with pytest.raises(M.MsxError) as err:
            plan.set_input("ids", np.zeros(4, dtype=np.int32))
        assert err.value.status == M.BAD_ARGUMENT
    finally:
        plan.destroy()


def test_an_op_without_a_kernel_is_refused_at_plan_creation(device):
    text = '%0: Tensor<f32, [4, 3]> = Input "p"\n%1: Tensor<f32, [3]> = SigregColumns %0\noutput %1\n'
    with pytest.raises(M.MsxError) as err:
        M.Plan(device, text)
    assert err.value.status == M.UNSUPPORTED and "SigregColumns" in str(err.value)


def test_a_raised_status_word_is_reported_by_the_lagged_loss_read_and_step_times_add_up(device):
    """A host that reads losses a few steps behind the one it submits learns of a bounded wait
    that ran out from that read, not only from a later sync: the status word is staged with each
    step's loss. The word is set here by a memset in stream order (no kernel misbehaves)."""
    import ctypes as C
    p = ProgramText()
    a = p.input("a", "f32", [8, 4]); b = p.input("b", "f32", [8, 4])
    loss = p.op("Mse", [], [a, b])
    p.output(loss)
    plan = M.Plan(device, p.text())
    try:
        plan.set_input("a", np.ones(32, dtype=np.float32)); plan.set_input("b", np.zeros(32, dtype=np.float32))
        for _ in range(3):
            plan.run()
        assert plan.loss_of(1) == np.float32(1.0)
        times = [plan.step_ms(k) for k in range(3)]
        assert all(0.0 < t < 50.0 for t in times), times
        raise_status = M.lib().msx_internal_raise_status
        raise_status.argtypes = [C.c_void_p, C.c_uint32]
        assert raise_status(plan.h, 2) == M.OK
        plan.run()
        plan.run()
        with pytest.raises(M.MsxError) as err:
            plan.loss_of(3)
        assert err.value.status == M.TIMEOUT
        # The report cleared the word: later steps run and read normally.
        plan.run()
        assert plan.loss_of(5) == np.float32(1.0)
        plan.sync()
    finally:
        plan.destroy()
