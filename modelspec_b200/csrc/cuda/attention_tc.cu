// Attention and its gradients on the tensor cores: each contraction is one batched tcgen05
// matmul over every (sequence, head) (gemm_tc.cu, 3xTF32), with two row kernels between them.
//
//   forward   S = Q_h K_h^T            -> P = masked softmax(S / sqrt(d))   -> O_h = P V_h
//   backward  P as the forward left it (or computed again as above);  dP = G_h V_h^T;  dS = scale P (dP - rowsum(P dP));
//             dV_h = P^T G_h;  dQ_h = dS K_h;  dK_h = dS^T Q_h
//
// Heads are addressed in place (row pitch H, head offset a * d), so nothing is gathered or
// transposed. The score matrices [B, A, L, S] live in scratch between the launches: 4 MB per
// layer at 32 x 2 heads x 128 x 128, which stays in the 126 MB L2 between producer and consumer.
// A masked key gets probability 0, so it adds exact zeros to every sum and its dK and dV rows
// are +0, as in the reference (crates/modelspec-runtime/src/cpu/interpreter.rs:1035-1119).
// Tolerance class: 3xTF32 products, warp-tree row sums, device expf.
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

// One warp per score row: p = softmax over the unmasked keys of acc * scale, in place.
__global__ void masked_softmax_kernel(float* __restrict__ scores, const float* __restrict__ mask, uint32_t rows,
                                      uint32_t rows_per_sequence, uint32_t s, float scale) {
    uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int lane = threadIdx.x & 31;
    float* p = scores + static_cast<uint64_t>(row) * s;
    const float* m = mask + static_cast<uint64_t>(row / rows_per_sequence) * s;
    float best = -INFINITY;
    for (uint32_t j = lane; j < s; j += 32)
        if (m[j] != 0.0f) best = fmaxf(best, p[j] * scale);
    best = warp_max(best);
    float total = 0.0f;
    for (uint32_t j = lane; j < s; j += 32) {
        float e = m[j] != 0.0f ? expf(p[j] * scale - best) : 0.0f;
        p[j] = e;
        total += e;
    }
    total = warp_sum(total);
    for (uint32_t j = lane; j < s; j += 32) p[j] = p[j] / total;
}

// dS = scale * P * (dP - sum_j P dP), written over dP.
__global__ void score_grad_kernel(const float* __restrict__ p, float* __restrict__ dp, uint32_t rows, uint32_t s, float scale) {
    uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int lane = threadIdx.x & 31;
    const float* pr = p + static_cast<uint64_t>(row) * s;
    float* dr = dp + static_cast<uint64_t>(row) * s;
    float dot = 0.0f;
    for (uint32_t j = lane; j < s; j += 32) dot = fmaf(pr[j], dr[j], dot);
    dot = warp_sum(dot);
    for (uint32_t j = lane; j < s; j += 32) dr[j] = pr[j] * (dr[j] - dot) * scale;
}

struct Heads {
    uint32_t b, l, s, a, d, h;
    float scale;
    BatchedOperand q(const float* x) const { return {x, h, static_cast<uint64_t>(l) * h, d, false}; }   // [L, d] of a head, row pitch H
    BatchedOperand kv(const float* x) const { return {x, h, static_cast<uint64_t>(s) * h, d, false}; }  // [S, d]
    BatchedOperand scores(const float* x) const { return {x, s, static_cast<uint64_t>(a) * l * s, static_cast<uint64_t>(l) * s, false}; }
    uint32_t rows() const { return b * a * l; }
};

Heads heads_of(AttentionShape sh) {
    Heads hd;
    hd.b = sh.batch; hd.l = sh.q_len; hd.s = sh.k_len; hd.a = sh.heads; hd.d = sh.head_dim; hd.h = sh.heads * sh.head_dim;
    hd.scale = 1.0f / sqrtf(static_cast<float>(sh.head_dim));
    return hd;
}

BatchedOperand transposed(BatchedOperand o) {
    o.transposed = true;
    return o;
}

void probabilities(cudaStream_t s, const float* q, const float* k, const float* mask, float* p, const Heads& hd, uint32_t* status) {
    // S[i, j] = sum_c q[i, c] k[j, c]: B is the keys stored [n, k].
    matmul_tc_batched(s, hd.q(q), transposed(hd.kv(k)), hd.scores(p), hd.l, hd.s, hd.d, hd.b, hd.a, status);
    uint32_t rows = hd.rows();
    masked_softmax_kernel<<<(rows + 7) / 8, 256, 0, s>>>(p, mask, rows, hd.a * hd.l, hd.s, hd.scale);
    check_launch("attention masked_softmax");
}

}  // namespace

uint64_t attention_tc_scratch_floats(AttentionShape sh) {
    return static_cast<uint64_t>(sh.batch) * sh.heads * sh.q_len * sh.k_len;
}

void attention_tc_forward(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask, float* out,
                          float* p, AttentionShape sh, uint32_t* status) {
    if (sh.batch == 0 || sh.q_len == 0) return;
    Heads hd = heads_of(sh);
    probabilities(s, q, k, mask, p, hd, status);
    // O[i, c] = sum_j P[i, j] v[j, c]
    matmul_tc_batched(s, hd.scores(p), hd.kv(v), hd.q(out), hd.l, hd.d, hd.s, hd.b, hd.a, status);
}

void attention_tc_backward(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask, const float* g,
                           float* dq, float* dk, float* dv, float* p, float* dp, AttentionShape sh, uint32_t* status, bool p_ready) {
    if (sh.batch == 0 || sh.q_len == 0) return;
    Heads hd = heads_of(sh);
    if (!p_ready) probabilities(s, q, k, mask, p, hd, status);
    // dV[j, c] = sum_i P[i, j] g[i, c]: A is P stored [k, m].
    if (dv) matmul_tc_batched(s, transposed(hd.scores(p)), hd.q(g), hd.kv(dv), hd.s, hd.d, hd.l, hd.b, hd.a, status);
    if (!dq && !dk) return;
    // dP[i, j] = sum_c g[i, c] v[j, c]
    matmul_tc_batched(s, hd.q(g), transposed(hd.kv(v)), hd.scores(dp), hd.l, hd.s, hd.d, hd.b, hd.a, status);
    uint32_t rows = hd.rows();
    score_grad_kernel<<<(rows + 7) / 8, 256, 0, s>>>(p, dp, rows, hd.s, hd.scale);
    check_launch("attention score_grad");
    // dQ[i, c] = sum_j dS[i, j] k[j, c];  dK[j, c] = sum_i dS[i, j] q[i, c]
    if (dq) matmul_tc_batched(s, hd.scores(dp), hd.kv(k), hd.q(dq), hd.l, hd.d, hd.s, hd.b, hd.a, status);
    if (dk) matmul_tc_batched(s, transposed(hd.scores(dp)), hd.q(q), hd.kv(dk), hd.s, hd.d, hd.l, hd.b, hd.a, status);
}

// ---- mixed precision ----------------------------------------------------------------------------
// The same launches for a plan that stores activations as bf16: the products run on the bf16
// kernel (gemm_bf16.cu), scores and their adjoints are written in f32 (a scratch matrix that only
// the row kernel after it reads), and the row kernels store the probabilities and the score
// gradients as bf16 for the products that follow.

namespace {

// One warp per score row: p = softmax over the unmasked keys of scores * scale, stored as bf16.
__global__ void masked_softmax_half_kernel(const float* __restrict__ scores, const float* __restrict__ mask, bf16* __restrict__ p,
                                           uint32_t rows, uint32_t rows_per_sequence, uint32_t s, float scale) {
    uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int lane = threadIdx.x & 31;
    const float* x = scores + static_cast<uint64_t>(row) * s;
    bf16* out = p + static_cast<uint64_t>(row) * s;
    const float* m = mask + static_cast<uint64_t>(row / rows_per_sequence) * s;
    float best = -INFINITY;
    for (uint32_t j = lane; j < s; j += 32)
        if (m[j] != 0.0f) best = fmaxf(best, x[j] * scale);
    best = warp_max(best);
    float total = 0.0f;
    for (uint32_t j = lane; j < s; j += 32) total += m[j] != 0.0f ? expf(x[j] * scale - best) : 0.0f;
    total = warp_sum(total);
    for (uint32_t j = lane; j < s; j += 32) out[j] = __float2bfloat16_rn(m[j] != 0.0f ? expf(x[j] * scale - best) / total : 0.0f);
}

// dS = scale * P * (dP - sum_j P dP), stored as bf16.
__global__ void score_grad_half_kernel(const bf16* __restrict__ p, const float* __restrict__ dp, bf16* __restrict__ ds, uint32_t rows,
                                       uint32_t s, float scale) {
    uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    int lane = threadIdx.x & 31;
    const bf16* pr = p + static_cast<uint64_t>(row) * s;
    const float* dr = dp + static_cast<uint64_t>(row) * s;
    bf16* out = ds + static_cast<uint64_t>(row) * s;
    float dot = 0.0f;
    for (uint32_t j = lane; j < s; j += 32) dot = fmaf(__bfloat162float(pr[j]), dr[j], dot);
    dot = warp_sum(dot);
    for (uint32_t j = lane; j < s; j += 32) out[j] = __float2bfloat16_rn(__bfloat162float(pr[j]) * (dr[j] - dot) * scale);
}

struct HalfHeads {
    Heads hd;
    HalfMatrix q(const void* x, bool transposed = false) const { return {x, hd.h, static_cast<uint64_t>(hd.l) * hd.h, hd.d, transposed}; }
    HalfMatrix kv(const void* x, bool transposed = false) const { return {x, hd.h, static_cast<uint64_t>(hd.s) * hd.h, hd.d, transposed}; }
    HalfMatrix scores(const void* x, bool transposed = false) const {
        return {x, hd.s, static_cast<uint64_t>(hd.a) * hd.l * hd.s, static_cast<uint64_t>(hd.l) * hd.s, transposed};
    }
    HalfResult to_q(void* x) const { return {x, true, hd.h, static_cast<uint64_t>(hd.l) * hd.h, hd.d}; }
    HalfResult to_kv(void* x) const { return {x, true, hd.h, static_cast<uint64_t>(hd.s) * hd.h, hd.d}; }
    HalfResult to_scores(float* x) const { return {x, false, hd.s, static_cast<uint64_t>(hd.a) * hd.l * hd.s, static_cast<uint64_t>(hd.l) * hd.s}; }
};

void half_probabilities(cudaStream_t s, const void* q, const void* k, const float* mask, void* p, float* scores, const HalfHeads& hh,
                        uint32_t* status) {
    const Heads& hd = hh.hd;
    // S[i, j] = sum_c q[i, c] k[j, c]: B is the keys stored [n, k].
    matmul_bf16(s, hh.q(q), hh.kv(k, true), hh.to_scores(scores), hd.l, hd.s, hd.d, hd.b, hd.a, nullptr, nullptr, status);
    const uint32_t rows = hd.rows();
    masked_softmax_half_kernel<<<(rows + 7) / 8, 256, 0, s>>>(scores, mask, static_cast<bf16*>(p), rows, hd.a * hd.l, hd.s, hd.scale);
    check_launch("attention masked_softmax");
}

}  // namespace

void attention_bf16_forward(cudaStream_t s, const void* q, const void* k, const void* v, const float* mask, void* out, void* p,
                            float* scores, AttentionShape sh, uint32_t* status) {
    if (sh.batch == 0 || sh.q_len == 0) return;
    const HalfHeads hh = {heads_of(sh)};
    const Heads& hd = hh.hd;
    half_probabilities(s, q, k, mask, p, scores, hh, status);
    // O[i, c] = sum_j P[i, j] v[j, c]
    matmul_bf16(s, hh.scores(p), hh.kv(v), hh.to_q(out), hd.l, hd.d, hd.s, hd.b, hd.a, nullptr, nullptr, status);
}

void attention_bf16_backward(cudaStream_t s, const void* q, const void* k, const void* v, const float* mask, const void* g, void* dq,
                             void* dk, void* dv, void* p, void* ds, float* scores, AttentionShape sh, uint32_t* status, bool p_ready) {
    if (sh.batch == 0 || sh.q_len == 0) return;
    const HalfHeads hh = {heads_of(sh)};
    const Heads& hd = hh.hd;
    if (!p_ready) half_probabilities(s, q, k, mask, p, scores, hh, status);
    // dV[j, c] = sum_i P[i, j] g[i, c]: A is P stored [k, m].
    if (dv) matmul_bf16(s, hh.scores(p, true), hh.q(g), hh.to_kv(dv), hd.s, hd.d, hd.l, hd.b, hd.a, nullptr, nullptr, status);
    if (!dq && !dk) return;
    // dP[i, j] = sum_c g[i, c] v[j, c], in f32.
    matmul_bf16(s, hh.q(g), hh.kv(v, true), hh.to_scores(scores), hd.l, hd.s, hd.d, hd.b, hd.a, nullptr, nullptr, status);
    const uint32_t rows = hd.rows();
    score_grad_half_kernel<<<(rows + 7) / 8, 256, 0, s>>>(static_cast<const bf16*>(p), scores, static_cast<bf16*>(ds), rows, hd.s, hd.scale);
    check_launch("attention score_grad");
    // dQ[i, c] = sum_j dS[i, j] k[j, c];  dK[j, c] = sum_i dS[i, j] q[i, c]
    if (dq) matmul_bf16(s, hh.scores(ds), hh.kv(k), hh.to_q(dq), hd.l, hd.d, hd.s, hd.b, hd.a, nullptr, nullptr, status);
    if (dk) matmul_bf16(s, hh.scores(ds, true), hh.q(q), hh.to_kv(dk), hd.s, hd.d, hd.l, hd.b, hd.a, nullptr, nullptr, status);
}

}  // namespace k
}  // namespace msx
