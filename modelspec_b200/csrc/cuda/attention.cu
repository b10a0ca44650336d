// Masked multi-head attention and its three gradients, f32 SIMT.
//
// One CTA of 128 threads takes 32 query rows (forward, grad-q) or 32 key rows (grad-k/v) of one
// (sequence, head). Scores are the reference's: the dot product over the head's columns as one
// fused chain from its first product, times 1/sqrt(d)
// (crates/modelspec-runtime/src/cpu/interpreter.rs:1459-1462), so they are bit-identical to the
// CPU's. The softmax sum and the row dot are warp trees and expf is the device's: tolerance
// class, deterministic. P V, dS K, dS^T Q and P^T G accumulate over ascending key (or query)
// index as fused chains, a masked key contributing an exact zero; masked keys get +0 rows in dK
// and dV (interpreter.rs:1035-1119). The probabilities are recomputed in the backward kernels,
// never stored. grad-q writes the row statistics (max, sum, row dot) that grad-k/v reads, the
// layout the reference's Vulkan kernels share (crates/modelspec-core/src/schedule.rs:1925-1997).
//
// A row of scores lives in shared memory, which bounds the keys of a sequence at 512, the
// reference's own device limit (schedule.rs:1925).
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

constexpr int QT = 32;       // query rows (or key rows) per CTA
constexpr int KT = 64;       // keys staged per tile in the query-major kernels
constexpr int THREADS = 128;
constexpr int MAXC = 32;     // columns per thread: head_dim <= 128

struct Dims {
    uint32_t l, s, heads, d, h, dc;  // dc = columns per column group = ceil(d / 4)
    float scale;
};

__device__ __forceinline__ void load_rows(float* dst, uint32_t dst_stride, const float* __restrict__ src,
                                          uint32_t first_row, uint32_t rows, uint32_t limit, uint32_t h,
                                          uint32_t col0, uint32_t d) {
    // dst[r][c] = src[(first_row + r) * h + col0 + c], zero past `limit` rows.
    for (uint32_t idx = threadIdx.x; idx < rows * d; idx += blockDim.x) {
        uint32_t r = idx / d, c = idx % d;
        dst[r * dst_stride + c] = first_row + r < limit ? src[static_cast<uint64_t>(first_row + r) * h + col0 + c] : 0.0f;
    }
}

// Scores of the CTA's 32 queries against every key of the sequence into ss[32][s + 1]; a masked
// key (or a query row past the end) gets -inf.
__device__ __forceinline__ void scores_phase(const float* __restrict__ k, const float* __restrict__ mask,
                                             const float* qs, float* ss, float* tile, Dims dm, uint32_t seq,
                                             uint32_t col0) {
    const uint32_t qi = threadIdx.x % QT, kg = threadIdx.x / QT;  // kg uniform per warp
    const uint32_t ds = dm.d + 1, sstride = dm.s + 1;
    for (uint32_t j0 = 0; j0 < dm.s; j0 += KT) {
        __syncthreads();
        load_rows(tile, ds, k, seq * dm.s + j0, KT, seq * dm.s + dm.s, dm.h, col0, dm.d);
        __syncthreads();
        for (uint32_t jj = kg * (KT / 4); jj < (kg + 1) * (KT / 4); ++jj) {
            uint32_t j = j0 + jj;
            if (j >= dm.s) break;
            float acc = -0.0f;
            for (uint32_t c = 0; c < dm.d; ++c) acc = fmaf(qs[qi * ds + c], tile[jj * ds + c], acc);
            bool keep = mask[seq * dm.s + j] != 0.0f;
            ss[qi * sstride + j] = keep ? acc * dm.scale : -INFINITY;
        }
    }
    __syncthreads();
}

// Per row: max, sum of exp(score - max), probabilities written over the scores. Returns nothing;
// row statistics land in stat_max / stat_sum (shared, 32 floats each).
__device__ __forceinline__ void softmax_phase(float* ss, float* stat_max, float* stat_sum, Dims dm) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, sstride = dm.s + 1;
    for (uint32_t r = warp; r < QT; r += THREADS / 32) {
        float* row = ss + r * sstride;
        float m = -INFINITY;
        for (uint32_t j = lane; j < dm.s; j += 32) m = fmaxf(m, row[j]);
        m = warp_max(m);
        float t = 0.0f;
        for (uint32_t j = lane; j < dm.s; j += 32) t += row[j] == -INFINITY ? 0.0f : expf(row[j] - m);
        t = warp_sum(t);
        for (uint32_t j = lane; j < dm.s; j += 32) row[j] = row[j] == -INFINITY ? 0.0f : expf(row[j] - m) / t;
        if (lane == 0) {
            stat_max[r] = m;
            stat_sum[r] = t;
        }
    }
    __syncthreads();
}

// out[qi][c] = sum_j w[qi][j] * src[j][c] over ascending j, for the CTA's 32 queries.
__device__ __forceinline__ void weighted_rows_phase(const float* __restrict__ src, const float* ws, float* tile,
                                                    float* acc, Dims dm, uint32_t seq, uint32_t col0) {
    const uint32_t qi = threadIdx.x % QT, cg = threadIdx.x / QT;
    const uint32_t ds = dm.d + 1, sstride = dm.s + 1;
#pragma unroll
    for (int c = 0; c < MAXC; ++c) acc[c] = -0.0f;
    for (uint32_t j0 = 0; j0 < dm.s; j0 += KT) {
        __syncthreads();
        load_rows(tile, ds, src, seq * dm.s + j0, KT, seq * dm.s + dm.s, dm.h, col0, dm.d);
        __syncthreads();
        uint32_t jn = min(static_cast<uint32_t>(KT), dm.s - j0);
        for (uint32_t jj = 0; jj < jn; ++jj) {
            float w = ws[qi * sstride + j0 + jj];
#pragma unroll
            for (int c = 0; c < MAXC; ++c)
                if (static_cast<uint32_t>(c) < dm.dc && cg * dm.dc + c < dm.d)
                    acc[c] = fmaf(w, tile[jj * ds + cg * dm.dc + c], acc[c]);
        }
    }
}

// Shared memory layout of the query-major kernels, in floats:
//   qs[32][d + 1], gs[32][d + 1] (grad-q only), tile[64][d + 1], ss[32][s + 1],
//   ds2[32][s + 1] (grad-q only), stat_max[32], stat_sum[32], stat_dot[32]
__global__ void __launch_bounds__(THREADS) forward_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                           const float* __restrict__ v, const float* __restrict__ mask,
                                                           float* __restrict__ out, Dims dm) {
    extern __shared__ float smem[];
    const uint32_t ds = dm.d + 1, sstride = dm.s + 1;
    float* qs = smem;
    float* tile = qs + QT * ds;
    float* ss = tile + KT * ds;
    float* stat_max = ss + QT * sstride;
    float* stat_sum = stat_max + QT;
    const uint32_t seq = blockIdx.z, head = blockIdx.y, q0 = blockIdx.x * QT, col0 = head * dm.d;
    load_rows(qs, ds, q, seq * dm.l + q0, QT, seq * dm.l + dm.l, dm.h, col0, dm.d);
    scores_phase(k, mask, qs, ss, tile, dm, seq, col0);
    softmax_phase(ss, stat_max, stat_sum, dm);
    float acc[MAXC];
    weighted_rows_phase(v, ss, tile, acc, dm, seq, col0);
    const uint32_t qi = threadIdx.x % QT, cg = threadIdx.x / QT;
    if (q0 + qi < dm.l) {
        float* o = out + static_cast<uint64_t>(seq * dm.l + q0 + qi) * dm.h + col0;
#pragma unroll
        for (int c = 0; c < MAXC; ++c)
            if (static_cast<uint32_t>(c) < dm.dc && cg * dm.dc + c < dm.d) o[cg * dm.dc + c] = acc[c] + 0.0f;
    }
}

__global__ void __launch_bounds__(THREADS) grad_q_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                          const float* __restrict__ v, const float* __restrict__ mask,
                                                          const float* __restrict__ g, float* __restrict__ stats,
                                                          float* __restrict__ dq, Dims dm) {
    extern __shared__ float smem[];
    const uint32_t ds = dm.d + 1, sstride = dm.s + 1;
    float* qs = smem;
    float* gs = qs + QT * ds;
    float* tile = gs + QT * ds;
    float* ss = tile + KT * ds;
    float* dp = ss + QT * sstride;
    float* stat_max = dp + QT * sstride;
    float* stat_sum = stat_max + QT;
    float* stat_dot = stat_sum + QT;
    const uint32_t seq = blockIdx.z, head = blockIdx.y, q0 = blockIdx.x * QT, col0 = head * dm.d;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    load_rows(qs, ds, q, seq * dm.l + q0, QT, seq * dm.l + dm.l, dm.h, col0, dm.d);
    load_rows(gs, ds, g, seq * dm.l + q0, QT, seq * dm.l + dm.l, dm.h, col0, dm.d);
    scores_phase(k, mask, qs, ss, tile, dm, seq, col0);
    softmax_phase(ss, stat_max, stat_sum, dm);
    // dP[i][j] = g_i . v_j over the head's columns.
    {
        const uint32_t qi = threadIdx.x % QT, kg = threadIdx.x / QT;
        for (uint32_t j0 = 0; j0 < dm.s; j0 += KT) {
            __syncthreads();
            load_rows(tile, ds, v, seq * dm.s + j0, KT, seq * dm.s + dm.s, dm.h, col0, dm.d);
            __syncthreads();
            for (uint32_t jj = kg * (KT / 4); jj < (kg + 1) * (KT / 4); ++jj) {
                uint32_t j = j0 + jj;
                if (j >= dm.s) break;
                float acc = -0.0f;
                for (uint32_t c = 0; c < dm.d; ++c) acc = fmaf(gs[qi * ds + c], tile[jj * ds + c], acc);
                dp[qi * sstride + j] = acc;
            }
        }
        __syncthreads();
    }
    // Row dot D_i = sum_j P dP, then dS = P (dP - D) written over P.
    for (uint32_t r = warp; r < QT; r += THREADS / 32) {
        float t = 0.0f;
        for (uint32_t j = lane; j < dm.s; j += 32) t = fmaf(ss[r * sstride + j], dp[r * sstride + j], t);
        t = warp_sum(t);
        for (uint32_t j = lane; j < dm.s; j += 32)
            ss[r * sstride + j] = ss[r * sstride + j] * (dp[r * sstride + j] - t);
        if (lane == 0) stat_dot[r] = t;
    }
    __syncthreads();
    if (threadIdx.x < QT && q0 + threadIdx.x < dm.l) {
        uint64_t at = (static_cast<uint64_t>(seq * dm.l + q0 + threadIdx.x) * dm.heads + head) * 3;
        stats[at] = stat_max[threadIdx.x];
        stats[at + 1] = stat_sum[threadIdx.x];
        stats[at + 2] = stat_dot[threadIdx.x];
    }
    if (dq == nullptr) return;
    float acc[MAXC];
    weighted_rows_phase(k, ss, tile, acc, dm, seq, col0);
    const uint32_t qi = threadIdx.x % QT, cg = threadIdx.x / QT;
    if (q0 + qi < dm.l) {
        float* o = dq + static_cast<uint64_t>(seq * dm.l + q0 + qi) * dm.h + col0;
#pragma unroll
        for (int c = 0; c < MAXC; ++c)
            if (static_cast<uint32_t>(c) < dm.dc && cg * dm.dc + c < dm.d) o[cg * dm.dc + c] = (acc[c] + 0.0f) * dm.scale;
    }
}

// Key-major: the CTA owns 32 keys and walks the queries of the sequence in ascending tiles.
// Shared, in floats: ks[32][d+1], vs[32][d+1], qs[32][d+1], gs[32][d+1], ps[32][33], dss[32][33],
// st[32][3].
__global__ void __launch_bounds__(THREADS) grad_kv_kernel(const float* __restrict__ q, const float* __restrict__ k,
                                                           const float* __restrict__ v, const float* __restrict__ mask,
                                                           const float* __restrict__ g, const float* __restrict__ stats,
                                                           float* __restrict__ dk, float* __restrict__ dv, Dims dm) {
    extern __shared__ float smem[];
    const uint32_t ds = dm.d + 1;
    float* ks = smem;
    float* vs = ks + QT * ds;
    float* qs = vs + QT * ds;
    float* gs = qs + QT * ds;
    float* ps = gs + QT * ds;
    float* dss = ps + QT * 33;
    float* st = dss + QT * 33;
    const uint32_t seq = blockIdx.z, head = blockIdx.y, j0 = blockIdx.x * QT, col0 = head * dm.d;
    load_rows(ks, ds, k, seq * dm.s + j0, QT, seq * dm.s + dm.s, dm.h, col0, dm.d);
    load_rows(vs, ds, v, seq * dm.s + j0, QT, seq * dm.s + dm.s, dm.h, col0, dm.d);
    const uint32_t jj = threadIdx.x % QT, grp = threadIdx.x / QT;
    const bool key_ok = j0 + jj < dm.s;
    const bool keep = key_ok && mask[seq * dm.s + j0 + jj] != 0.0f;
    float acc_k[MAXC], acc_v[MAXC];
#pragma unroll
    for (int c = 0; c < MAXC; ++c) acc_k[c] = acc_v[c] = -0.0f;
    for (uint32_t i0 = 0; i0 < dm.l; i0 += QT) {
        __syncthreads();
        load_rows(qs, ds, q, seq * dm.l + i0, QT, seq * dm.l + dm.l, dm.h, col0, dm.d);
        load_rows(gs, ds, g, seq * dm.l + i0, QT, seq * dm.l + dm.l, dm.h, col0, dm.d);
        if (threadIdx.x < QT * 3) {
            uint32_t r = threadIdx.x / 3, w = threadIdx.x % 3;
            st[threadIdx.x] = i0 + r < dm.l ? stats[(static_cast<uint64_t>(seq * dm.l + i0 + r) * dm.heads + head) * 3 + w] : 0.0f;
        }
        __syncthreads();
        // P and dS of key jj against the 8 queries of this thread's group.
        for (uint32_t ii = grp * (QT / 4); ii < (grp + 1) * (QT / 4); ++ii) {
            float p = 0.0f, dsv = 0.0f;
            if (keep && i0 + ii < dm.l) {
                float sc = -0.0f, dpv = -0.0f;
                for (uint32_t c = 0; c < dm.d; ++c) {
                    sc = fmaf(qs[ii * ds + c], ks[jj * ds + c], sc);
                    dpv = fmaf(gs[ii * ds + c], vs[jj * ds + c], dpv);
                }
                p = expf(sc * dm.scale - st[ii * 3]) / st[ii * 3 + 1];
                dsv = p * (dpv - st[ii * 3 + 2]);
            }
            ps[ii * 33 + jj] = p;
            dss[ii * 33 + jj] = dsv;
        }
        __syncthreads();
        uint32_t in = min(static_cast<uint32_t>(QT), dm.l - i0);
        for (uint32_t ii = 0; ii < in; ++ii) {
            float p = ps[ii * 33 + jj], dsv = dss[ii * 33 + jj];
#pragma unroll
            for (int c = 0; c < MAXC; ++c)
                if (static_cast<uint32_t>(c) < dm.dc && grp * dm.dc + c < dm.d) {
                    acc_v[c] = fmaf(p, gs[ii * ds + grp * dm.dc + c], acc_v[c]);
                    acc_k[c] = fmaf(dsv, qs[ii * ds + grp * dm.dc + c], acc_k[c]);
                }
        }
    }
    if (!key_ok) return;
    uint64_t row = static_cast<uint64_t>(seq * dm.s + j0 + jj) * dm.h + col0;
#pragma unroll
    for (int c = 0; c < MAXC; ++c)
        if (static_cast<uint32_t>(c) < dm.dc && grp * dm.dc + c < dm.d) {
            if (dv) dv[row + grp * dm.dc + c] = keep ? acc_v[c] + 0.0f : 0.0f;
            if (dk) dk[row + grp * dm.dc + c] = keep ? (acc_k[c] + 0.0f) * dm.scale : 0.0f;
        }
}

Dims dims_of(AttentionShape sh) {
    Dims dm;
    dm.l = sh.q_len;
    dm.s = sh.k_len;
    dm.heads = sh.heads;
    dm.d = sh.head_dim;
    dm.h = sh.heads * sh.head_dim;
    dm.dc = (sh.head_dim + 3) / 4;
    // 1 / sqrt(d), each correctly rounded, as the reference computes it once per call
    // (interpreter.rs:1404-1417).
    dm.scale = 1.0f / sqrtf(static_cast<float>(sh.head_dim));
    return dm;
}

void check_shape(AttentionShape sh) {
    if (sh.k_len > 512) throw std::runtime_error("attention: more than 512 keys per sequence has no CUDA kernel");
    if (sh.head_dim > 4 * MAXC) throw std::runtime_error("attention: a head wider than 128 has no CUDA kernel");
}

template <class K> void opt_in(K kernel, size_t bytes) {
    check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)),
          "attention shared memory");
}

}  // namespace

uint64_t attention_stats_floats(AttentionShape sh) {
    return static_cast<uint64_t>(sh.batch) * sh.q_len * sh.heads * 3;
}

void attention_forward(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask,
                       float* out, AttentionShape sh) {
    check_shape(sh);
    if (sh.batch == 0 || sh.q_len == 0) return;
    Dims dm = dims_of(sh);
    size_t floats = (QT + KT) * (dm.d + 1) + QT * (dm.s + 1) + 2 * QT;
    opt_in(forward_kernel, floats * sizeof(float));
    dim3 grid((sh.q_len + QT - 1) / QT, sh.heads, sh.batch);
    forward_kernel<<<grid, THREADS, floats * sizeof(float), s>>>(q, k, v, mask, out, dm);
    check_launch("attention_forward");
}

void attention_grad_q(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask,
                      const float* g, float* stats, float* dq, AttentionShape sh) {
    check_shape(sh);
    if (sh.batch == 0 || sh.q_len == 0) return;
    Dims dm = dims_of(sh);
    size_t floats = (2 * QT + KT) * (dm.d + 1) + 2 * QT * (dm.s + 1) + 3 * QT;
    opt_in(grad_q_kernel, floats * sizeof(float));
    dim3 grid((sh.q_len + QT - 1) / QT, sh.heads, sh.batch);
    grad_q_kernel<<<grid, THREADS, floats * sizeof(float), s>>>(q, k, v, mask, g, stats, dq, dm);
    check_launch("attention_grad_q");
}

void attention_grad_kv(cudaStream_t s, const float* q, const float* k, const float* v, const float* mask,
                       const float* g, const float* stats, float* dk, float* dv, AttentionShape sh) {
    check_shape(sh);
    if (sh.batch == 0 || sh.k_len == 0) return;
    Dims dm = dims_of(sh);
    size_t floats = 4 * QT * (dm.d + 1) + 2 * QT * 33 + 3 * QT;
    opt_in(grad_kv_kernel, floats * sizeof(float));
    dim3 grid((sh.k_len + QT - 1) / QT, sh.heads, sh.batch);
    grad_kv_kernel<<<grid, THREADS, floats * sizeof(float), s>>>(q, k, v, mask, g, stats, dk, dv, dm);
    check_launch("attention_grad_kv");
}

}  // namespace k
}  // namespace msx
