// Row kernels: layer_norm and its two gradients, softmax and its gradient, cross_entropy and its
// gradient. One warp per row for hidden-size rows, one block per row for vocabulary-size rows;
// row reductions are warp-shuffle trees, so sums round in another order than the reference's
// ascending-column loops (crates/modelspec-runtime/src/cpu/interpreter.rs:970-1034, :1172-1233,
// :1513-1527): tolerance class, deterministic. The per-element formulas keep the reference's
// operation order. All are HBM-bound; a row is read from L1/L2 on its second and third pass.
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

uint32_t sum_rows_chunks(uint64_t rows);

namespace {

#ifndef MSX_LN_BACKWARD_WIDE_BLOCKS
#define MSX_LN_BACKWARD_WIDE_BLOCKS 296
#endif
#ifndef MSX_LN_BACKWARD_BLOCKS
#define MSX_LN_BACKWARD_BLOCKS 592
#endif
constexpr float kLayerNormEps = 1e-12f;
constexpr int kWarpsPerBlock = 8;

__device__ __forceinline__ void row_moments(const float* __restrict__ row, uint32_t h, int lane,
                                            float* mean, float* rstd) {
    float s = 0.0f;
    for (uint32_t j = lane; j < h; j += 32) s += row[j];
    float m = warp_sum(s) / static_cast<float>(h);
    float q = 0.0f;
    for (uint32_t j = lane; j < h; j += 32) {
        float d = row[j] - m;
        q = fmaf(d, d, q);
    }
    float variance = warp_sum(q) / static_cast<float>(h);
    *mean = m;
    *rstd = 1.0f / sqrtf(variance + kLayerNormEps);
}

__global__ void layer_norm_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                  const float* __restrict__ beta, float* __restrict__ out, uint32_t rows,
                                  uint32_t h) {
    int lane = threadIdx.x & 31;
    uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* row = x + static_cast<uint64_t>(r) * h;
    float mean, rstd;
    row_moments(row, h, lane, &mean, &rstd);
    float* o = out + static_cast<uint64_t>(r) * h;
    for (uint32_t j = lane; j < h; j += 32) o[j] = (row[j] - mean) * rstd * gamma[j] + beta[j];
}

__global__ void layer_norm_grad_x_kernel(const float* __restrict__ x, const float* __restrict__ gamma,
                                         const float* __restrict__ g, float* __restrict__ out, uint32_t rows,
                                         uint32_t h) {
    int lane = threadIdx.x & 31;
    uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const float* row = x + static_cast<uint64_t>(r) * h;
    const float* grow = g + static_cast<uint64_t>(r) * h;
    float mean, rstd;
    row_moments(row, h, lane, &mean, &rstd);
    float s1 = 0.0f, s2 = 0.0f;
    for (uint32_t j = lane; j < h; j += 32) {
        float gx = grow[j] * gamma[j];
        float xhat = (row[j] - mean) * rstd;
        s1 += gx;
        s2 = fmaf(gx, xhat, s2);
    }
    float width = static_cast<float>(h);
    float mean_gx = warp_sum(s1) / width, mean_gx_xhat = warp_sum(s2) / width;
    float* o = out + static_cast<uint64_t>(r) * h;
    for (uint32_t j = lane; j < h; j += 32) {
        float gx = grow[j] * gamma[j];
        float xhat = (row[j] - mean) * rstd;
        o[j] = rstd * ((gx - mean_gx) - xhat * mean_gx_xhat);
    }
}

__global__ void row_stats_kernel(const float* __restrict__ x, float* __restrict__ stats, uint32_t rows,
                                 uint32_t h) {
    int lane = threadIdx.x & 31;
    uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    float mean, rstd;
    row_moments(x + static_cast<uint64_t>(r) * h, h, lane, &mean, &rstd);
    if (lane == 0) {
        stats[2 * r] = mean;
        stats[2 * r + 1] = rstd;
    }
}

// Block (32, 8) over a 32-column tile and a chunk of rows: partial column sums of g * xhat and,
// when wanted, of g.
__global__ void grad_gamma_stage1(const float* __restrict__ x, const float* __restrict__ g,
                                  const float* __restrict__ stats, uint32_t rows, uint32_t h,
                                  uint32_t rows_per_chunk, float* __restrict__ partial_gamma,
                                  float* __restrict__ partial_beta) {
    __shared__ float sg[8][32], sb[8][32];
    uint32_t c = blockIdx.x * 32 + threadIdx.x;
    uint32_t r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
    float acc_g = 0.0f, acc_b = 0.0f;
    if (c < h)
        for (uint32_t r = r0 + threadIdx.y; r < r1; r += 8) {
            float gv = g[static_cast<uint64_t>(r) * h + c];
            float xhat = (x[static_cast<uint64_t>(r) * h + c] - stats[2 * r]) * stats[2 * r + 1];
            acc_g = fmaf(gv, xhat, acc_g);
            acc_b += gv;
        }
    sg[threadIdx.y][threadIdx.x] = acc_g;
    sb[threadIdx.y][threadIdx.x] = acc_b;
    __syncthreads();
    if (threadIdx.y == 0 && c < h) {
        float tg = sg[0][threadIdx.x], tb = sb[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < 8; ++w) {
            tg += sg[w][threadIdx.x];
            tb += sb[w][threadIdx.x];
        }
        partial_gamma[static_cast<uint64_t>(blockIdx.y) * h + c] = tg;
        if (partial_beta) partial_beta[static_cast<uint64_t>(blockIdx.y) * h + c] = tb;
    }
}

__global__ void grad_gamma_stage2(const float* __restrict__ partial_gamma, const float* __restrict__ partial_beta,
                                  uint32_t chunks, uint32_t h, float* __restrict__ dgamma,
                                  float* __restrict__ dbeta) {
    uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= h) return;
    float tg = partial_gamma[c];
    for (uint32_t k = 1; k < chunks; ++k) tg += partial_gamma[static_cast<uint64_t>(k) * h + c];
    dgamma[c] = tg;
    if (dbeta) {
        float tb = partial_beta[c];
        for (uint32_t k = 1; k < chunks; ++k) tb += partial_beta[static_cast<uint64_t>(k) * h + c];
        dbeta[c] = tb;
    }
}

constexpr int kRowThreads = 256;

// Max of the row (the first element, replaced only by a greater one: NaN never wins) and the sum
// of exp(x - max), by a block.
template <class T>
__device__ __forceinline__ void block_row_softmax(const T* __restrict__ row, uint32_t v, float* shared,
                                                  float* max, float* total) {
    float m = -INFINITY;
    for (uint32_t c = threadIdx.x; c < v; c += blockDim.x) {
        float x = load1(row + c);
        if (x > m) m = x;
    }
    m = block_max(m, shared);
    float s = 0.0f;
    for (uint32_t c = threadIdx.x; c < v; c += blockDim.x) s += expf(load1(row + c) - m);
    *max = m;
    *total = block_sum(s, shared);
}

__global__ void softmax_kernel(const float* __restrict__ x, float* __restrict__ out, uint32_t k) {
    __shared__ float shared[33];
    const float* row = x + static_cast<uint64_t>(blockIdx.x) * k;
    float max, total;
    block_row_softmax(row, k, shared, &max, &total);
    float* o = out + static_cast<uint64_t>(blockIdx.x) * k;
    for (uint32_t c = threadIdx.x; c < k; c += blockDim.x) o[c] = expf(row[c] - max) / total;
}

__global__ void softmax_grad_kernel(const float* __restrict__ y, const float* __restrict__ g,
                                    float* __restrict__ out, uint32_t k) {
    __shared__ float shared[33];
    const float* yr = y + static_cast<uint64_t>(blockIdx.x) * k;
    const float* gr = g + static_cast<uint64_t>(blockIdx.x) * k;
    float acc = 0.0f;
    for (uint32_t c = threadIdx.x; c < k; c += blockDim.x) acc = fmaf(gr[c], yr[c], acc);
    float d = block_sum(acc, shared);
    float* o = out + static_cast<uint64_t>(blockIdx.x) * k;
    for (uint32_t c = threadIdx.x; c < k; c += blockDim.x) o[c] = yr[c] * (gr[c] - d);
}

template <class T>
__global__ void cross_entropy_rows_kernel(const T* __restrict__ logits, const int32_t* __restrict__ labels,
                                          const float* __restrict__ weights, float* __restrict__ row_loss,
                                          uint32_t v, uint32_t ld) {
    __shared__ float shared[33];
    uint32_t r = blockIdx.x;
    // A row of weight 0 adds w * l = 0 to the loss whatever its logits: skip its passes.
    if (weights[r] == 0.0f) {
        if (threadIdx.x == 0) row_loss[r] = 0.0f;
        return;
    }
    const T* row = logits + static_cast<uint64_t>(r) * ld;
    float max, total;
    block_row_softmax(row, v, shared, &max, &total);
    if (threadIdx.x == 0) {
        int32_t label = labels[r];
        float picked = (label >= 0 && static_cast<uint32_t>(label) < v) ? load1(row + label) : 0.0f;
        row_loss[r] = max + logf(total) - picked;
    }
}

// loss = sum_n w[n] l[n] / sum_n w[n], both sums in f64 (a tree over the block), one rounding.
__global__ void cross_entropy_loss_kernel(const float* __restrict__ row_loss, const float* __restrict__ weights,
                                          uint32_t rows, const float* __restrict__ global_den, float* __restrict__ loss) {
    __shared__ double shared[33];
    double num = 0.0, den = 0.0;
    for (uint32_t r = threadIdx.x; r < rows; r += blockDim.x) {
        double w = static_cast<double>(weights[r]);
        num = fma(w, static_cast<double>(row_loss[r]), num);
        den += w;
    }
    num = block_sum(num, shared);
    den = block_sum(den, shared);
    // Data parallel: the numerator of this shard over the weight sum of the whole batch.
    if (global_den) den = static_cast<double>(global_den[0]);
    if (threadIdx.x == 0) loss[0] = den == 0.0 ? 0.0f : static_cast<float>(num / den);
}

__global__ void weight_sum_kernel(const float* __restrict__ weights, uint32_t rows, float* __restrict__ out) {
    __shared__ double shared[33];
    double den = 0.0;
    for (uint32_t r = threadIdx.x; r < rows; r += blockDim.x) den += static_cast<double>(weights[r]);
    den = block_sum(den, shared);
    if (threadIdx.x == 0) out[0] = static_cast<float>(den);
}

__global__ void cross_entropy_grad_kernel(const float* __restrict__ logits, const int32_t* __restrict__ labels,
                                          const float* __restrict__ weights, const float* __restrict__ g,
                                          const float* __restrict__ denominator, float* __restrict__ out,
                                          uint32_t v, uint32_t ld, uint32_t ld_out) {
    __shared__ float shared[33];
    uint32_t r = blockIdx.x;
    float* o = out + static_cast<uint64_t>(r) * ld_out;
    float den = denominator[0], w = weights[r];
    if (den == 0.0f || w == 0.0f) {
        for (uint32_t c = threadIdx.x; c < v; c += blockDim.x) o[c] = 0.0f;
        return;
    }
    const float* row = logits + static_cast<uint64_t>(r) * ld;
    float max, total;
    block_row_softmax(row, v, shared, &max, &total);
    float scale = g[0] * w / den;
    uint32_t label = static_cast<uint32_t>(labels[r]);
    for (uint32_t c = threadIdx.x; c < v; c += blockDim.x) {
        float target = c == label ? 1.0f : 0.0f;
        o[c] = scale * (expf(row[c] - max) / total - target);
    }
}

// Loss row and gradient row in one visit of the logits row: max, sum of exp, then
// scale * (p - onehot) while the row is still in cache. The same formulas, in the same order, as
// the two separate kernels.
template <class T>
__global__ void cross_entropy_fused_kernel(const T* __restrict__ logits, const int32_t* __restrict__ labels,
                                           const float* __restrict__ weights, const float* __restrict__ g,
                                           const float* __restrict__ denominator, float* __restrict__ row_loss,
                                           T* __restrict__ out, uint32_t v, uint32_t ld, uint32_t ld_out) {
    __shared__ float shared[33];
    uint32_t r = blockIdx.x;
    T* o = out + static_cast<uint64_t>(r) * ld_out;
    float den = denominator[0], w = weights[r];
    if (w == 0.0f) {
        if (threadIdx.x == 0) row_loss[r] = 0.0f;
        for (uint32_t c = threadIdx.x; c < v; c += blockDim.x) store1(o + c, 0.0f);
        return;
    }
    const T* row = logits + static_cast<uint64_t>(r) * ld;
    float max, total;
    block_row_softmax(row, v, shared, &max, &total);
    uint32_t label = static_cast<uint32_t>(labels[r]);
    if (threadIdx.x == 0) row_loss[r] = max + logf(total) - (label < v ? load1(row + label) : 0.0f);
    if (den == 0.0f) {
        for (uint32_t c = threadIdx.x; c < v; c += blockDim.x) store1(o + c, 0.0f);
        return;
    }
    float scale = g[0] * w / den;
    for (uint32_t c = threadIdx.x; c < v; c += blockDim.x) {
        float target = c == label ? 1.0f : 0.0f;
        store1(o + c, scale * (expf(load1(row + c) - max) / total - target));
    }
}

// The same, for rows of up to 32 * 1024 logits, with the row held in registers: one read of the
// logits from memory (every load of the row in flight at once), one write of the gradient, and
// each exp computed once, by the hardware exponential (relative error about 2^-21, far inside the
// tolerance class every exp-based kernel is in), with one reciprocal of the row sum instead of a
// division per element: 30,522 exps and divisions per row are otherwise as long as the row's
// memory traffic.
// VEC = 4 reads and writes 16 bytes per thread (row pitches that are multiples of 4 floats).
constexpr int kWideThreads = 1024, kWideItems = 32;
template <int VEC, class T>
__global__ void __launch_bounds__(kWideThreads, 1)
cross_entropy_fused_wide_kernel(const T* __restrict__ logits, const int32_t* __restrict__ labels,
                                const float* __restrict__ weights, const float* __restrict__ g,
                                const float* __restrict__ denominator, float* __restrict__ row_loss,
                                T* __restrict__ out, uint32_t v, uint32_t ld, uint32_t ld_out,
                                uint32_t* __restrict__ counter, float* __restrict__ loss) {
    // Element i of this thread is column column_of(i): consecutive threads take consecutive
    // (groups of VEC) columns.
    auto column_of = [](int i, uint32_t tid) { return (static_cast<uint32_t>(i / VEC) * kWideThreads + tid) * VEC + i % VEC; };
    __shared__ float shared[33];
    __shared__ double shared64[33];
    __shared__ bool is_last;
    const uint32_t r = blockIdx.x, tid = threadIdx.x, rows = gridDim.x;
    T* o = out + static_cast<uint64_t>(r) * ld_out;
    // The weight sum: given (the whole batch's, data parallel), or summed here by every block in
    // the same order (f64 over the block, one rounding), so that no launch has to precede this one.
    float den;
    if (denominator != nullptr) {
        den = denominator[0];
    } else {
        double sum = 0.0;
        for (uint32_t j = tid; j < rows; j += kWideThreads) sum += static_cast<double>(weights[j]);
        den = static_cast<float>(block_sum(sum, shared64));
    }
    const float w = weights[r];
    float x[kWideItems];
    float total = 0.0f;
    uint32_t label = 0;
    if (w == 0.0f) {
        if (tid == 0) row_loss[r] = 0.0f;
    } else {
        const T* row = logits + static_cast<uint64_t>(r) * ld;
        if (VEC == 4) {
            // Unconditional loads from a clamped column (the pitch covers the whole float4 of the
            // last valid column), so that all eight are in flight together; what lies past v is
            // replaced afterwards.
            const uint32_t last = (v - 1) & ~3u;
#pragma unroll
            for (int i = 0; i < kWideItems; i += 4) {
                const float4 f = load4(row + min(column_of(i, tid), last));
                x[i] = f.x; x[i + 1] = f.y; x[i + 2] = f.z; x[i + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < kWideItems; ++i) x[i] = load1(row + min(column_of(i, tid), v - 1));
        }
#pragma unroll
        for (int i = 0; i < kWideItems; ++i)
            if (column_of(i, tid) >= v) x[i] = -INFINITY;
        float m = -INFINITY;
#pragma unroll
        for (int i = 0; i < kWideItems; ++i)
            if (x[i] > m) m = x[i];
        m = block_max(m, shared);
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < kWideItems; ++i) {
            const uint32_t c = column_of(i, tid);
            if (c < v) {
                x[i] = __expf(x[i] - m);
                sum += x[i];
            }
        }
        total = block_sum(sum, shared);
        label = static_cast<uint32_t>(labels[r]);
        if (tid == 0) row_loss[r] = m + logf(total) - (label < v ? load1(row + label) : 0.0f);
    }
    // The loss, by the last block to get here: sum of w * l over sum of w, f64 sums, one rounding.
    // Only thread 0's row loss has to be visible to that block, so only thread 0 fences, and the
    // gradient stores below are not waited for: they drain while the SM's next block loads.
    if (tid == 0) {
        __threadfence();
        const uint32_t before = atomicAdd(counter, 1u);
        is_last = before + 1u == rows;
        if (is_last) *counter = 0u;
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        double num = 0.0, den64 = 0.0;
        for (uint32_t j = tid; j < rows; j += kWideThreads) {
            double wj = static_cast<double>(weights[j]);
            num = fma(wj, static_cast<double>(__ldcg(row_loss + j)), num);
            den64 += wj;
        }
        num = block_sum(num, shared64);
        den64 = block_sum(den64, shared64);
        if (denominator != nullptr) den64 = static_cast<double>(denominator[0]);
        if (tid == 0) loss[0] = den64 == 0.0 ? 0.0f : static_cast<float>(num / den64);
    }
    const bool zero = den == 0.0f || w == 0.0f;
    const float scale = zero ? 0.0f : g[0] * w / den;
    const float inverse = zero ? 0.0f : 1.0f / total;
#pragma unroll
    for (int i = 0; i < kWideItems; ++i) {
        const uint32_t c = column_of(i, tid);
        const float target = c == label ? 1.0f : 0.0f;
        x[i] = zero ? 0.0f : scale * (x[i] * inverse - target);
    }
    if (VEC == 4) {
#pragma unroll
        for (int i = 0; i < kWideItems; i += 4) {
            const uint32_t c = column_of(i, tid);
            // Columns past v inside the pitch are padding nobody reads: the whole float4 is written.
            if (c < v) store4(o + c, make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]));
        }
    } else {
#pragma unroll
        for (int i = 0; i < kWideItems; ++i) {
            const uint32_t c = column_of(i, tid);
            if (c < v) store1(o + c, x[i]);
        }
    }
}

inline uint32_t warp_row_blocks(uint64_t rows) { return static_cast<uint32_t>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock); }

// The same for rows of 16-byte pitch, as two blocks per SM: 512 threads hold 32 elements each in
// registers and up to 32 more in shared memory (64 KB a block), so that one block's loads and
// stores run under the other's reductions and exponentials. Elements bound for shared memory go
// there straight from global memory (cp.async, 16 bytes), all in flight with the register loads;
// every thread reads back only what it copied itself.
constexpr int kSplitThreads = 512, kSplitRegisterItems = 32, kSplitSharedItems = 32;
constexpr int kSplitSharedBytes = kSplitSharedItems * kSplitThreads * 4;
__global__ void __launch_bounds__(kSplitThreads, 2)
cross_entropy_fused_split_kernel(const float* __restrict__ logits, const int32_t* __restrict__ labels,
                                 const float* __restrict__ weights, const float* __restrict__ g,
                                 const float* __restrict__ denominator, float* __restrict__ row_loss,
                                 float* __restrict__ out, uint32_t v, uint32_t ld, uint32_t ld_out,
                                 uint32_t* __restrict__ counter, float* __restrict__ loss) {
    // Group k of this thread is the four columns from (k * 512 + tid) * 4 on: groups 0..7 live in
    // registers, groups 8..15 in shared memory.
    extern __shared__ float4 parked[];  // [kSplitSharedItems / 4][kSplitThreads]
    __shared__ float shared[33];
    __shared__ double shared64[33];
    __shared__ bool is_last;
    constexpr int kRegisterGroups = kSplitRegisterItems / 4, kSharedGroups = kSplitSharedItems / 4;
    const uint32_t r = blockIdx.x, tid = threadIdx.x, rows = gridDim.x;
    auto column_of = [tid](int group) { return (static_cast<uint32_t>(group) * kSplitThreads + tid) * 4; };
    float* o = out + static_cast<uint64_t>(r) * ld_out;
    float den;
    if (denominator != nullptr) {
        den = denominator[0];
    } else {
        double sum = 0.0;
        for (uint32_t j = tid; j < rows; j += kSplitThreads) sum += static_cast<double>(weights[j]);
        den = static_cast<float>(block_sum(sum, shared64));
    }
    const float w = weights[r];
    float4 x[kRegisterGroups];
    float total = 0.0f;
    uint32_t label = 0;
    // How many of the parked groups hold columns of the row at all (the same for every thread of
    // a warp but the one the row ends in, whose later lanes have one fewer).
    int parked_groups = 0;
#pragma unroll
    for (int k = 0; k < kSharedGroups; ++k)
        if (column_of(kRegisterGroups + k) < v) parked_groups = k + 1;
    if (w == 0.0f) {
        if (tid == 0) row_loss[r] = 0.0f;
    } else {
        const float* row = logits + static_cast<uint64_t>(r) * ld;
        const uint32_t last = (v - 1) & ~3u;
#pragma unroll
        for (int k = 0; k < kSharedGroups; ++k)
            if (k < parked_groups) {
                const uint32_t to = static_cast<uint32_t>(__cvta_generic_to_shared(&parked[k * kSplitThreads + tid]));
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(row + column_of(kRegisterGroups + k)) : "memory");
            }
        asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
        for (int k = 0; k < kRegisterGroups; ++k) x[k] = __ldg(reinterpret_cast<const float4*>(row + min(column_of(k), last)));
        auto mask = [v](float4 f, uint32_t c) {
            if (c >= v) f.x = -INFINITY;
            if (c + 1 >= v) f.y = -INFINITY;
            if (c + 2 >= v) f.z = -INFINITY;
            if (c + 3 >= v) f.w = -INFINITY;
            return f;
        };
        float m = -INFINITY;
#pragma unroll
        for (int k = 0; k < kRegisterGroups; ++k) {
            x[k] = mask(x[k], column_of(k));
            m = fmaxf(fmaxf(m, fmaxf(x[k].x, x[k].y)), fmaxf(x[k].z, x[k].w));
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
        for (int k = 0; k < kSharedGroups; ++k)
            if (k < parked_groups) {
                const float4 f = mask(parked[k * kSplitThreads + tid], column_of(kRegisterGroups + k));
                parked[k * kSplitThreads + tid] = f;
                m = fmaxf(fmaxf(m, fmaxf(f.x, f.y)), fmaxf(f.z, f.w));
            }
        m = block_max(m, shared);
        // exp(-inf) is 0: the masked columns add nothing and need no test of their own.
        auto exponentials = [m](float4 f) { return make_float4(__expf(f.x - m), __expf(f.y - m), __expf(f.z - m), __expf(f.w - m)); };
        float sum = 0.0f;
#pragma unroll
        for (int k = 0; k < kRegisterGroups; ++k) {
            x[k] = exponentials(x[k]);
            sum += (x[k].x + x[k].y) + (x[k].z + x[k].w);
        }
#pragma unroll
        for (int k = 0; k < kSharedGroups; ++k)
            if (k < parked_groups) {
                const float4 f = exponentials(parked[k * kSplitThreads + tid]);
                parked[k * kSplitThreads + tid] = f;
                sum += (f.x + f.y) + (f.z + f.w);
            }
        total = block_sum(sum, shared);
        label = static_cast<uint32_t>(labels[r]);
        if (tid == 0) row_loss[r] = m + logf(total) - (label < v ? row[label] : 0.0f);
    }
    if (tid == 0) {
        __threadfence();
        const uint32_t before = atomicAdd(counter, 1u);
        is_last = before + 1u == rows;
        if (is_last) *counter = 0u;
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        double num = 0.0, den64 = 0.0;
        for (uint32_t j = tid; j < rows; j += kSplitThreads) {
            double wj = static_cast<double>(weights[j]);
            num = fma(wj, static_cast<double>(__ldcg(row_loss + j)), num);
            den64 += wj;
        }
        num = block_sum(num, shared64);
        den64 = block_sum(den64, shared64);
        if (denominator != nullptr) den64 = static_cast<double>(denominator[0]);
        if (tid == 0) loss[0] = den64 == 0.0 ? 0.0f : static_cast<float>(num / den64);
    }
    const bool zero = den == 0.0f || w == 0.0f;
    const float scale = zero ? 0.0f : g[0] * w / den;
    const float inverse = zero ? 0.0f : 1.0f / total;
    auto gradient = [=](float4 f, uint32_t c) {
        if (zero) return make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        return make_float4(scale * (f.x * inverse - (c == label ? 1.0f : 0.0f)), scale * (f.y * inverse - (c + 1 == label ? 1.0f : 0.0f)),
                           scale * (f.z * inverse - (c + 2 == label ? 1.0f : 0.0f)), scale * (f.w * inverse - (c + 3 == label ? 1.0f : 0.0f)));
    };
    // Columns past v inside the pitch are padding nobody reads: the whole float4 is written.
#pragma unroll
    for (int k = 0; k < kRegisterGroups; ++k) {
        const uint32_t c = column_of(k);
        if (c < v) *reinterpret_cast<float4*>(o + c) = gradient(x[k], c);
    }
#pragma unroll
    for (int k = 0; k < kSharedGroups; ++k)
        if (k < parked_groups) {
            const uint32_t c = column_of(kRegisterGroups + k);
            *reinterpret_cast<float4*>(o + c) = gradient(zero ? make_float4(0.0f, 0.0f, 0.0f, 0.0f) : parked[k * kSplitThreads + tid], c);
        }
}

// How a warp holds a row in registers: lane l keeps ITEMS values, V consecutive columns per turn of
// 32 V columns. V = 1 (one 4-byte load per value; the f32 layout) or V = 2 (a bf16 pair per 4-byte
// load, so that a warp's load still covers 128 contiguous bytes).
template <int V> __device__ __forceinline__ uint32_t column_of(int i, uint32_t lane) {
    return static_cast<uint32_t>(i / V) * (32u * V) + lane * V + static_cast<uint32_t>(i % V);
}
// The row's values from clamped columns (what a column past h reads is discarded by the caller):
// unconditional, so that every load of a row is in flight before the first use.
template <int ITEMS, int V, class T>
__device__ __forceinline__ void load_row(const T* __restrict__ row, uint32_t lane, uint32_t h, float (&to)[ITEMS]) {
    if constexpr (V == 1) {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) to[i] = load1(row + min(i * 32 + lane, h - 1));
    } else {
        static_assert(ITEMS % 2 == 0, "pairs");
#pragma unroll
        for (int j = 0; j < ITEMS / 2; ++j) {
            const float2 f = load2(row + min(j * 64 + lane * 2, h - 2));
            to[2 * j] = f.x;
            to[2 * j + 1] = f.y;
        }
    }
}
template <int ITEMS, int V, class T>
__device__ __forceinline__ void store_row(T* __restrict__ row, uint32_t lane, uint32_t h, const float (&from)[ITEMS]) {
    if constexpr (V == 1) {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i)
            if (i * 32 + lane < h) store1(row + i * 32 + lane, from[i]);
    } else {
#pragma unroll
        for (int j = 0; j < ITEMS / 2; ++j)
            if (j * 64 + lane * 2 < h) store2(row + j * 64 + lane * 2, make_float2(from[2 * j], from[2 * j + 1]));  // h is even
    }
}

// The keep decisions of one row as the warp holds it (bit i of `mask` = item i of this lane) to
// and from their stored form: word w of the row holds columns 32 w .. 32 w + 31, bit = column
// modulo 32. The row has a multiple of 32 columns, at most 1,024: one word per lane.
__device__ __forceinline__ uint32_t spread16(uint32_t x) {  // bit b of the low half to bit 2 b
    x = (x | (x << 8)) & 0x00FF00FFu;
    x = (x | (x << 4)) & 0x0F0F0F0Fu;
    x = (x | (x << 2)) & 0x33333333u;
    x = (x | (x << 1)) & 0x55555555u;
    return x;
}
template <int ITEMS, int V>
__device__ __forceinline__ void save_keep_bits(uint32_t* __restrict__ row_words, uint32_t lane, uint32_t h, uint32_t mask) {
    uint32_t mine = 0;
    if constexpr (V == 1) {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            const uint32_t word = __ballot_sync(0xffffffffu, (mask >> i) & 1u);  // columns 32 i + lane
            if (lane == static_cast<uint32_t>(i)) mine = word;
        }
    } else {
#pragma unroll
        for (int j = 0; j < ITEMS / 2; ++j) {
            // Lane l holds columns 64 j + 2 l and + 1: lanes 0-15 fill word 2 j, lanes 16-31 word 2 j + 1.
            const uint32_t even = __ballot_sync(0xffffffffu, (mask >> (2 * j)) & 1u), odd = __ballot_sync(0xffffffffu, (mask >> (2 * j + 1)) & 1u);
            if (lane == static_cast<uint32_t>(2 * j)) mine = spread16(even & 0xffffu) | (spread16(odd & 0xffffu) << 1);
            if (lane == static_cast<uint32_t>(2 * j + 1)) mine = spread16(even >> 16) | (spread16(odd >> 16) << 1);
        }
    }
    if (lane < h / 32) row_words[lane] = mine;
}
template <int ITEMS, int V>
__device__ __forceinline__ uint32_t load_keep_bits(const uint32_t* __restrict__ row_words, uint32_t lane, uint32_t h) {
    const uint32_t mine = lane < h / 32 ? __ldg(row_words + lane) : 0u;
    uint32_t mask = 0;
    if constexpr (V == 1) {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) mask |= ((__shfl_sync(0xffffffffu, mine, i) >> lane) & 1u) << i;
    } else {
#pragma unroll
        for (int j = 0; j < ITEMS / 2; ++j) {
            const uint32_t word = __shfl_sync(0xffffffffu, mine, 2 * j + static_cast<int>(lane >> 4));
            mask |= ((word >> (2 * (lane & 15u))) & 3u) << (2 * j);
        }
    }
    return mask;
}
// The keep decisions of a row for one site: read when an earlier launch of the step stored them,
// else drawn (element index_base + row h + column of Philox stream 4) and stored when asked.
template <int ITEMS, int V>
__device__ __forceinline__ uint32_t keep_mask(const DropoutDraw& draw, uint64_t row_at, uint32_t lane, uint32_t h) {
    uint32_t* const row_words = draw.bits ? draw.bits + row_at / 32 : nullptr;
    if (draw.stored && row_words != nullptr) return load_keep_bits<ITEMS, V>(row_words, lane, h);
    const uint32_t id_lo = static_cast<uint32_t>(draw.token[0]), id_hi = static_cast<uint32_t>(draw.token[1]);
    uint32_t mask = 0;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const uint32_t w0 = philox_word0(static_cast<uint32_t>(draw.index_base + row_at + column_of<V>(i, lane)), 4u, id_lo, id_hi,
                                         static_cast<uint32_t>(draw.seed), static_cast<uint32_t>(draw.seed >> 32));
        mask |= (w0 >= draw.threshold ? 1u : 0u) << i;
    }
    if (row_words != nullptr) save_keep_bits<ITEMS, V>(row_words, lane, h, mask);
    return mask;
}

// dropout(x) + residual, then layer_norm of the sum, one warp per row with the row in registers:
// the three launches of a transformer sublayer's tail as one. Every element goes through the same
// rounded operations as the separate kernels (the Philox draw of element index_base + r h + c, the
// scaled or zeroed value, one addition, the layer norm of the stored sum). Each part is optional:
// without a draw on x the sum is x + residual; without gamma the launch ends with the sum; with a
// draw on the result, dropout of the layer norm is written to out_dropped (and out may be null);
// sum_out may be null when only the layer norm is wanted.
template <int ITEMS, int V, class T>
__global__ void __launch_bounds__(256) dropout_add_layer_norm_kernel(
    const T* __restrict__ x, const T* __restrict__ residual, DropoutDraw x_draw, const float* __restrict__ gamma,
    const float* __restrict__ beta, T* __restrict__ sum_out, T* __restrict__ out, DropoutDraw out_draw,
    T* __restrict__ out_dropped, uint32_t rows, uint32_t h, bool gelu_first) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t r = blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (r >= rows) return;
    const uint64_t base = static_cast<uint64_t>(r) * h;
    // The loads first, so that all are in flight before the Philox rounds of the first element start.
    float v[ITEMS], xs[ITEMS];
    load_row<ITEMS, V>(x + base, lane, h, xs);
    if (residual != nullptr) load_row<ITEMS, V>(residual + base, lane, h, v);
    // gelu(x) in the place of the sum (the head's transform: dense, gelu, layer norm).
    if (gelu_first) {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) xs[i] = gelu_value_for<T>(xs[i]);
    }
    if (x_draw.token != nullptr) {
        const uint32_t keep = keep_mask<ITEMS, V>(x_draw, base, lane, h);
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) xs[i] = (keep >> i) & 1u ? xs[i] * x_draw.scale : 0.0f;
    }
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const uint32_t c = column_of<V>(i, lane);
        v[i] = c < h ? (residual != nullptr ? v[i] + xs[i] : xs[i]) : 0.0f;
        // What is stored is what the layer norm below reads: the sum as its storage type holds it.
        v[i] = stored_as(v[i], static_cast<const T*>(nullptr));
    }
    if (sum_out != nullptr) store_row<ITEMS, V>(sum_out + base, lane, h, v);
    if (gamma == nullptr) return;
    const float width = static_cast<float>(h);
    float sum = 0.0f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
        if (column_of<V>(i, lane) < h) sum += v[i];
    const float mean = warp_sum(sum) / width;
    float q = 0.0f;
#pragma unroll
    for (int i = 0; i < ITEMS; ++i)
        if (column_of<V>(i, lane) < h) {
            float d = v[i] - mean;
            q = fmaf(d, d, q);
        }
    const float rstd = 1.0f / sqrtf(warp_sum(q) / width + kLayerNormEps);
    const uint32_t keep_out = out_dropped != nullptr ? keep_mask<ITEMS, V>(out_draw, base, lane, h) : 0u;
    float dropped[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const uint32_t c = column_of<V>(i, lane);
        const uint32_t cc = min(c, h - 1);
        const float y = (v[i] - mean) * rstd * gamma[cc] + beta[cc];
        v[i] = y;
        dropped[i] = (out_dropped != nullptr && c < h && ((keep_out >> i) & 1u)) ? y * out_draw.scale : 0.0f;
    }
    if (out != nullptr) store_row<ITEMS, V>(out + base, lane, h, v);
    if (out_dropped != nullptr) store_row<ITEMS, V>(out_dropped + base, lane, h, dropped);
}

// layer_norm_grad_x, layer_norm_grad_gamma and the beta gradient in one launch. A block takes a
// chunk of rows, a warp one row at a time with the row of x and of g in registers (ITEMS values
// per lane): row moments, then the dx row, then this row's terms of the column sums. Warp sums of
// a chunk are added in warp order, chunk sums by the last block to finish: thread (lane, w) adds
// chunks w, w + 8, ... in ascending order and the eight sums are added in ascending w. Every
// output is a fixed expression of the inputs: deterministic, tolerance class against a
// sequential column sum. dx (with gamma), dgamma and dbeta may each be null.
// Rows of 512 or more elements (ITEMS >= 16) keep their column sums in shared memory instead of
// registers (the same additions in the same order), and gamma is read where it is used: with the
// sums and gamma in registers a thread needs about 250 of them, one block of 8 warps fills an SM's
// register file, and the loads of a row have nothing to hide behind.
template <int ITEMS, int V, class T>
__global__ void __launch_bounds__(256, ITEMS >= 16 ? 2 : 1) layer_norm_backward_kernel(
    const T* __restrict__ x, const float* __restrict__ gamma, const T* __restrict__ g, const T* __restrict__ g1,
    const T* __restrict__ g2, const T* __restrict__ g3, T* __restrict__ dx,
    float* __restrict__ partial, uint32_t* __restrict__ counter, float* __restrict__ dgamma, float* __restrict__ dbeta,
    uint32_t want, uint32_t rows, uint32_t h, uint32_t rows_per_chunk, DropoutDraw adjoint_draw, DropoutDraw dx_draw,
    T* __restrict__ dx_dropped, const T* __restrict__ pre_activation) {
    constexpr bool WIDE = ITEMS >= 16;
    extern __shared__ float backward_sums[];  // 8 * 32 * ITEMS floats, twice that for wide rows
    float* const buf = backward_sums;
    float* const buf_b = backward_sums + (WIDE ? 8 * 32 * ITEMS : 0);
    __shared__ bool is_last;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, chunks = gridDim.x;
    const uint32_t r0 = blockIdx.x * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
    const float width = static_cast<float>(h);
    // dx is formed when it is stored or when what is stored is a function of it.
    const bool want_dx = dx != nullptr || dx_dropped != nullptr;
    constexpr int HELD = WIDE ? 1 : ITEMS;
    float acc_g[HELD], acc_b[HELD], gam[HELD];
    // This thread's column sums when they live in shared memory: value i at [i * 32].
    float* const sum_g = buf + warp * ITEMS * 32 + lane;
    float* const sum_b = buf_b + (WIDE ? warp * ITEMS * 32 + lane : 0);
    if constexpr (WIDE) {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            sum_g[i * 32] = 0.0f;
            sum_b[i * 32] = 0.0f;
        }
    } else {
#pragma unroll
        for (int i = 0; i < ITEMS; ++i) {
            acc_g[i] = 0.0f;
            acc_b[i] = 0.0f;
            uint32_t c = column_of<V>(i, lane);
            gam[i] = (want_dx && c < h) ? gamma[c] : 0.0f;
        }
    }
    auto gamma_of = [&](int i) -> float {
        if constexpr (WIDE) {
            const uint32_t c = column_of<V>(i, lane);
            return (want_dx && c < h) ? __ldg(gamma + c) : 0.0f;
        } else {
            return gam[i];
        }
    };
    for (uint32_t r = r0 + warp; r < r1; r += 8) {
        // All loads of an array are issued before any is used: unconditional, from a clamped
        // column (what a column past h reads is discarded below), one array after another. A load
        // under a condition of its own would wait for the one before it.
        const uint64_t row_at = static_cast<uint64_t>(r) * h;
        float xv[ITEMS], gv[ITEMS];
        load_row<ITEMS, V>(x + row_at, lane, h, xv);
        load_row<ITEMS, V>(g + row_at, lane, h, gv);
        // The adjoint as a sum the program spells as a chain of Adds: ((g + g1) + g2) + g3.
        for (const T* more : {g1, g2, g3}) {
            if (more == nullptr) continue;
            float t[ITEMS];
            load_row<ITEMS, V>(more + row_at, lane, h, t);
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) gv[i] = gv[i] + t[i];
        }
        // An adjoint that the program passes through dropout_grad first: the draw of element
        // (r, c), on the sum.
        if (adjoint_draw.token != nullptr) {
            const uint32_t keep = keep_mask<ITEMS, V>(adjoint_draw, row_at, lane, h);
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) gv[i] = (keep >> i) & 1u ? gv[i] * adjoint_draw.scale : 0.0f;
        }
#pragma unroll
        for (int i = 0; i < ITEMS; ++i)
            if (column_of<V>(i, lane) >= h) {
                xv[i] = 0.0f;
                gv[i] = 0.0f;
            }
        float sum = 0.0f;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i)
            if (column_of<V>(i, lane) < h) sum += xv[i];
        const float mean = warp_sum(sum) / width;
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i)
            if (column_of<V>(i, lane) < h) {
                float d = xv[i] - mean;
                q = fmaf(d, d, q);
            }
        const float rstd = 1.0f / sqrtf(warp_sum(q) / width + kLayerNormEps);
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int i = 0; i < ITEMS; ++i)
            if (column_of<V>(i, lane) < h) {
                float xhat = (xv[i] - mean) * rstd;
                if constexpr (WIDE) {
                    sum_g[i * 32] = fmaf(gv[i], xhat, sum_g[i * 32]);
                    sum_b[i * 32] += gv[i];
                } else {
                    acc_g[i] = fmaf(gv[i], xhat, acc_g[i]);
                    acc_b[i] += gv[i];
                }
                float gx = gv[i] * gamma_of(i);
                s1 += gx;
                s2 = fmaf(gx, xhat, s2);
                // The dx row below is a function of these two: kept in the registers of x and g.
                xv[i] = xhat;
                gv[i] = gx;
            }
        if (want_dx) {
            const float mean_gx = warp_sum(s1) / width, mean_gx_xhat = warp_sum(s2) / width;
            // The pre-activations of a gelu_grad on dx: loaded together, before the first is used.
            float pre[ITEMS];
            if (pre_activation != nullptr) load_row<ITEMS, V>(pre_activation + row_at, lane, h, pre);
            float second[ITEMS];
            const uint32_t keep_dx = (pre_activation == nullptr && dx_dropped != nullptr) ? keep_mask<ITEMS, V>(dx_draw, row_at, lane, h) : 0u;
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) {
                const uint32_t c = column_of<V>(i, lane);
                const float gx = gv[i], xhat = xv[i];
                const float value = rstd * ((gx - mean_gx) - xhat * mean_gx_xhat);
                xv[i] = value;  // the dx row, in the registers of the x row
                second[i] = 0.0f;
                // A function of dx for the reader that wants that: gelu_grad (the dense layer
                // before a gelu and this layer norm), or dropout_grad (the projection before
                // this sublayer's dropout).
                if (pre_activation != nullptr) {
                    second[i] = gelu_grad_value_for<T>(pre[i], value);
                } else if (dx_dropped != nullptr && c < h) {
                    second[i] = (keep_dx >> i) & 1u ? value * dx_draw.scale : 0.0f;
                }
            }
            if (dx != nullptr) store_row<ITEMS, V>(dx + row_at, lane, h, xv);
            if (dx_dropped != nullptr) store_row<ITEMS, V>(dx_dropped + row_at, lane, h, second);
        }
    }
    if (want == 0) return;
    float* partial_gamma = partial + static_cast<uint64_t>(blockIdx.x) * h;
    float* partial_beta = partial + static_cast<uint64_t>(chunks + blockIdx.x) * h;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        if ((want & (1u << pass)) == 0) continue;
        __syncthreads();
        if constexpr (!WIDE) {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i) buf[(warp * ITEMS + i) * 32 + lane] = pass == 0 ? acc_g[i] : acc_b[i];
        }
        __syncthreads();
        const float* const sums = (WIDE && pass == 1) ? buf_b : buf;
        for (uint32_t c = threadIdx.x; c < h; c += 256) {
            // Column c is value i of lane l (the inverse of column_of).
            const uint32_t turn = c / (32u * V), within = c % (32u * V);
            const uint32_t i = turn * V + within % V, l = within / V;
            float total = sums[i * 32 + l];
#pragma unroll
            for (int w = 1; w < 8; ++w) total += sums[(w * ITEMS + i) * 32 + l];
            (pass == 0 ? partial_gamma : partial_beta)[c] = total;
        }
    }
    if (counter == nullptr) return;  // the chunk sums are added later, by finalize_sums
    if (!last_block_arrives(counter, chunks, &is_last)) return;
    for (int pass = 0; pass < 2; ++pass) {
        float* out = pass == 0 ? dgamma : dbeta;
        if ((want & (1u << pass)) == 0) continue;
        const float* from = partial + static_cast<uint64_t>(pass) * chunks * h;
        for (uint32_t c0 = 0; c0 < h; c0 += 32) {
            uint32_t c = c0 + lane;
            float total = 0.0f;
            if (c < h)
                for (uint32_t k = warp; k < chunks; k += 8) total += __ldcg(from + static_cast<uint64_t>(k) * h + c);
            __syncthreads();
            buf[warp * 32 + lane] = total;
            __syncthreads();
            if (warp == 0 && c < h) {
                float t = buf[lane];
#pragma unroll
                for (int w = 1; w < 8; ++w) t += buf[w * 32 + lane];
                out[c] = t;
            }
        }
    }
}

// The one-read kernels: f32 rows of more than 16,384 logits with a 16-byte pitch as two 512-thread
// blocks per SM, every other case as one 1,024-thread block with the row in registers.
void launch_cross_entropy_one_read(cudaStream_t s, const float* logits, const int32_t* labels, const float* weights, const float* g,
                                   const float* den, float* row_loss, float* grad, uint32_t vv, uint32_t l1, uint32_t l2, uint32_t* counter,
                                   float* loss, uint64_t rows, bool vec) {
    if (vec && vv > 16384) {
        static const bool configured = [] {
            cudaFuncSetAttribute(cross_entropy_fused_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSplitSharedBytes);
            return true;
        }();
        (void)configured;
        cross_entropy_fused_split_kernel<<<static_cast<uint32_t>(rows), kSplitThreads, kSplitSharedBytes, s>>>(logits, labels, weights, g, den,
                                                                                                              row_loss, grad, vv, l1, l2,
                                                                                                              counter, loss);
    } else if (vec) {
        cross_entropy_fused_wide_kernel<4><<<static_cast<uint32_t>(rows), kWideThreads, 0, s>>>(logits, labels, weights, g, den, row_loss,
                                                                                                grad, vv, l1, l2, counter, loss);
    } else {
        cross_entropy_fused_wide_kernel<1><<<static_cast<uint32_t>(rows), kWideThreads, 0, s>>>(logits, labels, weights, g, den, row_loss,
                                                                                                grad, vv, l1, l2, counter, loss);
    }
}
void launch_cross_entropy_one_read(cudaStream_t s, const bf16* logits, const int32_t* labels, const float* weights, const float* g,
                                   const float* den, float* row_loss, bf16* grad, uint32_t vv, uint32_t l1, uint32_t l2, uint32_t* counter,
                                   float* loss, uint64_t rows, bool vec) {
    if (vec)
        cross_entropy_fused_wide_kernel<4><<<static_cast<uint32_t>(rows), kWideThreads, 0, s>>>(logits, labels, weights, g, den, row_loss,
                                                                                                grad, vv, l1, l2, counter, loss);
    else
        cross_entropy_fused_wide_kernel<1><<<static_cast<uint32_t>(rows), kWideThreads, 0, s>>>(logits, labels, weights, g, den, row_loss,
                                                                                                grad, vv, l1, l2, counter, loss);
}

uint32_t backward_chunks(uint64_t rows, uint64_t h) {
    // Four blocks per SM: a warp walks its rows one after another, each row a chain of loads and
    // three warp reductions, so it is the number of warps in flight that hides that latency (4,096
    // rows of 128: a row a warp, 8.4 us; three blocks per SM left a quarter of the warps a second
    // row, 10.5 us). Rows
    // of more than 256 elements keep their column sums in shared memory, two blocks per SM: one wave
    // of 296 blocks instead of a full wave and a half one.
    const uint64_t blocks = h > 256 ? MSX_LN_BACKWARD_WIDE_BLOCKS : MSX_LN_BACKWARD_BLOCKS;
    uint64_t per = (rows + blocks - 1) / blocks;
    if (per < 8) per = 8;
    uint64_t chunks = (rows + per - 1) / per;
    return static_cast<uint32_t>(chunks < 1 ? 1 : chunks);
}

}  // namespace

void layer_norm(cudaStream_t s, const float* x, const float* gamma, const float* beta, float* out,
                uint64_t rows, uint64_t h) {
    if (rows == 0) return;
    layer_norm_kernel<<<warp_row_blocks(rows), kWarpsPerBlock * 32, 0, s>>>(x, gamma, beta, out,
                                                                            static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
    check_launch("layer_norm");
}

void layer_norm_grad_x(cudaStream_t s, const float* x, const float* gamma, const float* g, float* out,
                       uint64_t rows, uint64_t h) {
    if (rows == 0) return;
    layer_norm_grad_x_kernel<<<warp_row_blocks(rows), kWarpsPerBlock * 32, 0, s>>>(
        x, gamma, g, out, static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
    check_launch("layer_norm_grad_x");
}

uint64_t layer_norm_grad_gamma_scratch_floats(uint64_t rows, uint64_t h) {
    return 2 * rows + 2 * sum_rows_chunks(rows) * h;
}

void layer_norm_grad_gamma(cudaStream_t s, const float* x, const float* g, float* scratch, float* dgamma,
                           float* dbeta, uint64_t rows, uint64_t h) {
    if (h == 0) return;
    uint32_t chunks = sum_rows_chunks(rows);
    uint32_t rows_per_chunk = static_cast<uint32_t>((rows + chunks - 1) / chunks);
    float* stats = scratch;
    float* partial_gamma = scratch + 2 * rows;
    float* partial_beta = partial_gamma + static_cast<uint64_t>(chunks) * h;
    if (rows > 0) {
        row_stats_kernel<<<warp_row_blocks(rows), kWarpsPerBlock * 32, 0, s>>>(x, stats, static_cast<uint32_t>(rows),
                                                                                static_cast<uint32_t>(h));
        check_launch("layer_norm_grad_gamma");
    }
    dim3 grid(static_cast<uint32_t>((h + 31) / 32), chunks);
    grad_gamma_stage1<<<grid, dim3(32, 8), 0, s>>>(x, g, stats, static_cast<uint32_t>(rows), static_cast<uint32_t>(h),
                                                   rows_per_chunk, partial_gamma, dbeta ? partial_beta : nullptr);
    check_launch("layer_norm_grad_gamma");
    grad_gamma_stage2<<<static_cast<uint32_t>((h + 127) / 128), 128, 0, s>>>(partial_gamma, partial_beta, chunks,
                                                                              static_cast<uint32_t>(h), dgamma, dbeta);
    check_launch("layer_norm_grad_gamma");
}

namespace {
template <class T>
void launch_add_layer_norm(cudaStream_t s, const T* x, const T* residual, const DropoutDraw& first, const float* gamma, const float* beta,
                           T* sum_out, T* out, const DropoutDraw& second, T* out_dropped, uint64_t rows, uint64_t h, bool gelu_first) {
    const uint32_t items = static_cast<uint32_t>((h + 31) / 32), blocks = static_cast<uint32_t>((rows + kWarpsPerBlock - 1) / kWarpsPerBlock);
    const uint32_t r = static_cast<uint32_t>(rows), hh = static_cast<uint32_t>(h);
    // bf16 rows of even width are held as pairs (4-byte loads); everything else one value per load.
    constexpr int PAIR = sizeof(T) == 2 ? 2 : 1;
    const bool pairs = PAIR == 2 && h % 2 == 0 && items >= 2;
#define MSX_DROPOUT_LN(N) do { if (pairs) dropout_add_layer_norm_kernel<N, (N % 2 == 0 ? PAIR : 1)><<<blocks, 256, 0, s>>>(x, residual, first, gamma, beta, sum_out, out, second, out_dropped, r, hh, gelu_first); \
        else dropout_add_layer_norm_kernel<N, 1><<<blocks, 256, 0, s>>>(x, residual, first, gamma, beta, sum_out, out, second, out_dropped, r, hh, gelu_first); } while (0)
    if (items <= 1) MSX_DROPOUT_LN(1);
    else if (items <= 2) MSX_DROPOUT_LN(2);
    else if (items <= 4) MSX_DROPOUT_LN(4);
    else if (items <= 8) MSX_DROPOUT_LN(8);
    else if (items <= 16) MSX_DROPOUT_LN(16);
    else if (items <= 24) MSX_DROPOUT_LN(24);
    else MSX_DROPOUT_LN(32);
#undef MSX_DROPOUT_LN
    check_launch("add_layer_norm");
}
template <class T> const T* typed(In a) { return static_cast<const T*>(a.p); }
template <class T> T* typed(Out a) { return static_cast<T*>(a.p); }
}  // namespace

void add_layer_norm(cudaStream_t s, In x, In residual, const DropoutDraw* x_draw, const float* gamma,
                    const float* beta, Out sum_out, Out out, const DropoutDraw* out_draw, Out out_dropped, uint64_t rows,
                    uint64_t h, bool gelu_first) {
    if (rows == 0 || h == 0) return;
    const DropoutDraw none = {};
    const DropoutDraw first = x_draw ? *x_draw : none, second = out_draw ? *out_draw : none;
    if (out_draw == nullptr || gamma == nullptr) out_dropped = Out();
    // The element type of the launch is that of x; the optional operands that are present share it.
    const bool half = x.half;
    for (bool other : {residual ? residual.half : half, sum_out ? sum_out.half : half, out ? out.half : half, out_dropped ? out_dropped.half : half})
        if (other != half) throw std::invalid_argument("add_layer_norm: f32 and bf16 activation operands in one launch");
    if (half)
        launch_add_layer_norm(s, typed<bf16>(x), typed<bf16>(residual), first, gamma, beta, typed<bf16>(sum_out), typed<bf16>(out), second,
                              typed<bf16>(out_dropped), rows, h, gelu_first);
    else
        launch_add_layer_norm(s, typed<float>(x), typed<float>(residual), first, gamma, beta, typed<float>(sum_out), typed<float>(out), second,
                              typed<float>(out_dropped), rows, h, gelu_first);
}

void dropout_add_layer_norm(cudaStream_t s, In x, In residual, const int32_t* token, uint64_t seed,
                            uint32_t threshold, float scale, uint64_t index_base, const float* gamma, const float* beta,
                            Out sum_out, Out out, uint64_t rows, uint64_t h) {
    DropoutDraw draw;
    draw.token = token;
    draw.seed = seed;
    draw.threshold = threshold;
    draw.scale = scale;
    draw.index_base = index_base;
    add_layer_norm(s, x, residual, &draw, gamma, beta, sum_out, out, nullptr, Out(), rows, h, false);
}

bool layer_norm_backward_supported(uint64_t h) { return h >= 1 && h <= 1024; }
uint32_t layer_norm_backward_chunks(uint64_t rows, uint64_t h) { return backward_chunks(rows, h); }
uint64_t layer_norm_backward_scratch_floats(uint64_t rows, uint64_t h) { return 2ull * backward_chunks(rows, h) * h; }

namespace {
template <class T>
void launch_layer_norm_backward(cudaStream_t s, const T* x, const float* gamma, const T* g, T* dx, float* scratch, uint32_t* counter,
                                float* dgamma, float* dbeta, uint64_t rows, uint64_t h, const T* g1, const T* g2, const T* g3,
                                const DropoutDraw& in_draw, const DropoutDraw& out_draw, T* dx_dropped, const T* pre_activation) {
    uint32_t chunks = backward_chunks(rows, h);
    uint32_t per = static_cast<uint32_t>((rows + chunks - 1) / chunks);
    uint32_t items = static_cast<uint32_t>((h + 31) / 32);
    uint32_t r = static_cast<uint32_t>(rows), hh = static_cast<uint32_t>(h);
    uint32_t want = (dgamma ? 1u : 0u) | (dbeta ? 2u : 0u);
    constexpr int PAIR = sizeof(T) == 2 ? 2 : 1;
    const bool pairs = PAIR == 2 && h % 2 == 0 && items >= 2;
    // Shared memory of the column sums: one array of 8 x 32 x N floats, two for rows of 512 or more.
#define MSX_LN_BACKWARD_ONE(N, W) do { \
        auto kernel = layer_norm_backward_kernel<N, W, T>; \
        constexpr uint32_t bytes = (N >= 16 ? 2u : 1u) * 8u * 32u * N * 4u; \
        if (bytes > 40000u) { \
            static const bool configured = [kernel] { cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)); return true; }(); \
            (void)configured; \
        } \
        kernel<<<chunks, 256, bytes, s>>>(x, gamma, g, g1, g2, g3, dx, scratch, counter, dgamma, dbeta, want, r, hh, per, in_draw, out_draw, dx_dropped, pre_activation); } while (0)
#define MSX_LN_BACKWARD(N) do { if (pairs) MSX_LN_BACKWARD_ONE(N, (N % 2 == 0 ? PAIR : 1)); else MSX_LN_BACKWARD_ONE(N, 1); } while (0)
    if (items <= 1) MSX_LN_BACKWARD(1);
    else if (items <= 2) MSX_LN_BACKWARD(2);
    else if (items <= 4) MSX_LN_BACKWARD(4);
    else if (items <= 8) MSX_LN_BACKWARD(8);
    else if (items <= 16) MSX_LN_BACKWARD(16);
    else if (items <= 24) MSX_LN_BACKWARD(24);
    else MSX_LN_BACKWARD(32);
#undef MSX_LN_BACKWARD
#undef MSX_LN_BACKWARD_ONE
    check_launch("layer_norm_backward");
}
}  // namespace

void layer_norm_backward(cudaStream_t s, In x, const float* gamma, In g, Out dx, float* scratch,
                         uint32_t* counter, float* dgamma, float* dbeta, uint64_t rows, uint64_t h, In g1, In g2,
                         In g3, const DropoutDraw* adjoint_draw, const DropoutDraw* dx_draw, Out dx_dropped,
                         In pre_activation) {
    if (h == 0) return;
    const DropoutDraw none = {};
    const DropoutDraw in_draw = adjoint_draw ? *adjoint_draw : none, out_draw = dx_draw ? *dx_draw : none;
    if (dx_draw == nullptr && !pre_activation) dx_dropped = Out();
    if (!dx_dropped) pre_activation = In();
    const bool half = x.half;
    for (bool other : {g.half, g1 ? g1.half : half, g2 ? g2.half : half, g3 ? g3.half : half, dx ? dx.half : half,
                       dx_dropped ? dx_dropped.half : half, pre_activation ? pre_activation.half : half})
        if (other != half) throw std::invalid_argument("layer_norm_backward: f32 and bf16 activation operands in one launch");
    if (half)
        launch_layer_norm_backward(s, typed<bf16>(x), gamma, typed<bf16>(g), typed<bf16>(dx), scratch, counter, dgamma, dbeta, rows, h,
                                   typed<bf16>(g1), typed<bf16>(g2), typed<bf16>(g3), in_draw, out_draw, typed<bf16>(dx_dropped),
                                   typed<bf16>(pre_activation));
    else
        launch_layer_norm_backward(s, typed<float>(x), gamma, typed<float>(g), typed<float>(dx), scratch, counter, dgamma, dbeta, rows, h,
                                   typed<float>(g1), typed<float>(g2), typed<float>(g3), in_draw, out_draw, typed<float>(dx_dropped),
                                   typed<float>(pre_activation));
}

void softmax(cudaStream_t s, const float* x, float* out, uint64_t rows, uint64_t k) {
    if (rows == 0) return;
    softmax_kernel<<<static_cast<uint32_t>(rows), kRowThreads, 0, s>>>(x, out, static_cast<uint32_t>(k));
    check_launch("softmax");
}

void softmax_grad(cudaStream_t s, const float* y, const float* g, float* out, uint64_t rows, uint64_t k) {
    if (rows == 0) return;
    softmax_grad_kernel<<<static_cast<uint32_t>(rows), kRowThreads, 0, s>>>(y, g, out, static_cast<uint32_t>(k));
    check_launch("softmax_grad");
}

void weight_sum(cudaStream_t s, const float* weights, uint64_t rows, float* out) {
    weight_sum_kernel<<<1, 1024, 0, s>>>(weights, static_cast<uint32_t>(rows), out);
    check_launch("weight_sum");
}

void cross_entropy(cudaStream_t s, In logits, const int32_t* labels, const float* weights,
                   float* row_loss, const float* global_den, float* loss, uint64_t rows, uint64_t v, uint64_t ld) {
    if (ld == 0) ld = v;
    if (rows > 0) {
        if (logits.half)
            cross_entropy_rows_kernel<<<static_cast<uint32_t>(rows), kRowThreads, 0, s>>>(typed<bf16>(logits), labels, weights, row_loss,
                                                                                          static_cast<uint32_t>(v), static_cast<uint32_t>(ld));
        else
            cross_entropy_rows_kernel<<<static_cast<uint32_t>(rows), kRowThreads, 0, s>>>(typed<float>(logits), labels, weights, row_loss,
                                                                                          static_cast<uint32_t>(v), static_cast<uint32_t>(ld));
        check_launch("cross_entropy");
    }
    cross_entropy_loss_kernel<<<1, 1024, 0, s>>>(row_loss, weights, static_cast<uint32_t>(rows), global_den, loss);
    check_launch("cross_entropy");
}

namespace {
template <class T>
void launch_cross_entropy_with_grad(cudaStream_t s, const T* logits, const int32_t* labels, const float* weights, const float* g,
                                    bool denominator_ready, float* denominator, float* row_loss, float* loss, T* grad, uint64_t rows,
                                    uint64_t v, uint32_t* counter, uint64_t ld, uint64_t ld_grad) {
    const uint32_t vv = static_cast<uint32_t>(v), l1 = static_cast<uint32_t>(ld), l2 = static_cast<uint32_t>(ld_grad);
    if (rows > 0 && counter != nullptr && v <= static_cast<uint64_t>(kWideThreads) * kWideItems) {
        const float* den = denominator_ready ? denominator : nullptr;
        const bool vec = ld % 4 == 0 && ld_grad % 4 == 0 && aligned4(logits) && aligned4(grad);
        launch_cross_entropy_one_read(s, logits, labels, weights, g, den, row_loss, grad, vv, l1, l2, counter, loss, rows, vec);
        check_launch("cross_entropy_with_grad");
        return;
    }
    if (!denominator_ready) {
        weight_sum_kernel<<<1, 1024, 0, s>>>(weights, static_cast<uint32_t>(rows), denominator);
        check_launch("cross_entropy_with_grad");
    }
    if (rows > 0) {
        cross_entropy_fused_kernel<<<static_cast<uint32_t>(rows), kRowThreads, 0, s>>>(logits, labels, weights, g, denominator, row_loss,
                                                                                       grad, vv, l1, l2);
        check_launch("cross_entropy_with_grad");
    }
    cross_entropy_loss_kernel<<<1, 1024, 0, s>>>(row_loss, weights, static_cast<uint32_t>(rows), denominator_ready ? denominator : nullptr, loss);
    check_launch("cross_entropy_with_grad");
}
}  // namespace

void cross_entropy_with_grad(cudaStream_t s, In logits, const int32_t* labels, const float* weights,
                             const float* g, bool denominator_ready, float* denominator, float* row_loss, float* loss,
                             Out grad, uint64_t rows, uint64_t v, uint32_t* counter, uint64_t ld, uint64_t ld_grad) {
    if (ld == 0) ld = v;
    if (ld_grad == 0) ld_grad = v;
    if (all_half({logits.half, grad.half}, "cross_entropy_with_grad"))
        launch_cross_entropy_with_grad(s, typed<bf16>(logits), labels, weights, g, denominator_ready, denominator, row_loss, loss,
                                       typed<bf16>(grad), rows, v, counter, ld, ld_grad);
    else
        launch_cross_entropy_with_grad(s, typed<float>(logits), labels, weights, g, denominator_ready, denominator, row_loss, loss,
                                       typed<float>(grad), rows, v, counter, ld, ld_grad);
}

void cross_entropy_grad(cudaStream_t s, const float* logits, const int32_t* labels, const float* weights,
                        const float* g, bool denominator_ready, float* denominator, float* out, uint64_t rows,
                        uint64_t v, uint64_t ld, uint64_t ld_out) {
    if (rows == 0) return;
    if (ld == 0) ld = v;
    if (ld_out == 0) ld_out = v;
    if (!denominator_ready) {
        weight_sum_kernel<<<1, 1024, 0, s>>>(weights, static_cast<uint32_t>(rows), denominator);
        check_launch("cross_entropy_grad");
    }
    cross_entropy_grad_kernel<<<static_cast<uint32_t>(rows), kRowThreads, 0, s>>>(logits, labels, weights, g, denominator, out,
                                                                                  static_cast<uint32_t>(v), static_cast<uint32_t>(ld),
                                                                                  static_cast<uint32_t>(ld_out));
    check_launch("cross_entropy_grad");
}

}  // namespace k
}  // namespace msx
