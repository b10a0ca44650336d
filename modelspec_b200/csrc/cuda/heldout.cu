// The held-out reduction on the device: the logits [rows, classes] of one evaluated batch into the
// weighted sum of the row losses and the count of correct selected rows, so that an evaluation
// reads back one small state instead of every batch's logits.
//
// Counterpart of the reference's two kernels HeldOutRows and HeldOutSum
// (crates/modelspec-runtime/src/spirv/emit/heldout.rs:1-24, :57-117) and of the host tally they
// replace (crates/modelspec-runtime/src/train/eval.rs:420-470, row_nll :490-499). Here it is one
// launch: a block per row, and the block that finishes last adds the rows' terms in ascending row
// order, as the host tally does. The device has f64, so the numerator is the host's own f64 chain
// (each term w x nll is exact in f64: two 24-bit significands) instead of the reference's
// two-float sum.
//
// Per row n: the maximum (first logit, replaced only by a greater one), the first largest logit's
// class (the lowest among ties), whether the row holds a NaN, and whether every |x| < 5e37.
// A row of weight +0 whose logits are all that small adds +0 without its softmax, as the host
// tally skips it (eval.rs:436-442); every other row computes nll = max + ln(sum exp(x - max)) -
// x[label] in f32 and adds f64(w) x f64(nll). A row counts as correct when its weight is positive,
// it holds no NaN and the first largest logit is its label. The sum of exp is added in a fixed
// tree per block, not in ascending class order: the row loss is tolerance class, the count exact.
#include <cmath>

#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {
namespace {

constexpr int THREADS = 256;

// What one pass over a row learns, combined across the block in a fixed order.
struct RowFacts {
    float max;
    uint32_t at;      // class of the first largest logit
    uint32_t flags;   // bit 0: a NaN; bit 1: some |x| >= 5e37 (or not finite)
};

__device__ __forceinline__ RowFacts merge(RowFacts a, RowFacts b) {
    RowFacts r;
    const bool take_b = b.max > a.max || (b.max == a.max && b.at < a.at);
    r.max = take_b ? b.max : a.max;
    r.at = take_b ? b.at : a.at;
    r.flags = a.flags | b.flags;
    return r;
}

__device__ __forceinline__ void see(RowFacts& f, float x, uint32_t i) {
    if (x != x) f.flags |= 1u;
    if (!(fabsf(x) < 5.0e37f)) f.flags |= 2u;
    if (x > f.max) {
        f.max = x;
        f.at = i;
    }
}

// Visits the row's elements: every thread sees its own in ascending class order. The body is read
// 16 bytes at a time from the first 16-byte boundary of the row.
template <class F> __device__ __forceinline__ void visit(const float* row, uint32_t classes, F f) {
    const uint32_t head = min(classes, static_cast<uint32_t>((16u - (reinterpret_cast<uintptr_t>(row) & 15u)) & 15u) / 4u);
    if (threadIdx.x < head) f(__ldg(row + threadIdx.x), threadIdx.x);
    const uint32_t body = (classes - head) / 4;
    const float4* wide = reinterpret_cast<const float4*>(row + head);
    auto four = [&](const float4& v, uint32_t i) {
        f(v.x, i);
        f(v.y, i + 1);
        f(v.z, i + 2);
        f(v.w, i + 3);
    };
    uint32_t j = threadIdx.x;
    for (; j + 3 * THREADS < body; j += 4 * THREADS) {  // four loads in flight per thread
        const float4 a = __ldg(wide + j), b = __ldg(wide + j + THREADS), c = __ldg(wide + j + 2 * THREADS), d = __ldg(wide + j + 3 * THREADS);
        four(a, head + 4 * j);
        four(b, head + 4 * (j + THREADS));
        four(c, head + 4 * (j + 2 * THREADS));
        four(d, head + 4 * (j + 3 * THREADS));
    }
    for (; j < body; j += THREADS) four(__ldg(wide + j), head + 4 * j);
    const uint32_t tail = head + 4 * body;
    if (tail + threadIdx.x < classes) f(__ldg(row + tail + threadIdx.x), tail + threadIdx.x);
}

__global__ void __launch_bounds__(THREADS) heldout_rows_kernel(const float* __restrict__ logits, uint64_t pitch,
                                                                const int32_t* __restrict__ labels, const float* __restrict__ weights,
                                                                uint32_t rows, uint32_t classes, double* __restrict__ terms,
                                                                uint32_t* __restrict__ hits, HeldOutState* state) {
    __shared__ RowFacts warp_facts[THREADS / 32];
    __shared__ float warp_sums[THREADS / 32];
    __shared__ RowFacts row_facts;
    __shared__ float row_total;
    __shared__ uint32_t last;
    __shared__ double staged[4 * THREADS];
    __shared__ uint32_t warp_hits[THREADS / 32];

    const uint32_t n = blockIdx.x;
    const float* row = logits + static_cast<uint64_t>(n) * pitch;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;

    RowFacts mine = {-INFINITY, 0xffffffffu, 0u};
    visit(row, classes, [&](float x, uint32_t i) { see(mine, x, i); });
    for (int d = 16; d > 0; d >>= 1) {
        RowFacts other;
        other.max = __shfl_xor_sync(0xffffffffu, mine.max, d);
        other.at = __shfl_xor_sync(0xffffffffu, mine.at, d);
        other.flags = __shfl_xor_sync(0xffffffffu, mine.flags, d);
        mine = merge(mine, other);
    }
    if (lane == 0) warp_facts[warp] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        RowFacts all = warp_facts[0];
        for (int w = 1; w < THREADS / 32; ++w) all = merge(all, warp_facts[w]);
        // A row of nothing above -inf (or of NaNs only): the first class is the first largest.
        if (all.at == 0xffffffffu) all.at = 0;
        row_facts = all;
    }
    __syncthreads();
    const RowFacts facts = row_facts;
    const float weight = weights[n];
    const int32_t given = labels[n];
    const uint32_t label = given >= 0 && static_cast<uint32_t>(given) < classes ? static_cast<uint32_t>(given) : 0u;

    const bool skipped = __float_as_uint(weight) == 0u && facts.flags == 0u;
    float nll = 0.0f;
    if (!skipped) {  // uniform across the block
        if (facts.flags & 1u) {
            nll = nanf("");
        } else {
            float part = 0.0f;
            const float m = facts.max;
            visit(row, classes, [&](float x, uint32_t) { part += expf(x - m); });
            for (int d = 16; d > 0; d >>= 1) part += __shfl_xor_sync(0xffffffffu, part, d);
            if (lane == 0) warp_sums[warp] = part;
            __syncthreads();
            if (threadIdx.x == 0) {
                float total = warp_sums[0];
                for (int w = 1; w < THREADS / 32; ++w) total += warp_sums[w];
                row_total = total;
            }
            __syncthreads();
            nll = m + logf(row_total) - __ldg(row + label);
        }
    }
    if (threadIdx.x == 0) {
        terms[n] = skipped ? 0.0 : static_cast<double>(weight) * static_cast<double>(nll);
        hits[n] = (weight > 0.0f && !(facts.flags & 1u) && facts.at == label) ? 1u : 0u;
        __threadfence();
        last = atomicAdd(&state->arrived, 1u) == rows - 1 ? 1u : 0u;
    }
    __syncthreads();
    if (!last) return;

    // The last block of the batch: the rows' terms in ascending row order onto the state.
    __threadfence();
    uint32_t counted = 0;
    double sum = state->numerator;
    bool started = state->started != 0u;
    for (uint32_t base = 0; base < rows; base += 4 * THREADS) {
        const uint32_t here = min(static_cast<uint32_t>(4 * THREADS), rows - base);
        for (uint32_t i = threadIdx.x; i < here; i += THREADS) {
            staged[i] = __ldcg(terms + base + i);
            counted += __ldcg(hits + base + i);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            // The first term starts the sum; each later one is added (its product is exact, so
            // the host's fused multiply-add rounds to the same f64).
            uint32_t i = 0;
            if (!started) {
                sum = staged[0];
                started = true;
                i = 1;
            }
            for (; i + 8 <= here; i += 8) {
                double t[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) t[u] = staged[i + u];
#pragma unroll
                for (int u = 0; u < 8; ++u) sum += t[u];
            }
            for (; i < here; ++i) sum += staged[i];
        }
        __syncthreads();
    }
    for (int d = 16; d > 0; d >>= 1) counted += __shfl_xor_sync(0xffffffffu, counted, d);
    if (lane == 0) warp_hits[warp] = counted;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long correct = 0;
        for (int w = 0; w < THREADS / 32; ++w) correct += warp_hits[w];
        state->numerator = sum;
        state->started = started ? 1u : 0u;
        state->correct += correct;
        state->arrived = 0u;  // the next batch counts its own rows
    }
}

}  // namespace

void heldout_rows(cudaStream_t s, const float* logits, uint64_t pitch, const int32_t* labels, const float* weights, uint64_t rows,
                  uint64_t classes, double* terms, uint32_t* hits, HeldOutState* state) {
    if (rows == 0) return;
    heldout_rows_kernel<<<static_cast<unsigned>(rows), THREADS, 0, s>>>(logits, pitch ? pitch : classes, labels, weights,
                                                                         static_cast<uint32_t>(rows), static_cast<uint32_t>(classes), terms,
                                                                         hits, state);
    check_launch("heldout_rows");
}

}  // namespace k
}  // namespace msx
