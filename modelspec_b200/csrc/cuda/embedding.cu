// Embedding gather and its scatter-add gradient.
//
// The gather copies rows (bit-exact). The gradient adds row g[n] to row ids[n] of a zero tensor
// in ascending n, as the reference's sequential loop does
// (crates/modelspec-runtime/src/cpu/interpreter.rs:923-941), without atomics: a first kernel links
// the occurrences of each id into an ascending chain (next[n] = the next n' > n with the same id)
// and records the chain head of every table row; a second kernel writes every output element
// once, walking its row's chain in order. The result is bit-identical to the sequential loop,
// including `0 + g` for the first occurrence. The reference's Vulkan path reaches the same order
// with a rank sort of the ids (crates/modelspec-runtime/src/spirv/emit/rowwise.rs:1024-1190).
// HBM-bound: the output is written once (rows * h * 4 bytes), g is read once.
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

__global__ void embedding_kernel(const float* __restrict__ table, const int32_t* __restrict__ ids,
                                 float* __restrict__ out, uint64_t n, uint32_t rows, uint32_t h,
                                 uint32_t* __restrict__ status) {
    // One warp per output row, 128-bit copies when the row length allows.
    uint64_t row = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    uint64_t warps = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 5;
    for (; row < n; row += warps) {
        int32_t id = ids[row];
        bool ok = id >= 0 && static_cast<uint32_t>(id) < rows;
        if (!ok && lane == 0) atomicOr(status, 1u);
        const float* src = table + static_cast<uint64_t>(ok ? id : 0) * h;
        float* dst = out + row * h;
        if (h % 4 == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0) {
            for (uint32_t j = lane; j < h / 4; j += 32) {
                float4 v = ok ? reinterpret_cast<const float4*>(src)[j] : make_float4(0.f, 0.f, 0.f, 0.f);
                reinterpret_cast<float4*>(dst)[j] = v;
            }
        } else {
            for (uint32_t j = lane; j < h; j += 32) dst[j] = ok ? src[j] : 0.0f;
        }
    }
}

// next[n] = smallest n' > n with ids[n'] == ids[n], else -1; head[ids[n]] = n when no earlier
// occurrence exists. One thread per n; ids are staged through shared memory in tiles.
__global__ void link_kernel(const int32_t* __restrict__ ids, uint32_t n, uint32_t rows,
                            int32_t* __restrict__ next, int32_t* __restrict__ head,
                            uint32_t* __restrict__ status) {
    __shared__ int32_t tile[1024];
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    int32_t mine = i < n ? ids[i] : -1;
    bool valid = i < n && mine >= 0 && static_cast<uint32_t>(mine) < rows;
    if (i < n && !valid) atomicOr(status, 1u);
    bool first = true;
    int32_t nxt = -1;
    for (uint32_t t0 = 0; t0 < n; t0 += 1024) {
        __syncthreads();
        for (uint32_t j = threadIdx.x; j < 1024; j += blockDim.x) tile[j] = t0 + j < n ? ids[t0 + j] : -2;
        __syncthreads();
        if (!valid) continue;
        uint32_t t1 = min(n, t0 + 1024u);
        if (t1 <= i) {
            // Entirely before i: only asks whether an earlier occurrence exists.
            if (first)
                for (uint32_t j = t0; j < t1; ++j)
                    if (tile[j - t0] == mine) { first = false; break; }
        } else if (nxt < 0) {
            for (uint32_t j = t0; j < t1; ++j) {
                if (tile[j - t0] != mine) continue;
                if (j < i) first = false;
                else if (j > i) { nxt = static_cast<int32_t>(j); break; }
            }
        }
    }
    if (valid) {
        next[i] = nxt;
        if (first) head[mine] = static_cast<int32_t>(i);
    } else if (i < n) {
        next[i] = -1;
    }
}

__global__ void scatter_kernel(const float* __restrict__ g, const int32_t* __restrict__ next,
                               const int32_t* __restrict__ head, float* __restrict__ out, uint32_t rows,
                               uint32_t h) {
    // One warp per table row.
    uint64_t row = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    uint64_t warps = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 5;
    for (; row < rows; row += warps) {
        int32_t first = head[row];
        float* dst = out + row * h;
        for (uint32_t j = lane; j < h; j += 32) {
            float acc = 0.0f;
            for (int32_t n = first; n >= 0; n = next[n]) acc = acc + g[static_cast<uint64_t>(n) * h + j];
            dst[j] = acc;
        }
    }
}

}  // namespace

void embedding(cudaStream_t s, const float* table, const int32_t* ids, float* out, uint64_t n,
               uint64_t rows, uint64_t h, uint32_t* status) {
    if (n == 0 || h == 0) return;
    uint64_t blocks = (n * 32 + 255) / 256;
    uint32_t grid = static_cast<uint32_t>(blocks > 148 * 16 ? 148 * 16 : blocks);
    embedding_kernel<<<grid, 256, 0, s>>>(table, ids, out, n, static_cast<uint32_t>(rows), static_cast<uint32_t>(h), status);
    check_launch("embedding");
}

uint64_t embedding_grad_scratch_ints(uint64_t n, uint64_t rows) { return n + rows; }

void embedding_grad(cudaStream_t s, const int32_t* ids, const float* g, float* out, uint64_t n,
                    uint64_t rows, uint64_t h, int32_t* scratch, uint32_t* status) {
    if (rows == 0 || h == 0) return;
    int32_t* next = scratch;
    int32_t* head = scratch + n;
    check(cudaMemsetAsync(head, 0xff, rows * sizeof(int32_t), s), "embedding_grad memset");
    if (n > 0) {
        link_kernel<<<static_cast<uint32_t>((n + 255) / 256), 256, 0, s>>>(ids, static_cast<uint32_t>(n),
                                                                          static_cast<uint32_t>(rows), next, head, status);
        check_launch("embedding_grad");
    }
    uint64_t blocks = (rows * 32 + 255) / 256;
    uint32_t grid = static_cast<uint32_t>(blocks > 148 * 16 ? 148 * 16 : blocks);
    scatter_kernel<<<grid, 256, 0, s>>>(g, next, head, out, static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
    check_launch("embedding_grad");
}

}  // namespace k
}  // namespace msx
