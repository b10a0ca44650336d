// Embedding gather and its scatter-add gradient.
//
// The gather copies rows (bit-exact). The gradient adds row g[n] to row ids[n] of a zero tensor
// in ascending n, as the reference's sequential loop does
// (crates/modelspec-runtime/src/cpu/interpreter.rs:923-941), without floating-point atomics: a
// counting sort groups the occurrences of each id in ascending n (rank among earlier equal ids,
// per-id counts by integer atomics, an exclusive scan for the group offsets), and one warp per
// table row then adds its group's rows of g in that order, loads issued ahead of the dependent
// additions. The result is bit-identical to the sequential loop, including `0 + g` for the first
// occurrence and an exact zero row for an id never read. The reference's Vulkan path reaches the same order
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

// rank[n] = how many earlier n' hold the same id; count[id] = occurrences of id. One thread per
// n; the ids before it are staged through shared memory in tiles of 1024.
__global__ void rank_kernel(const int32_t* __restrict__ ids, uint32_t n, uint32_t rows, int32_t* __restrict__ rank,
                            int32_t* __restrict__ count, uint32_t* __restrict__ status) {
    __shared__ int32_t tile[1024];
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    int32_t mine = i < n ? ids[i] : -1;
    bool valid = i < n && mine >= 0 && static_cast<uint32_t>(mine) < rows;
    if (i < n && !valid) atomicOr(status, 1u);
    // Only ids before the block's last thread matter to anyone in the block.
    uint32_t block_last = min(n, (blockIdx.x + 1) * blockDim.x);
    int32_t earlier = 0;
    for (uint32_t t0 = 0; t0 < block_last; t0 += 1024) {
        __syncthreads();
        for (uint32_t j = threadIdx.x; j < 1024; j += blockDim.x) tile[j] = t0 + j < n ? ids[t0 + j] : -2;
        __syncthreads();
        if (!valid || t0 >= i) continue;
        uint32_t stop = min(i, t0 + 1024u) - t0;
        for (uint32_t j = 0; j < stop; ++j) earlier += tile[j] == mine ? 1 : 0;
    }
    if (valid) {
        rank[i] = earlier;
        atomicAdd(&count[mine], 1);  // integer: the total does not depend on the order
    } else if (i < n) {
        rank[i] = -1;
    }
}

// offset[r] = sum of count[0 .. r): one CTA, each thread a contiguous run of rows.
__global__ void offsets_kernel(const int32_t* __restrict__ count, uint32_t rows, int32_t* __restrict__ offset) {
    __shared__ int32_t sums[1024];
    uint32_t per = (rows + blockDim.x - 1) / blockDim.x;
    uint32_t begin = min(rows, threadIdx.x * per), end = min(rows, begin + per);
    int32_t local = 0;
    for (uint32_t r = begin; r < end; ++r) local += count[r];
    sums[threadIdx.x] = local;
    __syncthreads();
    // Hillis-Steele inclusive scan over the per-thread sums.
    for (uint32_t d = 1; d < blockDim.x; d <<= 1) {
        int32_t add = threadIdx.x >= d ? sums[threadIdx.x - d] : 0;
        __syncthreads();
        sums[threadIdx.x] += add;
        __syncthreads();
    }
    int32_t running = sums[threadIdx.x] - local;
    for (uint32_t r = begin; r < end; ++r) {
        offset[r] = running;
        running += count[r];
    }
}

// list[offset[id] + rank] = n: the occurrences of each id, ascending.
__global__ void list_kernel(const int32_t* __restrict__ ids, uint32_t n, const int32_t* __restrict__ rank,
                            const int32_t* __restrict__ offset, int32_t* __restrict__ list) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && rank[i] >= 0) list[offset[ids[i]] + rank[i]] = static_cast<int32_t>(i);
}

// One warp per table row: 0 + g[n0] + g[n1] + ... over the row's occurrences in ascending n, the
// additions in order, the loads ahead of them.
__global__ void scatter_kernel(const float* __restrict__ g, const int32_t* __restrict__ list,
                               const int32_t* __restrict__ offset, const int32_t* __restrict__ count,
                               float* __restrict__ out, uint32_t rows, uint32_t h) {
    uint64_t row = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    uint64_t warps = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 5;
    for (; row < rows; row += warps) {
        int32_t c = count[row];
        const int32_t* mine = list + offset[row];
        float* dst = out + row * h;
        for (uint32_t j0 = 0; j0 < h; j0 += 128) {
            // Up to four columns per lane at a time, so one pass over the list serves 128 columns.
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            int32_t i = 0;
            for (; i + 4 <= c; i += 4) {
                int32_t n0 = mine[i], n1 = mine[i + 1], n2 = mine[i + 2], n3 = mine[i + 3];
                float v[4][4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t j = j0 + q * 32 + lane;
                    bool in = j < h;
                    v[0][q] = in ? g[static_cast<uint64_t>(n0) * h + j] : 0.0f;
                    v[1][q] = in ? g[static_cast<uint64_t>(n1) * h + j] : 0.0f;
                    v[2][q] = in ? g[static_cast<uint64_t>(n2) * h + j] : 0.0f;
                    v[3][q] = in ? g[static_cast<uint64_t>(n3) * h + j] : 0.0f;
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[q] = (((acc[q] + v[0][q]) + v[1][q]) + v[2][q]) + v[3][q];
            }
            for (; i < c; ++i) {
                int32_t n = mine[i];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t j = j0 + q * 32 + lane;
                    if (j < h) acc[q] = acc[q] + g[static_cast<uint64_t>(n) * h + j];
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t j = j0 + q * 32 + lane;
                if (j < h) dst[j] = acc[q];
            }
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

uint64_t embedding_grad_scratch_ints(uint64_t n, uint64_t rows) { return 2 * n + 2 * rows; }

void embedding_grad(cudaStream_t s, const int32_t* ids, const float* g, float* out, uint64_t n,
                    uint64_t rows, uint64_t h, int32_t* scratch, uint32_t* status) {
    if (rows == 0 || h == 0) return;
    int32_t* rank = scratch;
    int32_t* list = scratch + n;
    int32_t* count = scratch + 2 * n;
    int32_t* offset = count + rows;
    check(cudaMemsetAsync(count, 0, rows * sizeof(int32_t), s), "embedding_grad memset");
    if (n > 0) {
        uint32_t blocks = static_cast<uint32_t>((n + 255) / 256);
        rank_kernel<<<blocks, 256, 0, s>>>(ids, static_cast<uint32_t>(n), static_cast<uint32_t>(rows), rank, count, status);
        check_launch("embedding_grad");
        offsets_kernel<<<1, 1024, 0, s>>>(count, static_cast<uint32_t>(rows), offset);
        check_launch("embedding_grad");
        list_kernel<<<blocks, 256, 0, s>>>(ids, static_cast<uint32_t>(n), rank, offset, list);
        check_launch("embedding_grad");
    }
    uint64_t blocks = (rows * 32 + 255) / 256;
    uint32_t grid = static_cast<uint32_t>(blocks > 148 * 16 ? 148 * 16 : blocks);
    scatter_kernel<<<grid, 256, 0, s>>>(g, list, offset, count, out, static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
    check_launch("embedding_grad");
}

}  // namespace k
}  // namespace msx
