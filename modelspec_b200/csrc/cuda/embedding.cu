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

// rank[n] = how many earlier n' hold the same id; count[id] = occurrences of id. Four lanes per
// n, each scanning a quarter of every 1024-id tile of the ids before it, staged through shared
// memory.
__global__ void rank_kernel(const int32_t* __restrict__ ids, uint32_t n, uint32_t rows, int32_t* __restrict__ rank,
                            int32_t* __restrict__ count, uint32_t* __restrict__ status) {
    __shared__ int32_t tile[1024];
    const uint32_t per_block = blockDim.x / 4;
    uint32_t i = blockIdx.x * per_block + threadIdx.x / 4, part = threadIdx.x & 3u;
    int32_t mine = i < n ? ids[i] : -1;
    bool valid = i < n && mine >= 0 && static_cast<uint32_t>(mine) < rows;
    if (i < n && !valid && part == 0) atomicOr(status, 1u);
    // Only ids before the block's last n matter to anyone in the block.
    uint32_t block_last = min(n, (blockIdx.x + 1) * per_block);
    int32_t earlier = 0;
    for (uint32_t t0 = 0; t0 < block_last; t0 += 1024) {
        __syncthreads();
        for (uint32_t j = threadIdx.x; j < 1024; j += blockDim.x) tile[j] = t0 + j < n ? ids[t0 + j] : -2;
        __syncthreads();
        if (!valid || t0 >= i) continue;
        uint32_t stop = min(i, t0 + 1024u) - t0;
        // Interleaved quarters keep the four lanes on different banks.
        for (uint32_t j = part; j < stop; j += 4) earlier += tile[j] == mine ? 1 : 0;
    }
    earlier += __shfl_xor_sync(0xffffffffu, earlier, 1);
    earlier += __shfl_xor_sync(0xffffffffu, earlier, 2);
    if (part != 0) return;
    if (valid) {
        rank[i] = earlier;
        atomicAdd(&count[mine], 1);  // integer: the total does not depend on the order
    } else if (i < n) {
        rank[i] = -1;
    }
}

// offset[r] = sum of count[0 .. r): one CTA of 1024 threads walks the rows 1024 at a time with
// coalesced loads, a warp-shuffle scan inside each warp and a scan of the 32 warp totals.
__global__ void offsets_kernel(const int32_t* __restrict__ count, uint32_t rows, int32_t* __restrict__ offset) {
    __shared__ int32_t warp_total[32], warp_prefix[32];
    __shared__ int32_t carry, chunk_total;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (uint32_t base = 0; base < rows; base += 1024) {
        uint32_t r = base + threadIdx.x;
        int32_t c = r < rows ? count[r] : 0;
        int32_t inclusive = c;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            int32_t up = __shfl_up_sync(0xffffffffu, inclusive, d);
            if (lane >= static_cast<uint32_t>(d)) inclusive += up;
        }
        if (lane == 31) warp_total[warp] = inclusive;
        __syncthreads();
        if (warp == 0) {
            int32_t t = warp_total[lane], scan = t;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                int32_t up = __shfl_up_sync(0xffffffffu, scan, d);
                if (lane >= static_cast<uint32_t>(d)) scan += up;
            }
            warp_prefix[lane] = scan - t;
            if (lane == 31) chunk_total = scan;
        }
        __syncthreads();
        if (r < rows) offset[r] = carry + warp_prefix[warp] + inclusive - c;
        __syncthreads();
        if (threadIdx.x == 0) carry += chunk_total;
        __syncthreads();
    }
}

// list[offset[id] + rank] = n: the occurrences of each id, ascending.
__global__ void list_kernel(const int32_t* __restrict__ ids, uint32_t n, const int32_t* __restrict__ rank,
                            const int32_t* __restrict__ offset, int32_t* __restrict__ list) {
    uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && rank[i] >= 0) list[offset[ids[i]] + rank[i]] = static_cast<int32_t>(i);
}

// One warp per (table row, group of 32 columns), lane = column: 0 + g[n0] + g[n1] + ... over the
// row's occurrences in ascending n. The additions stay in order; the loads of up to 32
// occurrences are issued together, so a row hit hundreds of times costs a few memory round
// trips, not one per occurrence.
__global__ void scatter_kernel(const float* __restrict__ g, const int32_t* __restrict__ list,
                               const int32_t* __restrict__ offset, const int32_t* __restrict__ count,
                               float* __restrict__ out, uint32_t rows, uint32_t h) {
    const uint32_t groups = (h + 31) / 32;
    const uint64_t items = static_cast<uint64_t>(rows) * groups;
    uint64_t item = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warps = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 5;
    for (; item < items; item += warps) {
        const uint32_t row = static_cast<uint32_t>(item / groups), col = static_cast<uint32_t>(item % groups) * 32 + lane;
        const int32_t c = count[row];
        const int32_t* mine = list + offset[row];
        const bool in = col < h;
        float acc = 0.0f;
        for (int32_t i0 = 0; i0 < c; i0 += 32) {
            const int32_t entry = i0 + static_cast<int32_t>(lane) < c ? mine[i0 + lane] : 0;
            const int32_t here = min(32, c - i0);
            float v[32];
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const int32_t n = __shfl_sync(0xffffffffu, entry, e);
                v[e] = (e < here && in) ? g[static_cast<uint64_t>(n) * h + col] : 0.0f;
            }
#pragma unroll
            for (int e = 0; e < 32; ++e)
                if (e < here) acc = acc + v[e];
        }
        if (in) out[static_cast<uint64_t>(row) * h + col] = acc;
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
        rank_kernel<<<static_cast<uint32_t>((n + 63) / 64), 256, 0, s>>>(ids, static_cast<uint32_t>(n), static_cast<uint32_t>(rows), rank, count, status);
        check_launch("embedding_grad");
        offsets_kernel<<<1, 1024, 0, s>>>(count, static_cast<uint32_t>(rows), offset);
        check_launch("embedding_grad");
        list_kernel<<<blocks, 256, 0, s>>>(ids, static_cast<uint32_t>(n), rank, offset, list);
        check_launch("embedding_grad");
    }
    uint64_t blocks = (rows * ((h + 31) / 32) * 32 + 255) / 256;
    uint32_t grid = static_cast<uint32_t>(blocks > 148 * 32 ? 148 * 32 : blocks);
    scatter_kernel<<<grid, 256, 0, s>>>(g, list, offset, count, out, static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
    check_launch("embedding_grad");
}

}  // namespace k
}  // namespace msx
