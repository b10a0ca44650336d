// Embedding gather and its scatter-add gradient.
//
// The gather copies rows (bit-exact). The gradient adds row g[n] to row ids[n] of a zero tensor
// in ascending n, as the reference's sequential loop does
// (crates/modelspec-runtime/src/cpu/interpreter.rs:923-941), without floating-point atomics: a
// sort by counting (the position of an occurrence is the number of occurrences that precede it in
// (id, n) order) groups the occurrences of each id in ascending n, and one warp per table row
// then finds its group by a search and adds those rows of g in that order, loads issued ahead of
// the dependent additions. The result is bit-identical to the sequential loop, including `0 + g` for the first
// occurrence and an exact zero row for an id never read. The reference's Vulkan path reaches the same order
// with a rank sort of the ids (crates/modelspec-runtime/src/spirv/emit/rowwise.rs:1024-1190).
// HBM-bound: the output is written once (rows * h * 4 bytes), g is read once. With `base` the
// result is base + that sum (one more rounded addition per element, the Add that follows the
// scatter when a tied weight has a second, dense gradient).
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

template <class TI, class TO>
__global__ void embedding_kernel(const TI* __restrict__ table, const int32_t* __restrict__ ids,
                                 TO* __restrict__ out, uint64_t n, uint32_t rows, uint32_t h,
                                 uint32_t* __restrict__ status) {
    // One warp per output row, 128-bit copies when the row length allows.
    uint64_t row = (static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    uint64_t warps = (static_cast<uint64_t>(gridDim.x) * blockDim.x) >> 5;
    for (; row < n; row += warps) {
        int32_t id = ids[row];
        bool ok = id >= 0 && static_cast<uint32_t>(id) < rows;
        if (!ok && lane == 0) atomicOr(status, 1u);
        const TI* src = table + static_cast<uint64_t>(ok ? id : 0) * h;
        TO* dst = out + row * h;
        if (h % 4 == 0 && reinterpret_cast<uintptr_t>(table) % (4 * sizeof(TI)) == 0 && reinterpret_cast<uintptr_t>(out) % (4 * sizeof(TO)) == 0) {
            for (uint32_t j = lane; j < h / 4; j += 32) store4(dst + 4 * j, ok ? load4(src + 4 * j) : make_float4(0.f, 0.f, 0.f, 0.f));
        } else {
            for (uint32_t j = lane; j < h; j += 32) store1(dst + j, ok ? load1(src + j) : 0.0f);
        }
    }
}

// Sorted position of occurrence i among all n: the number of occurrences with a smaller id, plus
// the earlier ones with the same id. Writing (id, i) there sorts the occurrences by id, ascending
// n within an id, without atomics. Eight lanes per occurrence each compare an eighth of every
// 4096-id tile, read from shared memory as broadcast int4; an id outside the table sorts last and
// is never matched by a row. n^2 / 8 comparisons per lane group: 2 M for n = 4096.
constexpr int kOrderTile = 4096;
__global__ void __launch_bounds__(256) order_kernel(const int32_t* __restrict__ ids, uint32_t n, uint32_t rows,
                                                    int32_t* __restrict__ sorted_id, int32_t* __restrict__ sorted_n,
                                                    uint32_t* __restrict__ status) {
    __shared__ int4 tile[kOrderTile / 4];
    const uint32_t i = blockIdx.x * 32 + threadIdx.x / 8, part = threadIdx.x & 7u;
    int32_t mine = i < n ? ids[i] : 0;
    const bool inside = i < n && mine >= 0 && static_cast<uint32_t>(mine) < rows;
    if (i < n && !inside) {
        if (part == 0) atomicOr(status, 1u);
        mine = INT32_MAX;
    }
    uint32_t before = 0;
    for (uint32_t t0 = 0; t0 < n; t0 += kOrderTile) {
        __syncthreads();
        for (uint32_t j = threadIdx.x; j < kOrderTile / 4; j += 256) {
            int4 v;
            int32_t* e = reinterpret_cast<int32_t*>(&v);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t at = t0 + 4 * j + q;
                int32_t id = at < n ? ids[at] : INT32_MAX;
                e[q] = (at < n && (id < 0 || static_cast<uint32_t>(id) >= rows)) ? INT32_MAX : id;
            }
            tile[j] = v;
        }
        __syncthreads();
        if (i >= n) continue;
        const uint32_t stop = min(n - t0, static_cast<uint32_t>(kOrderTile));
        for (uint32_t j = part; 4 * j < stop; j += 8) {
            const int4 v = tile[j];
            const int32_t* e = reinterpret_cast<const int32_t*>(&v);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint32_t at = t0 + 4 * j + q;
                // Padding past n holds INT32_MAX at an index above every i: never counted.
                before += (e[q] < mine || (e[q] == mine && at < i)) ? 1u : 0u;
            }
        }
    }
    before += __shfl_xor_sync(0xffffffffu, before, 1);
    before += __shfl_xor_sync(0xffffffffu, before, 2);
    before += __shfl_xor_sync(0xffffffffu, before, 4);
    if (part == 0 && i < n) {
        sorted_id[before] = mine;
        sorted_n[before] = static_cast<int32_t>(i);
    }
}

// First position in sorted_id[0 .. n) whose id is not below `row`, by a 32-way search: each
// round the lanes probe 32 evenly spaced positions of the remaining range.
__device__ __forceinline__ uint32_t warp_lower_bound(const int32_t* __restrict__ sorted_id, uint32_t n, int32_t row, uint32_t lane) {
    uint32_t lo = 0, hi = n;
    while (lo < hi) {
        const uint32_t step = (hi - lo + 31) / 32;
        const uint32_t probe = lo + lane * step;
        const bool below = probe < hi && sorted_id[probe] < row;
        const uint32_t count = __popc(__ballot_sync(0xffffffffu, below));
        if (count == 0) return lo;
        const uint32_t next_hi = min(hi, lo + count * step);
        lo = lo + (count - 1) * step + 1;
        hi = next_hi;
    }
    return lo;
}

// One warp per (table row, group of VEC * 32 columns), eight per block: base + (0 + g[n0] + g[n1]
// + ...) over the row's occurrences in ascending n. The additions stay in order. A row read up to
// 32 times is summed by its warp, the loads of 8 occurrences issued together. A hotter row (the
// mask token, a padding position: hundreds of occurrences) would be one warp waiting on memory
// hundreds of times: the block takes it together instead, all 256 threads streaming 32
// occurrences at a time into shared memory while one thread per column adds the previous 32 in
// order. A row nobody read gets `base` (or zero); when base is out itself, such a row is left
// alone and only the rows some id names are read and written. VEC = 4 reads and writes 16 bytes
// per lane and needs h % 4 == 0 and 16-byte aligned g, base and out.
constexpr uint32_t kHotRow = 32, kHotChunk = 32, kCachedIds = 4096;
template <int VEC, class TG, class TO>
__global__ void __launch_bounds__(256) scatter_kernel(const TG* __restrict__ g, const int32_t* __restrict__ sorted_id,
                                                      const int32_t* __restrict__ sorted_n, uint32_t n,
                                                      const float* base, TO* out, uint32_t rows, uint32_t h) {
    constexpr uint32_t span = VEC * 32;
    constexpr int LOADS = kHotChunk * span / VEC / 256;
    __shared__ float stage[kHotChunk][span];
    __shared__ int32_t cached_ids[kCachedIds];
    __shared__ uint32_t hot_item[8], hot_at[8], hot_count[8], hot_rows;
    // Every row's warp searches the sorted ids: up to 4096 of them are copied into shared memory
    // once per block (a block walks many rows), so that a search round is a shared-memory read.
    const int32_t* ids = sorted_id;
    if (n <= kCachedIds) {
        for (uint32_t j = threadIdx.x; j < n; j += blockDim.x) cached_ids[j] = sorted_id[j];
        ids = cached_ids;
        __syncthreads();
    }
    const uint32_t groups = (h + span - 1) / span;
    const uint64_t items = static_cast<uint64_t>(rows) * groups;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // Neighbouring rows go to different blocks: the hot rows of a vocabulary sit together (the most
    // frequent tokens have neighbouring ids), and each is a serial job for the block that gets it.
    for (uint64_t first = blockIdx.x; first < items; first += static_cast<uint64_t>(gridDim.x) * 8) {
        if (threadIdx.x == 0) hot_rows = 0;
        __syncthreads();
        const uint64_t item = first + static_cast<uint64_t>(warp) * gridDim.x;
        if (item < items) {
            const uint32_t row = static_cast<uint32_t>(item / groups), col = static_cast<uint32_t>(item % groups) * span + lane * VEC;
            const bool in = col < h;
            uint32_t at = n ? warp_lower_bound(ids, n, static_cast<int32_t>(row), lane) : 0u;
            uint32_t count = 0;
            if (at < n && ids[at] == static_cast<int32_t>(row))
                count = warp_lower_bound(ids, n, static_cast<int32_t>(row) + 1, lane) - at;
            if (count > kHotRow) {
                if (lane == 0) {
                    uint32_t slot = atomicAdd(&hot_rows, 1u);
                    hot_item[slot] = warp;
                    hot_at[slot] = at;
                    hot_count[slot] = count;
                }
            } else {
                float acc[VEC];
#pragma unroll
                for (int q = 0; q < VEC; ++q) acc[q] = 0.0f;
                for (uint32_t done = 0; done < count; done += 8) {
                    const uint32_t here = min(8u, count - done);
                    const int32_t entry = lane < here ? __ldg(sorted_n + at + done + lane) : 0;
                    float v[8][VEC];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int32_t src = __shfl_sync(0xffffffffu, entry, e);
                        const TG* from = g + static_cast<uint64_t>(src) * h + col;
                        if (static_cast<uint32_t>(e) < here && in) {
                            if (VEC == 4) {
                                const float4 f = load4(from);
                                v[e][0] = f.x; v[e][1 % VEC] = f.y; v[e][2 % VEC] = f.z; v[e][3 % VEC] = f.w;
                            } else {
                                v[e][0] = load1(from);
                            }
                        } else {
#pragma unroll
                            for (int q = 0; q < VEC; ++q) v[e][q] = 0.0f;
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (static_cast<uint32_t>(e) < here) {
#pragma unroll
                            for (int q = 0; q < VEC; ++q) acc[q] = acc[q] + v[e][q];
                        }
                }
                // In place (base is out): a row nobody read already holds its result.
                if (in && !(count == 0 && static_cast<const void*>(base) == static_cast<const void*>(out))) {
                    TO* to = out + static_cast<uint64_t>(row) * h + col;
                    if (VEC == 4) {
                        float4 r = make_float4(acc[0], acc[1 % VEC], acc[2 % VEC], acc[3 % VEC]);
                        if (base) {
                            const float4 b = *reinterpret_cast<const float4*>(base + static_cast<uint64_t>(row) * h + col);
                            r.x = b.x + r.x; r.y = b.y + r.y; r.z = b.z + r.z; r.w = b.w + r.w;
                        }
                        store4(to, r);
                    } else {
                        store1(to, base ? base[static_cast<uint64_t>(row) * h + col] + acc[0] : acc[0]);
                    }
                }
            }
        }
        __syncthreads();
        // The hot rows of this round, one after another, by the whole block (in slot order: which
        // warp took which slot does not change any sum).
        const uint32_t hot = hot_rows;
        for (uint32_t slot = 0; slot < hot; ++slot) {
            const uint64_t hot_id = first + static_cast<uint64_t>(hot_item[slot]) * gridDim.x;
            const uint32_t row = static_cast<uint32_t>(hot_id / groups), col0 = static_cast<uint32_t>(hot_id % groups) * span;
            const uint32_t at = hot_at[slot], count = hot_count[slot];
            // Two chunks of loads are in flight while a third is added: one round trip to memory
            // per chunk would otherwise be the whole cost of a hot row.
            float4 held4[2][VEC == 4 ? LOADS : 1];
            float held1[2][VEC == 1 ? LOADS : 1];
            auto fetch = [&](uint32_t chunk_start, int set) {
#pragma unroll
                for (int j = 0; j < LOADS; ++j) {
                    const uint32_t f = threadIdx.x + 256 * j;
                    const uint32_t r = f / (span / VEC), c = (f % (span / VEC)) * VEC;
                    const bool wanted = chunk_start + r < count && col0 + c < h;
                    const int32_t src = wanted ? __ldg(sorted_n + at + chunk_start + r) : 0;
                    const TG* from = g + static_cast<uint64_t>(src) * h + col0 + c;
                    if (VEC == 4) held4[set][j % (VEC == 4 ? LOADS : 1)] = wanted ? load4(from) : make_float4(0.f, 0.f, 0.f, 0.f);
                    else held1[set][j % (VEC == 1 ? LOADS : 1)] = wanted ? load1(from) : 0.0f;
                }
            };
            float acc = 0.0f;
            fetch(0, 0);
            if (kHotChunk < count) fetch(kHotChunk, 1);
            for (uint32_t pair = 0; pair < count; pair += 2 * kHotChunk) {
#pragma unroll
                for (int set = 0; set < 2; ++set) {
                    const uint32_t start = pair + set * kHotChunk;
                    if (start >= count) break;
#pragma unroll
                    for (int j = 0; j < LOADS; ++j) {
                        const uint32_t f = threadIdx.x + 256 * j;
                        const uint32_t r = f / (span / VEC), c = (f % (span / VEC)) * VEC;
                        if (VEC == 4) *reinterpret_cast<float4*>(&stage[r][c]) = held4[set][j % (VEC == 4 ? LOADS : 1)];
                        else stage[r][c] = held1[set][j % (VEC == 1 ? LOADS : 1)];
                    }
                    __syncthreads();
                    if (start + 2 * kHotChunk < count) fetch(start + 2 * kHotChunk, set);
                    if (threadIdx.x < span) {
                        const uint32_t here = min(kHotChunk, count - start);
                        if (here == kHotChunk) {
                            // A whole chunk: every value is read before the first is added (the additions
                            // are a chain; a read inside it would be a round trip each).
                            float t[kHotChunk];
#pragma unroll
                            for (uint32_t r = 0; r < kHotChunk; ++r) t[r] = stage[r][threadIdx.x];
#pragma unroll
                            for (uint32_t r = 0; r < kHotChunk; ++r) acc = acc + t[r];
                        } else {
                            for (uint32_t r = 0; r < here; ++r) acc = acc + stage[r][threadIdx.x];
                        }
                    }
                    __syncthreads();
                }
            }
            if (threadIdx.x < span && col0 + threadIdx.x < h) {
                const uint64_t where = static_cast<uint64_t>(row) * h + col0 + threadIdx.x;
                store1(out + where, base ? base[where] + acc : acc);
            }
        }
    }
}


// The in-place form (a tied table: `out` already holds the dense gradient and only the rows some
// id names change): one warp per sorted position instead of one per table row. The warp whose
// position starts a run of equal ids owns that row: it counts the run (the lanes compare the next
// 32 ids at a time) and adds `out[row] + (0 + g[n0] + g[n1] + ...)` exactly as the row walk above
// does; the other positions have nothing to do. A step names a few thousand of a vocabulary's
// 30,522 rows, so this visits n positions where the row walk visits every row twice (two
// searches); a hot row's run is long, so two hot rows never start within one block's eight
// positions and the block-wide path below takes at most one of them.
template <int VEC, class TG, class TO>
__global__ void __launch_bounds__(256) scatter_in_place_kernel(const TG* __restrict__ g, const int32_t* __restrict__ sorted_id,
                                                               const int32_t* __restrict__ sorted_n, uint32_t n, TO* out, uint32_t rows,
                                                               uint32_t h) {
    constexpr uint32_t span = VEC * 32;
    constexpr int LOADS = kHotChunk * span / VEC / 256;
    __shared__ float stage[kHotChunk][span];
    __shared__ uint32_t hot_row, hot_at, hot_count, hot_group;
    const uint32_t groups = (h + span - 1) / span;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint32_t group = 0; group < groups; ++group) {
        if (threadIdx.x == 0) hot_count = 0;
        __syncthreads();
        const uint32_t p = blockIdx.x * 8 + warp, col = group * span + lane * VEC;
        const bool in = col < h;
        const int32_t id = p < n ? sorted_id[p] : -1;
        const bool head = p < n && id >= 0 && static_cast<uint32_t>(id) < rows && (p == 0 || sorted_id[p - 1] != id);
        if (head) {  // the same for the whole warp
            // The run of this id: ids are sorted, so it ends at the first different one. The
            // next 32 positions are looked at side by side (most runs end there); a longer run's
            // end is searched for, 32 probes a round.
            const uint32_t probe = p + 1 + lane;
            const uint32_t same = __ballot_sync(0xffffffffu, probe < n && sorted_id[probe] == id);
            const uint32_t count = same == 0xffffffffu ? warp_lower_bound(sorted_id, n, id + 1, lane) - p : __ffs(~same);
            if (count > kHotRow) {
                if (lane == 0) {
                    hot_row = static_cast<uint32_t>(id);
                    hot_at = p;
                    hot_count = count;
                    hot_group = group;
                }
            } else {
                float acc[VEC];
#pragma unroll
                for (int q = 0; q < VEC; ++q) acc[q] = 0.0f;
                for (uint32_t done = 0; done < count; done += 8) {
                    const uint32_t here = min(8u, count - done);
                    const int32_t entry = lane < here ? __ldg(sorted_n + p + done + lane) : 0;
                    float v[8][VEC];
#pragma unroll
                    for (int e = 0; e < 8; ++e) {
                        const int32_t src = __shfl_sync(0xffffffffu, entry, e);
                        const TG* from = g + static_cast<uint64_t>(src) * h + col;
                        if (static_cast<uint32_t>(e) < here && in) {
                            if (VEC == 4) {
                                const float4 f = load4(from);
                                v[e][0] = f.x; v[e][1 % VEC] = f.y; v[e][2 % VEC] = f.z; v[e][3 % VEC] = f.w;
                            } else {
                                v[e][0] = load1(from);
                            }
                        } else {
#pragma unroll
                            for (int q = 0; q < VEC; ++q) v[e][q] = 0.0f;
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 8; ++e)
                        if (static_cast<uint32_t>(e) < here) {
#pragma unroll
                            for (int q = 0; q < VEC; ++q) acc[q] = acc[q] + v[e][q];
                        }
                }
                if (in) {
                    TO* to = out + static_cast<uint64_t>(id) * h + col;
                    if (VEC == 4) {
                        const float4 b = *reinterpret_cast<const float4*>(to);
                        store4(to, make_float4(b.x + acc[0], b.y + acc[1 % VEC], b.z + acc[2 % VEC], b.w + acc[3 % VEC]));
                    } else {
                        store1(to, static_cast<float>(*to) + acc[0]);
                    }
                }
            }
        }
        __syncthreads();
        // The block's hot row, if one starts here, by the whole block: 32 occurrences at a time
        // into shared memory, two chunks of loads in flight while a third is added in order.
        const uint32_t count = hot_count;
        if (count == 0) continue;
        const uint32_t row = hot_row, at = hot_at, col0 = hot_group * span;
        float4 held4[2][VEC == 4 ? LOADS : 1];
        float held1[2][VEC == 1 ? LOADS : 1];
        auto fetch = [&](uint32_t chunk_start, int set) {
#pragma unroll
            for (int j = 0; j < LOADS; ++j) {
                const uint32_t f = threadIdx.x + 256 * j;
                const uint32_t r = f / (span / VEC), c = (f % (span / VEC)) * VEC;
                const bool wanted = chunk_start + r < count && col0 + c < h;
                const int32_t src = wanted ? __ldg(sorted_n + at + chunk_start + r) : 0;
                const TG* from = g + static_cast<uint64_t>(src) * h + col0 + c;
                if (VEC == 4) held4[set][j % (VEC == 4 ? LOADS : 1)] = wanted ? load4(from) : make_float4(0.f, 0.f, 0.f, 0.f);
                else held1[set][j % (VEC == 1 ? LOADS : 1)] = wanted ? load1(from) : 0.0f;
            }
        };
        float acc = 0.0f;
        fetch(0, 0);
        if (kHotChunk < count) fetch(kHotChunk, 1);
        for (uint32_t pair = 0; pair < count; pair += 2 * kHotChunk) {
#pragma unroll
            for (int set = 0; set < 2; ++set) {
                const uint32_t start = pair + set * kHotChunk;
                if (start >= count) break;
#pragma unroll
                for (int j = 0; j < LOADS; ++j) {
                    const uint32_t f = threadIdx.x + 256 * j;
                    const uint32_t r = f / (span / VEC), c = (f % (span / VEC)) * VEC;
                    if (VEC == 4) *reinterpret_cast<float4*>(&stage[r][c]) = held4[set][j % (VEC == 4 ? LOADS : 1)];
                    else stage[r][c] = held1[set][j % (VEC == 1 ? LOADS : 1)];
                }
                __syncthreads();
                if (start + 2 * kHotChunk < count) fetch(start + 2 * kHotChunk, set);
                if (threadIdx.x < span) {
                    const uint32_t here = min(kHotChunk, count - start);
                    if (here == kHotChunk) {
                        // A whole chunk: every value is read before the first is added (the additions
                        // are a chain; a read inside it would be a round trip each).
                        float t[kHotChunk];
#pragma unroll
                        for (uint32_t r = 0; r < kHotChunk; ++r) t[r] = stage[r][threadIdx.x];
#pragma unroll
                        for (uint32_t r = 0; r < kHotChunk; ++r) acc = acc + t[r];
                    } else {
                        for (uint32_t r = 0; r < here; ++r) acc = acc + stage[r][threadIdx.x];
                    }
                }
                __syncthreads();
            }
        }
        if (threadIdx.x < span && col0 + threadIdx.x < h) {
            const uint64_t where = static_cast<uint64_t>(row) * h + col0 + threadIdx.x;
            store1(out + where, static_cast<float>(out[where]) + acc);
        }
    }
}

}  // namespace

void embedding(cudaStream_t s, In table, const int32_t* ids, Out out, uint64_t n,
               uint64_t rows, uint64_t h, uint32_t* status) {
    if (n == 0 || h == 0) return;
    uint64_t blocks = (n * 32 + 255) / 256;
    uint32_t grid = static_cast<uint32_t>(blocks > 148 * 16 ? 148 * 16 : blocks);
    const uint32_t r = static_cast<uint32_t>(rows), hh = static_cast<uint32_t>(h);
    // A mixed-precision plan gathers from an f32 parameter table or a bf16 activation into bf16.
    if (table.half && out.half) embedding_kernel<<<grid, 256, 0, s>>>(static_cast<const bf16*>(table.p), ids, static_cast<bf16*>(out.p), n, r, hh, status);
    else if (out.half) embedding_kernel<<<grid, 256, 0, s>>>(table.f32(), ids, static_cast<bf16*>(out.p), n, r, hh, status);
    else if (!table.half) embedding_kernel<<<grid, 256, 0, s>>>(table.f32(), ids, out.f32(), n, r, hh, status);
    else throw std::invalid_argument("embedding: a bf16 table gathered into f32");
    check_launch("embedding");
}

uint64_t embedding_grad_scratch_ints(uint64_t n, uint64_t rows) {
    (void)rows;
    return 2 * n;
}

void embedding_order(cudaStream_t s, const int32_t* ids, uint64_t n, uint64_t rows, int32_t* scratch, uint32_t* status) {
    if (n == 0 || rows == 0) return;
    order_kernel<<<static_cast<uint32_t>((n + 31) / 32), 256, 0, s>>>(ids, static_cast<uint32_t>(n), static_cast<uint32_t>(rows), scratch,
                                                                      scratch + n, status);
    check_launch("embedding_order");
}

namespace {
template <class TG, class TO>
void launch_scatter(cudaStream_t s, const TG* g, TO* out, uint64_t n, uint64_t rows, uint64_t h, const int32_t* scratch, const float* base) {
    const int32_t* sorted_id = scratch;
    const int32_t* sorted_n = scratch + n;
    const bool vec = h % 4 == 0 && aligned4(g) && aligned4(out) && reinterpret_cast<uintptr_t>(base) % 16 == 0;
    const uint64_t span = vec ? 128 : 32;
    if (n > 0 && static_cast<const void*>(base) == static_cast<const void*>(out)) {
        // In place: only the rows some id names change, a warp per sorted position.
        const uint32_t positions = static_cast<uint32_t>((n + 7) / 8);
        if (vec) scatter_in_place_kernel<4><<<positions, 256, 0, s>>>(g, sorted_id, sorted_n, static_cast<uint32_t>(n), out, static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
        else scatter_in_place_kernel<1><<<positions, 256, 0, s>>>(g, sorted_id, sorted_n, static_cast<uint32_t>(n), out, static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
        check_launch("embedding_grad");
        return;
    }
    const uint64_t blocks = (rows * ((h + span - 1) / span) + 7) / 8;
    const uint32_t grid = static_cast<uint32_t>(blocks > 148 * 6 ? 148 * 6 : blocks);
    if (vec) scatter_kernel<4><<<grid, 256, 0, s>>>(g, sorted_id, sorted_n, static_cast<uint32_t>(n), base, out, static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
    else scatter_kernel<1><<<grid, 256, 0, s>>>(g, sorted_id, sorted_n, static_cast<uint32_t>(n), base, out, static_cast<uint32_t>(rows), static_cast<uint32_t>(h));
    check_launch("embedding_grad");
}
}  // namespace

void embedding_scatter(cudaStream_t s, In g, Out out, uint64_t n, uint64_t rows, uint64_t h, const int32_t* scratch,
                       const float* base) {
    if (rows == 0 || h == 0) return;
    // A mixed-precision plan scatters a bf16 adjoint into an f32 parameter gradient (with or
    // without an f32 addend) or into a bf16 activation adjoint (the gathered rows of a head).
    if (g.half && out.half) {
        if (base) throw std::invalid_argument("embedding_grad: an f32 addend of a bf16 result");
        launch_scatter(s, static_cast<const bf16*>(g.p), static_cast<bf16*>(out.p), n, rows, h, scratch, base);
    } else if (g.half) {
        launch_scatter(s, static_cast<const bf16*>(g.p), out.f32(), n, rows, h, scratch, base);
    } else if (!out.half) {
        launch_scatter(s, g.f32(), out.f32(), n, rows, h, scratch, base);
    } else {
        throw std::invalid_argument("embedding_grad: an f32 adjoint scattered into bf16");
    }
}

void embedding_grad(cudaStream_t s, const int32_t* ids, In g, Out out, uint64_t n,
                    uint64_t rows, uint64_t h, int32_t* scratch, uint32_t* status, const float* base) {
    embedding_order(s, ids, n, rows, scratch, status);
    embedding_scatter(s, g, out, n, rows, h, scratch, base);
}

}  // namespace k
}  // namespace msx
