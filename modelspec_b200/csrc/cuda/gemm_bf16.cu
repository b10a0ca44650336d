// matmul on bf16 operands for mixed-precision plans: tcgen05.mma (kind::f16, bf16 inputs) fed by TMA,
// f32 accumulation in tensor memory, a persistent CTA per SM.
//
// The reference has no 16-bit type (crates/modelspec-core/src/ir/tensor.rs:38-51: f32 and i32); a
// plan made with MSX_PLAN_BF16 stores activations and the working copy of every weight as bf16
// and runs every product here. An operand needs no conversion on its way to the tensor core, so
// unlike the split-TF32 kernel (gemm_tc.cu) the tiles go from global to shared memory by TMA
// (cp.async.bulk.tensor, 128-byte swizzle) and no thread touches them:
//
//   warp 0      one thread issues the TMA loads of a k block (64 deep: A 128 x 64, B BN x 64) into
//               the next free stage and arms the stage's mbarrier with the byte count;
//   warp 1      allocates tensor memory; one thread issues four MMAs (128 x BN x 16) per k block,
//               releases the stage with tcgen05.commit, and after the last k block of a tile
//               commits the accumulator's barrier;
//   warps 2-5   drain: tcgen05.ld of their 32 lanes, bias, conversion, row stores to C (bf16 or
//               f32) or to the split-k workspace.
// The accumulator is double-buffered (2 x BN columns of tensor memory), so the drain of one tile
// runs under the MMAs of the next; a CTA walks tiles w, w + grid, ... of the launch.
//
// Storage forms: an operand is K-major when k is its contiguous index (A stored [m, k], B stored
// [n, k]) and MN-major otherwise (A stored [k, m], B stored [k, n]). Both are read in place: a
// K-major tile is rows of 128 bytes (64 k), an MN-major tile is panels of 64 m (or n) by 64 k
// rows of 128 bytes; the shared-memory descriptors name the layout, so NN, NT, TN and TT need no
// transposed copy. Batched products (attention heads) address (sequence, head) through two more
// tensor-map coordinates. Every tensor map covers this GPU's own memory only, and every load is a
// plain one to the issuing CTA.
//
// Every mbarrier wait is bounded: when one runs out the role raises bit 1 of the status word and
// sets a flag that makes the other roles leave their loops; the producer then waits (bounded) for
// the copies it still has in flight, the tensor memory is freed and the CTA returns.
#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <string>

#include "common.cuh"
#include "kernels.cuh"
#include "tcgen05.cuh"

namespace msx {
namespace k {

namespace {

using namespace tc;

constexpr int BM = 128, BK = 64;
constexpr int THREADS = 192;
constexpr uint32_t A_BYTES = BM * BK * 2;    // 16 KB
constexpr uint32_t PANEL_BYTES = 64 * BK * 2;  // an MN-major panel: 64 k rows of 64 elements

template <int BN> struct Cfg {
    static constexpr uint32_t B_BYTES = BN * BK * 2;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = BN == 256 ? 4 : (BN == 128 ? 6 : 8);
    static constexpr uint32_t STORE_BYTES = 4 * 2 * 4096;  // per drain warp two slabs of 32 rows x 128 bytes for its TMA stores
    static constexpr uint32_t TOTAL = STAGES * STAGE_BYTES + STORE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
    static constexpr uint32_t TMEM_COLUMNS = 2 * BN;
};

struct Bf16Args {
    void* c;             // C, or the split-k workspace [split][m][n] (f32)
    const float* bias;   // added to every row of C by the CTA that writes C; null for none
    uint32_t* status;
    uint32_t m, n, ldc;
    uint32_t m_tiles, n_tiles, splits, kblocks, kblocks_per_split;
    uint32_t batch, batch_inner;
    uint64_t c_outer, c_inner;  // elements between the C matrices of consecutive batch indices
    uint32_t out_half;          // C is bf16 (never the workspace)
    uint32_t c_vec;             // every row of C starts on a 16-byte boundary
    uint32_t c_tma;             // C is written by TMA stores through map_c (else by the threads' own stores)
    CoordOrder a_order, b_order, c_order;
};

// The work item `w` of a launch: its tile, batch index and k split.
struct Work {
    uint32_t tile_m, tile_n, z_inner, z_outer, split, kb0, kb1;
};
__device__ __forceinline__ Work work_of(const Bf16Args& a, uint32_t w) {
    Work k;
    k.split = w % a.splits;
    uint32_t t = w / a.splits;
    k.tile_m = t % a.m_tiles;
    t /= a.m_tiles;
    k.tile_n = t % a.n_tiles;
    const uint32_t z = t / a.n_tiles;
    k.z_inner = a.batch_inner ? z % a.batch_inner : 0u;
    k.z_outer = a.batch_inner ? z / a.batch_inner : 0u;
    k.kb0 = k.split * a.kblocks_per_split;
    k.kb1 = min(a.kblocks, k.kb0 + a.kblocks_per_split);
    if (k.kb0 > k.kb1) k.kb0 = k.kb1;
    return k;
}

__device__ __forceinline__ void place(const CoordOrder& order, uint32_t row, uint32_t inner, uint32_t outer, uint32_t (&upper)[3]) {
    upper[order.row] = row;
    upper[order.inner] = inner;
    upper[order.outer] = outer;
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(THREADS, 1)
matmul_bf16_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const __grid_constant__ CUtensorMap map_c,
                   const Bf16Args args) {
    using C = Cfg<BN>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ char smem_raw[];
    // 1024-byte alignment: the 128-byte swizzle pattern repeats every 8 rows of 128 bytes.
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    char* store_slabs = tiles + STAGES * C::STAGE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(store_slabs + C::STORE_BYTES);
    // bars[0, STAGES) full, [STAGES, 2 STAGES) empty, then accumulator full [2], accumulator empty [2].
    uint64_t* acc_full = bars + 2 * STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t total = args.m_tiles * args.n_tiles * args.batch * args.splits;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars[s]), 1);
            mbar_init(smem_u32(&bars[STAGES + s]), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), 4);  // one arrival per drain warp
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        if (args.c_tma) asm volatile("prefetch.tensormap [%0];" ::"l"(&map_c) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(C::TMEM_COLUMNS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---- producer: TMA loads, one thread --------------------------------------------------
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            uint32_t armed = 0, armed_phase = 0;  // bit s: stage s was armed, and with which parity last
            bool alive = true;
            for (uint32_t w = blockIdx.x; w < total && alive; w += gridDim.x) {
                const Work k = work_of(args, w);
                for (uint32_t kb = k.kb0; kb < k.kb1; ++kb) {
                    alive = mbar_wait(smem_u32(&bars[STAGES + stage]), phase ^ 1u, abort_flag, args.status);
                    if (!alive) break;
                    const uint32_t full = smem_u32(&bars[stage]);
                    const uint32_t a_dst = smem_u32(tiles + stage * C::STAGE_BYTES), b_dst = a_dst + A_BYTES;
                    mbar_expect_tx(full, C::STAGE_BYTES);
                    armed |= 1u << stage;
                    armed_phase = (armed_phase & ~(1u << stage)) | (phase << stage);
                    uint32_t upper[3];
                    if (A_MN) {  // stored [k, m]: two panels of 64 m
                        place(args.a_order, kb * BK, k.z_inner, k.z_outer, upper);
#pragma unroll
                        for (uint32_t p = 0; p < BM / 64; ++p) tma_load(a_dst + p * PANEL_BYTES, &map_a, full, k.tile_m * BM + p * 64, upper);
                    } else {     // stored [m, k]: 128 rows of 64 k
                        place(args.a_order, k.tile_m * BM, k.z_inner, k.z_outer, upper);
                        tma_load(a_dst, &map_a, full, kb * BK, upper);
                    }
                    if (B_MN) {  // stored [k, n]: BN / 64 panels of 64 n
                        place(args.b_order, kb * BK, k.z_inner, k.z_outer, upper);
#pragma unroll
                        for (uint32_t p = 0; p < BN / 64; ++p) tma_load(b_dst + p * PANEL_BYTES, &map_b, full, k.tile_n * BN + p * 64, upper);
                    } else {     // stored [n, k]: BN rows of 64 k
                        place(args.b_order, k.tile_n * BN, k.z_inner, k.z_outer, upper);
                        tma_load(b_dst, &map_b, full, kb * BK, upper);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!alive) {
                // Another role gave up: the copies already issued still write into this CTA's
                // shared memory, so each armed stage is waited for (bounded) before the CTA may go.
                for (uint32_t st = 0; st < static_cast<uint32_t>(STAGES); ++st) {
                    if (!(armed & (1u << st))) continue;
                    const uint32_t parity = (armed_phase >> st) & 1u;
                    for (uint32_t spin = 0; spin < WAIT_LIMIT && !mbar_try_wait(smem_u32(&bars[st]), parity); ++spin) {}
                }
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer --------------------------------------------------------------------------
        // Instruction descriptor: f32 accumulator (bits 4-5 = 1), bf16 A and B (bits 7-9 and 10-12
        // = 1), the operands' majors (bits 15 and 16: 1 = MN-major), N >> 3 at bit 17, M >> 4 at 24.
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((A_MN ? 1u : 0u) << 15) | ((B_MN ? 1u : 0u) << 16) |
                               (static_cast<uint32_t>(BN >> 3) << 17) | (static_cast<uint32_t>(BM >> 4) << 24);
        // Shared-memory matrix descriptors (sm_100 form: bit 46 set, 128-byte swizzle = 2 in bits
        // 61-63), all offsets in 16-byte units. K-major: 8-row groups 1024 bytes apart (stride
        // offset), the leading offset unused. MN-major: panels of 64 elements 8192 bytes apart
        // (leading offset), groups of 8 k rows 1024 bytes apart (stride offset).
        constexpr uint32_t a_lbo = A_MN ? PANEL_BYTES : 16u, b_lbo = B_MN ? PANEL_BYTES : 16u;
        constexpr uint32_t high = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
        constexpr uint32_t a_low = ((a_lbo >> 4) & 0x3FFFu) << 16, b_low = ((b_lbo >> 4) & 0x3FFFu) << 16;
        const uint32_t tiles16 = (smem_u32(tiles) & 0x3FFFFu) >> 4;
        auto desc = [](uint32_t hi, uint32_t lo) { return (static_cast<uint64_t>(hi) << 32) | lo; };
        uint32_t stage = 0, phase = 0, item = 0;
        bool alive = true;
        for (uint32_t w = blockIdx.x; w < total && alive; w += gridDim.x, ++item) {
            const Work k = work_of(args, w);
            const uint32_t acc = item & 1u, acc_phase = (item >> 1) & 1u;
            // The drain warps have emptied this half of the accumulator (first use: passes at once).
            alive = mbar_wait(smem_u32(&acc_empty[acc]), acc_phase ^ 1u, abort_flag, args.status);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t tmem_d = tmem_base + acc * BN;
            for (uint32_t kb = k.kb0; kb < k.kb1 && alive; ++kb) {
                alive = mbar_wait(smem_u32(&bars[stage]), phase, abort_flag, args.status);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const uint32_t a16 = a_low + tiles16 + stage * (C::STAGE_BYTES >> 4);
                    const uint32_t b16 = b_low + tiles16 + stage * (C::STAGE_BYTES >> 4) + (A_BYTES >> 4);
#pragma unroll
                    for (uint32_t ks = 0; ks < BK / 16; ++ks) {
                        // k = 16: 32 bytes along a K-major row, or 16 rows (2048 bytes) of an MN-major panel.
                        const uint32_t a_step = (A_MN ? ks * 2048u : ks * 32u) >> 4;
                        const uint32_t b_step = (B_MN ? ks * 2048u : ks * 32u) >> 4;
                        mma_bf16(tmem_d, desc(high, a16 + a_step), desc(high, b16 + b_step), idesc, (kb != k.kb0 || ks != 0u) ? 1u : 0u);
                    }
                    mma_commit(smem_u32(&bars[STAGES + stage]));  // frees the stage when these MMAs finish
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (alive && lane == 0) mma_commit(smem_u32(&acc_full[acc]));  // arrives at once when no MMA is pending
            __syncwarp();
        }
    } else {
        // ---- drain warps: tensor memory -> registers -> C ----------------------------------------
        const uint32_t quarter = warp & 3u;  // the 32 lanes of tensor memory this warp may read
        uint32_t item = 0;
        uint32_t turn = 0;  // TMA stores issued by this warp so far: they alternate between its two slabs
        bool alive = true;
        for (uint32_t w = blockIdx.x; w < total && alive; w += gridDim.x, ++item) {
            const Work k = work_of(args, w);
            const uint32_t acc = item & 1u, acc_phase = (item >> 1) & 1u;
            const bool partial = args.splits > 1;
            // The tile's bias values, lane l holding columns l, l + 32, ..., fetched before the
            // wait for the tile (a load issued inside the drain waits behind everything else the
            // SM has in flight) and handed round by shuffles.
            float held[BN / 32];
            if (args.bias != nullptr && !partial) {
#pragma unroll
                for (int i = 0; i < BN / 32; ++i) {
                    const uint32_t c = k.tile_n * BN + i * 32 + lane;
                    held[i] = c < args.n ? __ldg(args.bias + c) : 0.0f;
                }
            }
            alive = mbar_wait(smem_u32(&acc_full[acc]), acc_phase, abort_flag, args.status);
            alive = __all_sync(0xffffffffu, alive);  // tcgen05.ld is warp-wide: decide as a warp
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool has_k = k.kb1 > k.kb0;
            const uint32_t row = k.tile_m * BM + quarter * 32u + lane;
            const uint64_t z_at = static_cast<uint64_t>(k.z_outer) * args.c_outer + static_cast<uint64_t>(k.z_inner) * args.c_inner;
            const uint64_t row_at = (partial ? static_cast<uint64_t>(k.split) * args.m * args.n : z_at) + static_cast<uint64_t>(row) * args.ldc;
            const bool half_out = args.out_half != 0 && !partial;
            if (args.c_tma) {
                // Coalesced: the warp's 32 rows of a 128-byte column slab go to shared memory (each
                // lane its row, 16-byte pieces swizzled as the tensor map expects) and from there to
                // C by one TMA store, which clips what lies outside the matrix. Two slabs a warp:
                // one is being stored while the next is filled. No other warp takes part.
                const uint32_t slab_cols = half_out ? 64u : 32u;
                char* const my_slabs = store_slabs + quarter * 2 * 4096;
                uint32_t upper[3];
                place(args.c_order, k.tile_m * BM + quarter * 32u, partial ? 0u : k.z_inner, partial ? k.split : k.z_outer, upper);
                const bool rows_inside = k.tile_m * BM + quarter * 32u < args.m;  // else nothing of this warp's is stored
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < static_cast<uint32_t>(BN); c0 += slab_cols, ++turn) {
                    const uint32_t col = k.tile_n * BN + c0;
                    if (col >= args.n) break;  // the same for the whole warp
                    char* const slab = my_slabs + (turn & 1u) * 4096;
                    // The store that last read this slab (two turns ago) has finished reading it.
                    if (lane == 0) tma_store_wait_read<1>();
                    __syncwarp();
#pragma unroll
                    for (uint32_t part = 0; part < 2; ++part) {
                        if (part == 1 && !half_out) break;
                        uint32_t r[32];
                        if (has_k) {
                            tmem_load32(tmem_base + acc * BN + c0 + part * 32 + ((quarter * 32u) << 16), r);
                            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) r[j] = 0u;
                        }
                        float v[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                        if (args.bias != nullptr && !partial) {
                            const uint32_t group = (c0 + part * 32) >> 5;
                            float mine = held[0];
#pragma unroll
                            for (int q = 1; q < BN / 32; ++q)
                                if (group == static_cast<uint32_t>(q)) mine = held[q];
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] += __shfl_sync(0xffffffffu, mine, j);
                        }
                        if (half_out) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                float8 f;
                                f.lo = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                f.hi = make_float4(v[j + 4], v[j + 5], v[j + 6], v[j + 7]);
                                store8(reinterpret_cast<bf16*>(slab + swizzled_chunk(lane, part * 4 + (j >> 3))), f);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<float4*>(slab + swizzled_chunk(lane, j >> 2)) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0 && rows_inside) tma_store(&map_c, smem_u32(slab), col, upper);
                }
            } else {
#pragma unroll 1
                for (uint32_t c0 = 0; c0 < static_cast<uint32_t>(BN); c0 += 32) {
                    const uint32_t col = k.tile_n * BN + c0;
                    if (col >= args.n) break;  // the same for the whole warp
                    uint32_t r[32];
                    if (has_k) {
                        tmem_load32(tmem_base + acc * BN + c0 + ((quarter * 32u) << 16), r);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    } else {
    #pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = 0u;  // an empty k range is a zero product
                    }
                    if (row >= args.m) continue;
                    float v[32];
    #pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (args.bias != nullptr && !partial) {
    #pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col + j < args.n) v[j] += __ldg(args.bias + col + j);
                    }
                    const bool whole = col + 32 <= args.n && args.c_vec;
                    if (half_out) {
                        __nv_bfloat16* out = static_cast<__nv_bfloat16*>(args.c) + row_at + col;
                        if (whole) {
    #pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 packed;
                                __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
                                __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
                                packed.x = *reinterpret_cast<uint32_t*>(&p0);
                                packed.y = *reinterpret_cast<uint32_t*>(&p1);
                                packed.z = *reinterpret_cast<uint32_t*>(&p2);
                                packed.w = *reinterpret_cast<uint32_t*>(&p3);
                                *reinterpret_cast<uint4*>(out + j) = packed;
                            }
                        } else {
    #pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < args.n) out[j] = __float2bfloat16_rn(v[j]);
                        }
                    } else {
                        float* out = static_cast<float*>(args.c) + row_at + col;
                        if (whole) {
    #pragma unroll
                            for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(out + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                        } else {
    #pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < args.n) out[j] = v[j];
                        }
                    }
                }
            }
            // This half of the accumulator may be overwritten by the tile after next.
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
        }
        // The last stores still read this CTA's shared memory.
        if (lane == 0) tma_store_wait_read<0>();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::TMEM_COLUMNS) : "memory");
    }
}

// The sum of the split-k partial tiles, ascending split order, into C (either type) with the bias.
__global__ void splitk_reduce_bf16_kernel(const float* __restrict__ ws, void* __restrict__ c, uint32_t out_half, uint64_t m, uint32_t n,
                                          uint32_t ldc, uint32_t splits, const float* __restrict__ bias) {
    const uint64_t count = m * n, stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        float acc = ws[i];
        for (uint32_t s = 1; s < splits; ++s) acc += ws[static_cast<uint64_t>(s) * count + i];
        const uint32_t col = static_cast<uint32_t>(i % n);
        if (bias) acc += bias[col];
        const uint64_t at = i / n * ldc + col;
        if (out_half) static_cast<__nv_bfloat16*>(c)[at] = __float2bfloat16_rn(acc);
        else static_cast<float*>(c)[at] = acc;
    }
}

template <int BN, bool A_MN, bool B_MN>
void launch(cudaStream_t s, const CUtensorMap& map_a, const CUtensorMap& map_b, const CUtensorMap& map_c, const Bf16Args& args, uint32_t blocks) {
    auto kernel = matmul_bf16_kernel<BN, A_MN, B_MN>;
    static std::atomic<int> configured_device{-1};
    int device = 0;
    check(cudaGetDevice(&device), "cudaGetDevice");
    if (device != configured_device.load(std::memory_order_relaxed)) {
        check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Cfg<BN>::TOTAL)), "matmul_bf16 shared memory");
        configured_device.store(device, std::memory_order_relaxed);
    }
    kernel<<<blocks, THREADS, Cfg<BN>::TOTAL, s>>>(map_a, map_b, map_c, args);
    check_launch("matmul_bf16");
}

template <int BN>
void launch_forms(cudaStream_t s, const CUtensorMap& a, const CUtensorMap& b, const CUtensorMap& c, const Bf16Args& args, uint32_t blocks, bool a_mn,
                  bool b_mn) {
    if (a_mn && b_mn) launch<BN, true, true>(s, a, b, c, args, blocks);
    else if (a_mn) launch<BN, true, false>(s, a, b, c, args, blocks);
    else if (b_mn) launch<BN, false, true>(s, a, b, c, args, blocks);
    else launch<BN, false, false>(s, a, b, c, args, blocks);
}

int sm_count() {
    static std::mutex lock;
    static int counts[64] = {};
    int device = 0;
    check(cudaGetDevice(&device), "cudaGetDevice");
    std::lock_guard<std::mutex> hold(lock);
    if (device < 0 || device >= 64) return 148;
    if (counts[device] == 0) check(cudaDeviceGetAttribute(&counts[device], cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute");
    return counts[device];
}

}  // namespace

// Tile width and k split. A tile is 128 rows by 64, 128 or 256 columns; the widest width that
// still gives every SM a tile wins (it re-reads A least), and a product with too few tiles for the
// device splits its k range instead (weight gradients: few tiles, k = the batch's rows).
MatmulBf16Plan matmul_bf16_plan(uint64_t m, uint64_t n, uint64_t k, uint64_t problems) {
    const uint64_t kblocks = (k + BK - 1) / BK, m_tiles = (m + BM - 1) / BM;
    static const uint32_t widths[3] = {256, 128, 64};
    static const double per_kblock[3] = {1250.0, 830.0, 620.0};  // SM cycles: operand feed through the L2 bounds a k block
    MatmulBf16Plan best = {};
    double best_cost = 0.0;
    for (int w = 0; w < 3; ++w) {
        const uint32_t bn = widths[w];
        if (bn > 64 && n <= bn / 2) continue;  // a tile mostly outside the matrix
        const uint64_t tiles = m_tiles * ((n + bn - 1) / bn) * problems;
        uint64_t splits = 1;
        if (problems == 1 && tiles < 100 && kblocks >= 8) splits = std::min<uint64_t>(std::min<uint64_t>(148 / tiles, kblocks / 4), 32);
        if (splits < 1) splits = 1;
        const uint64_t per = (kblocks + splits - 1) / splits;
        if (kblocks) splits = (kblocks + per - 1) / per;
        const uint64_t waves = (tiles * splits + 147) / 148;
        double cost = static_cast<double>(waves) * (4000.0 + static_cast<double>(per) * per_kblock[w]);
        if (splits > 1) cost += 8000.0 + static_cast<double>(m * n * (splits + 1)) * 4.0 / 3000.0;
        if (best.bn == 0 || cost < best_cost) {
            best_cost = cost;
            best.bn = bn;
            best.splits = static_cast<uint32_t>(splits);
            best.kblocks_per_split = static_cast<uint32_t>(per == 0 ? 1 : per);
        }
    }
    best.workspace_floats = best.splits > 1 ? best.splits * m * n : 0;
    return best;
}

void matmul_bf16(cudaStream_t s, const HalfMatrix& a, const HalfMatrix& b, const HalfResult& c, uint64_t m, uint64_t n, uint64_t k,
                 uint32_t outer, uint32_t inner, float* workspace, const float* bias, uint32_t* status, bool leave_partials) {
    if (m == 0 || n == 0 || outer == 0 || inner == 0) return;
    const uint64_t problems = static_cast<uint64_t>(outer) * inner;
    const MatmulBf16Plan p = matmul_bf16_plan(m, n, k, problems);
    if (p.splits > 1 && workspace == nullptr) throw std::invalid_argument("matmul_bf16: a split k needs its workspace");
    Bf16Args args = {};
    CoordOrder a_order = {}, b_order = {};
    // A: stored [m, k] (K-major: loads of 128 rows) or [k, m] (MN-major: loads of 64 k rows).
    const CUtensorMap map_a = a.transposed ? encode(a, m, k, inner, outer, 64, &a_order, "A")
                                           : encode(a, k, m, inner, outer, BM, &a_order, "A");
    // B: stored [n, k] (K-major: loads of BN rows) or [k, n] (MN-major: loads of 64 k rows).
    const CUtensorMap map_b = b.transposed ? encode(b, k, n, inner, outer, p.bn, &b_order, "B")
                                           : encode(b, n, k, inner, outer, 64, &b_order, "B");
    const bool partial = p.splits > 1;
    args.c = partial ? static_cast<void*>(workspace) : c.base;
    args.bias = partial ? nullptr : bias;
    args.status = status;
    args.m = static_cast<uint32_t>(m);
    args.n = static_cast<uint32_t>(n);
    args.ldc = partial ? static_cast<uint32_t>(n) : (c.pitch ? c.pitch : static_cast<uint32_t>(n));
    args.m_tiles = static_cast<uint32_t>((m + BM - 1) / BM);
    args.n_tiles = static_cast<uint32_t>((n + p.bn - 1) / p.bn);
    args.splits = p.splits;
    args.kblocks = static_cast<uint32_t>((k + BK - 1) / BK);
    args.kblocks_per_split = p.kblocks_per_split;
    args.batch = static_cast<uint32_t>(problems);
    args.batch_inner = problems > 1 ? inner : 0;
    args.c_outer = c.stride_outer;
    args.c_inner = c.stride_inner;
    args.out_half = c.half ? 1u : 0u;
    const uint32_t unit = (c.half && !partial) ? 8u : 4u;  // elements in 16 bytes
    args.c_vec = reinterpret_cast<uintptr_t>(args.c) % 16 == 0 && args.ldc % unit == 0 &&
                 (partial ? (m * n) % 4 == 0 : (c.stride_outer % unit == 0 && c.stride_inner % unit == 0));
    args.a_order = a_order;
    args.b_order = b_order;
    // C through TMA stores when its rows can be addressed that way: the result matrices as the
    // operands are described, the split-k workspace as `splits` dense [m, n] matrices.
    CUtensorMap map_c = map_a;
    {
        const bool float_out = partial || !c.half;
        HalfMatrix target = {args.c, args.ldc, partial ? m * n : c.stride_outer, partial ? 0 : c.stride_inner, false};
        if (tma_addressable(target, float_out)) {
            CoordOrder c_order = {};
            map_c = encode(target, n, m, partial ? 1 : inner, partial ? p.splits : outer, 32, &c_order, "C", float_out);
            args.c_order = c_order;
            args.c_tma = 1;
        }
    }
    const uint64_t total = static_cast<uint64_t>(args.m_tiles) * args.n_tiles * problems * p.splits;
    const uint32_t blocks = static_cast<uint32_t>(std::min<uint64_t>(total, static_cast<uint64_t>(sm_count())));
    const bool a_mn = a.transposed, b_mn = !b.transposed;
    if (p.bn == 256) launch_forms<256>(s, map_a, map_b, map_c, args, blocks, a_mn, b_mn);
    else if (p.bn == 128) launch_forms<128>(s, map_a, map_b, map_c, args, blocks, a_mn, b_mn);
    else launch_forms<64>(s, map_a, map_b, map_c, args, blocks, a_mn, b_mn);
    if (partial && !leave_partials) {
        const uint64_t count = m * n, wanted = (count + 255) / 256;
        splitk_reduce_bf16_kernel<<<static_cast<uint32_t>(std::min<uint64_t>(wanted, 148 * 8)), 256, 0, s>>>(
            workspace, c.base, c.half ? 1u : 0u, m, static_cast<uint32_t>(n), c.pitch ? c.pitch : static_cast<uint32_t>(n), p.splits, bias);
        check_launch("splitk_reduce_bf16");
    }
}

}  // namespace k
}  // namespace msx
