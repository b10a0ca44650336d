// Fused attention for mixed-precision plans: forward in one kernel, the three gradients in one.
//
// The score matrix never reaches memory. What the op computes is the reference's
// (crates/modelspec-runtime/src/cpu/interpreter.rs:1035-1119, helper :1308-1510): per sequence b,
// head a and query i, s_ij = (q_i . k_j) / sqrt(d), a softmax over the unmasked keys,
// O_i = sum_j p_ij v_j; dS = p (dP - D_i) with dP = g_i . v_j and D_i = sum_j p_ij dP_ij,
// dQ_i = scale sum_j dS_ij k_j, dK_j = scale sum_i dS_ij q_i, dV_j = sum_i p_ij g_i; a masked key has
// probability 0 and zero gradient rows. Here q, k, v, g and every result are bf16 [rows, H] read and
// written in place (row pitch H, head a at columns a d ..), all products are tcgen05.mma kind::f16
// with f32 accumulation in tensor memory on TMA-loaded tiles, and softmax statistics are f32.
//
// Every operand tile is 128 rows of 64 head columns: 128 bytes a row, 128-byte swizzle, one TMA
// load. The same bytes serve as a K-major operand (k = head columns: Q K^T, G V^T) and as an
// MN-major one (k = rows: P^T G, dS^T Q, P V, dS K), so nothing is transposed or copied.
// Probabilities and score gradients are written by the softmax threads as bf16 into two such
// tiles (64 keys each) and read by the tensor core from there.
//
//   forward   one CTA per (128 queries, head, sequence); key tiles of 128 in turn: S = Q K^T into
//             tensor memory, online softmax by 128 threads (one query row each: running max and
//             sum, the row of O in registers, rescaled when the max moves), P to shared memory,
//             P V into tensor memory, added to the registers. Writes O and per (row, head) the
//             max and the sum. Two CTAs share an SM: one's softmax runs under the other's MMAs.
//   backward  one CTA per (head, sequence), at most 512 keys and 512 queries: for each key tile
//             j, for each query tile i: S and then dP through one region of tensor memory, P and
//             dS to shared memory, dV_j += P^T G_i, dK_j += dS^T Q_i, dQ_i += dS K_j. dV_j and dK_j
//             are drained after the i loop, the (up to four) dQ_i tiles stay in tensor memory
//             until the end: 128 + 128 + 4 x 64 = 512 columns. D_i comes from sum_c O g.
//
// Heads of up to 64 columns (a multiple of 8). Every mbarrier wait is bounded; when one runs out
// the role raises bit 1 of the status word, the other roles leave their loops, the producer waits
// (bounded) for its copies in flight, tensor memory is freed and the CTA returns.
#include "tcgen05.cuh"

namespace msx {
namespace k {

namespace {

using namespace tc;

constexpr uint32_t TILE = 128;                 // rows of a tile (queries or keys)
constexpr uint32_t TILE_BYTES = TILE * 128;    // 64 bf16 columns a row
constexpr int ROW_WARPS = 16;                  // four threads a row: 32 score columns, 16 result columns each
constexpr int THREADS = 64 + 32 * ROW_WARPS;   // warp 0 loads, warp 1 issues MMAs, warps 2-17 do the row work

struct FusedArgs {
    const float* mask;   // [batch, keys]
    void* out;           // forward: O; backward: unused
    float* stats;        // [(row * heads + head) * 2 + {0, 1}] = max, sum of exp
    const void* o;       // backward: the forward's O
    const void* g;       // backward: the adjoint of O (also read through its tensor map)
    void* dq;
    void* dk;
    void* dv;
    uint32_t* status;
    uint32_t batch, q_len, k_len, heads, d, h;
    float scale;
    CoordOrder order;    // of every [rows, H] operand's tensor map
};

// Which of the 32 keys from `first` on count (inside the sequence and not masked out): bit c for
// key first + c, the same word in every lane of the warp.
__device__ __forceinline__ uint32_t keys_that_count(const float* __restrict__ mask, uint32_t seq, uint32_t first, uint32_t k_len, uint32_t lane) {
    const uint32_t key = first + lane;
    const bool counts = key < k_len && mask[static_cast<uint64_t>(seq) * k_len + key] != 0.0f;
    return __ballot_sync(0xffffffffu, counts);
}

// One [128 rows, 64 columns] tile of a [rows, H] operand: rows row0.. of sequence `seq`, head `head`.
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar, const CoordOrder& order, uint32_t row0,
                                          uint32_t head, uint32_t seq) {
    uint32_t upper[3];
    upper[order.row] = row0;
    upper[order.inner] = head;
    upper[order.outer] = seq;
    tma_load(dst, map, bar, 0, upper);
}

// 32 lanes x 16 consecutive columns of tensor memory.
__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// 32 f32 values of row `row`, columns chunk * 32 .., as bf16 into a pair of [128 rows, 64 columns]
// tiles (columns 0-63 in the first, 64-127 in the second) in the layout the tensor core reads.
__device__ __forceinline__ void store_chunk_bf16(char* tile_pair, uint32_t row, uint32_t chunk, const float (&v)[32]) {
    char* to = tile_pair + (chunk >> 1) * TILE_BYTES;
    const uint32_t first16 = (chunk & 1u) * 4;  // 16-byte chunk index of column chunk * 32 within its tile row
#pragma unroll
    for (int c = 0; c < 32; c += 8) {
        float8 f;
        f.lo = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
        f.hi = make_float4(v[c + 4], v[c + 5], v[c + 6], v[c + 7]);
        store8(reinterpret_cast<bf16*>(to + swizzled_chunk(row, first16 + (c >> 3))), f);
    }
}

// 16 f32 values as bf16 to global memory (columns c0 .. c0 + 15 of a head's row, those below d).
__device__ __forceinline__ void store_part_bf16(void* base, uint64_t element, const float (&v)[16], uint32_t c0, uint32_t d) {
    bf16* to = static_cast<bf16*>(base) + element + c0;
#pragma unroll
    for (uint32_t c = 0; c < 16; c += 8) {
        if (c0 + c + 8 > d) break;
        float8 f;
        f.lo = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
        f.hi = make_float4(v[c + 4], v[c + 5], v[c + 6], v[c + 7]);
        store8(to + c, f);
    }
}

// ---- forward --------------------------------------------------------------------------------------
// Shared memory: Q, two stages of K, V, two stages of P (two tiles each): 128 KB, then barriers and
// the exchange of row maxima and sums between the four threads of a row.
// Tensor memory: S of even key tiles at columns [0, 128), of odd ones at [128, 256); P V of even key
// tiles at [256, 320), of odd ones at [320, 384). P and P V are double-buffered so that the rows
// add P_j V_j to their result one key tile late, after the softmax of tile j + 1: the product's
// latency is off their path.
constexpr uint32_t FWD_TILES = 8 * TILE_BYTES;
constexpr uint32_t FWD_SMEM = FWD_TILES + 1024 /* alignment slack */ + 256 /* barriers */ + 2 * 4 * TILE * 4 /* row exchange */;
constexpr uint32_t FWD_TMEM = 512;

__global__ void __launch_bounds__(THREADS, 1)
attention_forward_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v, const FusedArgs args) {
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    char* q_tile = tiles;
    auto k_tile = [&](uint32_t stage) { return tiles + (1 + stage) * TILE_BYTES; };
    char* v_tile = tiles + 3 * TILE_BYTES;
    auto p_tile = [&](uint32_t stage) { return tiles + (4 + 2 * stage) * TILE_BYTES; };  // two tiles a stage: keys 0-63 and 64-127 of the key tile
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + FWD_TILES);
    enum { Q_FULL, K_FULL0, K_FULL1, K_EMPTY0, K_EMPTY1, V_FULL, V_EMPTY, S_FULL0, S_FULL1, P_READY, PV_FULL0, PV_FULL1, ROWS_MET, BARS };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BARS);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
    float* exchange = reinterpret_cast<float*>(tiles + FWD_TILES + 256);  // [2][4 column chunks][128 rows]

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t q0 = blockIdx.x * TILE, head = blockIdx.y, seq = blockIdx.z;
    const uint32_t key_tiles = (args.k_len + TILE - 1) / TILE;
    auto bar = [&](int which) { return smem_u32(&bars[which]); };

    if (tid == 0) {
        for (int b = 0; b < BARS; ++b) mbar_init(bar(b), (b == P_READY || b == ROWS_MET) ? static_cast<uint32_t>(ROW_WARPS) : 1u);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(FWD_TMEM) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_pv = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0) {
            bool alive = true;
            uint32_t armed = 0, k_phase[2] = {0, 0}, v_phase = 0;  // armed: bit 0 Q, 1-2 the K stages, 3 V
            mbar_expect_tx(bar(Q_FULL), TILE_BYTES);
            load_tile(smem_u32(q_tile), &map_q, bar(Q_FULL), args.order, q0, head, seq);
            armed |= 1u;
            for (uint32_t j = 0; j < key_tiles && alive; ++j) {
                const uint32_t stage = j & 1u, use = j >> 1;
                alive = mbar_wait(bar(K_EMPTY0 + stage), (use & 1u) ^ 1u, abort_flag, args.status);
                if (!alive) break;
                mbar_expect_tx(bar(K_FULL0 + stage), TILE_BYTES);
                load_tile(smem_u32(k_tile(stage)), &map_k, bar(K_FULL0 + stage), args.order, j * TILE, head, seq);
                armed |= 2u << stage;
                k_phase[stage] = use & 1u;
                alive = mbar_wait(bar(V_EMPTY), (j & 1u) ^ 1u, abort_flag, args.status);
                if (!alive) break;
                mbar_expect_tx(bar(V_FULL), TILE_BYTES);
                load_tile(smem_u32(v_tile), &map_v, bar(V_FULL), args.order, j * TILE, head, seq);
                armed |= 8u;
                v_phase = j & 1u;
            }
            if (!alive) {
                // The copies already issued still write into this CTA's shared memory: wait (bounded).
                if (armed & 1u) for (uint32_t spin = 0; spin < WAIT_LIMIT && !mbar_try_wait(bar(Q_FULL), 0); ++spin) {}
                for (uint32_t stage = 0; stage < 2; ++stage)
                    if (armed & (2u << stage)) for (uint32_t spin = 0; spin < WAIT_LIMIT && !mbar_try_wait(bar(K_FULL0 + stage), k_phase[stage]); ++spin) {}
                if (armed & 8u) for (uint32_t spin = 0; spin < WAIT_LIMIT && !mbar_try_wait(bar(V_FULL), v_phase); ++spin) {}
            }
        }
    } else if (warp == 1) {
        const uint32_t idesc_s = instruction_descriptor(TILE, TILE, false, false);
        const uint32_t idesc_pv = instruction_descriptor(TILE, 64, false, true);
        // S_j = Q K_j^T into its half of the score columns: k runs over the 64 head columns, 16
        // (32 bytes of a row) per MMA. S_j+1 is issued before P_j V_j, so that it runs under the
        // softmax of tile j.
        auto scores = [&](uint32_t j) -> bool {
            const uint32_t stage = j & 1u;
            if (!mbar_wait(bar(K_FULL0 + stage), (j >> 1) & 1u, abort_flag, args.status)) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
#pragma unroll
                for (uint32_t ks = 0; ks < 4; ++ks)
                    mma_bf16(tmem_base + stage * 128, tile_descriptor(smem_u32(q_tile) + ks * 32, 16), tile_descriptor(smem_u32(k_tile(stage)) + ks * 32, 16),
                             idesc_s, ks != 0);
                mma_commit(bar(K_EMPTY0 + stage));
                mma_commit(bar(S_FULL0 + stage));
            }
            __syncwarp();
            return true;
        };
        bool alive = mbar_wait(bar(Q_FULL), 0, abort_flag, args.status);
        if (alive) alive = scores(0);
        for (uint32_t j = 0; j < key_tiles && alive; ++j) {
            const uint32_t ph = j & 1u;
            // The rows have read S_j-1 (they arrived at P_READY of tile j - 1 after it): its columns are free.
            if (j + 1 < key_tiles) alive = scores(j + 1);
            if (alive) alive = mbar_wait(bar(P_READY), ph, abort_flag, args.status);
            if (alive) alive = mbar_wait(bar(V_FULL), ph, abort_flag, args.status);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                // P V: k runs over the 128 keys, 16 per MMA: 32 bytes of a P row (two tiles of 64
                // keys), 16 rows (2048 bytes) of the V tile.
#pragma unroll
                for (uint32_t ks = 0; ks < 8; ++ks)
                    mma_bf16(tmem_pv + ph * 64, tile_descriptor(smem_u32(p_tile(ph)) + (ks >> 2) * TILE_BYTES + (ks & 3u) * 32, 16),
                             tile_descriptor(smem_u32(v_tile) + ks * 2048, TILE_BYTES), idesc_pv, ks != 0);
                mma_commit(bar(V_EMPTY));
                mma_commit(bar(PV_FULL0 + ph));
            }
            __syncwarp();
        }
    } else {
        // Four threads a query row: row q0 + t (lane t of tensor memory), score columns
        // chunk * 32 .. of a key tile and result columns chunk * 16 ... The lanes of tensor memory a
        // warp may read are those of its index modulo 4.
        const uint32_t quarter = warp & 3u, chunk = (warp - 2) >> 2, t = quarter * 32 + lane;
        const uint32_t lane_base = (quarter * 32u) << 16;
        const uint32_t row = q0 + t;
        float best = -INFINITY, total = 0.0f;  // total: over this thread's columns only, until the end
        float o[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) o[c] = 0.0f;
        bool alive = true;
        uint32_t meetings = 0;  // completed phases of ROWS_MET
        // The four threads of every row exchange a value each (the maximum of their columns, at the
        // end their sum) through shared memory; the warps meet at an mbarrier with a bounded wait.
        auto exchange_with_row = [&](float mine, float (&all)[4]) -> bool {
            float* slot = exchange + (meetings & 1u) * 4 * TILE;
            slot[chunk * TILE + t] = mine;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ROWS_MET));
            bool ok = mbar_wait(bar(ROWS_MET), meetings & 1u, abort_flag, args.status);
            ok = __all_sync(0xffffffffu, ok);
            ++meetings;
            if (!ok) return false;
#pragma unroll
            for (int c = 0; c < 4; ++c) all[c] = slot[c * TILE + t];
            return true;
        };
        // P_j V_j is added one key tile late (after the softmax of tile j + 1), with the factor by
        // which the maximum moved at tile j: o_j = o_j-1 * shrink_j + P_j V_j.
        float pending_shrink = 0.0f;
        auto add_product = [&](uint32_t j) -> bool {
            bool ok = mbar_wait(bar(PV_FULL0 + (j & 1u)), (j >> 1) & 1u, abort_flag, args.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) return false;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t pv[16];
            tmem_load16(tmem_pv + (j & 1u) * 64 + lane_base + chunk * 16, pv);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int c = 0; c < 16; ++c) o[c] = o[c] * pending_shrink + __uint_as_float(pv[c]);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            return true;
        };
        for (uint32_t j = 0; j < key_tiles; ++j) {
            const uint32_t stage = j & 1u;
            const uint32_t counts = keys_that_count(args.mask, seq, j * TILE + chunk * 32, args.k_len, lane);
            alive = mbar_wait(bar(S_FULL0 + stage), (j >> 1) & 1u, abort_flag, args.status);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r[32];
            tmem_load32(tmem_base + stage * 128 + lane_base + chunk * 32, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            float sc[32];
            float mine = -INFINITY;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                sc[c] = ((counts >> c) & 1u) ? __uint_as_float(r[c]) * args.scale : -INFINITY;
                mine = fmaxf(mine, sc[c]);
            }
            float parts[4];
            alive = exchange_with_row(mine, parts);
            if (!alive) break;
            const float new_best = fmaxf(fmaxf(best, fmaxf(parts[0], parts[1])), fmaxf(parts[2], parts[3]));
            // exp(-inf - -inf) never forms: a row that has seen no key yet keeps zeros.
            const float shrink = best == -INFINITY ? 0.0f : __expf(best - new_best);
            float tile_total = 0.0f;
#pragma unroll
            for (int c = 0; c < 32; ++c) {
                sc[c] = ((counts >> c) & 1u) ? __expf(sc[c] - new_best) : 0.0f;
                tile_total += sc[c];
            }
            total = total * shrink + tile_total;
            best = new_best;
            // This stage of P is free: P_j-2 V_j-2 was complete before this thread added it, a tile ago.
            store_chunk_bf16(p_tile(stage), t, chunk, sc);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_READY));
            // The product of the tile before, which ran under this tile's softmax.
            if (j > 0) {
                alive = add_product(j - 1);
                if (!alive) break;
            }
            pending_shrink = shrink;
        }
        if (alive && key_tiles > 0) alive = add_product(key_tiles - 1);
        if (alive) {
            float parts[4];
            alive = exchange_with_row(total, parts);
            if (alive && row < args.q_len) {
                const float sum = (parts[0] + parts[1]) + (parts[2] + parts[3]);
                const float inverse = sum > 0.0f ? 1.0f / sum : 0.0f;
#pragma unroll
                for (int c = 0; c < 16; ++c) o[c] *= inverse;
                const uint64_t global_row = static_cast<uint64_t>(seq) * args.q_len + row;
                store_part_bf16(args.out, global_row * args.h + head * args.d, o, chunk * 16, args.d);
                if (args.stats != nullptr && chunk == 0) {
                    float* st = args.stats + (global_row * args.heads + head) * 2;
                    st[0] = best;
                    st[1] = sum;
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(FWD_TMEM) : "memory");
}

// ---- backward -------------------------------------------------------------------------------------
// Shared memory: K_j, V_j, two stages of (Q_i, G_i), P (two tiles), dS (two tiles): 160 KB; then
// barriers and the row statistics of every query (max, 1 / sum, D).
// Tensor memory (512 columns): S / dP [0, 128), dV [128, 192), dK [192, 256), dQ_i [256 + 64 i, ..).
constexpr uint32_t BWD_TILES = 10 * TILE_BYTES;
constexpr uint32_t BWD_ROWS = 512;
constexpr uint32_t BWD_SMEM = BWD_TILES + 1024 /* alignment slack */ + 256 /* barriers */ + 3 * BWD_ROWS * 4;
constexpr uint32_t BWD_TMEM = 512;

__global__ void __launch_bounds__(THREADS, 1)
attention_backward_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                          const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_g, const FusedArgs args) {
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    char* k_tile = tiles;
    char* v_tile = tiles + TILE_BYTES;
    auto q_tile = [&](uint32_t stage) { return tiles + (2 + 2 * stage) * TILE_BYTES; };
    auto g_tile = [&](uint32_t stage) { return tiles + (3 + 2 * stage) * TILE_BYTES; };
    char* p_tile = tiles + 6 * TILE_BYTES;
    char* ds_tile = tiles + 8 * TILE_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + BWD_TILES);
    // KV_FULL/KV_EMPTY: the key tile's K and V. QG_FULL/QG_EMPTY [2]: a stage of Q_i and G_i. S_FULL,
    // DP_FULL: the S / dP region holds a product. P_DONE, DS_DONE: the row threads have written P
    // (and are done with S) / dS. P_FREE, DS_FREE: the MMAs that read the P / dS tiles are complete.
    // ACC_FULL: dV_j and dK_j are complete; ACC_EMPTY: they have been drained. DQ_FULL: everything is.
    // STATS_MET: every row's statistics are in shared memory.
    enum { KV_FULL, KV_EMPTY, QG_FULL0, QG_FULL1, QG_EMPTY0, QG_EMPTY1, S_FULL, DP_FULL, P_DONE, DS_DONE, P_FREE, DS_FREE, ACC_FULL, ACC_EMPTY,
           DQ_FULL, STATS_MET, BARS };
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + BARS);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(tmem_slot + 1);
    float* row_best = reinterpret_cast<float*>(tiles + BWD_TILES + 256);  // [BWD_ROWS]
    float* row_inverse = row_best + BWD_ROWS;                             // 1 / sum of exp
    float* row_dot = row_inverse + BWD_ROWS;                              // D_i

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t head = blockIdx.x, seq = blockIdx.y;
    const uint32_t key_tiles = (args.k_len + TILE - 1) / TILE, query_tiles = (args.q_len + TILE - 1) / TILE;
    auto bar = [&](int which) { return smem_u32(&bars[which]); };

    if (tid == 0) {
        for (int b = 0; b < BARS; ++b)
            mbar_init(bar(b), (b == P_DONE || b == DS_DONE || b == ACC_EMPTY || b == STATS_MET) ? static_cast<uint32_t>(ROW_WARPS) : 1u);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(BWD_TMEM) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_sp = tmem_base, tmem_dv = tmem_base + 128, tmem_dk = tmem_base + 192, tmem_dq = tmem_base + 256;

    if (warp == 0) {
        if (lane == 0) {
            bool alive = true;
            uint32_t pair = 0;  // (j, i) pairs issued so far: stage = pair & 1
            uint32_t armed = 0, armed_phase = 0;  // bit 0 KV, bits 1-2 the QG stages
            for (uint32_t j = 0; j < key_tiles && alive; ++j) {
                alive = mbar_wait(bar(KV_EMPTY), (j & 1u) ^ 1u, abort_flag, args.status);
                if (!alive) break;
                mbar_expect_tx(bar(KV_FULL), 2 * TILE_BYTES);
                load_tile(smem_u32(k_tile), &map_k, bar(KV_FULL), args.order, j * TILE, head, seq);
                load_tile(smem_u32(v_tile), &map_v, bar(KV_FULL), args.order, j * TILE, head, seq);
                armed |= 1u;
                armed_phase = (armed_phase & ~1u) | (j & 1u);
                for (uint32_t i = 0; i < query_tiles; ++i, ++pair) {
                    const uint32_t stage = pair & 1u, use = pair >> 1;
                    alive = mbar_wait(bar(QG_EMPTY0 + stage), (use & 1u) ^ 1u, abort_flag, args.status);
                    if (!alive) break;
                    mbar_expect_tx(bar(QG_FULL0 + stage), 2 * TILE_BYTES);
                    load_tile(smem_u32(q_tile(stage)), &map_q, bar(QG_FULL0 + stage), args.order, i * TILE, head, seq);
                    load_tile(smem_u32(g_tile(stage)), &map_g, bar(QG_FULL0 + stage), args.order, i * TILE, head, seq);
                    armed |= 2u << stage;
                    armed_phase = (armed_phase & ~(2u << stage)) | ((use & 1u) << (1 + stage));
                }
            }
            if (!alive) {
                if (armed & 1u) for (uint32_t spin = 0; spin < WAIT_LIMIT && !mbar_try_wait(bar(KV_FULL), armed_phase & 1u); ++spin) {}
                for (uint32_t stage = 0; stage < 2; ++stage)
                    if (armed & (2u << stage))
                        for (uint32_t spin = 0; spin < WAIT_LIMIT && !mbar_try_wait(bar(QG_FULL0 + stage), (armed_phase >> (1 + stage)) & 1u); ++spin) {}
            }
        }
    } else if (warp == 1) {
        const uint32_t idesc_scores = instruction_descriptor(TILE, TILE, false, false);   // Q K^T, G V^T
        const uint32_t idesc_keys = instruction_descriptor(TILE, 64, true, true);         // P^T G, dS^T Q
        const uint32_t idesc_queries = instruction_descriptor(TILE, 64, false, true);     // dS K
        bool alive = true;
        uint32_t pair = 0;
        for (uint32_t j = 0; j < key_tiles && alive; ++j) {
            alive = mbar_wait(bar(KV_FULL), j & 1u, abort_flag, args.status);
            // dV_j and dK_j start from zero: the previous key tile's must have been drained.
            if (alive) alive = mbar_wait(bar(ACC_EMPTY), (j & 1u) ^ 1u, abort_flag, args.status);
            for (uint32_t i = 0; i < query_tiles && alive; ++i, ++pair) {
                const uint32_t stage = pair & 1u, use = pair >> 1, ph = pair & 1u;
                const uint32_t q_at = smem_u32(q_tile(stage)), g_at = smem_u32(g_tile(stage));
                alive = mbar_wait(bar(QG_FULL0 + stage), use & 1u, abort_flag, args.status);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
#pragma unroll
                    for (uint32_t ks = 0; ks < 4; ++ks)
                        mma_bf16(tmem_sp, tile_descriptor(q_at + ks * 32, 16), tile_descriptor(smem_u32(k_tile) + ks * 32, 16), idesc_scores, ks != 0);
                    mma_commit(bar(S_FULL));
                }
                __syncwarp();
                // The row threads have read S and written P: dP may take the region, P^T G may read P.
                alive = mbar_wait(bar(P_DONE), ph, abort_flag, args.status);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
#pragma unroll
                    for (uint32_t ks = 0; ks < 4; ++ks)
                        mma_bf16(tmem_sp, tile_descriptor(g_at + ks * 32, 16), tile_descriptor(smem_u32(v_tile) + ks * 32, 16), idesc_scores, ks != 0);
                    mma_commit(bar(DP_FULL));
                    // dV_j += P^T G_i: m = keys (two panels of 64, 16 KB apart), k = the 128 queries, 16 rows per MMA.
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks)
                        mma_bf16(tmem_dv, tile_descriptor(smem_u32(p_tile) + ks * 2048, TILE_BYTES), tile_descriptor(g_at + ks * 2048, TILE_BYTES),
                                 idesc_keys, (i | ks) != 0);
                    mma_commit(bar(P_FREE));
                }
                __syncwarp();
                alive = mbar_wait(bar(DS_DONE), ph, abort_flag, args.status);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    // dK_j += dS^T Q_i, and dQ_i += dS K_j: k = the 128 keys, 16 per MMA (32 bytes of
                    // a dS row, 16 rows of the K tile).
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks)
                        mma_bf16(tmem_dk, tile_descriptor(smem_u32(ds_tile) + ks * 2048, TILE_BYTES), tile_descriptor(q_at + ks * 2048, TILE_BYTES),
                                 idesc_keys, (i | ks) != 0);
#pragma unroll
                    for (uint32_t ks = 0; ks < 8; ++ks)
                        mma_bf16(tmem_dq + 64 * i, tile_descriptor(smem_u32(ds_tile) + (ks >> 2) * TILE_BYTES + (ks & 3u) * 32, 16),
                                 tile_descriptor(smem_u32(k_tile) + ks * 2048, TILE_BYTES), idesc_queries, (j | ks) != 0);
                    mma_commit(bar(DS_FREE));
                    mma_commit(bar(QG_EMPTY0 + stage));
                    if (i + 1 == query_tiles) {
                        mma_commit(bar(ACC_FULL));
                        mma_commit(bar(KV_EMPTY));
                        if (j + 1 == key_tiles) mma_commit(bar(DQ_FULL));
                    }
                }
                __syncwarp();
            }
        }
    } else {
        // Four threads a row of a tile (lane t of tensor memory): score columns chunk * 32 .., and
        // columns chunk * 16 .. of the gradients when they are drained.
        const uint32_t quarter = warp & 3u, chunk = (warp - 2) >> 2, t = quarter * 32 + lane;
        const uint32_t lane_base = (quarter * 32u) << 16;
        bool alive = true;
        // Row statistics of every query of this (sequence, head), one row a thread: the forward's
        // max and sum, and D = sum_c O g over the head's columns.
        {
            const uint32_t row = chunk * TILE + t;
            float best = 0.0f, inverse = 0.0f, dot = 0.0f;
            if (row < args.q_len) {
                const uint64_t global_row = static_cast<uint64_t>(seq) * args.q_len + row;
                const float* st = args.stats + (global_row * args.heads + head) * 2;
                best = st[0];
                inverse = st[1] > 0.0f ? 1.0f / st[1] : 0.0f;
                const bf16* o = static_cast<const bf16*>(args.o) + global_row * args.h + head * args.d;
                const bf16* g = static_cast<const bf16*>(args.g) + global_row * args.h + head * args.d;
                for (uint32_t c = 0; c + 8 <= args.d; c += 8) {
                    const float8 a = load8(o + c), b = load8(g + c);
                    dot = fmaf(a.lo.x, b.lo.x, dot); dot = fmaf(a.lo.y, b.lo.y, dot); dot = fmaf(a.lo.z, b.lo.z, dot); dot = fmaf(a.lo.w, b.lo.w, dot);
                    dot = fmaf(a.hi.x, b.hi.x, dot); dot = fmaf(a.hi.y, b.hi.y, dot); dot = fmaf(a.hi.z, b.hi.z, dot); dot = fmaf(a.hi.w, b.hi.w, dot);
                }
            }
            row_best[row] = best;
            row_inverse[row] = inverse;  // 0 for a row past the end: its probabilities are zeros
            row_dot[row] = dot;
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(STATS_MET));
            alive = mbar_wait(bar(STATS_MET), 0, abort_flag, args.status);
            alive = __all_sync(0xffffffffu, alive);
        }
        uint32_t pair = 0;
        for (uint32_t j = 0; j < key_tiles && alive; ++j) {
            const uint32_t counts = keys_that_count(args.mask, seq, j * TILE + chunk * 32, args.k_len, lane);
            for (uint32_t i = 0; i < query_tiles; ++i, ++pair) {
                const uint32_t ph = pair & 1u;
                const uint32_t row = i * TILE + t;
                const float best = row_best[row], inverse = row_inverse[row], dot = row_dot[row];
                alive = mbar_wait(bar(S_FULL), ph, abort_flag, args.status);
                // The P tile is free once the P^T G of the previous pair has been read by the tensor core.
                if (alive) alive = mbar_wait(bar(P_FREE), ph ^ 1u, abort_flag, args.status);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t r[32];
                tmem_load32(tmem_sp + lane_base + chunk * 32, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float p[32];
#pragma unroll
                for (int c = 0; c < 32; ++c) p[c] = ((counts >> c) & 1u) ? __expf(__uint_as_float(r[c]) * args.scale - best) * inverse : 0.0f;
                store_chunk_bf16(p_tile, t, chunk, p);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(P_DONE));
                alive = mbar_wait(bar(DP_FULL), ph, abort_flag, args.status);
                if (alive) alive = mbar_wait(bar(DS_FREE), ph ^ 1u, abort_flag, args.status);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                tmem_load32(tmem_sp + lane_base + chunk * 32, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int c = 0; c < 32; ++c) p[c] = p[c] * (__uint_as_float(r[c]) - dot) * args.scale;  // dS
                store_chunk_bf16(ds_tile, t, chunk, p);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(DS_DONE));
            }
            if (!alive) break;
            // dV_j and dK_j are complete: rows are keys now. Drain them, then free the accumulators.
            alive = mbar_wait(bar(ACC_FULL), j & 1u, abort_flag, args.status);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t key = j * TILE + t;
            const uint64_t key_at = (static_cast<uint64_t>(seq) * args.k_len + key) * args.h + head * args.d;
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                uint32_t raw[16];
                tmem_load16((which == 0 ? tmem_dv : tmem_dk) + lane_base + chunk * 16, raw);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float v[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(raw[c]);
                void* to = which == 0 ? args.dv : args.dk;
                if (to != nullptr && key < args.k_len) store_part_bf16(to, key_at, v, chunk * 16, args.d);
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(ACC_EMPTY));
        }
        if (alive) {
            alive = mbar_wait(bar(DQ_FULL), 0, abort_flag, args.status);
            alive = __all_sync(0xffffffffu, alive);
        }
        if (alive && args.dq != nullptr) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (uint32_t i = 0; i < query_tiles; ++i) {
                uint32_t raw[16];
                tmem_load16(tmem_dq + 64 * i + lane_base + chunk * 16, raw);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                float v[16];
#pragma unroll
                for (int c = 0; c < 16; ++c) v[c] = __uint_as_float(raw[c]);
                const uint32_t row = i * TILE + t;
                if (row < args.q_len) store_part_bf16(args.dq, (static_cast<uint64_t>(seq) * args.q_len + row) * args.h + head * args.d, v, chunk * 16, args.d);
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(BWD_TMEM) : "memory");
}

// The tensor map of a [batch * rows, H] operand read head by head in tiles of 128 rows.
CUtensorMap head_map(const void* base, uint32_t rows, const AttentionShape& sh, CoordOrder* order, const char* what) {
    const uint32_t h = sh.heads * sh.head_dim;
    const HalfMatrix x = {base, h, static_cast<uint64_t>(rows) * h, sh.head_dim, false};
    return encode(x, sh.head_dim, rows, sh.heads, sh.batch, TILE, order, what);
}

FusedArgs fused_args(const float* mask, AttentionShape sh, uint32_t* status) {
    FusedArgs a = {};
    a.mask = mask;
    a.status = status;
    a.batch = sh.batch;
    a.q_len = sh.q_len;
    a.k_len = sh.k_len;
    a.heads = sh.heads;
    a.d = sh.head_dim;
    a.h = sh.heads * sh.head_dim;
    a.scale = 1.0f / sqrtf(static_cast<float>(sh.head_dim));
    return a;
}

template <class K> void opt_in(K kernel, uint32_t bytes) {
    check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes)), "attention_fused shared memory");
}

}  // namespace

bool attention_fused_supported(AttentionShape sh) {
    return sh.head_dim <= 64 && sh.head_dim % 8 == 0 && sh.k_len <= BWD_ROWS && sh.q_len <= BWD_ROWS && sh.batch > 0 && sh.q_len > 0;
}

uint64_t attention_fused_stats_floats(AttentionShape sh) { return static_cast<uint64_t>(sh.batch) * sh.q_len * sh.heads * 2; }

void attention_fused_forward(cudaStream_t s, const void* q, const void* k, const void* v, const float* mask, void* out, float* stats,
                             AttentionShape sh, uint32_t* status) {
    if (!attention_fused_supported(sh)) throw std::invalid_argument("attention_fused_forward: heads of up to 64 columns, up to 512 keys and queries");
    FusedArgs args = fused_args(mask, sh, status);
    args.out = out;
    args.stats = stats;
    CoordOrder order = {}, same = {};
    const CUtensorMap map_q = head_map(q, sh.q_len, sh, &order, "q");
    const CUtensorMap map_k = head_map(k, sh.k_len, sh, &same, "k");
    const CUtensorMap map_v = head_map(v, sh.k_len, sh, &same, "v");
    args.order = order;
    opt_in(attention_forward_kernel, FWD_SMEM);
    const dim3 grid((sh.q_len + TILE - 1) / TILE, sh.heads, sh.batch);
    attention_forward_kernel<<<grid, THREADS, FWD_SMEM, s>>>(map_q, map_k, map_v, args);
    check_launch("attention_fused_forward");
}

void attention_fused_backward(cudaStream_t s, const void* q, const void* k, const void* v, const float* mask, const void* g, const void* o,
                              const float* stats, void* dq, void* dk, void* dv, AttentionShape sh, uint32_t* status) {
    if (!attention_fused_supported(sh)) throw std::invalid_argument("attention_fused_backward: heads of up to 64 columns, up to 512 keys and queries");
    FusedArgs args = fused_args(mask, sh, status);
    args.stats = const_cast<float*>(stats);
    args.o = o;
    args.g = g;
    args.dq = dq;
    args.dk = dk;
    args.dv = dv;
    CoordOrder order = {}, same = {};
    const CUtensorMap map_q = head_map(q, sh.q_len, sh, &order, "q");
    const CUtensorMap map_k = head_map(k, sh.k_len, sh, &same, "k");
    const CUtensorMap map_v = head_map(v, sh.k_len, sh, &same, "v");
    const CUtensorMap map_g = head_map(g, sh.q_len, sh, &same, "g");
    args.order = order;
    opt_in(attention_backward_kernel, BWD_SMEM);
    const dim3 grid(sh.heads, sh.batch);
    attention_backward_kernel<<<grid, THREADS, BWD_SMEM, s>>>(map_q, map_k, map_v, map_g, args);
    check_launch("attention_fused_backward");
}

}  // namespace k
}  // namespace msx
