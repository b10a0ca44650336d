// matmul on the 5th-generation tensor cores: tcgen05.mma with the accumulator in tensor memory,
// f32 operands as a split-TF32 product (tolerance class).
//
// Each f32 operand x is split into hi (its top 11 significant bits) and lo = x - hi, both exact
// tf32 values (the tensor core keeps 11 significant bits of lo, so x is represented to about
// 2^-21 |x|), and a product is summed as hi*hi + hi*lo + lo*hi (+ lo*lo where it comes for free,
// in the 64-row tile) in f32 accumulators: two orders below the kernel tolerance 1e-5 + 1e-4 r.
// The exact kernel (gemm.cu) stays for bit-level parity runs.
//
// Two kernels. Products whose operands TMA can address (bases on 16 bytes, row pitches multiples
// of 16 bytes: every product of a BERT-shaped step but the batched ones of its attention) run on
// 128 x 128 tiles in a persistent kernel fed by TMA, described where it is defined further down.
// The rest run on the 64-row tiles described here.
//
// On the 64-row tile the four partial products are not four MMAs: the hi and lo halves of A are
// stacked along M (64 rows each of one 128-row operand) and those of B along N (BN columns each of
// one 2 BN-wide operand). One MMA per 8-deep k slice then yields all four products, in four
// quadrants of tensor memory that the epilogue adds.
//
// One CTA computes a 64 x BN tile (BN = 32, 64 or 128) over a range of 32-deep k blocks:
//   warps 0-7  load the A and B blocks from global memory, split them and store hi and lo in the
//              128-byte-swizzled shared-memory layouts tcgen05 reads (K-major or MN-major by how
//              the operand is stored, so NN, TN and NT need no transposed copy), then drain the
//              accumulator: tcgen05.ld, the quadrant sums, row-wise stores to C or to the
//              split-K workspace;
//   warp 8     allocates tensor memory, issues 4 MMAs per k block from one thread, and releases
//              each shared-memory stage with tcgen05.commit.
//
// Shared memory stays under half an SM's (2 to 4 stages of 24 to 48 KB) and registers under
// half its file, so two CTAs share an SM and one drains while the other loads. Stage hand-off is
// by mbarriers; every wait is bounded and, when it runs out, raises bit 1 of the status word,
// makes every role leave its loop, frees the tensor memory and returns. A k range split across
// CTAs (grid.z, k blocks dealt out round-robin) writes partial tiles that `splitk_reduce_kernel`
// or the step's finalize launch adds in ascending split order (deterministic).
#include <atomic>
#include <cstdlib>

#include "common.cuh"
#include "kernels.cuh"
#include "tcgen05.cuh"

namespace msx {
namespace k {

namespace {

constexpr int BK = 32;
constexpr int LOADER_THREADS = 256, THREADS = LOADER_THREADS + 32;
constexpr uint32_t WAIT_LIMIT = 1u << 24;  // try_wait polls before a wait gives up
#ifndef MSX_TC_JOB_KBLOCKS
#define MSX_TC_JOB_KBLOCKS 32  // k blocks a unit of matmul_tc_jobs gets (BERT-tiny's 13 weight gradients on the 128 x 128 tile: 33 us with 8, 43 with 16, 34 with 32, which leaves the fewest partial tiles)
#endif

// The cost model of matmul_tc_plan, in SM cycles (tuning builds may override).
#ifndef MSX_TC_FIXED
#define MSX_TC_FIXED 5000.0
// Per k block of one CTA, bounded by how far ahead its loads run (SETS - 1 blocks) ...
#define MSX_TC_LATENCY32 700.0
#define MSX_TC_LATENCY64 950.0
#define MSX_TC_LATENCY128 1900.0
// ... and per k block of an SM, however many CTAs share it, bounded by the tensor pipe: a tf32
// MMA of 128 x 256 x 8 was measured at about 275 cycles (half that for 128 wide, a floor of
// about 100 below), four of them per k block.
#define MSX_TC_KB32 400.0
#define MSX_TC_KB64 560.0
#define MSX_TC_KB128 1100.0
// The 128 x 128 tile (a persistent CTA per SM): per launch, per k block (twelve MMAs of
// 128 x 128 x 8) and per tile.
#define MSX_TC_FIXED_WIDE 8000.0
#define MSX_TC_KB_WIDE 1550.0
#define MSX_TC_TILE_WIDE 500.0
#define MSX_TC_DRAIN_WIDE 5000.0  // a tile's drain, which bounds a tile of few k blocks
// Operand bytes all SMs together pull through the L2 per SM cycle.
#define MSX_TC_BYTES_PER_CYCLE 3800.0
#define MSX_TC_REDUCE_FIXED 8000.0
#define MSX_TC_REDUCE_BYTES_PER_CYCLE 3000.0
#endif

// The 64-row tile described above, two CTAs per SM (the 128 x 128 tile is a kernel of its own,
// further down).
template <int BM, int BN> struct Config {
    static_assert(BM == 64, "the stacked-A tile has 64 rows");
    static constexpr int STAGES = BN == 128 ? 2 : (BN == 64 ? 3 : 4);  // shared-memory stages
    static constexpr int SETS = BN == 32 ? 4 : (BN == 128 ? 2 : 3);    // register sets of loads in flight
    static constexpr int CTAS_PER_SM = 2;
    static constexpr uint32_t A_BYTES = 2 * BM * BK * 4;  // hi rows 0-63, lo rows 64-127
    static constexpr uint32_t B_BYTES = 2 * BN * BK * 4;  // hi columns 0..BN-1, lo columns BN..2BN-1
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t TOTAL = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
    static constexpr uint32_t TMEM_COLUMNS = 2 * BN;
};

constexpr int MAX_GROUP = 4;  // products of one shape that one launch can carry
constexpr int MAX_JOBS = 24;  // products of different shapes that one launch can carry

struct TcArgs {
    // Per product of the group (grid.z = product * splits + split when not batched):
    const float* a[MAX_GROUP];
    const float* b[MAX_GROUP];
    float* c[MAX_GROUP];           // C, or the split-K workspace [splits][m][n]
    const float* bias[MAX_GROUP];  // added to every row of C by the CTA that writes C; null for none
    uint32_t splits;
    uint32_t products;             // how many of a[], b[], c[] are used
    uint32_t m, n, k;
    uint32_t lda, ldb, ldc;        // row pitch, in elements, of each matrix as stored
    uint32_t kblocks_per_split;
    uint32_t a_vec, b_vec, c_vec;  // 16-byte accesses are aligned for this operand
    uint32_t c_padded;             // the columns of C between n and ldc are padding that may be overwritten
    uint32_t c_tma;                // the 128 x 128 tile writes C (or the split-k workspace) by TMA stores
    tc::CoordOrder c_order;        // where the row and split coordinates sit in the tensor maps of C
    tc::CoordOrder a_order, b_order;  // the same for the operands of the 128 x 128 tile
    // Batched products: grid.z = batch index z, split as (z / inner, z % inner); each matrix of
    // problem z starts at outer * stride_outer + inner * stride_inner elements. inner = 0: not batched.
    uint32_t batch_inner;
    uint64_t a_outer, a_inner, b_outer, b_inner, c_outer, c_inner;
    uint32_t* status;
    // Products of different shapes in one launch (one storage form, one tile width): a 1-D grid
    // whose block b belongs to the job whose block range holds it; `job_count` = 0 otherwise.
    uint32_t job_count;
    struct Job {
        const float* a;
        const float* b;
        float* c;  // C, or the job's split-K workspace
        uint32_t m, n, k, lda, ldb, ldc, splits, first_block;  // first_block: the job's first block, or unit of the 128 x 128 tile
        tc::CoordOrder c_order;                               // the 128 x 128 tile: as TcArgs::c_order, of this job's result
    } jobs[MAX_JOBS];
    uint32_t units;  // the 128 x 128 tile: tiles x splits over all products or jobs of the launch
};

#ifdef MSX_TC_TRACE
// Phase timestamps of the first 16 CTAs, for tuning builds only.
__device__ long long g_trace[16][16];
#define TRACE(slot) do { if (blockIdx.x + blockIdx.y * gridDim.x + blockIdx.z * gridDim.x * gridDim.y < 16) \
    g_trace[blockIdx.x + blockIdx.y * gridDim.x + blockIdx.z * gridDim.x * gridDim.y][slot] = clock64(); } while (0)
#else
#define TRACE(slot) do { } while (0)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for `parity` of `bar`; false when the wait ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status) {
    for (uint32_t spin = 0; spin < WAIT_LIMIT; ++spin) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spin & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicOr(status, 2u);
    return false;
}

// The same, polled by one lane for its warp (all lanes must call it together).
__device__ __forceinline__ bool warp_mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, uint32_t* status) {
    uint32_t ok = 0;
    if ((threadIdx.x & 31u) == 0) ok = mbar_wait(bar, parity, abort_flag, status) ? 1u : 0u;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    // The lanes that did not poll observe the phase themselves before they touch what it guards.
    if (ok) mbar_try_wait(bar, parity);
    return ok != 0;
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 32 lanes x 32 consecutive columns of tensor memory: r[j] = column `taddr.column + j` of this
// thread's lane.
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_load16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// Byte offset of the 16-byte chunk holding elements (row, 4 c16 .. 4 c16 + 3) of a K-major tile:
// 128-byte rows, 8-row groups of 1024 bytes, chunk index xor-ed with the row within its group.
__device__ __forceinline__ uint32_t k_major_offset(uint32_t row, uint32_t c16) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((c16 ^ (row & 7u)) << 4);
}
// The same for an MN-major tile: for each k a 128-byte row of 32 consecutive MN elements, the
// 32 k rows of a block forming one 4096-byte panel per 32 MN elements; within a row the 32-byte
// chunk index is xor-ed with the k row modulo 4 (groups of 4 rows, 512 bytes). `c` counts 16-byte
// chunks along MN.
__device__ __forceinline__ uint32_t mn_major_offset(uint32_t krow, uint32_t c) {
    uint32_t in_panel = c & 7u;
    return (c >> 3) * (BK * 128u) + krow * 128u + (((in_panel >> 1) ^ (krow & 3u)) << 5) + ((in_panel & 1u) << 4);
}

__device__ __forceinline__ float4 load4(const float* __restrict__ p, uint64_t index, uint32_t valid, bool vec) {
    // `valid` = how many of the 4 elements from `index` are inside the matrix (0..4).
    // Volatile asm keeps every load where it is written: the prefetch depth is the point, and
    // the compiler otherwise sinks the loads to their first use.
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    const float* at = p + index;
    if (valid == 4 && vec) {
        asm volatile("ld.global.nc.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(at));
        return v;
    }
    if (valid > 0) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v.x) : "l"(at));
    if (valid > 1) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v.y) : "l"(at + 1));
    if (valid > 2) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v.z) : "l"(at + 2));
    if (valid > 3) asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v.w) : "l"(at + 3));
    return v;
}

// hi = x with the 13 mantissa bits below tf32 cleared (an exact tf32, whatever rounding the tensor
// core would apply to a wider value), lo = x - hi exactly (at most 13 significant bits, below
// 2^-10 |x|). One logic op and one subtraction per element: the split must not cost more than
// the MMAs it feeds.
__device__ __forceinline__ float top_tf32(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }

__device__ __forceinline__ void store_split(char* tile, uint32_t hi_offset, uint32_t lo_offset, float4 v) {
    float4 h, l;
    h.x = top_tf32(v.x); h.y = top_tf32(v.y); h.z = top_tf32(v.z); h.w = top_tf32(v.w);
    l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
    *reinterpret_cast<float4*>(tile + hi_offset) = h;
    *reinterpret_cast<float4*>(tile + lo_offset) = l;
}

__device__ __forceinline__ uint32_t in_range(uint32_t start, uint32_t limit) {
    return start >= limit ? 0u : (limit - start >= 4u ? 4u : limit - start);
}

__device__ __forceinline__ void loaders_barrier(uint32_t threads) {
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

template <int BM, int BN, bool A_T, bool B_T>
__global__ void __launch_bounds__(THREADS, Config<BM, BN>::CTAS_PER_SM) matmul_tc_kernel(TcArgs args) {
    using Cfg = Config<BM, BN>;
    constexpr int STAGES = Cfg::STAGES, SETS = Cfg::SETS;
    extern __shared__ char smem_raw[];
    // Tiles need 1024-byte alignment for the swizzle pattern to line up with address bits.
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(tiles + STAGES * Cfg::STAGE_BYTES);
    // bars[0 .. STAGES) full, bars[STAGES .. 2 STAGES) empty, bars[2 STAGES] accumulator ready;
    // then the TMEM address and the abort flag.
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 1);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * STAGES + 2);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) TRACE(0);
    // The problem this CTA works on: the launch's own, or one job of a launch that carries several.
    uint32_t pm = args.m, pn = args.n, pk = args.k, plda = args.lda, pldb = args.ldb, pldc = args.ldc, psplits = args.splits;
    uint32_t tile_x = blockIdx.x, tile_y = blockIdx.y, tile_z = blockIdx.z;
    const float* job_a = nullptr;
    const float* job_b = nullptr;
    float* job_c = nullptr;
    if (args.job_count) {
        uint32_t j = 0;
        while (j + 1 < args.job_count && args.jobs[j + 1].first_block <= blockIdx.x) ++j;
        const TcArgs::Job& job = args.jobs[j];
        pm = job.m; pn = job.n; pk = job.k; plda = job.lda; pldb = job.ldb; pldc = job.ldc; psplits = job.splits;
        job_a = job.a; job_b = job.b; job_c = job.c;
        const uint32_t local = blockIdx.x - job.first_block, across = (pn + BN - 1) / BN, down = (pm + BM - 1) / BM;
        tile_x = local % across;
        tile_y = (local / across) % down;
        tile_z = local / (across * down);
    }
    const uint32_t m0 = tile_y * BM, n0 = tile_x * BN;
    const uint32_t kblocks_total = (pk + BK - 1) / BK;
    const bool batched = args.batch_inner != 0;
    const uint32_t z_outer = batched ? tile_z / args.batch_inner : 0, z_inner = batched ? tile_z % args.batch_inner : 0;
    const uint32_t product = (batched || args.job_count) ? 0 : tile_z / psplits, split = batched ? 0 : tile_z % psplits;
    // A split k is dealt out block by block: split s takes k blocks s, s + splits, ... The CTAs of
    // the splits of one tile run side by side, so at any time they read neighbouring 128-byte
    // pieces of the same operand rows (one DRAM page) instead of pieces a whole k range apart.
    const uint32_t stride = batched ? 1u : psplits;
    const uint32_t kblocks = kblocks_total > split ? (kblocks_total - split + stride - 1) / stride : 0;

    // ---- loaders, first part: where this thread's chunks sit, and the first loads. They are issued
    // before the barriers and the tensor memory are set up, so that the set-up hides under them.
    const float* __restrict__ a = job_a ? job_a : args.a[product] + z_outer * args.a_outer + z_inner * args.a_inner;
    const float* __restrict__ b = job_b ? job_b : args.b[product] + z_outer * args.b_outer + z_inner * args.b_inner;
    constexpr int A_CHUNKS = BM * BK / 4 / LOADER_THREADS, B_CHUNKS = BN * BK / 4 / LOADER_THREADS;
    // Where this thread's chunks sit in a block does not depend on the block: the shared-memory
    // offsets, the address of each chunk in the first k block and whether all four of its elements
    // lie inside the matrix rows are computed once. A k block that lies wholly inside k then costs
    // one pointer addition and one 16-byte load per chunk: address arithmetic and bounds checks
    // per block would be as many instructions again as the split itself. The lo half of an operand
    // lies half the operand's bytes after the hi half (64 rows, BN rows, or as many 32-element
    // panels).
    uint32_t aoff[A_CHUNKS], boff[B_CHUNKS];
    const float* a_at[A_CHUNKS];
    const float* b_at[B_CHUNKS];
    bool a_whole[A_CHUNKS], b_whole[B_CHUNKS];
    constexpr uint32_t a_per_k_row = BM / 4, b_per_k_row = BN / 4;  // 16-byte chunks of one k row of an MN-major tile
    auto a_place = [&](int i, uint32_t* row, uint32_t* col) {
        const uint32_t q = tid + i * LOADER_THREADS;
        if (A_T) { *row = q / a_per_k_row; *col = (q % a_per_k_row) * 4; }  // (k, m)
        else     { *row = q >> 3; *col = (q & 7u) * 4; }                    // (m, k)
    };
    auto b_place = [&](int i, uint32_t* row, uint32_t* col) {
        const uint32_t q = tid + i * LOADER_THREADS;
        if (B_T) { *row = q >> 3; *col = (q & 7u) * 4; }                    // (n, k)
        else     { *row = q / b_per_k_row; *col = (q % b_per_k_row) * 4; }  // (k, n)
    };
    const uint32_t first_k = split * BK;
#pragma unroll
    for (int i = 0; i < A_CHUNKS; ++i) {
        uint32_t row, col;
        a_place(i, &row, &col);
        aoff[i] = A_T ? mn_major_offset(row, col / 4) : k_major_offset(row, col / 4);
        a_at[i] = A_T ? a + static_cast<uint64_t>(first_k + row) * plda + m0 + col
                      : a + static_cast<uint64_t>(m0 + row) * plda + first_k + col;
        a_whole[i] = args.a_vec && (A_T ? m0 + col + 4 <= pm : m0 + row < pm);
    }
#pragma unroll
    for (int i = 0; i < B_CHUNKS; ++i) {
        uint32_t row, col;
        b_place(i, &row, &col);
        boff[i] = B_T ? k_major_offset(row, col / 4) : mn_major_offset(row, col / 4);
        b_at[i] = B_T ? b + static_cast<uint64_t>(n0 + row) * pldb + first_k + col
                      : b + static_cast<uint64_t>(first_k + row) * pldb + n0 + col;
        b_whole[i] = args.b_vec && (B_T ? n0 + row < pn : n0 + col + 4 <= pn);
    }
    // Elements from one k block of this CTA to its next.
    const uint64_t a_step = static_cast<uint64_t>(BK) * stride * (A_T ? plda : 1u);
    const uint64_t b_step = static_cast<uint64_t>(BK) * stride * (B_T ? 1u : pldb);
    auto fetch = [&](uint32_t kb, float4 (&av)[A_CHUNKS], float4 (&bv)[B_CHUNKS]) {
        const uint32_t k0 = (kb * stride + split) * BK;
        const bool inside = k0 + BK <= pk;
#pragma unroll
        for (int i = 0; i < A_CHUNKS; ++i) {
            if (inside && a_whole[i]) {
                av[i] = load4(a_at[i] + kb * a_step, 0, 4, true);
                continue;
            }
            uint32_t row, col;
            a_place(i, &row, &col);
            if (A_T) {  // stored [k, m]: 4 consecutive m of one k row
                uint32_t gk = k0 + row, gm = m0 + col;
                uint32_t valid = gk < pk ? in_range(gm, pm) : 0u;
                av[i] = load4(a, static_cast<uint64_t>(gk) * plda + gm, valid, args.a_vec);
            } else {    // stored [m, k]: 4 consecutive k of one row
                uint32_t gm = m0 + row, gk = k0 + col;
                uint32_t valid = gm < pm ? in_range(gk, pk) : 0u;
                av[i] = load4(a, static_cast<uint64_t>(gm) * plda + gk, valid, args.a_vec);
            }
        }
#pragma unroll
        for (int i = 0; i < B_CHUNKS; ++i) {
            if (inside && b_whole[i]) {
                bv[i] = load4(b_at[i] + kb * b_step, 0, 4, true);
                continue;
            }
            uint32_t row, col;
            b_place(i, &row, &col);
            if (B_T) {  // stored [n, k]
                uint32_t gn = n0 + row, gk = k0 + col;
                uint32_t valid = gn < pn ? in_range(gk, pk) : 0u;
                bv[i] = load4(b, static_cast<uint64_t>(gn) * pldb + gk, valid, args.b_vec);
            } else {    // stored [k, n]
                uint32_t gk = k0 + row, gn = n0 + col;
                uint32_t valid = gk < pk ? in_range(gn, pn) : 0u;
                bv[i] = load4(b, static_cast<uint64_t>(gk) * pldb + gn, valid, args.b_vec);
            }
        }
    };
    // SETS register sets: the loads of the next SETS - 1 blocks are in flight while a block is
    // split and stored.
    float4 av[SETS][A_CHUNKS], bv[SETS][B_CHUNKS];
    // The four bias values this thread adds in the epilogue, fetched with the first loads: a load
    // issued in the epilogue would be a round trip to memory with nothing to hide behind.
    const float* __restrict__ bias_row = (job_c || args.job_count) ? nullptr : args.bias[product];
    float bias_mine[4] = {0.f, 0.f, 0.f, 0.f};
    if (warp < 8) {
        if (bias_row) {
            const uint32_t gn = n0 + (lane % (BN / 4)) * 4;
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (gn + q < pn) bias_mine[q] = __ldg(bias_row + gn + q);
        }
#pragma unroll
        for (int s = 0; s < SETS - 1; ++s)
            if (static_cast<uint32_t>(s) < kblocks) fetch(s, av[s], bv[s]);
    }

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&bars[s]), LOADER_THREADS);
            mbar_init(smem_u32(&bars[STAGES + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * STAGES]), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Cfg::TMEM_COLUMNS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    if (tid == 0) TRACE(1);

    if (warp < 8) {
        // ---- loaders: global -> (hi, lo) -> swizzled shared memory ---------------------------
        bool alive = true;
        auto deposit = [&](uint32_t kb, const float4 (&a_regs)[A_CHUNKS], const float4 (&b_regs)[B_CHUNKS]) -> bool {
            const uint32_t stage = kb % STAGES, round = kb / STAGES;
            char* a_tile = tiles + stage * Cfg::STAGE_BYTES;
            char* b_tile = a_tile + Cfg::A_BYTES;
            // The stage is free once the MMAs that read its previous contents have completed.
            if (!mbar_wait(smem_u32(&bars[STAGES + stage]), (round & 1u) ^ 1u, abort_flag, args.status)) return false;
#pragma unroll
            for (int i = 0; i < A_CHUNKS; ++i) store_split(a_tile, aoff[i], aoff[i] + Cfg::A_BYTES / 2, a_regs[i]);
#pragma unroll
            for (int i = 0; i < B_CHUNKS; ++i) store_split(b_tile, boff[i], boff[i] + Cfg::B_BYTES / 2, b_regs[i]);
            // Make the generic-proxy stores visible to the tensor core's async-proxy reads.
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(&bars[stage]));
            if (tid == 0 && kb < 4) TRACE(2 + kb);
            return true;
        };
        for (uint32_t kb0 = 0; kb0 < kblocks && alive; kb0 += SETS) {
#pragma unroll
            for (int s = 0; s < SETS; ++s) {
                const uint32_t kb = kb0 + s;
                if (kb >= kblocks || !alive) break;
                if (kb + SETS - 1 < kblocks) fetch(kb + SETS - 1, av[(s + SETS - 1) % SETS], bv[(s + SETS - 1) % SETS]);
                alive = deposit(kb, av[s], bv[s]);
            }
        }
        // ---- epilogue: tensor memory -> shared memory -> global --------------------------------
        // Lanes 0-63 of tensor memory hold the A_hi rows, 64-127 the A_lo rows of the same 64 tile
        // rows; columns [0, BN) the products with B_hi, [BN, 2 BN) those with B_lo. A warp reads
        // its lane quarter, adds the two column halves and writes the sums, row-major, into one of
        // two shared-memory tiles (hi rows, lo rows; the stages are free by now). After a barrier
        // all eight warps add the two tiles and write C a whole tile row at a time, 16 bytes per
        // lane where the pitch of C allows.
        if (alive && kblocks > 0) alive = mbar_wait(smem_u32(&bars[2 * STAGES]), 0, abort_flag, args.status);
        alive = __all_sync(0xffffffffu, alive);  // tcgen05.ld is warp-wide: decide as a warp
        if (tid == 0) TRACE(6);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t quarter = warp & 3u, half = warp >> 2;
        constexpr int PARTS = BN == 128 ? 2 : 1;
        constexpr uint32_t PITCH = BN + 4;  // 16-byte phases of consecutive rows fall on distinct banks
        const bool drains = BN != 32 || half == 0;  // a 32-column tile is one block per lane quarter
        float* tile_hi = reinterpret_cast<float*>(tiles);
        float* tile_lo = tile_hi + 64 * PITCH;  // the sums of the A_lo rows
        if (drains) {
            // Lane quarters 0-1 hold the A_hi rows, 2-3 the A_lo rows.
            float* to_row = (quarter < 2 ? tile_hi : tile_lo) + ((quarter & 1u) * 32u + lane) * PITCH;
#pragma unroll
            for (int part = 0; part < PARTS; ++part) {
                const uint32_t col = BN == 128 ? half * 64u + part * 32u : (BN == 64 ? half * 32u : 0u);
                uint32_t r1[32], r2[32];
                if (alive && kblocks > 0) {
                    const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + col;
                    tmem_load32(taddr, r1);
                    tmem_load32(taddr + BN, r2);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) { r1[j] = 0u; r2[j] = 0u; }  // an empty k range contributes zeros
                }
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    float4 v;
                    v.x = __uint_as_float(r1[j]) + __uint_as_float(r2[j]);
                    v.y = __uint_as_float(r1[j + 1]) + __uint_as_float(r2[j + 1]);
                    v.z = __uint_as_float(r1[j + 2]) + __uint_as_float(r2[j + 2]);
                    v.w = __uint_as_float(r1[j + 3]) + __uint_as_float(r2[j + 3]);
                    *reinterpret_cast<float4*>(to_row + col + j) = v;
                }
            }
        }
        loaders_barrier(LOADER_THREADS);
        if (tid == 0) TRACE(13);
        float* __restrict__ out = batched ? args.c[0] + z_outer * args.c_outer + z_inner * args.c_inner
                                          : (job_c ? job_c : args.c[product]) + static_cast<uint64_t>(split) * pm * pldc;
        constexpr uint32_t LANES_PER_ROW = BN / 4, ROWS_PER_PASS = 32 / LANES_PER_ROW;
        const uint32_t c4 = (lane % LANES_PER_ROW) * 4, gn = n0 + c4;
#pragma unroll 4
        for (uint32_t r = warp * ROWS_PER_PASS + lane / LANES_PER_ROW; r < BM; r += 8 * ROWS_PER_PASS) {
            const uint32_t gm = m0 + r;
            if (gm >= pm || gn >= pn) continue;
            const float4 h = *reinterpret_cast<const float4*>(tile_hi + r * PITCH + c4);
            const float4 l = *reinterpret_cast<const float4*>(tile_lo + r * PITCH + c4);
            // `x + 0` turns a -0 sum of zero products into the +0 a skipped term gives.
            float v[4] = {(h.x + l.x) + 0.0f, (h.y + l.y) + 0.0f, (h.z + l.z) + 0.0f, (h.w + l.w) + 0.0f};
            if (bias_row) {
#pragma unroll
                for (int q = 0; q < 4; ++q) v[q] = v[q] + bias_mine[q];
            }
            float* dst = out + static_cast<uint64_t>(gm) * pldc + gn;
            // Inside the pitch a whole float4 may be written: what lies past n is padding.
            if (args.c_vec && (gn + 4 <= pn || (args.c_padded && gn + 4 <= pldc))) {
                *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    if (gn + q < pn) dst[q] = v[q];
            }
        }
    } else {
        // ---- the MMA warp: one thread issues, the tensor core runs asynchronously ---------------
        // Instruction descriptor: f32 accumulator, tf32 A and B, their majors, N >> 3, M >> 4, for
        // the stacked operands: M = 128 (hi and lo rows), N = 2 BN (hi and lo columns).
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_T ? 1u : 0u) << 15) | ((B_T ? 0u : 1u) << 16) |
                               (static_cast<uint32_t>((2 * BN) >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
        // The shared-memory matrix descriptor of tcgen05 (version 1): start address (bits 0-13),
        // leading (16-29) and stride (32-45) byte offsets, all in 16-byte units, bit 46 set (the
        // sm_100 version), and in bits 61-63 the swizzle of the tile: 2 = 128-byte swizzle of
        // 16-byte chunks (K-major tiles), 1 = 128-byte swizzle of 32-byte chunks, the one layout
        // the tensor core reads MN-major 32-bit operands from. The descriptors of a k block differ
        // only in the start address: everything else is built once.
        constexpr uint32_t a_lbo = A_T ? BK * 128u : 16u, b_lbo = B_T ? 16u : BK * 128u;
        constexpr uint32_t a_sbo = A_T ? 512u : 1024u, b_sbo = B_T ? 1024u : 512u;
        constexpr uint32_t a_type = A_T ? 1u : 2u, b_type = B_T ? 2u : 1u;
        constexpr uint32_t a_high = ((a_sbo >> 4) & 0x3FFFu) | (1u << 14) | (a_type << 29);
        constexpr uint32_t b_high = ((b_sbo >> 4) & 0x3FFFu) | (1u << 14) | (b_type << 29);
        constexpr uint32_t a_low = ((a_lbo >> 4) & 0x3FFFu) << 16, b_low = ((b_lbo >> 4) & 0x3FFFu) << 16;
        const uint32_t tiles16 = (smem_u32(tiles) & 0x3FFFFu) >> 4;
        auto desc = [](uint32_t high, uint32_t low) { return (static_cast<uint64_t>(high) << 32) | low; };
        bool alive = true;
        uint32_t stage = 0, parity = 0;
        for (uint32_t kb = 0; kb < kblocks && alive; ++kb) {
            alive = mbar_wait(smem_u32(&bars[stage]), parity, abort_flag, args.status);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (lane == 0) {
                const uint32_t a16 = a_low + tiles16 + stage * (Cfg::STAGE_BYTES >> 4);
                const uint32_t b16 = b_low + tiles16 + stage * (Cfg::STAGE_BYTES >> 4) + (Cfg::A_BYTES >> 4);
#pragma unroll
                for (uint32_t ks = 0; ks < BK / 8; ++ks) {
                    // One MMA covers k = 8: 32 bytes along a K-major row (8-row groups 1024 bytes
                    // apart), or 8 rows of an MN-major panel (4-row groups 512 bytes apart, panels
                    // of 32 MN elements 4096 bytes apart).
                    const uint32_t a_step = (A_T ? ks * 1024u : ks * 32u) >> 4;
                    const uint32_t b_step = (B_T ? ks * 32u : ks * 1024u) >> 4;
                    mma_tf32(tmem_base, desc(a_high, a16 + a_step), desc(b_high, b16 + b_step), idesc, (kb | ks) != 0u);
                }
                mma_commit(smem_u32(&bars[STAGES + stage]));                   // frees the stage when they finish
                if (kb < 4) TRACE(8 + kb);
                if (kb + 1 == kblocks) mma_commit(smem_u32(&bars[2 * STAGES]));  // and, at the end, the accumulator
            }
            if (++stage == STAGES) { stage = 0; parity ^= 1u; }
            __syncwarp();
        }
    }
    if (tid == 0) TRACE(7);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0) TRACE(12);
    if (warp == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::TMEM_COLUMNS) : "memory");
    }
}

#ifdef MSX_TC_TRACE
// Phase timestamps of CTA 0 of the persistent kernel, for tuning builds only.
#define WTRACE(slot) do { if (blockIdx.x == 0 && (slot) < 256) (&g_trace[0][0])[(slot)] = clock64(); } while (0)
#else
#define WTRACE(slot) do { } while (0)
#endif

// ---- the 128 x 128 tile as a persistent kernel ---------------------------------------------------
// For every product whose operands TMA can address. The hi and lo halves of A are two 128-row
// operands, those of B two 128-column ones; per 8-deep k slice three MMAs of 128 x 128 x 8 add
// hi*hi, hi*lo and lo*hi into one accumulator (lo*lo, below 2^-20 of a product, is left out). One CTA per SM
// walks the launch's tiles (block b takes units b, b + grid, ...), so the set-up of a CTA is paid
// once and the drain of a tile runs under the k loop of the next one. The raw f32 blocks come in
// by TMA (zero-filled past the matrix edges, so no role checks bounds): loads issued by threads
// kept too few bytes in flight to hide their latency (a k block took 1,860 cycles to load, split
// and store against 1,070 for its MMAs).
//   warps 0-7   split: read a raw k block (A 128 x 32, B 128 x 32) from its shared-memory slot,
//               store the hi and lo halves in the layouts tcgen05 reads, free the slot;
//   warp 8      issues the MMAs into one of two accumulators of 128 tensor-memory columns;
//   warp 9      issues the TMA loads of the k blocks of all the CTA's tiles as one sequence, two
//               blocks ahead of the splitters;
//   warps 12-15 drain the other accumulator: a lane quarter each, 32 columns at a time into a
//               shared-memory slab of their own (two per warp), which a TMA store writes to C
//               while the next slab is filled.
struct Wide {
    static constexpr int STAGES = 2, DRAIN_WARPS = 4;  // split stages, and as many raw slots
    // Four groups of four warps: two of splitters, one with the MMA and the TMA warp, one of drain
    // warps.
    static constexpr int THREADS = 512, DRAIN_FIRST_WARP = 12;
    static constexpr uint32_t A_BYTES = 2 * 128 * BK * 4;  // hi tile, lo tile
    static constexpr uint32_t B_BYTES = 2 * 128 * BK * 4;  // hi columns 0-127, lo columns 128-255
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t RAW_OPERAND_BYTES = 128 * BK * 4, RAW_BYTES = 2 * RAW_OPERAND_BYTES;  // A block, B block
    static constexpr uint32_t SLAB_BYTES = 32 * 128;                     // 32 rows of 32 floats
    static constexpr uint32_t DRAIN_BYTES = DRAIN_WARPS * 2 * SLAB_BYTES;  // two slabs per drain warp
    static constexpr uint32_t TOTAL = STAGES * (STAGE_BYTES + RAW_BYTES) + DRAIN_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
    static constexpr uint32_t ACC_COLUMNS = 128, TMEM_COLUMNS = 256;
};

// Which tile, split and product (or job) unit `u` of a launch is, with that product's sizes: the
// tiles of one column of tiles are neighbours (they share their B block), then the splits of a
// tile, then the columns; the jobs of a launch that carries several follow one another.
struct WideUnit {
    uint32_t m0, n0, split, product, kblocks;
    uint32_t m, n, ldc, splits;
    float* c;
    const float* bias;
    tc::CoordOrder c_order;
};
__device__ __forceinline__ WideUnit wide_unit(const TcArgs& args, uint32_t u) {
    WideUnit w;
    uint32_t k;
    if (args.job_count) {
        uint32_t j = 0;
        while (j + 1 < args.job_count && args.jobs[j + 1].first_block <= u) ++j;
        const TcArgs::Job& job = args.jobs[j];
        u -= job.first_block;
        w.product = j;
        w.m = job.m; w.n = job.n; k = job.k; w.ldc = job.ldc; w.splits = job.splits;
        w.c = job.c;
        w.bias = nullptr;
        w.c_order = job.c_order;
    } else {
        w.m = args.m; w.n = args.n; k = args.k; w.ldc = args.ldc; w.splits = args.splits;
        w.c_order = args.c_order;
    }
    const uint32_t down = (w.m + 127) / 128, across = (w.n + 127) / 128, kblocks_total = (k + BK - 1) / BK;
    w.m0 = (u % down) * 128u;
    u /= down;
    w.split = u % w.splits;
    u /= w.splits;
    w.n0 = (u % across) * 128u;
    if (!args.job_count) {
        w.product = u / across;
        w.c = args.c[w.product];
        w.bias = args.bias[w.product];
    }
    w.kblocks = kblocks_total > w.split ? (kblocks_total - w.split + w.splits - 1) / w.splits : 0u;
    return w;
}

// The tensor maps of a launch's products: the operands as stored (boxes of 32 floats by 128 rows
// for an operand stored with k along its rows, by 32 rows for one stored with k down its columns)
// and the results (or their split-k workspaces).
struct WideMaps {
    CUtensorMap a[MAX_JOBS], b[MAX_JOBS], c[MAX_JOBS];
};

template <bool A_T, bool B_T>
__global__ void __launch_bounds__(Wide::THREADS, 1) matmul_tc_wide_kernel(TcArgs args, const __grid_constant__ WideMaps maps) {
    constexpr int STAGES = Wide::STAGES;
    extern __shared__ char smem_raw[];
    char* tiles = reinterpret_cast<char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
    char* raw_blocks = tiles + STAGES * Wide::STAGE_BYTES;
    char* drain_slabs = raw_blocks + STAGES * Wide::RAW_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(drain_slabs + Wide::DRAIN_BYTES);
    // Barriers: split stage s filled / free, raw slot s filled / free, accumulator b ready /
    // drained; then the TMEM address and the abort flag.
    uint64_t* split_full = bars;
    uint64_t* split_empty = bars + STAGES;
    uint64_t* raw_full = bars + 2 * STAGES;
    uint64_t* raw_empty = bars + 3 * STAGES;
    uint64_t* acc_full = bars + 4 * STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(acc_empty + 3);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t units = args.units;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(&split_full[s]), LOADER_THREADS);
            mbar_init(smem_u32(&split_empty[s]), 1);
            mbar_init(smem_u32(&raw_full[s]), 1);  // the TMA warp's arrival, with the bytes it expects
            mbar_init(smem_u32(&raw_empty[s]), LOADER_THREADS);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(smem_u32(&acc_full[b]), 1);
            mbar_init(smem_u32(&acc_empty[b]), Wide::DRAIN_WARPS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(Wide::TMEM_COLUMNS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 8) {
        // ---- the splitters: raw block -> (hi, lo) -> the swizzled tiles tcgen05 reads -------------
        // How many k blocks this CTA works through in all: the sequence the stages count along.
        uint32_t total = 0;
        for (uint32_t u = blockIdx.x; u < units; u += gridDim.x) total += wide_unit(args, u).kblocks;
        // A raw block lies as its TMA load left it, in the 128-byte swizzle: an operand stored
        // with k along its rows as 128 rows of 128 bytes, one stored with k down its columns as
        // four panels of 32 k rows of 128 bytes (32 of the 128 tile rows or columns each). Chunk i
        // of a thread lies a fixed number of rows after its chunk 0, in the raw block and in the
        // split tile alike.
        constexpr int CHUNKS = 128 * BK / 4 / LOADER_THREADS;  // 16-byte chunks of one operand block a thread moves
        constexpr uint32_t A_TILE_STEP = A_T ? (LOADER_THREADS / 32) * 128u : (LOADER_THREADS / 64) * 1024u;
        constexpr uint32_t B_TILE_STEP = B_T ? (LOADER_THREADS / 64) * 1024u : (LOADER_THREADS / 32) * 128u;
        constexpr uint32_t A_RAW_STEP = A_T ? 1024u : 4096u, B_RAW_STEP = B_T ? 4096u : 1024u;  // 8 k rows, or 32 rows
        const uint32_t a_row = A_T ? tid >> 5 : tid >> 3, a_chunk = A_T ? tid & 31u : tid & 7u;  // (k, m) or (m, k)
        const uint32_t b_row = B_T ? tid >> 3 : tid >> 5, b_chunk = B_T ? tid & 7u : tid & 31u;  // (n, k) or (k, n)
        const uint32_t aoff = A_T ? mn_major_offset(a_row, a_chunk) : k_major_offset(a_row, a_chunk);
        const uint32_t boff = B_T ? k_major_offset(b_row, b_chunk) : mn_major_offset(b_row, b_chunk);
        const uint32_t a_raw = A_T ? (a_chunk >> 3) * 4096u + tc::swizzled_chunk(a_row, a_chunk & 7u) : tc::swizzled_chunk(a_row, a_chunk);
        const uint32_t b_raw = B_T ? tc::swizzled_chunk(b_row, b_chunk) : (b_chunk >> 3) * 4096u + tc::swizzled_chunk(b_row, b_chunk & 7u);
        bool alive = true;
        uint32_t stage = 0, parity = 0;
        for (uint32_t g = 0; g < total && alive; ++g) {
            const char* raw = raw_blocks + stage * Wide::RAW_BYTES;
            char* a_tile = tiles + stage * Wide::STAGE_BYTES;
            char* b_tile = a_tile + Wide::A_BYTES;
            if (tid == 0 && g < 24) WTRACE(64 + 2 * g);
            // The raw block has landed, and the MMAs that read the stage's previous contents have completed.
            alive = mbar_wait(smem_u32(&raw_full[stage]), parity, abort_flag, args.status) &&
                    mbar_wait(smem_u32(&split_empty[stage]), parity ^ 1u, abort_flag, args.status);
            if (!alive) break;
            if (tid == 0 && g < 24) WTRACE(65 + 2 * g);
            float4 av[CHUNKS], bv[CHUNKS];
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) av[i] = *reinterpret_cast<const float4*>(raw + a_raw + i * A_RAW_STEP);
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) bv[i] = *reinterpret_cast<const float4*>(raw + Wide::RAW_OPERAND_BYTES + b_raw + i * B_RAW_STEP);
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) store_split(a_tile, aoff + i * A_TILE_STEP, aoff + i * A_TILE_STEP + Wide::A_BYTES / 2, av[i]);
#pragma unroll
            for (int i = 0; i < CHUNKS; ++i) store_split(b_tile, boff + i * B_TILE_STEP, boff + i * B_TILE_STEP + Wide::B_BYTES / 2, bv[i]);
            // The raw slot may be loaded again (its values are in registers or stored); the split
            // stores are visible to the tensor core's async-proxy reads before the MMA warp is told.
            mbar_arrive(smem_u32(&raw_empty[stage]));
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            mbar_arrive(smem_u32(&split_full[stage]));
            if (++stage == STAGES) { stage = 0; parity ^= 1u; }
        }
    } else if (warp < Wide::DRAIN_FIRST_WARP) {
        if (warp == 8) {
        // ---- the MMA warp ---------------------------------------------------------------------------
        // Instruction descriptors: f32 accumulator, tf32 A and B, their majors, N >> 3, M >> 4.
        const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((A_T ? 1u : 0u) << 15) | ((B_T ? 0u : 1u) << 16) |
                               (static_cast<uint32_t>(128 >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
        constexpr uint32_t a_lbo = A_T ? BK * 128u : 16u, b_lbo = B_T ? 16u : BK * 128u;
        constexpr uint32_t a_sbo = A_T ? 512u : 1024u, b_sbo = B_T ? 1024u : 512u;
        constexpr uint32_t a_type = A_T ? 1u : 2u, b_type = B_T ? 2u : 1u;
        constexpr uint32_t a_high = ((a_sbo >> 4) & 0x3FFFu) | (1u << 14) | (a_type << 29);
        constexpr uint32_t b_high = ((b_sbo >> 4) & 0x3FFFu) | (1u << 14) | (b_type << 29);
        constexpr uint32_t a_low = ((a_lbo >> 4) & 0x3FFFu) << 16, b_low = ((b_lbo >> 4) & 0x3FFFu) << 16;
        const uint32_t tiles16 = (smem_u32(tiles) & 0x3FFFFu) >> 4;
        auto desc = [](uint32_t high, uint32_t low) { return (static_cast<uint64_t>(high) << 32) | low; };
        bool alive = true;
        uint32_t stage = 0, parity = 0, turn = 0;
        for (uint32_t u = blockIdx.x; u < units && alive; u += gridDim.x, ++turn) {
            const uint32_t kblocks = wide_unit(args, u).kblocks;
            if (kblocks == 0) continue;
            const uint32_t acc = turn & 1u;
            // The accumulator is free once the drain warps have read its previous tile.
            if (lane == 0 && turn < 8) WTRACE(32 + 3 * turn);
            alive = mbar_wait(smem_u32(&acc_empty[acc]), ((turn >> 1) & 1u) ^ 1u, abort_flag, args.status);
            if (lane == 0 && turn < 8) WTRACE(33 + 3 * turn);
            for (uint32_t kb = 0; kb < kblocks && alive; ++kb) {
                alive = mbar_wait(smem_u32(&split_full[stage]), parity, abort_flag, args.status);
                if (!alive) break;
                if (lane == 0 && turn < 8 && kb + 1 == kblocks) WTRACE(34 + 3 * turn);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const uint32_t a16 = a_low + tiles16 + stage * (Wide::STAGE_BYTES >> 4);
                    const uint32_t b16 = b_low + tiles16 + stage * (Wide::STAGE_BYTES >> 4) + (Wide::A_BYTES >> 4);
                    const uint32_t to = tmem_base + acc * Wide::ACC_COLUMNS;
#pragma unroll
                    for (uint32_t ks = 0; ks < BK / 8; ++ks) {
                        const uint32_t a_at = (A_T ? ks * 1024u : ks * 32u) >> 4;
                        const uint32_t b_at = (B_T ? ks * 32u : ks * 1024u) >> 4;
                        const uint64_t a_hi = desc(a_high, a16 + a_at), a_lo = desc(a_high, a16 + (Wide::A_BYTES >> 5) + a_at);
                        const uint64_t b_hi = desc(b_high, b16 + b_at), b_lo = desc(b_high, b16 + (Wide::B_BYTES >> 5) + b_at);
                        mma_tf32(to, a_hi, b_hi, idesc, (kb | ks) != 0u);
                        mma_tf32(to, a_hi, b_lo, idesc, 1u);
                        mma_tf32(to, a_lo, b_hi, idesc, 1u);
                    }
                    mma_commit(smem_u32(&split_empty[stage]));                     // frees the stage when they finish
                    if (kb + 1 == kblocks) mma_commit(smem_u32(&acc_full[acc]));  // and, at the end, hands the tile to the drain
                }
                if (++stage == STAGES) { stage = 0; parity ^= 1u; }
                __syncwarp();
            }
        }
        } else if (warp == 9) {
        // ---- the TMA warp: the raw k blocks of every tile of this CTA, in order ---------------------
        bool alive = true;
        uint32_t stage = 0, parity = 1;  // the parity a free slot shows
        uint32_t issued = 0;
        for (uint32_t u = blockIdx.x; u < units && alive; u += gridDim.x) {
            const WideUnit w = wide_unit(args, u);
            for (uint32_t kb = 0; kb < w.kblocks && alive; ++kb, ++issued) {
                alive = mbar_wait(smem_u32(&raw_empty[stage]), parity, abort_flag, args.status);
                if (!alive) break;
                if (lane == 0) {
                    const uint32_t bar = smem_u32(&raw_full[stage]);
                    const uint32_t to_a = smem_u32(raw_blocks + stage * Wide::RAW_BYTES), to_b = to_a + Wide::RAW_OPERAND_BYTES;
                    const uint32_t k0 = (kb * w.splits + w.split) * BK;
                    tc::mbar_expect_tx(bar, Wide::RAW_BYTES);
                    uint32_t upper[3] = {0u, 0u, 0u};
                    if (A_T) {  // stored [k, m]: four boxes of 32 m by 32 k
                        upper[args.a_order.row] = k0;
#pragma unroll
                        for (uint32_t p = 0; p < 4; ++p) tc::tma_load(to_a + p * 4096u, &maps.a[w.product], bar, w.m0 + 32u * p, upper);
                    } else {    // stored [m, k]: one box of 32 k by 128 m
                        upper[args.a_order.row] = w.m0;
                        tc::tma_load(to_a, &maps.a[w.product], bar, k0, upper);
                    }
                    upper[0] = upper[1] = upper[2] = 0u;
                    if (B_T) {  // stored [n, k]
                        upper[args.b_order.row] = w.n0;
                        tc::tma_load(to_b, &maps.b[w.product], bar, k0, upper);
                    } else {    // stored [k, n]
                        upper[args.b_order.row] = k0;
#pragma unroll
                        for (uint32_t p = 0; p < 4; ++p) tc::tma_load(to_b + p * 4096u, &maps.b[w.product], bar, w.n0 + 32u * p, upper);
                    }
                }
                if (++stage == STAGES) { stage = 0; parity ^= 1u; }
                __syncwarp();
            }
        }
        // A role gave up: the loads still in flight land (a bounded wait each) before the CTA, and
        // with it their shared-memory destination, goes away.
        if (*abort_flag && lane == 0) {
            for (uint32_t back = 0; back < static_cast<uint32_t>(STAGES) && back < issued; ++back) {
                const uint32_t i = issued - 1 - back;
                for (uint32_t spin = 0; spin < WAIT_LIMIT; ++spin)
                    if (mbar_try_wait(smem_u32(&raw_full[i % STAGES]), (i / STAGES) & 1u)) break;
            }
        }
        }
    } else {
        // ---- the drain warps: tensor memory -> a shared-memory slab -> C ---------------------------
        // A warp reads its lane quarter (the tensor-memory lanes a warp may read are 32 (warp % 4)
        // ..) 32 columns at a time: the sums (with the bias) go row
        // by row into a slab of 32 rows x 128 bytes in the 128-byte swizzle (the 16-byte chunks of
        // a row xor-ed with the row), which one TMA store then writes (what lies outside C is not
        // written), or, where C cannot be a TMA target, the warp itself as 128-byte row segments.
        const uint32_t quarter = warp & 3u;
        char* const my_slabs = drain_slabs + (warp - Wide::DRAIN_FIRST_WARP) * 2 * Wide::SLAB_BYTES;
        bool alive = true;
        uint32_t turn = 0, filled = 0;
        for (uint32_t u = blockIdx.x; u < units && alive; u += gridDim.x, ++turn) {
            const WideUnit w = wide_unit(args, u);
            if (w.kblocks == 0) continue;
            const uint32_t acc = turn & 1u;
            // The tile's 128 bias values, four per lane, fetched before the wait for the tile: a
            // load issued inside the drain would queue behind everything else the SM has in flight.
            const float* __restrict__ bias_row = w.bias;
            const uint32_t pm = w.m, pn = w.n, pldc = w.ldc;
            float4 bias4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (bias_row) {
                const uint32_t at = w.n0 + 4 * lane;
                if (at + 4 <= pn && reinterpret_cast<uintptr_t>(bias_row) % 16 == 0) {
                    bias4 = __ldg(reinterpret_cast<const float4*>(bias_row + at));
                } else {
                    if (at < pn) bias4.x = __ldg(bias_row + at);
                    if (at + 1 < pn) bias4.y = __ldg(bias_row + at + 1);
                    if (at + 2 < pn) bias4.z = __ldg(bias_row + at + 2);
                    if (at + 3 < pn) bias4.w = __ldg(bias_row + at + 3);
                }
            }
            if (warp == Wide::DRAIN_FIRST_WARP && lane == 0 && turn < 8) WTRACE(4 * turn);
            alive = warp_mbar_wait(smem_u32(&acc_full[acc]), (turn >> 1) & 1u, abort_flag, args.status);
            if (!alive) break;
            if (warp == Wide::DRAIN_FIRST_WARP && lane == 0 && turn < 8) WTRACE(4 * turn + 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* __restrict__ out = w.c + static_cast<uint64_t>(w.split) * pm * pldc;
            const uint32_t first_row = w.m0 + quarter * 32u;
            uint32_t upper[3] = {0u, 0u, 0u};
            upper[w.c_order.row] = first_row;
            upper[w.c_order.outer] = w.split;
#pragma unroll 1
            for (uint32_t col = 0; col < 128; col += 32, ++filled) {
                char* const slab = my_slabs + (filled & 1u) * Wide::SLAB_BYTES;
                // The store that last read this slab (two chunks ago) has finished reading it.
                if (args.c_tma) {
                    if (lane == 0) tc::tma_store_wait_read<1>();
                    __syncwarp();
                }
                uint32_t r[32];
                tmem_load32(tmem_base + ((quarter * 32u) << 16) + acc * Wide::ACC_COLUMNS + col, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (col == 96) {
                    // The whole accumulator is in registers or stored: the MMA warp may write it again.
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&acc_empty[acc]));
                    if (warp == Wide::DRAIN_FIRST_WARP && lane == 0 && turn < 8) WTRACE(4 * turn + 2);
                }
                const uint32_t gn0 = w.n0 + col;
                if (gn0 >= pn) continue;  // the same for the whole warp
#pragma unroll
                for (uint32_t j = 0; j < 32; j += 4) {
                    // One addition an element: the bias (columns col + j .. + 3 are held by lane
                    // (col + j) / 4, zeros past n), or the `x + 0` that turns a -0 sum of zero
                    // products into the +0 a skipped term gives (as a bias of +0 does).
                    float4 add = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (bias_row) {
                        const uint32_t holder = (col + j) >> 2;
                        add.x = __shfl_sync(0xffffffffu, bias4.x, holder);
                        add.y = __shfl_sync(0xffffffffu, bias4.y, holder);
                        add.z = __shfl_sync(0xffffffffu, bias4.z, holder);
                        add.w = __shfl_sync(0xffffffffu, bias4.w, holder);
                    }
                    float4 v;
                    v.x = __uint_as_float(r[j]) + add.x;
                    v.y = __uint_as_float(r[j + 1]) + add.y;
                    v.z = __uint_as_float(r[j + 2]) + add.z;
                    v.w = __uint_as_float(r[j + 3]) + add.w;
                    *reinterpret_cast<float4*>(slab + tc::swizzled_chunk(lane, j >> 2)) = v;
                }
                if (args.c_tma) {
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0 && first_row < pm) tc::tma_store(&maps.c[w.product], smem_u32(slab), gn0, upper);
                    continue;
                }
                __syncwarp();
                const uint32_t c4 = (lane & 7u) * 4, gn = gn0 + c4;
#pragma unroll
                for (uint32_t pass = 0; pass < 8; ++pass) {
                    const uint32_t row = pass * 4 + (lane >> 3), gm = first_row + row;
                    if (gm >= pm || gn >= pn) continue;
                    const float4 v = *reinterpret_cast<const float4*>(slab + tc::swizzled_chunk(row, lane & 7u));
                    float* dst = out + static_cast<uint64_t>(gm) * pldc + gn;
                    // Inside the pitch a whole float4 may be written: what lies past n is padding.
                    if (args.c_vec && (gn + 4 <= pn || (args.c_padded && gn + 4 <= pldc))) {
                        *reinterpret_cast<float4*>(dst) = v;
                    } else {
                        if (gn < pn) dst[0] = v.x;
                        if (gn + 1 < pn) dst[1] = v.y;
                        if (gn + 2 < pn) dst[2] = v.z;
                        if (gn + 3 < pn) dst[3] = v.w;
                    }
                }
                __syncwarp();
            }
            if (warp == Wide::DRAIN_FIRST_WARP && lane == 0 && turn < 8) WTRACE(4 * turn + 3);
        }
        // The slabs must outlive the stores that read them.
        if (args.c_tma && lane == 0) tc::tma_store_wait_read<0>();
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 8) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Wide::TMEM_COLUMNS) : "memory");
    }
}

__global__ void splitk_reduce_kernel(const float* __restrict__ ws, float* __restrict__ c, uint64_t count, uint32_t splits,
                                     const float* __restrict__ bias, uint32_t n) {
    uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        float acc = ws[i];
        for (uint32_t s = 1; s < splits; ++s) acc += ws[static_cast<uint64_t>(s) * count + i];
        c[i] = bias ? acc + bias[i % n] : acc;
    }
}

template <int BM, int BN, bool A_T, bool B_T> void launch(cudaStream_t s, const TcArgs& args, dim3 grid) {
    auto kernel = matmul_tc_kernel<BM, BN, A_T, B_T>;
    // The attribute is per device: set it when the device changes (a second thread that sees a
    // stale value only sets it once more).
    static std::atomic<int> configured_device{-1};
    int device = 0;
    check(cudaGetDevice(&device), "cudaGetDevice");
    if (device != configured_device.load(std::memory_order_relaxed)) {
        check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Config<BM, BN>::TOTAL)), "matmul_tc shared memory");
        configured_device.store(device, std::memory_order_relaxed);
    }
    kernel<<<grid, THREADS, Config<BM, BN>::TOTAL, s>>>(args);
    check_launch("matmul_tc");
}

template <int BM, int BN> void launch_forms(cudaStream_t s, const TcArgs& args, dim3 grid, bool a_t, bool b_t) {
    if (a_t && b_t) launch<BM, BN, true, true>(s, args, grid);
    else if (a_t) launch<BM, BN, true, false>(s, args, grid);
    else if (b_t) launch<BM, BN, false, true>(s, args, grid);
    else launch<BM, BN, false, false>(s, args, grid);
}

template <bool A_T, bool B_T> void launch_wide(cudaStream_t s, const TcArgs& args, const WideMaps& maps, uint32_t units) {
    auto kernel = matmul_tc_wide_kernel<A_T, B_T>;
    static std::atomic<int> configured_device{-1};
    static std::atomic<int> sm_count{0};
    int device = 0;
    check(cudaGetDevice(&device), "cudaGetDevice");
    if (device != configured_device.load(std::memory_order_relaxed)) {
        check(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(Wide::TOTAL)), "matmul_tc_wide shared memory");
        int sms = 0;
        check(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device), "cudaDeviceGetAttribute");
        sm_count.store(sms, std::memory_order_relaxed);
        configured_device.store(device, std::memory_order_relaxed);
    }
    // One CTA per SM, each walking its share of the units.
    uint32_t sms = static_cast<uint32_t>(sm_count.load(std::memory_order_relaxed));
#ifdef MSX_TC_TRACE
    if (const char* forced = std::getenv("MSX_TC_WIDE_GRID")) sms = static_cast<uint32_t>(std::atoi(forced));
#endif
    kernel<<<units < sms ? units : sms, Wide::THREADS, Wide::TOTAL, s>>>(args, maps);
    check_launch("matmul_tc_wide");
}

void launch_tile(cudaStream_t s, const TcArgs& args, dim3 grid, uint32_t bm, uint32_t bn, bool a_t, bool b_t, const WideMaps* maps = nullptr) {
    if (bm == 128) {
        (void)grid;
        const uint32_t units = args.units;
        if (a_t && b_t) launch_wide<true, true>(s, args, *maps, units);
        else if (a_t) launch_wide<true, false>(s, args, *maps, units);
        else if (b_t) launch_wide<false, true>(s, args, *maps, units);
        else launch_wide<false, false>(s, args, *maps, units);
    }
    else if (bn == 32) launch_forms<64, 32>(s, args, grid, a_t, b_t);
    else if (bn == 64) launch_forms<64, 64>(s, args, grid, a_t, b_t);
    else launch_forms<64, 128>(s, args, grid, a_t, b_t);
}

#ifdef MSX_TC_TRACE
}  // namespace
extern "C" void msx_tc_trace_read(long long* out) { cudaMemcpyFromSymbol(out, g_trace, sizeof(long long) * 256); }
namespace {
#endif

bool aligned16(const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; }

}  // namespace

// Tile width and k split by a cost model in SM cycles, fitted to measured phase times of this
// kernel. A CTA costs a fixed latency (set-up, first loads, drain) plus a latency-bound time per
// k block; two CTAs share an SM and overlap, so an SM's CTAs run in pairs; shared-memory
// bandwidth bounds the k blocks an SM gets through whatever the overlap; a split k adds the
// reduce launch. Narrow tiles win when the problem is small (more SMs share the latency-bound
// work) or k is long (their loads run further ahead), wide ones when the product is large (less
// operand re-reading).
MatmulTcPlan matmul_tc_plan(uint64_t m, uint64_t n, uint64_t k, uint64_t problems, uint64_t group, bool wide_ok) {
    // Candidates: 64-row tiles of width 32, 64, 128 (two CTAs per SM) and the 128 x 128 tile.
    static const uint32_t rows[4] = {64, 64, 64, 128}, widths[4] = {32, 64, 128, 128};
    static const double per_block[4] = {MSX_TC_KB32, MSX_TC_KB64, MSX_TC_KB128, MSX_TC_KB_WIDE};
    static const double latency[4] = {MSX_TC_LATENCY32, MSX_TC_LATENCY64, MSX_TC_LATENCY128, MSX_TC_KB_WIDE};
    const uint64_t kblocks = (k + BK - 1) / BK;
    MatmulTcPlan best = {};
    double best_cost = 0.0;
    for (int w = 0; w < 4; ++w) {
#ifdef MSX_TC_TRACE
        if (const char* forced = std::getenv("MSX_TC_FORCE_BN"))
            if (static_cast<uint32_t>(std::atoi(forced)) != widths[w]) continue;
        if (const char* forced = std::getenv("MSX_TC_FORCE_BM"))
            if (static_cast<uint32_t>(std::atoi(forced)) != rows[w]) continue;
#endif
        if (rows[w] == 128 && (problems > 1 || kblocks == 0 || !wide_ok)) continue;  // batched and empty products stay on the narrow tiles, and operands TMA cannot address
        const uint64_t m_tiles = (m + rows[w] - 1) / rows[w], n_tiles = (n + widths[w] - 1) / widths[w];
        const uint64_t tiles = m_tiles * n_tiles * problems * group;
        const uint64_t most = problems > 1 ? 1 : (kblocks / 2 > 0 ? kblocks / 2 : 1);
        for (uint64_t splits = 1; splits <= most && splits <= 64; ++splits) {
            const uint64_t per = (kblocks + splits - 1) / splits;
            const uint64_t used = kblocks == 0 ? 1 : (kblocks + per - 1) / per;
            if (used != splits) continue;  // the same partition as a smaller count
            const uint64_t per_sm = (tiles * splits + 147) / 148;
            const uint64_t together = rows[w] == 128 ? 1 : 2;  // CTAs that share an SM and overlap
            const double fixed = MSX_TC_FIXED;
            const double paired = static_cast<double>((per_sm + together - 1) / together) * (fixed + static_cast<double>(per) * latency[w]);
            const double streamed = static_cast<double>(per_sm * per) * per_block[w];
            // Every tile reads its rows of A and columns of B over k; what the SMs can pull
            // through the L2 in a cycle bounds a product with many tiles.
            const double bytes = 4.0 * static_cast<double>(problems * group) *
                                 (static_cast<double>(m * k * n_tiles) + static_cast<double>(n * k * m_tiles) +
                                  static_cast<double>(m * n * (splits > 1 ? splits : 1)));
            const double traffic = bytes / MSX_TC_BYTES_PER_CYCLE;
            double cost = paired > streamed ? paired : streamed;
            // The persistent kernel pays its set-up and its last drain once; a tile's drain runs
            // under the next tile's k loop.
            if (rows[w] == 128) {
                const double k_loop = static_cast<double>(per) * MSX_TC_KB_WIDE;
                cost = MSX_TC_FIXED_WIDE + static_cast<double>(per_sm) * ((k_loop > MSX_TC_DRAIN_WIDE ? k_loop : MSX_TC_DRAIN_WIDE) + MSX_TC_TILE_WIDE);
            }
            if (traffic > cost) cost = traffic;
            if (splits > 1) cost += MSX_TC_REDUCE_FIXED + static_cast<double>(m * n * (splits + 1)) * 4.0 / MSX_TC_REDUCE_BYTES_PER_CYCLE;
            if (best.bn == 0 || cost < best_cost) {
                best_cost = cost;
                best.bm = rows[w];
                best.bn = widths[w];
                best.splits = static_cast<uint32_t>(splits);
                best.kblocks_per_split = static_cast<uint32_t>(per == 0 ? 1 : per);
            }
        }
    }
    best.workspace_floats = best.splits > 1 ? best.splits * m * n : 0;
    return best;
}

void matmul_tc_group(cudaStream_t s, const MatmulOperands* products, uint32_t count, bool a_t, bool b_t, uint64_t m, uint64_t n,
                     uint64_t k, uint32_t* status, bool leave_partials, MatmulPitches pitches) {
    if (m == 0 || n == 0 || count == 0) return;
    if (count > MAX_GROUP) throw std::invalid_argument("matmul_tc_group: more products than one launch carries");
    // The 128 x 128 tile loads its operands by TMA: bases on 16 bytes, rows a multiple of 16 bytes apart.
    bool wide_ok = (pitches.a ? pitches.a : (a_t ? m : k)) % 4 == 0 && (pitches.b ? pitches.b : (b_t ? k : n)) % 4 == 0;
    for (uint32_t g = 0; g < count; ++g) wide_ok = wide_ok && aligned16(products[g].a) && aligned16(products[g].b);
    MatmulTcPlan p = matmul_tc_plan(m, n, k, 1, count, wide_ok);
    TcArgs args = {};
    args.m = static_cast<uint32_t>(m);
    args.n = static_cast<uint32_t>(n);
    args.k = static_cast<uint32_t>(k);
    args.lda = pitches.a ? pitches.a : static_cast<uint32_t>(a_t ? m : k);
    args.ldb = pitches.b ? pitches.b : static_cast<uint32_t>(b_t ? k : n);
    // Partial tiles of a split k are dense; the pitch of C applies to the CTAs that write C itself.
    args.ldc = (pitches.c && p.splits == 1) ? pitches.c : static_cast<uint32_t>(n);
    if (pitches.c && p.splits > 1) throw std::invalid_argument("matmul_tc_group: a pitched result with a split k");
    args.splits = p.splits;
    args.products = count;
    args.kblocks_per_split = p.kblocks_per_split;
    // A float4 read starts at a multiple of 4 elements within a row, so rows must keep that phase.
    args.a_vec = args.lda % 4 == 0;
    args.b_vec = args.ldb % 4 == 0;
    args.c_vec = args.ldc % 4 == 0;
    args.c_padded = pitches.c != 0 && p.splits == 1;
    for (uint32_t g = 0; g < count; ++g) {
        args.c_vec = args.c_vec && aligned16(p.splits > 1 ? products[g].workspace : products[g].c);
        args.a[g] = products[g].a;
        args.b[g] = products[g].b;
        args.c[g] = p.splits > 1 ? products[g].workspace : products[g].c;
        args.bias[g] = p.splits > 1 ? nullptr : products[g].bias;
        args.a_vec = args.a_vec && aligned16(products[g].a);
        args.b_vec = args.b_vec && aligned16(products[g].b);
    }
    args.status = status;
    dim3 grid(static_cast<uint32_t>((n + p.bn - 1) / p.bn), static_cast<uint32_t>((m + p.bm - 1) / p.bm), p.splits * count);
    args.units = grid.x * grid.y * grid.z;
    WideMaps maps = {};
    if (p.bm == 128) {
        // C through TMA stores when its rows can be addressed that way: the result as it is
        // stored, the split-k workspace as `splits` dense [m, n] matrices.
        for (uint32_t g = 0; g < count; ++g) {
            const HalfMatrix a_stored = {args.a[g], args.lda, 0, 0, false}, b_stored = {args.b[g], args.ldb, 0, 0, false};
            // Rows of 32 floats: 128 of them for an operand stored with k along its rows, 32 for
            // one stored with k down its columns (its tile is four such boxes side by side).
            maps.a[g] = a_t ? tc::encode(a_stored, m, k, 1, 1, 32, &args.a_order, "A", true) : tc::encode(a_stored, k, m, 1, 1, 128, &args.a_order, "A", true);
            maps.b[g] = b_t ? tc::encode(b_stored, k, n, 1, 1, 128, &args.b_order, "B", true) : tc::encode(b_stored, n, k, 1, 1, 32, &args.b_order, "B", true);
        }
        const bool partial = p.splits > 1;
        bool addressable = true;
        for (uint32_t g = 0; g < count; ++g) {
            const HalfMatrix target = {args.c[g], args.ldc, partial ? m * n : 0, 0, false};
            addressable = addressable && tc::tma_addressable(target, true);
        }
        if (addressable) {
            for (uint32_t g = 0; g < count; ++g) {
                const HalfMatrix target = {args.c[g], args.ldc, partial ? m * n : 0, 0, false};
                maps.c[g] = tc::encode(target, n, m, 1, partial ? p.splits : 1, 32, &args.c_order, "C", true);
            }
            args.c_tma = 1;
        }
    }
    launch_tile(s, args, grid, p.bm, p.bn, a_t, b_t, &maps);
    if (p.splits > 1 && !leave_partials) {
        uint64_t total = m * n;
        uint64_t blocks = (total + 255) / 256;
        for (uint32_t g = 0; g < count; ++g) {
            splitk_reduce_kernel<<<static_cast<uint32_t>(blocks > 148 * 8 ? 148 * 8 : blocks), 256, 0, s>>>(
                products[g].workspace, products[g].c, total, p.splits, products[g].bias, static_cast<uint32_t>(n));
            check_launch("splitk_reduce");
        }
    }
}

void matmul_tc(cudaStream_t s, const float* a, bool a_t, const float* b, bool b_t, float* c, uint64_t m, uint64_t n,
               uint64_t k, float* workspace, uint32_t* status, const float* bias, bool leave_partials) {
    MatmulOperands one = {a, b, c, bias, workspace};
    matmul_tc_group(s, &one, 1, a_t, b_t, m, n, k, status, leave_partials);
}

// One job of matmul_tc_jobs: k split so that a unit (a 128 x 128 tile of one split, or a CTA of
// the 64 x 64 tiles where TMA cannot address the job) gets about MSX_TC_JOB_KBLOCKS k blocks (the
// jobs of a launch fill the device together, so a job does not have to on its own).
MatmulTcPlan matmul_tc_job_plan(uint64_t m, uint64_t n, uint64_t k) {
    const uint64_t kblocks = (k + BK - 1) / BK;
    uint64_t splits = kblocks / MSX_TC_JOB_KBLOCKS;
    if (splits < 1) splits = 1;
    if (splits > 32) splits = 32;
    MatmulTcPlan p = {};
    p.bm = 64;
    p.bn = 64;
    p.kblocks_per_split = static_cast<uint32_t>((kblocks + splits - 1) / splits);
    p.splits = static_cast<uint32_t>(kblocks == 0 ? 1 : (kblocks + p.kblocks_per_split - 1) / p.kblocks_per_split);
    p.workspace_floats = p.splits > 1 ? p.splits * m * n : 0;
    return p;
}

namespace {
// The jobs of one launch on the persistent 128 x 128 tile, when TMA can address every operand and
// every result (or split-k workspace); false when it cannot, and the 64 x 64 tiles take them.
bool wide_jobs(cudaStream_t s, const MatmulJob* jobs, uint32_t count, bool a_t, bool b_t, uint32_t* status) {
    TcArgs args = {};
    WideMaps maps = {};
    args.status = status;
    args.c_tma = 1;
    args.c_vec = 1;
    for (uint32_t j = 0; j < count; ++j) {
        const MatmulJob& job = jobs[j];
        const MatmulTcPlan p = matmul_tc_job_plan(job.m, job.n, job.k);
        const bool partial = p.splits > 1;
        TcArgs::Job& to = args.jobs[args.job_count++];
        to.a = job.a;
        to.b = job.b;
        to.c = partial ? job.workspace : job.c;
        to.m = static_cast<uint32_t>(job.m);
        to.n = static_cast<uint32_t>(job.n);
        to.k = static_cast<uint32_t>(job.k);
        to.lda = static_cast<uint32_t>(a_t ? job.m : job.k);
        to.ldb = static_cast<uint32_t>(b_t ? job.k : job.n);
        to.ldc = to.n;
        to.splits = p.splits;
        to.first_block = args.units;
        args.units += static_cast<uint32_t>(((job.m + 127) / 128) * ((job.n + 127) / 128)) * p.splits;
        const HalfMatrix a_stored = {to.a, to.lda, 0, 0, false}, b_stored = {to.b, to.ldb, 0, 0, false};
        const HalfMatrix target = {to.c, to.ldc, partial ? job.m * job.n : 0, 0, false};
        if (job.k == 0 || !tc::tma_addressable(a_stored, true) || !tc::tma_addressable(b_stored, true) || !tc::tma_addressable(target, true)) return false;
        maps.a[j] = a_t ? tc::encode(a_stored, job.m, job.k, 1, 1, 32, &args.a_order, "A", true) : tc::encode(a_stored, job.k, job.m, 1, 1, 128, &args.a_order, "A", true);
        maps.b[j] = b_t ? tc::encode(b_stored, job.k, job.n, 1, 1, 128, &args.b_order, "B", true) : tc::encode(b_stored, job.n, job.k, 1, 1, 32, &args.b_order, "B", true);
        maps.c[j] = tc::encode(target, job.n, job.m, 1, partial ? p.splits : 1, 32, &to.c_order, "C", true);
    }
    launch_tile(s, args, dim3(args.units), 128, 128, a_t, b_t, &maps);
    return true;
}
}  // namespace

void matmul_tc_jobs(cudaStream_t s, const MatmulJob* jobs, uint32_t count, bool a_t, bool b_t, uint32_t* status) {
    if (count == 0) return;
    if (count > MAX_JOBS) throw std::invalid_argument("matmul_tc_jobs: more jobs than one launch carries");
    for (uint32_t j = 0; j < count; ++j)
        if (jobs[j].m == 0 || jobs[j].n == 0) throw std::invalid_argument("matmul_tc_jobs: an empty product");
    if (wide_jobs(s, jobs, count, a_t, b_t, status)) return;
    TcArgs args = {};
    args.splits = 1;
    args.a_vec = args.b_vec = args.c_vec = 1;
    args.status = status;
    uint32_t blocks = 0;
    for (uint32_t j = 0; j < count; ++j) {
        const MatmulJob& job = jobs[j];
        if (job.m == 0 || job.n == 0) throw std::invalid_argument("matmul_tc_jobs: an empty product");
        const MatmulTcPlan p = matmul_tc_job_plan(job.m, job.n, job.k);
        TcArgs::Job& to = args.jobs[args.job_count++];
        to.a = job.a;
        to.b = job.b;
        to.c = p.splits > 1 ? job.workspace : job.c;
        to.m = static_cast<uint32_t>(job.m);
        to.n = static_cast<uint32_t>(job.n);
        to.k = static_cast<uint32_t>(job.k);
        to.lda = static_cast<uint32_t>(a_t ? job.m : job.k);
        to.ldb = static_cast<uint32_t>(b_t ? job.k : job.n);
        to.ldc = to.n;
        to.splits = p.splits;
        to.first_block = blocks;
        blocks += static_cast<uint32_t>(((job.m + 63) / 64) * ((job.n + 63) / 64)) * p.splits;
        args.a_vec = args.a_vec && aligned16(job.a) && to.lda % 4 == 0;
        args.b_vec = args.b_vec && aligned16(job.b) && to.ldb % 4 == 0;
        args.c_vec = args.c_vec && aligned16(to.c) && to.ldc % 4 == 0;
    }
    launch_tile(s, args, dim3(blocks), 64, 64, a_t, b_t);
}

void matmul_tc_batched(cudaStream_t s, const BatchedOperand& a, const BatchedOperand& b, const BatchedOperand& c, uint64_t m,
                       uint64_t n, uint64_t k, uint32_t outer, uint32_t inner, uint32_t* status) {
    if (m == 0 || n == 0 || outer == 0 || inner == 0) return;
    TcArgs args = {};
    args.a[0] = a.base;
    args.b[0] = b.base;
    args.c[0] = const_cast<float*>(c.base);
    args.splits = 1;
    args.m = static_cast<uint32_t>(m);
    args.n = static_cast<uint32_t>(n);
    args.k = static_cast<uint32_t>(k);
    args.lda = a.pitch;
    args.ldb = b.pitch;
    args.ldc = c.pitch;
    args.kblocks_per_split = static_cast<uint32_t>((k + BK - 1) / BK) + 1;
    auto vec = [](const BatchedOperand& o) {
        return aligned16(o.base) && o.pitch % 4 == 0 && o.stride_outer % 4 == 0 && o.stride_inner % 4 == 0;
    };
    args.a_vec = vec(a);
    args.b_vec = vec(b);
    args.c_vec = vec(c);
    args.batch_inner = inner;
    args.a_outer = a.stride_outer; args.a_inner = a.stride_inner;
    args.b_outer = b.stride_outer; args.b_inner = b.stride_inner;
    args.c_outer = c.stride_outer; args.c_inner = c.stride_inner;
    args.status = status;
    const MatmulTcPlan p = matmul_tc_plan(m, n, k, static_cast<uint64_t>(outer) * inner);
    dim3 grid(static_cast<uint32_t>((n + p.bn - 1) / p.bn), static_cast<uint32_t>((m + p.bm - 1) / p.bm), outer * inner);
    launch_tile(s, args, grid, p.bm, p.bn, a.transposed, b.transposed);
}

}  // namespace k
}  // namespace msx
