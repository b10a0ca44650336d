// Whole-tensor sums (reduce_sum, mean, mse) and column sums (sum_rows).
//
// The reference sums a whole tensor sequentially in f64 and rounds once to f32
// (crates/modelspec-runtime/src/cpu/interpreter.rs:903-917, :1913-1921). Here the f64 partial
// sums are combined as a tree; the f64 result differs from the sequential one by a few units of
// 2^-53 relative, so the rounded f32 is the same except across a rounding boundary (tolerance
// class, deterministic). Column sums (the bias gradients, interpreter.rs:943-958) are f32 in two
// stages: rows are split into chunks summed in ascending order, then the chunk sums are added in
// ascending order; the split changes the rounding sequence (tolerance class, deterministic).
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

constexpr int kThreads = 256;
constexpr uint32_t kMaxBlocks = 592;  // 4 per SM

enum class Whole : int { Sum, SquaredDifference };

template <Whole KIND>
__global__ void whole_stage1(const float* __restrict__ a, const float* __restrict__ b, uint64_t n,
                             double* __restrict__ partial) {
    __shared__ double shared[33];
    double acc = 0.0;
    uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t j = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride) {
        if (KIND == Whole::Sum) {
            acc += static_cast<double>(a[j]);
        } else {
            double d = static_cast<double>(a[j]) - static_cast<double>(b[j]);
            acc = fma(d, d, acc);
        }
    }
    double total = block_sum(acc, shared);
    if (threadIdx.x == 0) partial[blockIdx.x] = total;
}

__global__ void whole_stage2(const double* __restrict__ partial, uint32_t blocks, double divisor,
                             float* __restrict__ out) {
    __shared__ double shared[33];
    double acc = 0.0;
    for (uint32_t j = threadIdx.x; j < blocks; j += blockDim.x) acc += partial[j];
    double total = block_sum(acc, shared);
    if (threadIdx.x == 0) out[0] = static_cast<float>(total / divisor);
}

uint32_t whole_blocks(uint64_t n) {
    uint64_t b = (n + kThreads * 4 - 1) / (kThreads * 4);
    return static_cast<uint32_t>(b < 1 ? 1 : (b > kMaxBlocks ? kMaxBlocks : b));
}

// Block (32, 8): lane = column of a 32-column tile, each of the 8 warps takes every 8th row of
// the block's row chunk.
// `counters`, when not null, holds one zeroed word per column block: the last chunk block of a
// column block to finish adds the chunk sums in ascending chunk order (what sum_rows_stage2 does
// as a second launch) and writes `out`.
template <class T>
__global__ void sum_rows_stage1(const T* __restrict__ g, uint32_t rows, uint32_t h, uint32_t ld, uint32_t rows_per_chunk,
                                float* __restrict__ partial, uint32_t* __restrict__ counters, float* __restrict__ out) {
    __shared__ float shared[8][32];
    __shared__ bool is_last;
    uint32_t c = blockIdx.x * 32 + threadIdx.x;
    uint32_t r0 = blockIdx.y * rows_per_chunk;
    uint32_t r1 = min(rows, r0 + rows_per_chunk);
    float acc = 0.0f;
    if (c < h) {
        // Eight loads in flight per thread; the additions stay in row order.
        uint32_t r = r0 + threadIdx.y;
        for (; r + 56 < r1; r += 64) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = load1(g + static_cast<uint64_t>(r + 8 * j) * ld + c);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc += v[j];
        }
        for (; r < r1; r += 8) acc += load1(g + static_cast<uint64_t>(r) * ld + c);
    }
    shared[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < h) {
        float total = shared[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < 8; ++w) total += shared[w][threadIdx.x];
        partial[static_cast<uint64_t>(blockIdx.y) * h + c] = total;
    }
    if (counters == nullptr) return;
    if (!last_block_arrives(counters + blockIdx.x, gridDim.y, &is_last)) return;
    if (threadIdx.y == 0 && c < h) {
        float total = __ldcg(partial + c);
        for (uint32_t k = 1; k < gridDim.y; ++k) total += __ldcg(partial + static_cast<uint64_t>(k) * h + c);
        out[c] = total;
    }
}

// The same with four columns per lane (16-byte loads) for matrices whose rows start on 16-byte
// boundaries: a block covers 128 columns. Only the chunk sums are written (the second stage is
// the step's finalize launch or sum_rows_stage2).
template <class T>
__global__ void sum_rows_stage1_wide(const T* __restrict__ g, uint32_t rows, uint32_t h, uint32_t ld, uint32_t rows_per_chunk,
                                     float* __restrict__ partial) {
    __shared__ float4 shared[8][32];
    const uint32_t c = (blockIdx.x * 32 + threadIdx.x) * 4;
    const uint32_t r0 = blockIdx.y * rows_per_chunk, r1 = min(rows, r0 + rows_per_chunk);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < h) {  // the pitch covers the whole float4; columns past h hold padding and are not written below
        uint32_t r = r0 + threadIdx.y;
        for (; r + 24 < r1; r += 32) {
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = load4(g + static_cast<uint64_t>(r + 8 * j) * ld + c);
#pragma unroll
            for (int j = 0; j < 4; ++j) { acc.x += v[j].x; acc.y += v[j].y; acc.z += v[j].z; acc.w += v[j].w; }
        }
        for (; r < r1; r += 8) {
            const float4 v = load4(g + static_cast<uint64_t>(r) * ld + c);
            acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
    }
    shared[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < h) {
        float4 total = shared[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < 8; ++w) {
            const float4 v = shared[w][threadIdx.x];
            total.x += v.x; total.y += v.y; total.z += v.z; total.w += v.w;
        }
        float* to = partial + static_cast<uint64_t>(blockIdx.y) * h + c;
        to[0] = total.x;
        if (c + 1 < h) to[1] = total.y;
        if (c + 2 < h) to[2] = total.z;
        if (c + 3 < h) to[3] = total.w;
    }
}

// The job whose block range holds this block: the last one whose first block is not past it. Thread
// t looks at job t, so the whole table costs the block one round trip to memory, not one per job.
template <class Job>
__device__ __forceinline__ uint32_t job_of_block(const Job* __restrict__ jobs, uint32_t count, uint32_t* which) {
    const uint32_t threads = blockDim.x * blockDim.y;
    for (uint32_t t = threadIdx.y * blockDim.x + threadIdx.x; t < count; t += threads) {
        const bool begun = jobs[t].first_block <= blockIdx.x;
        const bool last = t + 1 == count || jobs[t + 1].first_block > blockIdx.x;
        if (begun && last) *which = t;
    }
    __syncthreads();
    return *which;
}

// The first stage of many column sums in one launch: block b works on the job whose block range
// holds it, on one 32-column block and one chunk of rows, exactly as sum_rows_stage1 does.
__global__ void sum_rows_batched_kernel(const RowSumJob* __restrict__ jobs, uint32_t count) {
    __shared__ float shared[8][32];
    __shared__ uint32_t which;
    const RowSumJob job = jobs[job_of_block(jobs, count, &which)];
    const uint32_t local = blockIdx.x - job.first_block, column_blocks = (job.width + 31) / 32;
    const uint32_t c = (local % column_blocks) * 32 + threadIdx.x, chunk = local / column_blocks;
    const uint32_t r0 = chunk * job.rows_per_chunk, r1 = min(job.rows, r0 + job.rows_per_chunk);
    float acc = 0.0f;
    // The same loop for either element type of the job's matrix (one type per block).
    auto column_sum = [&](auto* g) {
        uint32_t r = r0 + threadIdx.y;
        for (; r + 56 < r1; r += 64) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = load1(g + static_cast<uint64_t>(r + 8 * j) * job.ld + c);
#pragma unroll
            for (int j = 0; j < 8; ++j) acc += v[j];
        }
        for (; r < r1; r += 8) acc += load1(g + static_cast<uint64_t>(r) * job.ld + c);
    };
    if (c < job.width) {
        if (job.half) column_sum(static_cast<const bf16*>(job.g));
        else column_sum(static_cast<const float*>(job.g));
    }
    shared[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < job.width) {
        float total = shared[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < 8; ++w) total += shared[w][threadIdx.x];
        job.partial[static_cast<uint64_t>(chunk) * job.width + c] = total;
    }
}

__global__ void sum_rows_stage2(const float* __restrict__ partial, uint32_t chunks, uint32_t h,
                                float* __restrict__ out) {
    uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= h) return;
    float total = partial[c];
    for (uint32_t k = 1; k < chunks; ++k) total += partial[static_cast<uint64_t>(k) * h + c];
    out[c] = total;
}

__global__ void finalize_sums_kernel(const SumJob* __restrict__ jobs, uint32_t count) {
    __shared__ float shared[8][32];
    __shared__ uint32_t which;
    const SumJob job = jobs[job_of_block(jobs, count, &which)];
    const uint32_t block = blockIdx.x - job.first_block;
    if (job.chunks <= 64) {
        // Plain ascending order, one thread per column (what the two-launch forms of sum_rows and
        // the split-K reduction do).
        const uint32_t c = block * 256 + threadIdx.y * 32 + threadIdx.x;
        if (c >= job.width) return;
        float acc = 0.0f;
#pragma unroll 8
        for (uint32_t k = 0; k < job.chunks; ++k) acc += job.partial[static_cast<uint64_t>(k) * job.width + c];
        job.out[c] = acc;
        return;
    }
    const uint32_t c = block * 32 + threadIdx.x;
    float acc = 0.0f;
    if (c < job.width) {
#pragma unroll 4
        for (uint32_t k = threadIdx.y; k < job.chunks; k += 8) acc += job.partial[static_cast<uint64_t>(k) * job.width + c];
    }
    shared[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < job.width) {
        float total = shared[0][threadIdx.x];
#pragma unroll
        for (int w = 1; w < 8; ++w) total += shared[w][threadIdx.x];
        job.out[c] = total;
    }
}

}  // namespace

RowSumJob row_sum_job(In g, float* partial, uint64_t rows, uint64_t h, uint64_t ld, uint32_t first_block) {
    RowSumJob job = {};
    job.g = g.p;
    job.half = g.half ? 1u : 0u;
    job.partial = partial;
    job.rows = static_cast<uint32_t>(rows);
    job.width = static_cast<uint32_t>(h);
    job.ld = static_cast<uint32_t>(ld ? ld : h);
    const uint32_t chunks = sum_rows_chunks(rows);
    job.rows_per_chunk = static_cast<uint32_t>((rows + chunks - 1) / chunks);
    job.first_block = first_block;
    return job;
}
uint32_t row_sum_job_blocks(uint64_t rows, uint64_t h) { return static_cast<uint32_t>((h + 31) / 32) * sum_rows_chunks(rows); }

void sum_rows_batched(cudaStream_t s, const RowSumJob* d_jobs, uint32_t jobs, uint32_t blocks) {
    if (jobs == 0 || blocks == 0) return;
    sum_rows_batched_kernel<<<blocks, dim3(32, 8), 0, s>>>(d_jobs, jobs);
    check_launch("sum_rows_batched");
}

void finalize_sums(cudaStream_t s, const SumJob* d_jobs, uint32_t jobs, uint32_t blocks) {
    if (jobs == 0 || blocks == 0) return;
    finalize_sums_kernel<<<blocks, dim3(32, 8), 0, s>>>(d_jobs, jobs);
    check_launch("finalize_sums");
}

uint32_t sum_rows_chunks(uint64_t rows) {
    uint64_t chunks = (rows + 127) / 128;
    return static_cast<uint32_t>(chunks < 1 ? 1 : (chunks > 64 ? 64 : chunks));
}

uint64_t reduce_scratch_doubles() { return kMaxBlocks; }

void reduce_sum(cudaStream_t s, const float* a, uint64_t n, bool mean, double* scratch, float* out) {
    uint32_t blocks = whole_blocks(n);
    whole_stage1<Whole::Sum><<<blocks, kThreads, 0, s>>>(a, nullptr, n, scratch);
    check_launch("reduce_sum");
    whole_stage2<<<1, kThreads, 0, s>>>(scratch, blocks, mean ? static_cast<double>(n) : 1.0, out);
    check_launch("reduce_sum");
}

void mse(cudaStream_t s, const float* a, const float* b, uint64_t n, double* scratch, float* out) {
    uint32_t blocks = whole_blocks(n);
    whole_stage1<Whole::SquaredDifference><<<blocks, kThreads, 0, s>>>(a, b, n, scratch);
    check_launch("mse");
    whole_stage2<<<1, kThreads, 0, s>>>(scratch, blocks, static_cast<double>(n), out);
    check_launch("mse");
}

uint64_t sum_rows_scratch_floats(uint64_t rows, uint64_t h) { return sum_rows_chunks(rows) * h; }

uint64_t sum_rows_counters(uint64_t h) { return (h + 31) / 32; }

namespace {
template <class T>
void launch_sum_rows(cudaStream_t s, const T* g, uint64_t rows, uint64_t h, float* scratch, float* out, uint32_t* counters, uint64_t ld) {
    uint32_t chunks = sum_rows_chunks(rows);
    uint32_t rows_per_chunk = static_cast<uint32_t>((rows + chunks - 1) / chunks);
    // Wide matrices whose rows can be read four elements at a time: four columns per lane, chunk sums only.
    const bool wide = h >= 1024 && ld % 4 == 0 && aligned4(g) && (out == nullptr || counters == nullptr) && !(chunks == 1 && out);
    if (wide) {
        dim3 grid(static_cast<uint32_t>((h + 127) / 128), chunks);
        sum_rows_stage1_wide<<<grid, dim3(32, 8), 0, s>>>(g, static_cast<uint32_t>(rows), static_cast<uint32_t>(h), static_cast<uint32_t>(ld),
                                                          rows_per_chunk, scratch);
        check_launch("sum_rows");
    } else {
        dim3 grid(static_cast<uint32_t>((h + 31) / 32), chunks);
        sum_rows_stage1<<<grid, dim3(32, 8), 0, s>>>(g, static_cast<uint32_t>(rows), static_cast<uint32_t>(h), static_cast<uint32_t>(ld),
                                                     rows_per_chunk, (chunks == 1 && out) ? out : scratch,
                                                     (chunks > 1 && out) ? counters : nullptr, out);
        check_launch("sum_rows");
    }
    if (chunks > 1 && counters == nullptr && out != nullptr) {
        sum_rows_stage2<<<static_cast<uint32_t>((h + 127) / 128), 128, 0, s>>>(scratch, chunks,
                                                                                static_cast<uint32_t>(h), out);
        check_launch("sum_rows");
    }
}
}  // namespace

void sum_rows(cudaStream_t s, In g, uint64_t rows, uint64_t h, float* scratch, float* out, uint32_t* counters,
              uint64_t ld) {
    if (h == 0) return;
    if (ld == 0) ld = h;
    if (g.half) launch_sum_rows(s, static_cast<const bf16*>(g.p), rows, h, scratch, out, counters, ld);
    else launch_sum_rows(s, g.f32(), rows, h, scratch, out, counters, ld);
}

}  // namespace k
}  // namespace msx
