// All-reduce of a gradient bucket over peer memory: every rank's copy of the bucket is mapped into
// every other rank's address space (CUDA IPC over NVLink / NVSwitch), rank r sums slice r of all
// copies in rank order and stores the sum into slice r of all copies. One kernel per rank, two
// rendezvous through flag words in peer memory (the copies are complete; the sums have landed).
//
// The reference trains on one device and has nothing like it: this is the exchange between the
// backward pass and the optimizer step of a data-parallel run. The sum of an element is formed by
// one rank only, in rank order 0 .. world - 1, so every rank holds the same bits and a run is
// repeatable.
//
// Why not the library's all-reduce: at 8 ranks it takes 100 us for the 16 MB of a tied embedding
// table's gradient and 39 us for 4 bytes; each rank here reads 7/8 of the bucket's bytes once and
// writes them once, all eight NVLink directions busy at the same time.
//
// Every wait is bounded by the global timer: a rank that gives up raises bit 1 of *status, marks
// the channel failed (later launches return at once) and leaves its copy unsummed.
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

constexpr uint32_t kThreads = 512;
constexpr uint64_t kWaitNanoseconds = 10ull * 1000 * 1000 * 1000;

__device__ __forceinline__ void store_release_system(uint32_t* at, uint32_t value) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(at), "r"(value) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_system(const uint32_t* at) {
    uint32_t value;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(value) : "l"(at) : "memory");
    return value;
}
__device__ __forceinline__ uint64_t global_timer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ float4 load_peer(const float* at) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(at) : "memory");
    return v;
}
__device__ __forceinline__ float load_peer_scalar(const float* at) {
    float v;
    asm volatile("ld.volatile.global.f32 %0, [%1];" : "=f"(v) : "l"(at) : "memory");
    return v;
}

// Thread q < world waits until rank q has written at least `value` into this rank's flag word q.
// False when the wait ran out.
__device__ bool wait_for_ranks(const PeerReduceArgs& a, uint32_t value, bool* gave_up) {
    if (threadIdx.x == 0) *gave_up = false;
    __syncthreads();
    if (threadIdx.x < a.world) {
        const uint32_t* flag = a.flags[a.rank] + threadIdx.x;
        const uint64_t start = global_timer();
        // Flag values only grow; the difference is compared so that a wrap of the counter is harmless.
        while (static_cast<int32_t>(load_acquire_system(flag) - value) < 0) {
            if (global_timer() - start > (a.wait_nanoseconds ? a.wait_nanoseconds : kWaitNanoseconds)) {
                *gave_up = true;
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();
    return !*gave_up;
}

template <int WORLD>
__device__ __forceinline__ void reduce_slice(const PeerReduceArgs& a, uint64_t lo, uint64_t hi) {
    // 16 bytes per thread, rank and group, GROUPS groups a turn: all WORLD x GROUPS loads are issued
    // before the first sum (a load from a peer takes microseconds; what bounds the kernel is how
    // many are in flight). A group past the end of the slice reads the turn's first group again
    // and stores nothing.
    constexpr int GROUPS = WORLD <= 2 ? 4 : 2;
    const uint64_t lo4 = (lo + 3) & ~3ull, hi4 = hi & ~3ull;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * kThreads * 4;
    for (uint64_t first = lo4 + (static_cast<uint64_t>(blockIdx.x) * kThreads + threadIdx.x) * 4; first < hi4; first += stride * GROUPS) {
        float4 v[GROUPS][WORLD];
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            const uint64_t i = first + g * stride < hi4 ? first + g * stride : first;
#pragma unroll
            for (int q = 0; q < WORLD; ++q) v[g][q] = load_peer(a.buffers[q] + i);
        }
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
            const uint64_t i = first + g * stride;
            if (i >= hi4) break;
            float4 sum = v[g][0];
#pragma unroll
            for (int q = 1; q < WORLD; ++q) {
                sum.x += v[g][q].x;
                sum.y += v[g][q].y;
                sum.z += v[g][q].z;
                sum.w += v[g][q].w;
            }
            sum.x *= a.scale;
            sum.y *= a.scale;
            sum.z *= a.scale;
            sum.w *= a.scale;
#pragma unroll
            for (int q = 0; q < WORLD; ++q) *reinterpret_cast<float4*>(a.buffers[q] + i) = sum;
        }
    }
    // The ragged ends of the slice, one element per thread.
    if (blockIdx.x == 0 && threadIdx.x < 8) {
        // At most three elements before lo4 and three from hi4 on (all of a slice shorter than four).
        const uint64_t head = min(lo4, hi) - lo;
        const uint64_t i = threadIdx.x < 4 ? lo + threadIdx.x : max(hi4, min(lo4, hi)) + (threadIdx.x - 4);
        const bool mine = threadIdx.x < 4 ? threadIdx.x < head : i < hi;
        if (mine) {
            float sum = load_peer_scalar(a.buffers[0] + i);
            for (int q = 1; q < WORLD; ++q) sum += load_peer_scalar(a.buffers[q] + i);
            sum *= a.scale;
            for (int q = 0; q < WORLD; ++q) a.buffers[q][i] = sum;
        }
    }
}

__global__ void __launch_bounds__(kThreads) peer_all_reduce_kernel(PeerReduceArgs a) {
    __shared__ bool gave_up;
    __shared__ bool is_last;
    // The channel's launch count: the same on every rank, read by every block before any block
    // of this launch can have finished (the last block to finish is the one that advances it).
    const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch);
    const uint32_t begun = 2 * epoch + 1, done = 2 * epoch + 2;
    bool ok = *reinterpret_cast<volatile uint32_t*>(a.failed) == 0;
    if (ok) {
        // This rank's copy is complete (the launches before this one wrote it): tell every rank.
        if (blockIdx.x == 0 && threadIdx.x < a.world) {
            __threadfence_system();
            store_release_system(a.flags[threadIdx.x] + a.rank, begun);
        }
        ok = wait_for_ranks(a, begun, &gave_up);
    }
    if (ok) {
        // Slices are multiples of four elements so that 16-byte accesses stay aligned.
        const uint64_t per = ((a.count + a.world - 1) / a.world + 3) & ~3ull;
        const uint64_t lo = min(a.count, per * a.rank), hi = min(a.count, lo + per);
        switch (a.world) {
            case 2: reduce_slice<2>(a, lo, hi); break;
            case 3: reduce_slice<3>(a, lo, hi); break;
            case 4: reduce_slice<4>(a, lo, hi); break;
            case 5: reduce_slice<5>(a, lo, hi); break;
            case 6: reduce_slice<6>(a, lo, hi); break;
            case 7: reduce_slice<7>(a, lo, hi); break;
            default: reduce_slice<8>(a, lo, hi); break;
        }
    }
    // A block that gave up marks the channel before it counts itself as finished: the last block
    // then knows that this rank's slice was not summed everywhere, whichever block it is.
    if (!ok && threadIdx.x == 0) {
        atomicOr(a.status, 2u);
        atomicOr(a.failed, 1u);
    }
    // The block's stores are out before it counts itself as finished.
    __threadfence_system();
    __syncthreads();
    if (!last_block_arrives(a.arrivals, gridDim.x, &is_last)) return;
    // The last block of this rank: every sum of this rank's slice has been stored everywhere,
    // unless some block gave up. Then the second rendezvous is not announced: the peers' waits for
    // it run out and they fail too, instead of going on with a partly summed bucket.
    ok = ok && *reinterpret_cast<volatile uint32_t*>(a.failed) == 0;
    if (ok) {
        if (threadIdx.x < a.world) {
            __threadfence_system();
            store_release_system(a.flags[threadIdx.x] + a.rank, done);
        }
        ok = wait_for_ranks(a, done, &gave_up);
    }
    if (threadIdx.x == 0) {
        if (!ok) {
            atomicOr(a.status, 2u);
            *reinterpret_cast<volatile uint32_t*>(a.failed) = 1;
        }
        *reinterpret_cast<volatile uint32_t*>(a.epoch) = epoch + 1;
    }
}

}  // namespace

void peer_all_reduce(cudaStream_t s, const PeerReduceArgs& args) {
    if (args.count == 0 || args.world < 2) return;
    const uint64_t per = (args.count + args.world - 1) / args.world;
    const uint64_t wanted = (per / 4 + kThreads - 1) / kThreads;
    const uint32_t blocks = static_cast<uint32_t>(wanted < 1 ? 1 : (wanted > 128 ? 128 : wanted));
    peer_all_reduce_kernel<<<blocks, kThreads, 0, s>>>(args);
    check_launch("peer_all_reduce");
}

}  // namespace k
}  // namespace msx
