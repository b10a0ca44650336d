// Shared device helpers and the host-side launch check.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <initializer_list>
#include <stdexcept>
#include <string>

namespace msx {
namespace k {

struct CudaError : std::runtime_error {
    cudaError_t code;
    CudaError(const std::string& what, cudaError_t c) : std::runtime_error(what), code(c) {}
};

inline void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess)
        throw CudaError(std::string(what) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")", e);
}

// After a kernel launch: reports a launch-configuration error without synchronising. The error
// is taken (cudaGetLastError), not peeked at, so a non-sticky error that this thread left behind
// earlier (the host application's own, or an earlier launch here) is reported once and does not
// fail every later launch.
inline void check_launch(const char* kernel) { check(cudaGetLastError(), kernel); }

// ---- elements of either storage type ------------------------------------------------------------
// A mixed-precision plan stores activations as bf16; the kernels that touch them are templates on
// the element type and compute in f32 whatever it is. One element, or four consecutive ones (16
// bytes of f32, 8 bytes of bf16; the address a multiple of that).
using bf16 = __nv_bfloat16;
__device__ __forceinline__ float load1(const float* p) { return __ldg(p); }
__device__ __forceinline__ float load1(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void store1(float* p, float v) { *p = v; }
__device__ __forceinline__ void store1(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
// Two consecutive elements (the address a multiple of their size).
__device__ __forceinline__ float2 load2(const float* p) { return __ldg(reinterpret_cast<const float2*>(p)); }
__device__ __forceinline__ float2 load2(const bf16* p) {
    const uint32_t raw = __ldg(reinterpret_cast<const uint32_t*>(p));
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw));
}
__device__ __forceinline__ void store2(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
__device__ __forceinline__ void store2(bf16* p, float2 v) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(v.x, v.y);
    *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<const uint32_t*>(&pair);
}
__device__ __forceinline__ float4 load4(const float* p) { return __ldg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ float4 load4(const bf16* p) {
    const uint2 raw = __ldg(reinterpret_cast<const uint2*>(p));
    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    return make_float4(lo.x, lo.y, hi.x, hi.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(bf16* p, float4 v) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&lo);
    raw.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = raw;
}
// Eight consecutive bf16 elements (16 bytes; the address a multiple of 16).
struct float8 {
    float4 lo, hi;
};
__device__ __forceinline__ float8 load8(const bf16* p) {
    const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
    const float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.z));
    const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.w));
    return {make_float4(a.x, a.y, b.x, b.y), make_float4(c.x, c.y, d.x, d.y)};
}
__device__ __forceinline__ void store8(bf16* p, const float8& v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.lo.x, v.lo.y), b = __floats2bfloat162_rn(v.lo.z, v.lo.w);
    const __nv_bfloat162 c = __floats2bfloat162_rn(v.hi.x, v.hi.y), d = __floats2bfloat162_rn(v.hi.z, v.hi.w);
    uint4 raw;
    raw.x = *reinterpret_cast<const uint32_t*>(&a);
    raw.y = *reinterpret_cast<const uint32_t*>(&b);
    raw.z = *reinterpret_cast<const uint32_t*>(&c);
    raw.w = *reinterpret_cast<const uint32_t*>(&d);
    *reinterpret_cast<uint4*>(p) = raw;
}
// `v` as an array of that element type would hold it.
__device__ __forceinline__ float stored_as(float v, const float*) { return v; }
__device__ __forceinline__ float stored_as(float v, const bf16*) { return __bfloat162float(__float2bfloat16_rn(v)); }
// Whether `p` may be read or written four elements at a time.
template <class T> inline bool aligned4(const T* p) { return reinterpret_cast<uintptr_t>(p) % (4 * sizeof(T)) == 0; }

// The activation operands of one launch share one storage type: true when all are bf16.
inline bool all_half(std::initializer_list<bool> halves, const char* kernel) {
    bool any = false, all = true;
    for (bool h : halves) {
        any = any || h;
        all = all && h;
    }
    if (any && !all) throw std::invalid_argument(std::string(kernel) + ": f32 and bf16 activation operands in one launch");
    return all;
}

// ---- GELU, the tanh form evaluated as x / (1 + exp(-2u)) -------------------------------------
// The operation order is the reference's (crates/modelspec-runtime/src/cpu/interpreter.rs:
// 1553-1587); the constants are the nearest f32 to sqrt(2/pi) and 0.044715.
__device__ __forceinline__ float gelu_twice_inner(float x) {
    const float scale = 0.7978845608028654f, cubic = 0.044715f;
    return 2.0f * scale * (x + cubic * x * x * x);
}
__device__ __forceinline__ float logistic(float v) { return 1.0f / (1.0f + expf(0.0f - v)); }
__device__ __forceinline__ float gelu_value(float x) { return x * logistic(gelu_twice_inner(x)); }
__device__ __forceinline__ float gelu_grad_value(float x, float g) {
    const float scale = 0.7978845608028654f, cubic = 0.044715f;
    float v = gelu_twice_inner(x);
    float s = logistic(v), r = logistic(0.0f - v);
    float slope = scale * (1.0f + 3.0f * cubic * x * x);
    return (s + 2.0f * (s * x) * r * slope) * g;
}

// The same two functions where the result is stored as bf16 (mixed-precision plans, which have no
// reference bits to keep): the hardware exponential and reciprocal, about 2^-21 relative, far
// inside the 2^-9 of the stored value, and r = 1 - s instead of a second exponential. Half the
// special-function work per element: gelu_grad over a [16384, 3072] matrix is otherwise bound by
// it, not by memory.
__device__ __forceinline__ float logistic_fast(float v) { return __fdividef(1.0f, 1.0f + __expf(0.0f - v)); }
template <class T> __device__ __forceinline__ float gelu_value_for(float x) {
    if constexpr (sizeof(T) == 2) return x * logistic_fast(gelu_twice_inner(x));
    else return gelu_value(x);
}
template <class T> __device__ __forceinline__ float gelu_grad_value_for(float x, float g) {
    if constexpr (sizeof(T) == 2) {
        const float scale = 0.7978845608028654f, cubic = 0.044715f;
        const float s = logistic_fast(gelu_twice_inner(x)), r = 1.0f - s;
        const float slope = scale * (1.0f + 3.0f * cubic * x * x);
        return (s + 2.0f * (s * x) * r * slope) * g;
    } else {
        return gelu_grad_value(x, g);
    }
}

// ---- Philox4x32-10, word 0 of the block ------------------------------------------------------
// Counter [c0, c1, c2, c3], key [k0, k1] (Salmon et al., SC 2011); the reference draws a dropout
// decision from word 0 alone (crates/modelspec-runtime/src/train/init.rs:91-112, :160-165).
__device__ __forceinline__ uint32_t philox_word0(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                 uint32_t k0, uint32_t k1) {
    const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
    for (int round = 0; round < 10; ++round) {
        if (round > 0) {
            k0 += W0;
            k1 += W1;
        }
        uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
        uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
        uint32_t n0 = hi1 ^ c1 ^ k0, n2 = hi0 ^ c3 ^ k1;
        c0 = n0;
        c1 = lo1;
        c2 = n2;
        c3 = lo0;
    }
    return c0;
}

// ---- reductions ------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `shared` holds 33 T.
template <class T> __device__ __forceinline__ T block_sum(T v, T* shared) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) shared[warp] = v;
    __syncthreads();
    if (warp == 0) {
        T t = lane < warps ? shared[lane] : T(0);
        t = warp_sum(t);
        if (lane == 0) shared[32] = t;
    }
    __syncthreads();
    return shared[32];
}
__device__ __forceinline__ float block_max(float v, float* shared) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) shared[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? shared[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) shared[32] = t;
    }
    __syncthreads();
    return shared[32];
}

// One-launch two-stage reductions: every block publishes its partial result, then calls this; the
// block that arrives last at `counter` (true for all its threads) sees every block's partials and
// finishes the job. The counter goes back to 0 for the next launch. Partials written by other
// blocks must be read with __ldcg (they may sit in another SM's path, never in this SM's L1).
__device__ __forceinline__ bool last_block_arrives(uint32_t* counter, uint32_t expected, bool* shared_flag) {
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        uint32_t before = atomicAdd(counter, 1u);
        bool last = before + 1u == expected;
        if (last) *counter = 0u;
        *shared_flag = last;
    }
    __syncthreads();
    bool last = *shared_flag;
    if (last) __threadfence();
    return last;
}

}  // namespace k
}  // namespace msx
