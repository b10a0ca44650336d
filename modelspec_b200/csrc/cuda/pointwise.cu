// Element-by-element kernels: the arithmetic ops, relu and gelu with their gradients, add_rows,
// transpose, the scalar broadcast and the Philox dropout. All are HBM-bound: 128-bit loads and
// stores where the element count allows, grids sized to a few waves of the 148 SMs.
//
// Every op here is one or a few rounded f32 operations per element in the order of the
// reference's interpreter (crates/modelspec-runtime/src/cpu/interpreter.rs:895-969, :1538-1587),
// so results are bit-identical to it except where expf differs from the host libm.
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

constexpr int kThreads = 256;

inline uint32_t blocks_for(uint64_t work_items) {
    uint64_t b = (work_items + kThreads - 1) / kThreads;
    const uint64_t cap = 148ull * 16;  // grid-stride beyond a few waves
    return static_cast<uint32_t>(b < 1 ? 1 : (b > cap ? cap : b));
}

__device__ __forceinline__ float apply(Binary op, float a, float b) {
    switch (op) {
        case Binary::Add: return a + b;
        case Binary::Sub: return a - b;
        case Binary::Mul: return a * b;
        default: return a / b;
    }
}

template <bool A_SCALAR, bool B_SCALAR>
__global__ void binary_kernel(Binary op, const float* __restrict__ a, const float* __restrict__ b,
                              float* __restrict__ out, uint64_t n) {
    uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    float sa = A_SCALAR ? a[0] : 0.0f, sb = B_SCALAR ? b[0] : 0.0f;
    uint64_t n4 = n / 4;
    bool vec = (reinterpret_cast<uintptr_t>(out) % 16 == 0) &&
               (A_SCALAR || reinterpret_cast<uintptr_t>(a) % 16 == 0) &&
               (B_SCALAR || reinterpret_cast<uintptr_t>(b) % 16 == 0);
    if (vec) {
        for (uint64_t j = i; j < n4; j += stride) {
            float4 va = A_SCALAR ? make_float4(sa, sa, sa, sa) : reinterpret_cast<const float4*>(a)[j];
            float4 vb = B_SCALAR ? make_float4(sb, sb, sb, sb) : reinterpret_cast<const float4*>(b)[j];
            float4 r;
            r.x = apply(op, va.x, vb.x);
            r.y = apply(op, va.y, vb.y);
            r.z = apply(op, va.z, vb.z);
            r.w = apply(op, va.w, vb.w);
            reinterpret_cast<float4*>(out)[j] = r;
        }
        for (uint64_t j = n4 * 4 + i; j < n; j += stride)
            out[j] = apply(op, A_SCALAR ? sa : a[j], B_SCALAR ? sb : b[j]);
    } else {
        for (uint64_t j = i; j < n; j += stride)
            out[j] = apply(op, A_SCALAR ? sa : a[j], B_SCALAR ? sb : b[j]);
    }
}

template <class T> __device__ __forceinline__ float apply_as(Unary op, float x) {
    switch (op) {
        case Unary::Relu: return x > 0.0f ? x : 0.0f;
        case Unary::Sqrt: return sqrtf(x);
        case Unary::Gelu: return gelu_value_for<T>(x);
        default: return x;
    }
}

template <class T>
__global__ void unary_kernel(Unary op, const T* __restrict__ a, T* __restrict__ out, uint64_t n) {
    uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if constexpr (sizeof(T) == 2) {
        // bf16: 16 bytes (eight elements) per thread and turn.
        if (reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0) {
            const uint64_t n8 = n / 8;
            for (uint64_t j = i; j < n8; j += stride) {
                float8 v = load8(a + 8 * j);
                v.lo.x = apply_as<T>(op, v.lo.x); v.lo.y = apply_as<T>(op, v.lo.y); v.lo.z = apply_as<T>(op, v.lo.z); v.lo.w = apply_as<T>(op, v.lo.w);
                v.hi.x = apply_as<T>(op, v.hi.x); v.hi.y = apply_as<T>(op, v.hi.y); v.hi.z = apply_as<T>(op, v.hi.z); v.hi.w = apply_as<T>(op, v.hi.w);
                store8(out + 8 * j, v);
            }
            for (uint64_t j = n8 * 8 + i; j < n; j += stride) store1(out + j, apply_as<T>(op, load1(a + j)));
            return;
        }
    }
    bool vec = reinterpret_cast<uintptr_t>(out) % (4 * sizeof(T)) == 0 && reinterpret_cast<uintptr_t>(a) % (4 * sizeof(T)) == 0;
    uint64_t n4 = vec ? n / 4 : 0;
    for (uint64_t j = i; j < n4; j += stride) {
        float4 v = load4(a + 4 * j);
        v.x = apply_as<T>(op, v.x);
        v.y = apply_as<T>(op, v.y);
        v.z = apply_as<T>(op, v.z);
        v.w = apply_as<T>(op, v.w);
        store4(out + 4 * j, v);
    }
    for (uint64_t j = n4 * 4 + i; j < n; j += stride) store1(out + j, apply_as<T>(op, load1(a + j)));
}

template <bool GELU, class T>
__global__ void act_grad_kernel(const T* __restrict__ a, const T* __restrict__ g,
                                T* __restrict__ out, uint64_t n) {
    uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    auto one = [](float x, float gg) { return GELU ? gelu_grad_value_for<T>(x, gg) : (x > 0.0f ? gg : 0.0f); };
    if constexpr (sizeof(T) == 2) {
        // bf16: 16 bytes (eight elements) of each array per thread and turn.
        if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(g)) % 16 == 0) {
            const uint64_t n8 = n / 8;
            for (uint64_t j = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n8; j += stride) {
                const float8 x = load8(a + 8 * j), gg = load8(g + 8 * j);
                float8 r;
                r.lo = make_float4(one(x.lo.x, gg.lo.x), one(x.lo.y, gg.lo.y), one(x.lo.z, gg.lo.z), one(x.lo.w, gg.lo.w));
                r.hi = make_float4(one(x.hi.x, gg.hi.x), one(x.hi.y, gg.hi.y), one(x.hi.z, gg.hi.z), one(x.hi.w, gg.hi.w));
                store8(out + 8 * j, r);
            }
            for (uint64_t j = n8 * 8 + static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride)
                store1(out + j, one(load1(a + j), load1(g + j)));
            return;
        }
    }
    if constexpr (sizeof(T) == 4) {
        // f32: 16 bytes (four elements) of each array per thread and turn.
        if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(g)) % 16 == 0) {
            const uint64_t n4 = n / 4;
            for (uint64_t j = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n4; j += stride) {
                const float4 x = load4(a + 4 * j), gg = load4(g + 4 * j);
                store4(out + 4 * j, make_float4(one(x.x, gg.x), one(x.y, gg.y), one(x.z, gg.z), one(x.w, gg.w)));
            }
            for (uint64_t j = n4 * 4 + static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride)
                store1(out + j, one(load1(a + j), load1(g + j)));
            return;
        }
    }
    for (uint64_t j = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride) {
        float x = load1(a + j), gg = load1(g + j);
        store1(out + j, one(x, gg));
    }
}

__global__ void fill_kernel(const float* __restrict__ scalar, float* __restrict__ out, uint64_t n) {
    float v = scalar[0];
    uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t j = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride) out[j] = v;
}

__global__ void add_rows_kernel(const float* __restrict__ x, const float* __restrict__ b,
                                float* __restrict__ out, uint64_t n, uint64_t h) {
    uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t j = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride)
        out[j] = x[j] + b[j % h];
}

// 32 x 32 tiles through shared memory, padded against bank conflicts.
__global__ void transpose_kernel(const float* __restrict__ a, float* __restrict__ out, uint32_t rows,
                                 uint32_t cols) {
    __shared__ float tile[32][33];
    uint32_t tiles_x = (cols + 31) / 32, tiles_y = (rows + 31) / 32;
    for (uint32_t t = blockIdx.x; t < tiles_x * tiles_y; t += gridDim.x) {
        uint32_t c0 = (t % tiles_x) * 32, r0 = (t / tiles_x) * 32;
        for (uint32_t dy = threadIdx.y; dy < 32; dy += blockDim.y) {
            uint32_t r = r0 + dy, c = c0 + threadIdx.x;
            if (r < rows && c < cols) tile[dy][threadIdx.x] = a[static_cast<uint64_t>(r) * cols + c];
        }
        __syncthreads();
        for (uint32_t dy = threadIdx.y; dy < 32; dy += blockDim.y) {
            uint32_t c = c0 + dy, r = r0 + threadIdx.x;
            if (r < rows && c < cols) out[static_cast<uint64_t>(c) * rows + r] = tile[threadIdx.x][dy];
        }
        __syncthreads();
    }
}

template <class T>
__global__ void dropout_kernel(const T* __restrict__ x, const int32_t* __restrict__ token,
                               uint32_t seed_lo, uint32_t seed_hi, uint32_t threshold, float scale,
                               uint64_t index_base, T* __restrict__ out, uint64_t n) {
    uint32_t id_lo = static_cast<uint32_t>(token[0]), id_hi = static_cast<uint32_t>(token[1]);
    uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t j = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; j < n; j += stride) {
        uint32_t w0 = philox_word0(static_cast<uint32_t>(index_base + j), 4u, id_lo, id_hi, seed_lo, seed_hi);
        store1(out + j, w0 >= threshold ? load1(x + j) * scale : 0.0f);
    }
}

}  // namespace

void binary(cudaStream_t s, Binary op, const float* a, bool a_scalar, const float* b, bool b_scalar,
            float* out, uint64_t n) {
    if (n == 0) return;
    uint32_t grid = blocks_for((n + 3) / 4);
    if (a_scalar && b_scalar) binary_kernel<true, true><<<grid, kThreads, 0, s>>>(op, a, b, out, n);
    else if (a_scalar) binary_kernel<true, false><<<grid, kThreads, 0, s>>>(op, a, b, out, n);
    else if (b_scalar) binary_kernel<false, true><<<grid, kThreads, 0, s>>>(op, a, b, out, n);
    else binary_kernel<false, false><<<grid, kThreads, 0, s>>>(op, a, b, out, n);
    check_launch("binary");
}

void unary(cudaStream_t s, Unary op, In a, Out out, uint64_t n) {
    if (n == 0) return;
    if (all_half({a.half, out.half}, "unary"))
        unary_kernel<<<blocks_for((n + 7) / 8), kThreads, 0, s>>>(op, static_cast<const bf16*>(a.p), static_cast<bf16*>(out.p), n);
    else
        unary_kernel<<<blocks_for((n + 3) / 4), kThreads, 0, s>>>(op, a.f32(), out.f32(), n);
    check_launch("unary");
}

void relu_grad(cudaStream_t s, const float* a, const float* g, float* out, uint64_t n) {
    if (n == 0) return;
    act_grad_kernel<false, float><<<blocks_for((n + 3) / 4), kThreads, 0, s>>>(a, g, out, n);
    check_launch("relu_grad");
}

void gelu_grad(cudaStream_t s, In a, In g, Out out, uint64_t n) {
    if (n == 0) return;
    if (all_half({a.half, g.half, out.half}, "gelu_grad"))
        act_grad_kernel<true, bf16><<<blocks_for((n + 7) / 8), kThreads, 0, s>>>(static_cast<const bf16*>(a.p), static_cast<const bf16*>(g.p),
                                                                       static_cast<bf16*>(out.p), n);
    else
        act_grad_kernel<true, float><<<blocks_for((n + 3) / 4), kThreads, 0, s>>>(a.f32(), g.f32(), out.f32(), n);
    check_launch("gelu_grad");
}

void fill_from_scalar(cudaStream_t s, const float* scalar, float* out, uint64_t n) {
    if (n == 0) return;
    fill_kernel<<<blocks_for(n), kThreads, 0, s>>>(scalar, out, n);
    check_launch("fill_from_scalar");
}

void add_rows(cudaStream_t s, const float* x, const float* b, float* out, uint64_t rows, uint64_t h) {
    if (rows * h == 0) return;
    add_rows_kernel<<<blocks_for(rows * h), kThreads, 0, s>>>(x, b, out, rows * h, h);
    check_launch("add_rows");
}

void transpose(cudaStream_t s, const float* a, float* out, uint64_t rows, uint64_t cols) {
    if (rows * cols == 0) return;
    uint64_t tiles = ((rows + 31) / 32) * ((cols + 31) / 32);
    uint32_t grid = static_cast<uint32_t>(tiles < 148 * 8 ? tiles : 148 * 8);
    transpose_kernel<<<grid, dim3(32, 8), 0, s>>>(a, out, static_cast<uint32_t>(rows), static_cast<uint32_t>(cols));
    check_launch("transpose");
}

void dropout(cudaStream_t s, In x, const int32_t* token, uint64_t seed, uint32_t threshold,
             float scale, uint64_t index_base, Out out, uint64_t n) {
    if (n == 0) return;
    const uint32_t lo = static_cast<uint32_t>(seed), hi = static_cast<uint32_t>(seed >> 32);
    if (all_half({x.half, out.half}, "dropout"))
        dropout_kernel<<<blocks_for(n), kThreads, 0, s>>>(static_cast<const bf16*>(x.p), token, lo, hi, threshold, scale, index_base,
                                                          static_cast<bf16*>(out.p), n);
    else
        dropout_kernel<<<blocks_for(n), kThreads, 0, s>>>(x.f32(), token, lo, hi, threshold, scale, index_base, out.f32(), n);
    check_launch("dropout");
}

}  // namespace k
}  // namespace msx
