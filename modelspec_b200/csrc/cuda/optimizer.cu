// The parameter update: one launch over every parameter tensor of the step.
//
// AdamW is the reference's 16 rounded f32 operations per element, in its order
// (crates/modelspec-core/src/ir/training.rs:925-980):
//   m' = beta1 * m + (1 - beta1) * g
//   v' = beta2 * v + ((1 - beta2) * g) * g
//   p' = p - lr_t * ((m' * c1) / (sqrt(v' * c2) + eps) + weight_decay * p)
// with sqrt and the division correctly rounded and no contraction (the file is compiled with
// -fmad=false), so given the same gradient the new p, m and v are bit-identical to the CPU's.
// The reference's Vulkan path runs one dispatch per parameter
// (crates/modelspec-core/src/ir/kernel.rs:869-894); here a chunk table maps each CTA to 4096
// elements of one tensor, so 41 tensors are one launch. HBM-bound: 16 bytes read and 12 written
// per element.
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

__global__ void __launch_bounds__(256) adamw_kernel(const UpdateTensor* __restrict__ tensors,
                                                     const uint32_t* __restrict__ chunk_tensor,
                                                     const uint32_t* __restrict__ chunk_start, AdamWConstants c,
                                                     const float* __restrict__ lr_t, const float* __restrict__ c1,
                                                     const float* __restrict__ c2) {
    UpdateTensor t = tensors[chunk_tensor[blockIdx.x]];
    uint64_t start = static_cast<uint64_t>(chunk_start[blockIdx.x]) * kUpdateChunk;
    uint64_t stop = start + kUpdateChunk < t.count ? start + kUpdateChunk : t.count;
    float lr = lr_t[0], k1 = c1[0], k2 = c2[0];
    auto update = [&](float g, float& p, float& m, float& v) {
        float m_next = c.beta1 * m + c.rest1 * g;
        float v_next = c.beta2 * v + (c.rest2 * g) * g;
        float direction = (m_next * k1) / (sqrtf(v_next * k2) + c.eps);
        float step = direction + c.weight_decay * p;
        p = p - lr * step;
        m = m_next;
        v = v_next;
    };
    const bool aligned = ((reinterpret_cast<uintptr_t>(t.g) | reinterpret_cast<uintptr_t>(t.p) | reinterpret_cast<uintptr_t>(t.m) |
                           reinterpret_cast<uintptr_t>(t.v)) & 15) == 0;
    if (aligned && stop - start == kUpdateChunk) {
        // A whole chunk of 16-byte-aligned tensors: two float4 per thread and array at a time,
        // all eight loads issued before the first update.
        constexpr int kVectors = 2, kTurns = kUpdateChunk / (256 * 4 * kVectors);
#pragma unroll 1
        for (int turn = 0; turn < kTurns; ++turn) {
            float4 g[kVectors], p[kVectors], m[kVectors], v[kVectors];
#pragma unroll
            for (int j = 0; j < kVectors; ++j) {
                const uint64_t i = start + ((turn * kVectors + j) * 256 + threadIdx.x) * 4;
                g[j] = *reinterpret_cast<const float4*>(t.g + i);
                p[j] = *reinterpret_cast<const float4*>(t.p + i);
                m[j] = *reinterpret_cast<const float4*>(t.m + i);
                v[j] = *reinterpret_cast<const float4*>(t.v + i);
            }
#pragma unroll
            for (int j = 0; j < kVectors; ++j) {
                const uint64_t i = start + ((turn * kVectors + j) * 256 + threadIdx.x) * 4;
                update(g[j].x, p[j].x, m[j].x, v[j].x);
                update(g[j].y, p[j].y, m[j].y, v[j].y);
                update(g[j].z, p[j].z, m[j].z, v[j].z);
                update(g[j].w, p[j].w, m[j].w, v[j].w);
                *reinterpret_cast<float4*>(t.p + i) = p[j];
                *reinterpret_cast<float4*>(t.m + i) = m[j];
                *reinterpret_cast<float4*>(t.v + i) = v[j];
                // The bf16 working copy the next step's matmuls read (mixed-precision plans).
                if (t.p16 != nullptr) store4(static_cast<bf16*>(t.p16) + i, p[j]);
            }
        }
        return;
    }
    for (uint64_t i = start + threadIdx.x; i < stop; i += blockDim.x) {
        float g = t.g[i], p = t.p[i], m = t.m[i], v = t.v[i];
        update(g, p, m, v);
        t.p[i] = p;
        t.m[i] = m;
        t.v[i] = v;
        if (t.p16 != nullptr) store1(static_cast<bf16*>(t.p16) + i, p);
    }
}

// The bf16 working copy of a parameter from its f32 master (after an upload).
__global__ void working_copy_kernel(const float* __restrict__ p, bf16* __restrict__ p16, uint64_t n) {
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) store1(p16 + i, p[i]);
}

__global__ void __launch_bounds__(256) sgd_kernel(const UpdateTensor* __restrict__ tensors,
                                                   const uint32_t* __restrict__ chunk_tensor,
                                                   const uint32_t* __restrict__ chunk_start,
                                                   const float* __restrict__ lr) {
    UpdateTensor t = tensors[chunk_tensor[blockIdx.x]];
    uint64_t start = static_cast<uint64_t>(chunk_start[blockIdx.x]) * kUpdateChunk;
    uint64_t stop = start + kUpdateChunk < t.count ? start + kUpdateChunk : t.count;
    float rate = lr[0];
    for (uint64_t i = start + threadIdx.x; i < stop; i += blockDim.x) {
        const float p = t.p[i] - rate * t.g[i];
        t.p[i] = p;
        if (t.p16 != nullptr) store1(static_cast<bf16*>(t.p16) + i, p);
    }
}

}  // namespace

void adamw(cudaStream_t s, const UpdateTensor* d_tensors, const uint32_t* d_chunk_tensor,
           const uint32_t* d_chunk_start, uint32_t chunks, AdamWConstants c, const float* lr_t,
           const float* c1, const float* c2) {
    if (chunks == 0) return;
    adamw_kernel<<<chunks, 256, 0, s>>>(d_tensors, d_chunk_tensor, d_chunk_start, c, lr_t, c1, c2);
    check_launch("adamw");
}

void working_copy(cudaStream_t s, const float* p, void* p16, uint64_t n) {
    if (n == 0) return;
    const uint64_t blocks = (n + 255) / 256;
    working_copy_kernel<<<static_cast<uint32_t>(blocks > 148 * 8 ? 148 * 8 : blocks), 256, 0, s>>>(p, static_cast<bf16*>(p16), n);
    check_launch("working_copy");
}

void sgd(cudaStream_t s, const UpdateTensor* d_tensors, const uint32_t* d_chunk_tensor,
         const uint32_t* d_chunk_start, uint32_t chunks, const float* lr) {
    if (chunks == 0) return;
    sgd_kernel<<<chunks, 256, 0, s>>>(d_tensors, d_chunk_tensor, d_chunk_start, lr);
    check_launch("sgd");
}

}  // namespace k
}  // namespace msx
