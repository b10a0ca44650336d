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
    for (uint64_t i = start + threadIdx.x; i < stop; i += blockDim.x) {
        float g = t.g[i], p = t.p[i], m = t.m[i], v = t.v[i];
        float m_next = c.beta1 * m + c.rest1 * g;
        float v_next = c.beta2 * v + (c.rest2 * g) * g;
        float direction = (m_next * k1) / (sqrtf(v_next * k2) + c.eps);
        float step = direction + c.weight_decay * p;
        t.p[i] = p - lr * step;
        t.m[i] = m_next;
        t.v[i] = v_next;
    }
}

__global__ void __launch_bounds__(256) sgd_kernel(const UpdateTensor* __restrict__ tensors,
                                                   const uint32_t* __restrict__ chunk_tensor,
                                                   const uint32_t* __restrict__ chunk_start,
                                                   const float* __restrict__ lr) {
    UpdateTensor t = tensors[chunk_tensor[blockIdx.x]];
    uint64_t start = static_cast<uint64_t>(chunk_start[blockIdx.x]) * kUpdateChunk;
    uint64_t stop = start + kUpdateChunk < t.count ? start + kUpdateChunk : t.count;
    float rate = lr[0];
    for (uint64_t i = start + threadIdx.x; i < stop; i += blockDim.x) t.p[i] = t.p[i] - rate * t.g[i];
}

}  // namespace

void adamw(cudaStream_t s, const UpdateTensor* d_tensors, const uint32_t* d_chunk_tensor,
           const uint32_t* d_chunk_start, uint32_t chunks, AdamWConstants c, const float* lr_t,
           const float* c1, const float* c2) {
    if (chunks == 0) return;
    adamw_kernel<<<chunks, 256, 0, s>>>(d_tensors, d_chunk_tensor, d_chunk_start, c, lr_t, c1, c2);
    check_launch("adamw");
}

void sgd(cudaStream_t s, const UpdateTensor* d_tensors, const uint32_t* d_chunk_tensor,
         const uint32_t* d_chunk_start, uint32_t chunks, const float* lr) {
    if (chunks == 0) return;
    sgd_kernel<<<chunks, 256, 0, s>>>(d_tensors, d_chunk_tensor, d_chunk_start, lr);
    check_launch("sgd");
}

}  // namespace k
}  // namespace msx
