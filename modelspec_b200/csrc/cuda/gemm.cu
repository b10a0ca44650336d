// matmul, f32, exact class: C[i, j] is one fused-multiply-add chain over ascending k that starts
// from the rounded first product, the element the reference's CPU loop computes
// (crates/modelspec-runtime/src/cpu/matmul.rs:268-292) and its GPU kernels chain with Fma
// (crates/modelspec-core/src/ir/kernel.rs:228-322). The accumulator starts at -0.0, so the first
// fmaf(a, b, -0.0) is the rounded product a * b, sign of zero included.
//
// 64 x 64 output tile per CTA, 16-deep k slices staged in shared memory, 4 x 4 outputs per
// thread. Either operand may be read as the transpose of its stored matrix, which is how the
// backward products G x W^T and X^T x G arrive (the reference folds the Transpose node into the
// matmul the same way, crates/modelspec-core/src/schedule.rs:526-551).
#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {

namespace {

constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

template <bool A_T, bool B_T>
__global__ void __launch_bounds__(256) matmul_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                     float* __restrict__ c, uint32_t m, uint32_t n, uint32_t k,
                                                     const float* __restrict__ bias) {
    __shared__ float as[BK][BM + 4];
    __shared__ float bs[BK][BN + 4];
    const uint32_t tid = threadIdx.x;
    const uint32_t tx = tid % 16, ty = tid / 16;
    const uint32_t m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = -0.0f;

    for (uint32_t k0 = 0; k0 < k; k0 += BK) {
        // Stage the A slice: element (mm, kk) of the tile.
#pragma unroll
        for (int e = 0; e < (BM * BK) / 256; ++e) {
            uint32_t idx = tid + e * 256;
            uint32_t mm, kk;
            if (A_T) { mm = idx % BM; kk = idx / BM; }   // stored [k, m]: m runs fastest
            else     { kk = idx % BK; mm = idx / BK; }   // stored [m, k]: k runs fastest
            uint32_t gm = m0 + mm, gk = k0 + kk;
            float v = 0.0f;
            if (gm < m && gk < k) v = A_T ? a[static_cast<uint64_t>(gk) * m + gm] : a[static_cast<uint64_t>(gm) * k + gk];
            as[kk][mm] = v;
        }
#pragma unroll
        for (int e = 0; e < (BN * BK) / 256; ++e) {
            uint32_t idx = tid + e * 256;
            uint32_t nn, kk;
            if (B_T) { kk = idx % BK; nn = idx / BK; }   // stored [n, k]: k runs fastest
            else     { nn = idx % BN; kk = idx / BN; }   // stored [k, n]: n runs fastest
            uint32_t gn = n0 + nn, gk = k0 + kk;
            float v = 0.0f;
            if (gn < n && gk < k) v = B_T ? b[static_cast<uint64_t>(gn) * k + gk] : b[static_cast<uint64_t>(gk) * n + gn];
            bs[kk][nn] = v;
        }
        __syncthreads();
        const uint32_t depth = min(static_cast<uint32_t>(BK), k - k0);
        if (depth == BK) {
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                float ar[TM], br[TN];
#pragma unroll
                for (int i = 0; i < TM; ++i) ar[i] = as[kk][ty * TM + i];
#pragma unroll
                for (int j = 0; j < TN; ++j) br[j] = bs[kk][tx * TN + j];
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(ar[i], br[j], acc[i][j]);
            }
        } else {
            // The last, short slice: stop at k so no padded product joins the chain.
            for (uint32_t kk = 0; kk < depth; ++kk) {
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j)
                        acc[i][j] = fmaf(as[kk][ty * TM + i], bs[kk][tx * TN + j], acc[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        uint32_t gm = m0 + ty * TM + i;
        if (gm >= m) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            uint32_t gn = n0 + tx * TN + j;
            // k = 0 leaves the -0.0 start; the reference writes +0 then.
            if (gn < n) {
                float value = k == 0 ? 0.0f : acc[i][j];
                c[static_cast<uint64_t>(gm) * n + gn] = bias ? value + bias[gn] : value;
            }
        }
    }
}

}  // namespace

void matmul(cudaStream_t s, const float* a, bool a_t, const float* b, bool b_t, float* c,
            uint64_t m, uint64_t n, uint64_t k, const float* bias) {
    if (m == 0 || n == 0) return;
    dim3 grid(static_cast<uint32_t>((n + BN - 1) / BN), static_cast<uint32_t>((m + BM - 1) / BM));
    uint32_t mm = static_cast<uint32_t>(m), nn = static_cast<uint32_t>(n), kk = static_cast<uint32_t>(k);
    if (a_t && b_t) matmul_kernel<true, true><<<grid, 256, 0, s>>>(a, b, c, mm, nn, kk, bias);
    else if (a_t) matmul_kernel<true, false><<<grid, 256, 0, s>>>(a, b, c, mm, nn, kk, bias);
    else if (b_t) matmul_kernel<false, true><<<grid, 256, 0, s>>>(a, b, c, mm, nn, kk, bias);
    else matmul_kernel<false, false><<<grid, 256, 0, s>>>(a, b, c, mm, nn, kk, bias);
    check_launch("matmul");
}

}  // namespace k
}  // namespace msx
