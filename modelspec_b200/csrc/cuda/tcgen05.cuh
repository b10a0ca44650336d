// The tcgen05 / TMA / mbarrier primitives of the bf16 tensor-core kernels (gemm_bf16.cu,
// attention_fused.cu): inline PTX wrappers, bounded waits, the shared-memory tile layout, and the
// host-side tensor-map encoding. Every tensor map covers this GPU's own memory only and every
// load is a plain one to the issuing CTA.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>

#include <algorithm>
#include <string>

#include "common.cuh"
#include "kernels.cuh"

namespace msx {
namespace k {
namespace tc {

constexpr uint32_t WAIT_LIMIT = 1u << 24;  // try_wait polls before a wait gives up

// Where the row, inner-batch and outer-batch coordinates of an operand sit among the tensor map's
// dimensions 1..3 (dimension 0 is the contiguous one): the dimensions are ordered by stride.
struct CoordOrder {
    uint8_t row, inner, outer, reserved;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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

// One tile of a 4-dimensional tensor map into shared memory; the stage's mbarrier counts the bytes.
__device__ __forceinline__ void tma_load(uint32_t dst, const CUtensorMap* map, uint32_t bar, uint32_t x, const uint32_t (&upper)[3]) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(upper[0]), "r"(upper[1]), "r"(upper[2])
        : "memory");
}

__device__ __forceinline__ void mma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
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


// One box of a 4-dimensional tensor map from shared memory to global memory (what lies outside the
// tensor is not written), as a bulk group of the issuing thread.
__device__ __forceinline__ void tma_store(const CUtensorMap* map, uint32_t src, uint32_t x, const uint32_t (&upper)[3]) {
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(x), "r"(upper[0]), "r"(upper[1]), "r"(upper[2])
                 : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Waits until all but the newest `Pending` store groups of this thread have read their shared memory.
template <int Pending> __device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(Pending) : "memory");
}

// Byte offset of the 16-byte chunk `c16` (8 bf16 elements) of row `row` in a tile of 128-byte rows
// with the 128-byte swizzle TMA writes and tcgen05 reads: 8-row groups of 1024 bytes, the chunk
// index xor-ed with the row within its group.
__device__ __forceinline__ uint32_t swizzled_chunk(uint32_t row, uint32_t c16) {
    return (row >> 3) * 1024u + (row & 7u) * 128u + ((c16 ^ (row & 7u)) << 4);
}

// The shared-memory matrix descriptor (sm_100 form: bit 46 set, 128-byte swizzle = 2 in bits
// 61-63; offsets in 16-byte units) of a tile at shared address `addr`: 8-row groups 1024 bytes
// apart (stride offset); `leading` is the distance between 64-element panels of an MN-major
// operand (unused for a K-major one).
__device__ __forceinline__ uint64_t tile_descriptor(uint32_t addr, uint32_t leading) {
    const uint32_t high = ((1024u >> 4) & 0x3FFFu) | (1u << 14) | (2u << 29);
    const uint32_t low = (((leading >> 4) & 0x3FFFu) << 16) | ((addr & 0x3FFFFu) >> 4);
    return (static_cast<uint64_t>(high) << 32) | low;
}
// Instruction descriptor of tcgen05.mma kind::f16 with bf16 operands and an f32 accumulator:
// bits 4-5 = 1 (f32), 7-9 and 10-12 = 1 (bf16), 15 / 16 = 1 for an MN-major A / B, N >> 3 at 17,
// M >> 4 at 24.
__device__ __forceinline__ uint32_t instruction_descriptor(uint32_t m, uint32_t n, bool a_mn, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point query: the library does not
// link the driver.
using EncodeTiled = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                 const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult found;
        check(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &found), "cudaGetDriverEntryPoint");
        if (found != cudaDriverEntryPointSuccess || p == nullptr) throw std::runtime_error("the driver has no cuTensorMapEncodeTiled");
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

// The tensor map of one operand as stored: `cols` contiguous elements per row, `rows` rows `pitch`
// elements apart, `inner` x `outer` such matrices. `box_rows` rows of 64 elements make one load.
// The three upper dimensions are listed by ascending stride; `order` says where each went.
// `float_elements`: the matrix holds f32 (a result tile written by a TMA store: 32 elements, 128
// bytes, a box row) instead of bf16 (64 elements a box row).
inline bool tma_addressable(const HalfMatrix& x, bool float_elements = false) {
    const uint64_t unit = float_elements ? 4 : 8;  // elements in 16 bytes
    return reinterpret_cast<uintptr_t>(x.base) % 16 == 0 && x.pitch % unit == 0 && x.stride_inner % unit == 0 && x.stride_outer % unit == 0;
}
inline CUtensorMap encode(const HalfMatrix& x, uint64_t cols, uint64_t rows, uint32_t inner, uint32_t outer, uint32_t box_rows, CoordOrder* order,
                   const char* what, bool float_elements = false) {
    if (!tma_addressable(x, float_elements))
        throw std::invalid_argument(std::string("matmul_bf16: operand ") + what +
                                    " is not a TMA source (base on 16 bytes, pitch and batch strides multiples of 16 bytes)");
    const uint64_t esize = float_elements ? 4 : 2;
    struct Dim { uint64_t size, stride; int which; };  // which: 0 row, 1 inner, 2 outer
    const uint64_t whole = static_cast<uint64_t>(x.pitch) * rows;
    Dim dims[3] = {{rows, x.pitch, 0}, {inner, inner > 1 ? x.stride_inner : 0, 1}, {outer, outer > 1 ? x.stride_outer : 0, 2}};
    // A dimension of one element may carry any stride: give it one above every real stride.
    uint64_t top = whole;
    for (const Dim& d : dims) top = std::max(top, d.size * d.stride);
    for (Dim& d : dims)
        if (d.size <= 1 && d.which != 0) d.stride = top;
    std::stable_sort(dims, dims + 3, [](const Dim& l, const Dim& r) { return l.stride < r.stride; });
    cuuint64_t gdim[4] = {cols, dims[0].size, dims[1].size, dims[2].size};
    cuuint64_t gstride[3] = {dims[0].stride * esize, dims[1].stride * esize, dims[2].stride * esize};
    cuuint32_t box[4] = {float_elements ? 32u : 64u, 1, 1, 1}, estride[4] = {1, 1, 1, 1};
    for (int d = 0; d < 3; ++d) {
        if (dims[d].which == 0) { order->row = static_cast<uint8_t>(d); box[d + 1] = box_rows; }
        if (dims[d].which == 1) order->inner = static_cast<uint8_t>(d);
        if (dims[d].which == 2) order->outer = static_cast<uint8_t>(d);
    }
    CUtensorMap map;
    CUresult r = encode_tiled()(&map, float_elements ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                                const_cast<void*>(x.base), gdim, gstride, box, estride,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::invalid_argument(std::string("matmul_bf16: cuTensorMapEncodeTiled refused operand ") + what + " (" + std::to_string(static_cast<int>(r)) + ")");
    return map;
}


}  // namespace tc
}  // namespace k
}  // namespace msx
