// msx_sum_rows_static: column sums of a row-major matrix through a scratch area that is part of
// the library image, for callers that must not allocate device memory.
//
// Some hosts that embed this library run inside a memory budget fixed before they start: a
// process that has handed all device memory to its own pool, a real-time loop that may not
// enter the driver's allocator, or a plug-in whose host forbids cudaMalloc after start-up. The
// plan API allocates its arena when a plan is built, which such hosts cannot do. This entry
// point gives them one reduction (the bias-gradient column sum, `SumRows`) that touches no
// allocator at all: its partial sums live in the file-scope device array below, which every GPU
// that loads the library carries from load to exit (1 MiB).
//
// It runs the two-launch form of the column sum (a first stage that leaves chunk sums, the wide
// one for rows of 1,024 or more columns on 16-byte boundaries, and a second stage that adds the
// chunks in ascending order). A plan runs the same first stage and adds the chunks in the same
// order inside that launch or in its finalize launch, so the results agree bit for bit.
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>
#include <string>

#include "../../../include/msx.h"
#include "kernels.cuh"

namespace {

// Partial column sums: at most 64 row chunks of at most 4096 columns.
constexpr uint64_t kMaxColumns = 4096;
constexpr uint64_t kMaxChunks = 64;
static __device__ __align__(256) float g_partial_sums[kMaxChunks * kMaxColumns];

// The device address of g_partial_sums on each device, looked up once per device. In host code
// the array's name stands for the symbol, not for memory a kernel can use: the address a kernel
// takes comes from cudaGetSymbolAddress with that device current.
constexpr int kMaxDevices = 64;
float* g_partial_address[kMaxDevices] = {};
std::mutex g_setup_lock;
thread_local std::string g_static_error;

int fail(int status, const std::string& what) {
    g_static_error = what;
    return status;
}

}  // namespace

extern "C" {

const char* msx_static_last_error() { return g_static_error.c_str(); }

int msx_sum_rows_static(const float* device_g, uint64_t rows, uint64_t columns, float* device_out, void* stream) {
    if (!device_g || !device_out) return fail(MSX_BAD_ARGUMENT, "msx_sum_rows_static: null matrix or result pointer");
    if (columns == 0 || columns > kMaxColumns)
        return fail(MSX_BAD_ARGUMENT, "msx_sum_rows_static: " + std::to_string(columns) + " columns; the static scratch holds 1 to " +
                                          std::to_string(kMaxColumns));
    if (rows > (1ull << 31)) return fail(MSX_BAD_ARGUMENT, "msx_sum_rows_static: more than 2^31 rows");
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return fail(MSX_NO_DEVICE, std::string("msx_sum_rows_static: cudaGetDevice: ") + cudaGetErrorString(e));
    if (device < 0 || device >= kMaxDevices) return fail(MSX_BAD_ARGUMENT, "msx_sum_rows_static: device ordinal out of range");
    float* partial = nullptr;
    {
        std::lock_guard<std::mutex> hold(g_setup_lock);
        if (!g_partial_address[device]) {
            // First call on this device: resolve the symbol with this device current.
            float* address = nullptr;
            e = cudaGetSymbolAddress(reinterpret_cast<void**>(&address), g_partial_sums);
            if (e != cudaSuccess || !address)
                return fail(MSX_LAUNCH_FAILED, std::string("msx_sum_rows_static: cudaGetSymbolAddress: ") + cudaGetErrorString(e));
            g_partial_address[device] = address;
        }
        partial = g_partial_address[device];
    }
    // Every partial sum a call reads is written by the same call first (stage 1 fills
    // [chunks, columns] before stage 2 reads it), so nothing has to start at zero and what an
    // earlier call left behind is never seen.
    try {
        msx::k::sum_rows(static_cast<cudaStream_t>(stream), device_g, rows, columns, partial, device_out);
    } catch (const std::exception& err) {
        return fail(MSX_LAUNCH_FAILED, err.what());
    }
    return MSX_OK;
}

}  // extern "C"
