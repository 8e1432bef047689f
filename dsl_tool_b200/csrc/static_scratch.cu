// A block-scaled FP4 GEMM entry point for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand the GEMM a scratch buffer: code running
// inside a stream capture or another framework's memory-planned region, plugins whose host
// interface only passes inputs and outputs, and processes that must not touch cudaMalloc
// after start-up.  For decode-sized problems (few activation rows, long K) the GEMM wants
// scratch for its split-K partial sums; here that scratch is a fixed array in the library's
// own device image, so the call needs nothing but its inputs and outputs.
#include <cuda_runtime.h>

#include <mutex>

#include "dslgemm.h"

// Held by every GPU that loads the library, until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[DSL_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
void* g_scratch_addr[kMaxDevices] = {};
std::mutex g_scratch_mutex;

// The array's name is only a host-side handle; the device address has to be asked for, once
// per device, with that device current.
cudaError_t scratch_address(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (g_scratch_addr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess) return e;
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return cudaSuccess;
}
}  // namespace

extern "C" int dsl_gemm_fp4_static_scratch(const uint8_t* A, const uint8_t* B, const uint8_t* sfa, const uint8_t* sfb,
                                           int format, void* C, long long ldc, long long M, int N, int K,
                                           const dsl_epilogue* ep, uint32_t* status, void* stream) {
    if (ep == nullptr) return DSL_ERR_NULL;
    if (M < 0 || N < 0) return DSL_ERR_SHAPE;
    // two K-slices of fp32 partial sums must fit, otherwise the scratch would be of no use
    if (static_cast<unsigned long long>(M) * static_cast<unsigned long long>(N) * sizeof(float) * 2ull >
        static_cast<unsigned long long>(DSL_STATIC_SCRATCH_BYTES))
        return DSL_ERR_TOO_LARGE;
    void* scratch = nullptr;
    cudaError_t e = scratch_address(&scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    dsl_epilogue local = *ep;
    local.workspace = scratch;
    local.workspace_bytes = DSL_STATIC_SCRATCH_BYTES;
    return dsl_gemm_fp4(A, B, sfa, sfb, format, C, ldc, M, N, K, nullptr, 1, &local, status, stream);
}
