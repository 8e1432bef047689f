// A block-scaled FP4 GEMM entry point for callers that cannot allocate device memory.
//
// Some hosts of this library have no way to hand the GEMM a scratch buffer: code running
// inside a stream capture or another framework's memory-planned region, plugins whose host
// interface only passes inputs and outputs, and processes that must not touch cudaMalloc
// after start-up.  For decode-sized problems (few activation rows, long K) the GEMM cuts K
// over the SMs and wants scratch for the partial sums and their arrival words; here that
// scratch is a fixed array in the library's own device image, so the call needs nothing but
// its inputs and outputs.
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
    if (M < 0 || N < 0 || K <= 0) return DSL_ERR_SHAPE;
    if (format != DSL_FP4_NV && format != DSL_FP4_MX) return DSL_ERR_ENUM;
    // what the kernels serving this problem would take from a workspace must fit the array
    if (dsl_workspace_bytes(format == DSL_FP4_NV ? DSL_OP_GEMM_FP4_NV : DSL_OP_GEMM_FP4_MX, M, N, K, 1) >
        static_cast<size_t>(DSL_STATIC_SCRATCH_BYTES))
        return DSL_ERR_TOO_LARGE;
    void* scratch = nullptr;
    cudaError_t e = scratch_address(&scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    dsl_epilogue local = *ep;
    local.workspace = scratch;
    local.workspace_bytes = DSL_STATIC_SCRATCH_BYTES;
    return dsl_gemm_fp4(A, B, sfa, sfb, format, C, ldc, M, N, K, nullptr, 1, &local, status, stream);
}

// Test hook: copies between the static array and a caller's device buffer (to_array != 0: into the
// array), ordered on `stream`, so that a test can fill the array with foreign bytes before a call and
// see afterwards which parts the call wrote.
extern "C" int dsl_selftest_static_scratch_copy(void* user, size_t offset, size_t bytes, int to_array, void* stream) {
    if (user == nullptr) return DSL_ERR_NULL;
    if (offset > DSL_STATIC_SCRATCH_BYTES || bytes > DSL_STATIC_SCRATCH_BYTES - offset) return DSL_ERR_TOO_LARGE;
    void* scratch = nullptr;
    cudaError_t e = scratch_address(&scratch);
    if (e != cudaSuccess) return static_cast<int>(e);
    unsigned char* at = static_cast<unsigned char*>(scratch) + offset;
    e = cudaMemcpyAsync(to_array ? static_cast<void*>(at) : user, to_array ? user : static_cast<void*>(at), bytes,
                        cudaMemcpyDeviceToDevice, reinterpret_cast<cudaStream_t>(stream));
    return static_cast<int>(e);
}
