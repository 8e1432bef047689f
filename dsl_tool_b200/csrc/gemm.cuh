// Kernel argument block and host launchers of the tcgen05 GEMM kernels (gemm.cu, gemm_groupwise.cu).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "dslgemm.h"

namespace dsl {

enum { KIND_F8 = 0, KIND_NVF4 = 1, KIND_MXF4 = 2, KIND_BF16 = 3 };

struct GemmArgs {
    int m_total;                 // rows of A / C over all row groups
    int n;                       // columns of C (rows of each group's weight)
    int k_bytes;                 // bytes per operand row: K for FP8, K/2 for FP4, 2K for BF16
    int num_groups;
    const int* group_offsets;    // device int32[num_groups+1] row offsets, or nullptr (one group of m_total rows)
    const uint8_t* sfa;          // tiled block scales of A / B (FP4 kinds)
    const uint8_t* sfb;
    int sf_katoms;               // 512-byte scale tiles along K per 128 rows = ceil(nblk/4)
    int sfb_tiles_per_group;     // ceil(n/128)
    const float* gsa;            // FP8 groupwise: A scales [m_total, K/128]
    const float* gsb;            //                B scales (see sb_block)
    int sb_block;                // 1: [G, ceil(n/128), K/128] block scales, 0: [G, K/128, n] per column
    float s1, s2;                // epilogue scales (host values) ...
    const float* s1_dev;         // ... overridden by these device scalars when non-null
    const float* s2_dev;
    int scale_product;           // 1: multiply by (s1*s2) once; 0: (acc*s1)*s2
    const float* row_scale;
    const float* col_scale;
    void* c;
    long long ldc;
    int out_bf16;
    int band;                    // column tiles per raster band (L2 reuse)
    int whole_tiles_only;        // 1: the tiles after the last full round are not cut into narrow pieces (measurements)
    int split_k;                 // > 1: K is cut into this many slices whose fp32 partial sums go to `partial`
    float* partial;              // [split_k, m_total, n] scratch (dense problems only): the caller's workspace
                                 // after its first DSL_WS_HEADER_BYTES
    size_t partial_bytes;        // capacity of `partial`
    unsigned long long* ws_words;   // the workspace's header: DSL_WS_HEADER_BYTES / 8 arrival words (gemm_decode.cu)
    int b_static;                // B was complete before the preceding kernel of the stream was launched
    int act;                     // DSL_ACT_*: SWIGLU turns column pairs (gate, up) into one output column
    uint8_t* out_sf;             // non-null: the result is quantised to NVFP4 (c = packed bytes, out_sf = scale tiles)
    float out_gs;                // its global scale (host value) ...
    const float* out_gs_dev;     // ... overridden by this device scalar when non-null
    int out_sf_katoms;           // 512-byte scale tiles along the output row = ceil(ceil(Nout/16)/4)
    uint32_t* status;
};

// A caller's workspace starts with a header that only the weight-streaming kernel's arrival words ever
// occupy (one 64-bit word per 128-column tile, tagged with a per-launch epoch); partial sums of every
// kernel start behind it.  Because the words sit at the same place whatever the problem's shape, no
// call can leave floating-point data where a later call looks for its words.
constexpr size_t DSL_WS_HEADER_BYTES = 64 * 1024;

// State that belongs to a device's context (function attributes, occupancy, SM count) is kept per
// device: one process may drive several GPUs.
constexpr int DSL_MAX_DEVICES = 64;
struct PerDeviceInt {
    std::atomic<int> v[DSL_MAX_DEVICES];
};
// Index of the current device, or -1 when it cannot serve as an index of PerDeviceInt.
inline int current_device_slot() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= DSL_MAX_DEVICES) return -1;
    return dev;
}
int sm_count();   // of the current device

constexpr int DSL_DECODE_MAX_ROWS = 128;   // activation rows the weight-streaming kernel (gemm_decode.cu) takes
constexpr int DSL_NOT_SERVED = -1000;      // launch_gemm_decode: problem outside its domain, use the tiled kernels

int launch_gemm_decode(int kind, const void* A, const void* B, const GemmArgs& args, cudaStream_t st);
// Scratch bytes (behind the header) the weight-streaming kernel would use for this problem; 0 when it
// combines inside clusters or does not serve the problem (*served says which).
size_t decode_scratch_bytes(int kind, const GemmArgs& args, bool* served);
size_t gemm_workspace_bytes(int kind, const GemmArgs& args);
int choose_split_k(const GemmArgs& args, long long tiles);
int launch_gemm(int kind, const void* A, const void* B, GemmArgs args, cudaStream_t st);
int launch_gemm_pair(int kind, const void* A, const void* B, GemmArgs args, cudaStream_t st);
int launch_gemm_fp8_groupwise_pair(const void* A, const void* B, GemmArgs args, cudaStream_t st);
int groupwise_pair_schedule_host(const int* group_offsets, int groups, int m_total, int n, int pairs, int band, int whole_tiles_only,
                                 int* out, int max_items);
int launch_gemm_fp8_groupwise(const void* A, const void* B, GemmArgs args, cudaStream_t st);
int launch_bounded_wait_selftest(uint32_t* status, unsigned limit_us, cudaStream_t st);
bool make_tmap_u8(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t box0,
                  uint32_t box1);

}  // namespace dsl
