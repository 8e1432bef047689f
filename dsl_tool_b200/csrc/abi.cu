// extern "C" entry points of libdslgemm: argument validation, then the kernel launchers.
#include <cuda_runtime.h>

#include "dslgemm.h"
#include "gemm.cuh"
#include "quant.cuh"

using namespace dsl;

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

extern "C" {

const char* dsl_version(void) { return "dslgemm 0.1 (sm_100a)"; }

size_t dsl_sf_bytes(long long rows, long long nblk) {
    if (rows <= 0 || nblk <= 0) return 0;
    return static_cast<size_t>((rows + 127) / 128) * static_cast<size_t>((nblk + 3) / 4) * 512;
}

size_t dsl_sf_bytes_grouped(long long rows, long long nblk, int groups) {
    if (rows < 0 || nblk <= 0 || groups < 0) return 0;
    return static_cast<size_t>((rows + 127) / 128 + groups) * static_cast<size_t>((nblk + 3) / 4) * 512;
}

int dsl_quant_fp8(const void* x, int dtype, long long rows, long long cols, int mode, float* scale_io,
                  int scale_given, uint8_t* q_out, void* ws, void* stream) {
    if (x == nullptr || scale_io == nullptr || q_out == nullptr) return DSL_ERR_NULL;
    if (dtype < DSL_F32 || dtype > DSL_F16) return DSL_ERR_ENUM;
    if (mode < DSL_FP8_PER_TENSOR || mode > DSL_FP8_BLOCK_128X128) return DSL_ERR_ENUM;
    if (rows < 0 || cols < 0 || rows > (1ll << 31) || cols > (1ll << 31)) return DSL_ERR_SHAPE;
    if (mode != DSL_FP8_PER_TENSOR && cols % 16 != 0) return DSL_ERR_SHAPE;
    if (mode == DSL_FP8_PER_TENSOR && !scale_given && ws == nullptr) return DSL_ERR_NULL;
    if (!aligned16(x) || !aligned16(q_out)) return DSL_ERR_ALIGN;
    if (rows == 0 || cols == 0) return 0;
    return static_cast<int>(launch_quant_fp8(x, dtype, rows, cols, mode, scale_io, scale_given, q_out,
                                             static_cast<uint32_t*>(ws), as_stream(stream)));
}

int dsl_quant_fp4(const void* x, int dtype, long long rows, long long cols, int format, float* gs_io,
                  int gs_given, uint8_t* q_out, uint8_t* sf_out, const int* group_offsets, int groups,
                  void* ws, void* stream) {
    if (x == nullptr || q_out == nullptr || sf_out == nullptr) return DSL_ERR_NULL;
    if (dtype < DSL_F32 || dtype > DSL_F16) return DSL_ERR_ENUM;
    if (format != DSL_FP4_NV && format != DSL_FP4_MX) return DSL_ERR_ENUM;
    if (format == DSL_FP4_NV && gs_io == nullptr) return DSL_ERR_NULL;
    if (format == DSL_FP4_NV && !gs_given && ws == nullptr) return DSL_ERR_NULL;
    if (rows < 0 || cols < 0 || rows > (1ll << 31) || cols > (1ll << 31) || cols % 32 != 0) return DSL_ERR_SHAPE;
    if (group_offsets != nullptr && (groups < 1 || groups > DSL_MAX_GROUPS)) return DSL_ERR_TOO_LARGE;
    if (!aligned16(x) || !aligned16(q_out) || !aligned16(sf_out)) return DSL_ERR_ALIGN;
    if (rows == 0 || cols == 0) return 0;
    const long long nblk = format == DSL_FP4_NV ? cols / 16 : cols / 32;
    size_t sf_bytes;
    int clear;
    if (group_offsets != nullptr) {
        sf_bytes = dsl_sf_bytes_grouped(rows, nblk, groups);
        clear = 1;
    } else {
        sf_bytes = dsl_sf_bytes(rows, nblk);
        clear = (rows % 128 != 0 || nblk % 4 != 0) ? 1 : 0;   // padding bytes must read as zero
    }
    return static_cast<int>(launch_quant_fp4(x, dtype, rows, cols, format, gs_io, gs_given, q_out, sf_out, sf_bytes,
                                             clear, group_offsets, groups, static_cast<uint32_t*>(ws),
                                             as_stream(stream)));
}

int dsl_quant_fp4_per_token(const void* x, int dtype, long long rows, long long cols, float* gs_out, uint8_t* q_out,
                            uint8_t* sf_out, const int* group_offsets, int groups, void* stream) {
    if (x == nullptr || q_out == nullptr || sf_out == nullptr || gs_out == nullptr) return DSL_ERR_NULL;
    if (dtype < DSL_F32 || dtype > DSL_F16) return DSL_ERR_ENUM;
    if (rows < 0 || cols < 0 || rows > (1ll << 31) || cols % 32 != 0) return DSL_ERR_SHAPE;
    if (cols > DSL_PER_TOKEN_MAX_COLS) return DSL_ERR_TOO_LARGE;      // a row is held in one CTA's registers
    if (group_offsets != nullptr && (groups < 1 || groups > DSL_MAX_GROUPS)) return DSL_ERR_TOO_LARGE;
    if (!aligned16(x) || !aligned16(q_out) || !aligned16(sf_out)) return DSL_ERR_ALIGN;
    if (rows == 0 || cols == 0) return 0;
    const long long nblk = cols / 16;
    size_t sf_bytes;
    int clear;
    if (group_offsets != nullptr) {
        sf_bytes = dsl_sf_bytes_grouped(rows, nblk, groups);
        clear = 1;
    } else {
        sf_bytes = dsl_sf_bytes(rows, nblk);
        clear = (rows % 128 != 0 || nblk % 4 != 0) ? 1 : 0;
    }
    return static_cast<int>(launch_quant_nvfp4_per_token(x, dtype, rows, cols, gs_out, q_out, sf_out, sf_bytes, clear, group_offsets,
                                                         groups, as_stream(stream)));
}

int dsl_transpose_u8(const uint8_t* in, uint8_t* out, int R, int C, void* stream) {
    if (in == nullptr || out == nullptr) return DSL_ERR_NULL;
    if (R < 0 || C < 0) return DSL_ERR_SHAPE;
    if (R == 0 || C == 0) return 0;
    return static_cast<int>(launch_transpose_u8(in, out, R, C, as_stream(stream)));
}

static int fill_common(GemmArgs& a, const void* A, const void* B, void* C, long long ldc, long long M_total, int N,
                       long long k_bytes, const int* group_offsets, int groups, const dsl_epilogue* ep,
                       uint32_t* status) {
    if (A == nullptr || B == nullptr || C == nullptr || ep == nullptr) return DSL_ERR_NULL;
    if (ep->activation != DSL_ACT_NONE && ep->activation != DSL_ACT_SWIGLU && ep->activation != DSL_ACT_GEGLU) return DSL_ERR_ENUM;
    const bool glu = ep->activation != DSL_ACT_NONE;
    if (glu && N % 2 != 0) return DSL_ERR_SHAPE;
    if (M_total < 0 || N < 0 || k_bytes <= 0 || M_total > 0x7FFFFFFFll || ldc < (glu ? N / 2 : N)) return DSL_ERR_SHAPE;
    if (k_bytes % 16 != 0) return DSL_ERR_SHAPE;
    if (group_offsets != nullptr && (groups < 1 || groups > DSL_MAX_GROUPS)) return DSL_ERR_TOO_LARGE;
    if (ep->out_dtype != DSL_F32 && ep->out_dtype != DSL_BF16 && ep->out_dtype != DSL_OUT_NVFP4) return DSL_ERR_ENUM;
    const int n_out = glu ? N / 2 : N;
    if (ep->out_dtype == DSL_OUT_NVFP4) {
        if (ep->out_sf == nullptr) return DSL_ERR_NULL;
        if (n_out % 16 != 0 || ldc % 16 != 0) return DSL_ERR_SHAPE;
        if (!aligned16(ep->out_sf)) return DSL_ERR_ALIGN;
        if (ep->out_gs_dev == nullptr && !(ep->out_gs_host > 0.f)) return DSL_ERR_SHAPE;
    }
    if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return DSL_ERR_ALIGN;
    a = GemmArgs{};
    a.m_total = static_cast<int>(M_total);
    a.n = N;
    a.k_bytes = static_cast<int>(k_bytes);
    a.num_groups = group_offsets != nullptr ? groups : 1;
    a.group_offsets = group_offsets;
    a.s1 = ep->scale_a_host;
    a.s2 = ep->scale_b_host;
    a.s1_dev = ep->scale_a_dev;
    a.s2_dev = ep->scale_b_dev;
    a.row_scale = ep->row_scale;
    a.col_scale = ep->col_scale;
    a.c = C;
    a.ldc = ldc;
    a.out_bf16 = ep->out_dtype == DSL_BF16;
    a.status = status;
    a.b_static = ep->b_is_static != 0;
    a.act = ep->activation;
    if (ep->out_dtype == DSL_OUT_NVFP4) {
        a.out_sf = static_cast<uint8_t*>(ep->out_sf);
        a.out_gs = ep->out_gs_host;
        a.out_gs_dev = ep->out_gs_dev;
        a.out_sf_katoms = (n_out / 16 + 3) / 4;
    }
    if (ep->workspace != nullptr && aligned16(ep->workspace) && ep->workspace_bytes > DSL_WS_HEADER_BYTES) {
        // header: arrival words of the weight-streaming kernel; behind it: fp32 partial sums
        a.ws_words = static_cast<unsigned long long*>(ep->workspace);
        a.partial = reinterpret_cast<float*>(static_cast<uint8_t*>(ep->workspace) + DSL_WS_HEADER_BYTES);
        a.partial_bytes = ep->workspace_bytes - DSL_WS_HEADER_BYTES;
    }
    return 0;
}

int dsl_gemm_fp8(const uint8_t* A, const uint8_t* B, void* C, long long ldc, long long M_total, int N, int K,
                 const int* group_offsets, int groups, const dsl_epilogue* ep, uint32_t* status, void* stream) {
    GemmArgs a;
    int rc = fill_common(a, A, B, C, ldc, M_total, N, K, group_offsets, groups, ep, status);
    if (rc != 0) return rc;
    a.scale_product = 0;   // (acc * scale_a) * scale_b, as the registered reference kernel does
    return launch_gemm(KIND_F8, A, B, a, as_stream(stream));
}

int dsl_gemm_bf16(const void* A, const void* B, void* C, long long ldc, long long M_total, int N, int K,
                  const int* group_offsets, int groups, const dsl_epilogue* ep, uint32_t* status, void* stream) {
    GemmArgs a;
    if (K <= 0 || K % 8 != 0) return DSL_ERR_SHAPE;
    int rc = fill_common(a, A, B, C, ldc, M_total, N, 2ll * K, group_offsets, groups, ep, status);
    if (rc != 0) return rc;
    a.scale_product = 0;
    return launch_gemm(KIND_BF16, A, B, a, as_stream(stream));
}

int dsl_gemm_fp8_groupwise(const uint8_t* A, const uint8_t* B, const float* sa, const float* sb, int sb_block,
                           void* C, long long ldc, long long M_total, int N, int K, const int* group_offsets,
                           int groups, const dsl_epilogue* ep, uint32_t* status, void* stream) {
    GemmArgs a;
    if (sa == nullptr || sb == nullptr) return DSL_ERR_NULL;
    if (K % 128 != 0) return DSL_ERR_SHAPE;
    int rc = fill_common(a, A, B, C, ldc, M_total, N, K, group_offsets, groups, ep, status);
    if (rc != 0) return rc;
    if (a.out_sf != nullptr) return DSL_ERR_ENUM;    // quantised output: not in the group-scaled kernels
    a.gsa = sa;
    a.gsb = sb;
    a.sb_block = sb_block != 0;
    a.scale_product = 0;
    return launch_gemm_fp8_groupwise(A, B, a, as_stream(stream));
}

int dsl_gemm_fp4(const uint8_t* A, const uint8_t* B, const uint8_t* sfa, const uint8_t* sfb, int format, void* C,
                 long long ldc, long long M_total, int N, int K, const int* group_offsets, int groups,
                 const dsl_epilogue* ep, uint32_t* status, void* stream) {
    GemmArgs a;
    if (sfa == nullptr || sfb == nullptr) return DSL_ERR_NULL;
    if (format != DSL_FP4_NV && format != DSL_FP4_MX) return DSL_ERR_ENUM;
    if (K <= 0 || K % 32 != 0) return DSL_ERR_SHAPE;
    if (!aligned16(sfa) || !aligned16(sfb)) return DSL_ERR_ALIGN;
    int rc = fill_common(a, A, B, C, ldc, M_total, N, K / 2, group_offsets, groups, ep, status);
    if (rc != 0) return rc;
    const int nblk = format == DSL_FP4_NV ? K / 16 : K / 32;
    a.sfa = sfa;
    a.sfb = sfb;
    a.sf_katoms = (nblk + 3) / 4;
    a.sfb_tiles_per_group = (N + 127) / 128;
    a.scale_product = 1;   // the two global scales multiply the accumulator once, as one factor
    return launch_gemm(format == DSL_FP4_NV ? KIND_NVF4 : KIND_MXF4, A, B, a, as_stream(stream));
}

size_t dsl_workspace_bytes(int op, long long M, int N, int K, int groups) {
    if (M <= 0 || N <= 0 || K <= 0 || M > 0x7FFFFFFFll) return 0;
    if (groups > 1) return 0;                         // row groups: no kernel uses scratch
    long long k_bytes;
    int kind;
    switch (op) {
        case DSL_OP_GEMM_FP8: kind = KIND_F8; k_bytes = K; break;
        case DSL_OP_GEMM_BF16: kind = KIND_BF16; k_bytes = 2ll * K; break;
        case DSL_OP_GEMM_FP4_NV: kind = KIND_NVF4; k_bytes = K / 2; break;
        case DSL_OP_GEMM_FP4_MX: kind = KIND_MXF4; k_bytes = K / 2; break;
        default: return 0;                            // the group-scaled FP8 GEMM and the quantisers use none
    }
    if (k_bytes <= 0 || k_bytes > 0x7FFFFFFFll) return 0;
    GemmArgs a{};
    a.m_total = static_cast<int>(M);
    a.n = N;
    a.k_bytes = static_cast<int>(k_bytes);
    a.num_groups = 1;
    a.partial = reinterpret_cast<float*>(uintptr_t(16));   // "a workspace is there": never dereferenced
    a.partial_bytes = ~size_t(0) >> 2;
    return gemm_workspace_bytes(kind, a);
}

int dsl_selftest_bounded_wait(uint32_t* status, unsigned limit_us, void* stream) {
    if (status == nullptr) return DSL_ERR_NULL;
    return launch_bounded_wait_selftest(status, limit_us, as_stream(stream));
}

int dsl_selftest_groupwise_schedule(const int32_t* group_offsets, int num_groups, long long m_total, int N, int pairs,
                                    int band, int whole_tiles_only, int32_t* out, int max_items) {
    if (out == nullptr) return DSL_ERR_NULL;
    if (m_total < 0 || m_total > 0x7FFFFFFF || N <= 0 || pairs <= 0 || max_items < 0) return DSL_ERR_SHAPE;
    // malformed offsets (out of range, decreasing) are let through on purpose: the kernel cannot refuse
    // what it reads from device memory, it sanitises it, and this is the way to see what it then does
    if (group_offsets != nullptr && (num_groups < 1 || num_groups > DSL_MAX_GROUPS)) return DSL_ERR_SHAPE;
    const long long tiles = ((m_total + 255) / 256 + (group_offsets != nullptr ? num_groups : 0)) * ((N + 255LL) / 256);
    if (tiles > (1ll << 29)) return DSL_ERR_SHAPE;
    const int n = groupwise_pair_schedule_host(group_offsets, num_groups, static_cast<int>(m_total), N, pairs, band,
                                               whole_tiles_only, out, max_items);
    return n < 0 ? DSL_ERR_TOO_LARGE : n;
}

}  // extern "C"
