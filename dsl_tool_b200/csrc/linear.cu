// dsl_linear: activation quantise + GEMM against a packed weight in ONE call of the C ABI.
//
// The two launches of a step (quantise / scale-pack the activations, multiply) used to be two
// calls from the host language with the quantised activations allocated in between; for decode
// shapes and for column shards of a large GEMM the host time of that pair exceeded the kernels'.
// Here the caller hands over one scratch area for the quantised activations (it is consumed by
// the GEMM of the same call, so a caller that issues its calls on one stream can reuse the area
// call after call) and both launches go out back to back, which is also what lets the GEMM's
// programmatic dependent launch overlap its set-up with the quantiser.
#include <cuda_runtime.h>

#include "dslgemm.h"

namespace {
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Carve {
    size_t q_bytes, scale_bytes, total;
    size_t off_scale, off_gs, off_ws, off_rows;
};

// Layout of the activation scratch: quantised bytes | scales | global / tensor scale (4 B) | amax cell (16 B) |
// per-token global scales (NVFP4 only)
bool carve(int format, long long M, int K, int groups, Carve* c) {
    if (M < 0 || K <= 0) return false;
    const size_t m = static_cast<size_t>(M);
    switch (format) {
        case DSL_W_FP8: c->q_bytes = m * K; c->scale_bytes = 0; break;
        case DSL_W_FP8_BLOCK128: c->q_bytes = m * K; c->scale_bytes = m * ((K + 127) / 128) * sizeof(float); break;
        case DSL_W_NVFP4:
            c->q_bytes = m * (K / 2);
            c->scale_bytes = groups > 1 ? dsl_sf_bytes_grouped(M, K / 16, groups) : dsl_sf_bytes(M, K / 16);
            break;
        case DSL_W_MXFP4:
            c->q_bytes = m * (K / 2);
            c->scale_bytes = groups > 1 ? dsl_sf_bytes_grouped(M, K / 32, groups) : dsl_sf_bytes(M, K / 32);
            break;
        case DSL_W_BF16: c->q_bytes = 0; c->scale_bytes = 0; break;
        default: return false;
    }
    c->off_scale = align_up(c->q_bytes, 256);
    c->off_gs = c->off_scale + align_up(c->scale_bytes, 256);
    c->off_ws = c->off_gs + 256;
    c->off_rows = c->off_ws + 256;                       // per-token global scales (NVFP4, act_scale_per_token)
    c->total = c->off_rows + (format == DSL_W_NVFP4 ? align_up(m * sizeof(float), 256) : 0);
    return true;
}
}  // namespace

extern "C" size_t dsl_linear_scratch_bytes(int format, long long M, int K, int groups) {
    Carve c;
    if (!carve(format, M, K, groups, &c)) return 0;
    return format == DSL_W_BF16 ? 0 : c.total;
}

extern "C" int dsl_linear(const void* x, int x_dtype, long long M, const dsl_weight* w, const int* group_offsets,
                          void* act_scratch, size_t act_scratch_bytes, void* C, long long ldc, const dsl_epilogue* ep,
                          uint32_t* status, void* stream) {
    if (x == nullptr || w == nullptr || C == nullptr || ep == nullptr || w->q == nullptr) return DSL_ERR_NULL;
    if (w->groups < 1 || w->n <= 0 || w->k <= 0) return DSL_ERR_SHAPE;
    if (w->groups > 1 && group_offsets == nullptr) return DSL_ERR_NULL;
    const int* offs = w->groups > 1 ? group_offsets : nullptr;
    dsl_epilogue e = *ep;
    e.b_is_static = 1;                      // a packed weight is complete long before this call
    if (w->format == DSL_W_BF16) {
        if (x_dtype != DSL_BF16) return DSL_ERR_ENUM;
        return dsl_gemm_bf16(x, w->q, C, ldc, M, w->n, w->k, offs, w->groups, &e, status, stream);
    }
    Carve c;
    if (!carve(w->format, M, w->k, w->groups, &c)) return DSL_ERR_ENUM;
    if (M == 0) return 0;
    if (act_scratch == nullptr) return DSL_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(act_scratch) & 255u) != 0) return DSL_ERR_ALIGN;
    if (act_scratch_bytes < c.total) return DSL_ERR_TOO_LARGE;
    uint8_t* base = static_cast<uint8_t*>(act_scratch);
    uint8_t* qa = base;
    void* scales = base + c.off_scale;
    float* gs = reinterpret_cast<float*>(base + c.off_gs);
    void* ws = base + c.off_ws;
    int rc;
    switch (w->format) {
        case DSL_W_FP8:
            if (w->scale == nullptr) return DSL_ERR_NULL;
            rc = dsl_quant_fp8(x, x_dtype, M, w->k, DSL_FP8_PER_TENSOR, gs, 0, qa, ws, stream);
            if (rc != 0) return rc;
            e.scale_a_dev = gs;
            e.scale_b_dev = static_cast<const float*>(w->scale);
            return dsl_gemm_fp8(qa, static_cast<const uint8_t*>(w->q), C, ldc, M, w->n, w->k, offs, w->groups, &e, status, stream);
        case DSL_W_FP8_BLOCK128:
            if (w->scale == nullptr) return DSL_ERR_NULL;
            rc = dsl_quant_fp8(x, x_dtype, M, w->k, DSL_FP8_GROUP_1X128, static_cast<float*>(scales), 0, qa, ws, stream);
            if (rc != 0) return rc;
            return dsl_gemm_fp8_groupwise(qa, static_cast<const uint8_t*>(w->q), static_cast<const float*>(scales),
                                          static_cast<const float*>(w->scale), 1, C, ldc, M, w->n, w->k, offs, w->groups, &e,
                                          status, stream);
        case DSL_W_NVFP4:
        case DSL_W_MXFP4: {
            if (w->scale == nullptr) return DSL_ERR_NULL;
            const int fmt = w->format == DSL_W_NVFP4 ? DSL_FP4_NV : DSL_FP4_MX;
            if (fmt == DSL_FP4_NV && w->global_scale == nullptr) return DSL_ERR_NULL;
            // NVFP4: a global scale handed in through ep->scale_a_dev (calibrated, or known from the producer of x)
            // is used as it is, which makes the quantiser ONE pass over x; otherwise it comes from an amax pass
            if (ep->act_scale_per_token) {
                if (fmt != DSL_FP4_NV) return DSL_ERR_ENUM;
                if (ep->row_scale != nullptr) return DSL_ERR_ENUM;      // the per-token factor occupies that slot
                float* gs_rows = reinterpret_cast<float*>(base + c.off_rows);
                rc = dsl_quant_fp4_per_token(x, x_dtype, M, w->k, gs_rows, qa, static_cast<uint8_t*>(scales), offs, w->groups, stream);
                if (rc != 0) return rc;
                e.scale_a_dev = nullptr;
                e.scale_a_host = 1.0f;
                e.scale_b_dev = w->global_scale;
                e.row_scale = gs_rows;
                return dsl_gemm_fp4(qa, static_cast<const uint8_t*>(w->q), static_cast<const uint8_t*>(scales),
                                    static_cast<const uint8_t*>(w->scale), fmt, C, ldc, M, w->n, w->k, offs, w->groups, &e, status,
                                    stream);
            }
            const bool gs_given = fmt == DSL_FP4_NV && ep->scale_a_dev != nullptr;
            float* gs_io = gs_given ? const_cast<float*>(ep->scale_a_dev) : gs;
            rc = dsl_quant_fp4(x, x_dtype, M, w->k, fmt, gs_io, gs_given ? 1 : 0, qa, static_cast<uint8_t*>(scales), offs, w->groups,
                               ws, stream);
            if (rc != 0) return rc;
            if (fmt == DSL_FP4_NV) {
                e.scale_a_dev = gs_io;
                e.scale_b_dev = w->global_scale;
            } else {
                e.scale_a_dev = e.scale_b_dev = nullptr;
                e.scale_a_host = e.scale_b_host = 1.0f;
            }
            return dsl_gemm_fp4(qa, static_cast<const uint8_t*>(w->q), static_cast<const uint8_t*>(scales),
                                static_cast<const uint8_t*>(w->scale), fmt, C, ldc, M, w->n, w->k, offs, w->groups, &e, status,
                                stream);
        }
        default:
            return DSL_ERR_ENUM;
    }
}
