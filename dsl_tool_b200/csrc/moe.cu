// The steps either side of the grouped GEMM in a mixture-of-experts layer: router top-k, the
// expert-sorted row plan, dispatch of already quantised rows, and the weighted combine.
//
// Everything is deterministic (no atomics decide an order): the plan is the stable sort of the
// (token, slot) entries by expert, the combine adds a token's slots in slot order.
//
// Dispatch moves QUANTISED rows: the activations are quantised once per token (T rows) and the
// packed bytes and scale bytes are then copied to their expert-sorted places (T * k rows), which
// moves K/2 + K/16 bytes per routed row instead of quantising 2 * K bytes per routed row again.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <float.h>

#include "dslgemm.h"
#include "ptx.cuh"

namespace dsl {

// ---- router: softmax over the experts, top-k ------------------------------------------------
// One warp per token.  Ties go to the lower expert index.  weights = softmax probabilities of the
// chosen experts, divided by their sum when `renorm` is set.
template <typename T>
__global__ void __launch_bounds__(256)
moe_route_kernel(const T* __restrict__ logits, int tokens, int experts, int k, int renorm, int* __restrict__ ids,
                 float* __restrict__ weights) {
    extern __shared__ float s_vals[];                     // [warps per block][experts]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens) return;
    float* v = s_vals + warp * experts;
    float mx = -FLT_MAX;
    for (int e = lane; e < experts; e += 32) {
        float x;
        if (sizeof(T) == 4) x = reinterpret_cast<const float*>(logits)[static_cast<size_t>(t) * experts + e];
        else x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(logits)[static_cast<size_t>(t) * experts + e]);
        v[e] = x;
        mx = fmaxf(mx, x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < experts; e += 32) sum += expf(v[e] - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    __syncwarp();
    float chosen_p = 0.f;       // lane j keeps the j-th choice (k <= 32)
    int chosen_e = 0;
    float psum = 0.f;
    for (int j = 0; j < k; ++j) {
        float best = -FLT_MAX;
        int bi = 0x7FFFFFFF;
        for (int e = lane; e < experts; e += 32) {
            const float x = v[e];
            if (x > best) { best = x; bi = e; }           // ascending e: the first maximum wins inside a lane
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        const float p = __fdiv_rn(expf(best - mx), sum);
        psum += p;
        if (lane == j) { chosen_p = p; chosen_e = bi; }
        if (lane == (bi & 31)) v[bi] = -FLT_MAX;
        __syncwarp();
    }
    if (lane < k) {
        ids[static_cast<size_t>(t) * k + lane] = chosen_e;
        weights[static_cast<size_t>(t) * k + lane] = renorm ? __fdiv_rn(chosen_p, psum) : chosen_p;
    }
}

// ---- plan: stable sort of the (token, slot) entries by expert ---------------------------------
// One CTA per expert walks all entries in order.  Pass `count` writes how many entries name the
// expert; pass `place` (second launch) turns the counts into offsets and gives every entry of the
// expert its row: offsets[e] + (number of earlier entries of e).
__global__ void __launch_bounds__(256) moe_count_kernel(const int* __restrict__ ids, int entries, int* __restrict__ counts) {
    __shared__ int s_part[8];
    const int e = blockIdx.x;
    int c = 0;
    for (int i = threadIdx.x; i < entries; i += 256) c += ids[i] == e;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) c += __shfl_xor_sync(0xFFFFFFFFu, c, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        int s = 0;
        for (int w = 0; w < 8; ++w) s += s_part[w];
        counts[e] = s;
    }
}

__global__ void __launch_bounds__(256)
moe_place_kernel(const int* __restrict__ ids, int entries, int experts, const int* __restrict__ counts,
                 int* __restrict__ offsets, int* __restrict__ tile0, int* __restrict__ dest) {
    __shared__ int s_base;
    __shared__ int s_warp[8];
    const int e = blockIdx.x;
    if (threadIdx.x == 0) {
        int rows = 0, tiles = 0;
        for (int j = 0; j < e; ++j) { rows += counts[j]; tiles += (counts[j] + 127) >> 7; }
        s_base = rows;
        offsets[e] = rows;
        tile0[e] = tiles;
        if (e == experts - 1) { offsets[experts] = rows + counts[e]; tile0[experts] = tiles + ((counts[e] + 127) >> 7); }
    }
    __syncthreads();
    int running = s_base;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i0 = 0; i0 < entries; i0 += 256) {
        const int i = i0 + threadIdx.x;
        const bool mine = i < entries && ids[i] == e;
        const unsigned bal = __ballot_sync(0xFFFFFFFFu, mine);
        if (lane == 0) s_warp[warp] = __popc(bal);
        __syncthreads();
        int before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) { const int c = s_warp[w]; before += w < warp ? c : 0; total += c; }
        if (mine) dest[i] = running + before + __popc(bal & ((1u << lane) - 1u));
        running += total;
        __syncthreads();
    }
}

// ---- dispatch of quantised FP4 rows ------------------------------------------------------------
// Entry i = token * k + slot goes to row dest[i] - offsets[first_expert] of the local expert-sorted
// buffers when its expert is one of [first_expert, last_expert).  Packed bytes are copied as 16-byte
// vectors; scale bytes move word-wise from the token-major tile layout to the expert-sorted one, in
// which every expert starts a fresh 128-row tile.  One warp per entry.
__global__ void __launch_bounds__(256)
moe_dispatch_fp4_kernel(const uint8_t* __restrict__ q_in, const uint8_t* __restrict__ sf_in, const int* __restrict__ ids,
                        const int* __restrict__ dest, const int* __restrict__ offsets, const int* __restrict__ tile0,
                        int entries, int k, int row_bytes, int katoms, int first_expert, int last_expert,
                        uint8_t* __restrict__ q_out, uint8_t* __restrict__ sf_out) {
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i >= entries) return;
    const int e = ids[i];
    if (e < first_expert || e >= last_expert) return;
    const int t = i / k;
    const int base = offsets[first_expert];
    const int d = dest[i] - base;
    const uint4* src = reinterpret_cast<const uint4*>(q_in + static_cast<size_t>(t) * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(q_out + static_cast<size_t>(d) * row_bytes);
    for (int j = lane; j < row_bytes / 16; j += 32) dst[j] = src[j];
    const int rg = dest[i] - offsets[e];                      // row inside its expert
    const int tile_d = tile0[e] - tile0[first_expert] + (rg >> 7);
    const int rin_d = rg & 127, rin_s = t & 127;
    const uint8_t* s_tile = sf_in + static_cast<size_t>(t >> 7) * katoms * 512 + (rin_s & 31) * 16 + (rin_s >> 5) * 4;
    uint8_t* d_tile = sf_out + static_cast<size_t>(tile_d) * katoms * 512 + (rin_d & 31) * 16 + (rin_d >> 5) * 4;
    for (int a = lane; a < katoms; a += 32)
        *reinterpret_cast<uint32_t*>(d_tile + static_cast<size_t>(a) * 512) = *reinterpret_cast<const uint32_t*>(s_tile + static_cast<size_t>(a) * 512);
}

// Plain rows (bf16 activations, E4M3 bytes, ...): same mapping, row_bytes % 16 == 0.
__global__ void __launch_bounds__(256)
moe_dispatch_rows_kernel(const uint8_t* __restrict__ x, const int* __restrict__ ids, const int* __restrict__ dest,
                         const int* __restrict__ offsets, int entries, int k, int row_bytes, int first_expert,
                         int last_expert, uint8_t* __restrict__ out) {
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i >= entries) return;
    const int e = ids[i];
    if (e < first_expert || e >= last_expert) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(i / k) * row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(dest[i] - offsets[first_expert]) * row_bytes);
    for (int j = lane; j < row_bytes / 16; j += 32) dst[j] = src[j];
}

// ---- combine -----------------------------------------------------------------------------------
// out[t, :] = sum over the token's slots, in slot order, of weight * y[row of that slot, :], taking
// only slots whose expert is local (the others are another rank's share of the sum).
template <typename TY, typename TO>
__global__ void __launch_bounds__(256)
moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ ids, const int* __restrict__ dest,
                   const int* __restrict__ offsets, const float* __restrict__ weights, int tokens, int k, int d_model,
                   int first_expert, int last_expert, TO* __restrict__ out) {
    __shared__ int s_row[32];
    __shared__ float s_w[32];
    const int t = blockIdx.x;
    const int base = offsets[first_expert];
    if (threadIdx.x < k) {                                  // the token's slots, once per CTA (k <= 32)
        const int i = t * k + threadIdx.x;
        const int e = ids[i];
        s_row[threadIdx.x] = (e >= first_expert && e < last_expert) ? dest[i] - base : -1;
        s_w[threadIdx.x] = weights[i];
    }
    __syncthreads();
    constexpr int VEC = 16 / sizeof(TY);                    // elements per 16-byte load
    const bool vec_ok = d_model % VEC == 0 && (reinterpret_cast<uintptr_t>(y) & 15u) == 0;
    if (vec_ok) {
        for (int c0 = threadIdx.x * VEC; c0 < d_model; c0 += 256 * VEC) {
            float acc[VEC];
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
            for (int s = 0; s < k; ++s) {
                const int r = s_row[s];
                if (r < 0) continue;
                const float w = s_w[s];
                const uint4 v = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(r) * d_model + c0);
                if (sizeof(TY) == 4) {
                    const float* f = reinterpret_cast<const float*>(&v);
#pragma unroll
                    for (int j = 0; j < VEC; ++j) acc[j] = fmaf(w, f[j], acc[j]);
                } else {
                    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
                    for (int j = 0; j < VEC / 2; ++j) {
                        const float2 f = __bfloat1622float2(h[j]);
                        acc[2 * j] = fmaf(w, f.x, acc[2 * j]);
                        acc[2 * j + 1] = fmaf(w, f.y, acc[2 * j + 1]);
                    }
                }
            }
            if (sizeof(TO) == 4 && (reinterpret_cast<uintptr_t>(out) & 15u) == 0) {
                float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + static_cast<size_t>(t) * d_model + c0);
#pragma unroll
                for (int j = 0; j < VEC / 4; ++j) o[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < VEC; ++j) {
                    if (sizeof(TO) == 4) reinterpret_cast<float*>(out)[static_cast<size_t>(t) * d_model + c0 + j] = acc[j];
                    else reinterpret_cast<__nv_bfloat16*>(out)[static_cast<size_t>(t) * d_model + c0 + j] = __float2bfloat16_rn(acc[j]);
                }
            }
        }
        return;
    }
    for (int c = threadIdx.x; c < d_model; c += 256) {
        float acc = 0.f;
        for (int s = 0; s < k; ++s) {
            const int r = s_row[s];
            if (r < 0) continue;
            const TY v = y[static_cast<size_t>(r) * d_model + c];
            float f;
            if (sizeof(TY) == 4) f = *reinterpret_cast<const float*>(&v);
            else f = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(&v));
            acc = fmaf(s_w[s], f, acc);
        }
        if (sizeof(TO) == 4) reinterpret_cast<float*>(out)[static_cast<size_t>(t) * d_model + c] = acc;
        else reinterpret_cast<__nv_bfloat16*>(out)[static_cast<size_t>(t) * d_model + c] = __float2bfloat16_rn(acc);
    }
}

}  // namespace dsl

using namespace dsl;

static inline cudaStream_t st_of(void* s) { return reinterpret_cast<cudaStream_t>(s); }

extern "C" int dsl_moe_route(const void* logits, int dtype, int tokens, int experts, int k, int renorm, int* ids_out,
                             float* weights_out, void* stream) {
    if (logits == nullptr || ids_out == nullptr || weights_out == nullptr) return DSL_ERR_NULL;
    if (dtype != DSL_F32 && dtype != DSL_BF16) return DSL_ERR_ENUM;
    if (tokens < 0 || experts < 1 || experts > DSL_MAX_GROUPS || k < 1 || k > 32 || k > experts) return DSL_ERR_SHAPE;
    if (tokens == 0) return 0;
    const unsigned grid = (tokens + 7) / 8;
    const size_t smem = 8 * static_cast<size_t>(experts) * sizeof(float);
    if (dtype == DSL_F32)
        moe_route_kernel<float><<<grid, 256, smem, st_of(stream)>>>(static_cast<const float*>(logits), tokens, experts, k, renorm, ids_out, weights_out);
    else
        moe_route_kernel<__nv_bfloat16><<<grid, 256, smem, st_of(stream)>>>(static_cast<const __nv_bfloat16*>(logits), tokens, experts, k, renorm, ids_out, weights_out);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int dsl_moe_plan(const int* ids, int entries, int experts, int* counts_scratch, int* offsets_out, int* tile0_out,
                            int* dest_out, void* stream) {
    if (ids == nullptr || counts_scratch == nullptr || offsets_out == nullptr || tile0_out == nullptr || dest_out == nullptr) return DSL_ERR_NULL;
    if (entries < 0 || experts < 1 || experts > DSL_MAX_GROUPS) return DSL_ERR_SHAPE;
    moe_count_kernel<<<experts, 256, 0, st_of(stream)>>>(ids, entries, counts_scratch);
    moe_place_kernel<<<experts, 256, 0, st_of(stream)>>>(ids, entries, experts, counts_scratch, offsets_out, tile0_out, dest_out);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int dsl_moe_dispatch_fp4(const uint8_t* q_in, const uint8_t* sf_in, const int* ids, const int* dest, const int* offsets,
                                    const int* tile0, int tokens, int k, int K, int format, int first_expert, int last_expert,
                                    uint8_t* q_out, uint8_t* sf_out, void* stream) {
    if (q_in == nullptr || sf_in == nullptr || ids == nullptr || dest == nullptr || offsets == nullptr || tile0 == nullptr ||
        q_out == nullptr || sf_out == nullptr)
        return DSL_ERR_NULL;
    if (format != DSL_FP4_NV && format != DSL_FP4_MX) return DSL_ERR_ENUM;
    if (tokens < 0 || k < 1 || K <= 0 || K % 32 != 0 || first_expert < 0 || last_expert < first_expert) return DSL_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(q_in) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(sf_in) |
         reinterpret_cast<uintptr_t>(sf_out)) & 15u)
        return DSL_ERR_ALIGN;
    const long long entries = static_cast<long long>(tokens) * k;
    if (entries == 0 || last_expert == first_expert) return 0;
    if (entries > 0x7FFFFFFFll) return DSL_ERR_TOO_LARGE;
    const int nblk = format == DSL_FP4_NV ? K / 16 : K / 32;
    moe_dispatch_fp4_kernel<<<static_cast<unsigned>((entries + 7) / 8), 256, 0, st_of(stream)>>>(
        q_in, sf_in, ids, dest, offsets, tile0, static_cast<int>(entries), k, K / 2, (nblk + 3) / 4, first_expert, last_expert, q_out, sf_out);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int dsl_moe_dispatch_rows(const void* x, const int* ids, const int* dest, const int* offsets, int tokens, int k,
                                     long long row_bytes, int first_expert, int last_expert, void* out, void* stream) {
    if (x == nullptr || ids == nullptr || dest == nullptr || offsets == nullptr || out == nullptr) return DSL_ERR_NULL;
    if (tokens < 0 || k < 1 || row_bytes <= 0 || row_bytes % 16 != 0 || row_bytes > 0x7FFFFFFFll || first_expert < 0 ||
        last_expert < first_expert)
        return DSL_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(out)) & 15u) return DSL_ERR_ALIGN;
    const long long entries = static_cast<long long>(tokens) * k;
    if (entries == 0 || last_expert == first_expert) return 0;
    if (entries > 0x7FFFFFFFll) return DSL_ERR_TOO_LARGE;
    moe_dispatch_rows_kernel<<<static_cast<unsigned>((entries + 7) / 8), 256, 0, st_of(stream)>>>(
        static_cast<const uint8_t*>(x), ids, dest, offsets, static_cast<int>(entries), k, static_cast<int>(row_bytes), first_expert,
        last_expert, static_cast<uint8_t*>(out));
    return static_cast<int>(cudaGetLastError());
}

extern "C" int dsl_moe_combine(const void* y, int y_dtype, const int* ids, const int* dest, const int* offsets, const float* weights,
                               int tokens, int k, int d_model, int first_expert, int last_expert, void* out, int out_dtype,
                               void* stream) {
    if (y == nullptr || ids == nullptr || dest == nullptr || offsets == nullptr || weights == nullptr || out == nullptr) return DSL_ERR_NULL;
    if ((y_dtype != DSL_F32 && y_dtype != DSL_BF16) || (out_dtype != DSL_F32 && out_dtype != DSL_BF16)) return DSL_ERR_ENUM;
    if (tokens < 0 || k < 1 || k > 32 || d_model < 1 || first_expert < 0 || last_expert < first_expert) return DSL_ERR_SHAPE;
    if (tokens == 0) return 0;
    cudaStream_t st = st_of(stream);
#define DSL_COMBINE(TY, TO)                                                                                              \
    moe_combine_kernel<TY, TO><<<tokens, 256, 0, st>>>(static_cast<const TY*>(y), ids, dest, offsets, weights, tokens, k, \
                                                         d_model, first_expert, last_expert, static_cast<TO*>(out))
    if (y_dtype == DSL_F32 && out_dtype == DSL_F32) DSL_COMBINE(float, float);
    else if (y_dtype == DSL_F32) DSL_COMBINE(float, __nv_bfloat16);
    else if (out_dtype == DSL_F32) DSL_COMBINE(__nv_bfloat16, float);
    else DSL_COMBINE(__nv_bfloat16, __nv_bfloat16);
#undef DSL_COMBINE
    return static_cast<int>(cudaGetLastError());
}
