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

// The same router for up to 64 experts with the logits in registers (lane l holds experts l and l + 32): no shared
// memory, no warp barrier per round.  Every sum, comparison and division is the one of the kernel above, in the same
// order, so ids and weights are bit-identical; the shared-memory form issued 1160 instructions per token.
template <typename T>
__global__ void __launch_bounds__(256)
moe_route64_kernel(const T* __restrict__ logits, int tokens, int experts, int k, int renorm, int* __restrict__ ids,
                   float* __restrict__ weights) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= tokens) return;
    const bool has0 = lane < experts, has1 = lane + 32 < experts;
    float v0 = -FLT_MAX, v1 = -FLT_MAX;
    if (sizeof(T) == 4) {
        const float* row = reinterpret_cast<const float*>(logits) + static_cast<size_t>(t) * experts;
        if (has0) v0 = row[lane];
        if (has1) v1 = row[lane + 32];
    } else {
        const __nv_bfloat16* row = reinterpret_cast<const __nv_bfloat16*>(logits) + static_cast<size_t>(t) * experts;
        if (has0) v0 = __bfloat162float(row[lane]);
        if (has1) v1 = __bfloat162float(row[lane + 32]);
    }
    float mx = -FLT_MAX;
    if (has0) mx = fmaxf(mx, v0);
    if (has1) mx = fmaxf(mx, v1);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xFFFFFFFFu, mx, o));
    float sum = 0.f;
    if (has0) sum += expf(v0 - mx);
    if (has1) sum += expf(v1 - mx);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xFFFFFFFFu, sum, o);
    float chosen_p = 0.f;
    int chosen_e = 0;
    float psum = 0.f;
    for (int j = 0; j < k; ++j) {
        float best = -FLT_MAX;
        int bi = 0x7FFFFFFF;
        if (has0 && v0 > best) { best = v0; bi = lane; }
        if (has1 && v1 > best) { best = v1; bi = lane + 32; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        const float p = __fdiv_rn(expf(best - mx), sum);
        psum += p;
        if (lane == j) { chosen_p = p; chosen_e = bi; }
        if (lane == (bi & 31)) {
            if (bi < 32) v0 = -FLT_MAX; else v1 = -FLT_MAX;
        }
    }
    if (lane < k) {
        ids[static_cast<size_t>(t) * k + lane] = chosen_e;
        weights[static_cast<size_t>(t) * k + lane] = renorm ? __fdiv_rn(chosen_p, psum) : chosen_p;
    }
}

// ---- plan: stable sort of the (token, slot) entries by expert ---------------------------------
// Three small launches, no atomics that could decide an order:
//   count   every CTA histograms its block of kPlanBlock consecutive entries (shared-memory counters: sums do
//           not depend on the order of the additions) -> block_counts[block][expert]
//   scan    one CTA: per expert the running sum over the blocks, then offsets / tile0 over the experts;
//           block_counts becomes the first row of (block, expert)
//   place   every CTA walks its block in order; an entry's row = first row of (block, expert) + number of
//           earlier entries of the block with the same expert (warp match + warps committed in order)
constexpr int kPlanBlock = 2048;

__global__ void __launch_bounds__(256)
moe_count_kernel(const int* __restrict__ ids, int entries, int experts, int* __restrict__ block_counts) {
    extern __shared__ int s_bins[];
    for (int e = threadIdx.x; e < experts; e += 256) s_bins[e] = 0;
    __syncthreads();
    const int i0 = blockIdx.x * kPlanBlock;
    for (int i = i0 + threadIdx.x; i < min(entries, i0 + kPlanBlock); i += 256) {
        const int e = ids[i];
        if (e >= 0 && e < experts) atomicAdd(&s_bins[e], 1);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += 256) block_counts[static_cast<size_t>(blockIdx.x) * experts + e] = s_bins[e];
}

// The running sums update block_counts in place, so the compiler must keep every load behind the store before it; with
// one expert per thread that made the loop a chain of dependent L2 round trips (64 blocks: 20 us for 2900 instructions).
// Loads and stores are therefore issued in batches of 16: the 16 loads of a batch are independent and in flight together.
__global__ void __launch_bounds__(1024)
moe_scan_kernel(int* __restrict__ block_counts, int blocks, int experts, int* __restrict__ offsets, int* __restrict__ tile0) {
    __shared__ int s_cnt[DSL_MAX_GROUPS];
    constexpr int B = 16;
    for (int e = threadIdx.x; e < experts; e += 1024) {
        int run = 0;
        for (int b0 = 0; b0 < blocks; b0 += B) {
            int c[B];
#pragma unroll
            for (int j = 0; j < B; ++j)
                c[j] = b0 + j < blocks ? __ldcg(block_counts + static_cast<size_t>(b0 + j) * experts + e) : 0;
#pragma unroll
            for (int j = 0; j < B; ++j) {
                if (b0 + j < blocks) block_counts[static_cast<size_t>(b0 + j) * experts + e] = run;
                run += c[j];
            }
        }
        s_cnt[e] = run;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int rows = 0, tiles = 0;
        for (int e = 0; e < experts; ++e) {
            const int c = s_cnt[e];
            offsets[e] = rows;
            tile0[e] = tiles;
            s_cnt[e] = rows;
            rows += c;
            tiles += (c + 127) >> 7;
        }
        offsets[experts] = rows;
        tile0[experts] = tiles;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < experts; e += 1024) {
        const int base = s_cnt[e];
        for (int b0 = 0; b0 < blocks; b0 += B) {
            int c[B];
#pragma unroll
            for (int j = 0; j < B; ++j)
                c[j] = b0 + j < blocks ? __ldcg(block_counts + static_cast<size_t>(b0 + j) * experts + e) : 0;
#pragma unroll
            for (int j = 0; j < B; ++j)
                if (b0 + j < blocks) block_counts[static_cast<size_t>(b0 + j) * experts + e] = c[j] + base;
        }
    }
}

__global__ void __launch_bounds__(256)
moe_place_kernel(const int* __restrict__ ids, int entries, int experts, const int* __restrict__ block_first,
                 int* __restrict__ dest) {
    extern __shared__ int s_next[];                        // next free row of every expert, for this block
    for (int e = threadIdx.x; e < experts; e += 256) s_next[e] = block_first[static_cast<size_t>(blockIdx.x) * experts + e];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int i0 = blockIdx.x * kPlanBlock;
    for (int c0 = i0; c0 < min(entries, i0 + kPlanBlock); c0 += 256) {
        const int i = c0 + threadIdx.x;
        const bool valid = i < entries;
        int e = valid ? ids[i] : -1;
        if (e < 0 || e >= experts) e = -1;                 // out-of-range ids get no row
        const unsigned peers = __match_any_sync(0xFFFFFFFFu, e);
        const int rank = __popc(peers & ((1u << lane) - 1u));
        const int leader = __ffs(peers) - 1;
        for (int w = 0; w < 8; ++w) {                      // warps commit in order: entries stay in sequence
            if (warp == w) {
                int base = 0;
                if (e >= 0 && lane == leader) {
                    base = s_next[e];
                    s_next[e] = base + __popc(peers);
                }
                base = __shfl_sync(0xFFFFFFFFu, base, leader);
                if (e >= 0) dest[i] = base + rank;
            }
            __syncthreads();
        }
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

// ---- rows on the wire (token all-to-all) --------------------------------------------------------
// A routed row travels between GPUs as one record: the packed e2m1 bytes followed by the row's scale bytes in
// plain K order (one 32-bit word per 512-byte scale tile of the row, i.e. four scale bytes; zero padding included),
// padded to a multiple of 16 bytes.  pack: entry i = token * k + slot -> record dest[i] (all experts, expert-sorted).
__global__ void __launch_bounds__(256)
moe_pack_wire_fp4_kernel(const uint8_t* __restrict__ q_in, const uint8_t* __restrict__ sf_in, const int* __restrict__ dest,
                         int entries, int k, int row_bytes, int katoms, int wire_bytes, uint8_t* __restrict__ wire) {
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i >= entries) return;
    const int t = i / k;
    const uint4* src = reinterpret_cast<const uint4*>(q_in + static_cast<size_t>(t) * row_bytes);
    uint8_t* rec = wire + static_cast<size_t>(dest[i]) * wire_bytes;
    uint4* dst = reinterpret_cast<uint4*>(rec);
    for (int j = lane; j < row_bytes / 16; j += 32) dst[j] = src[j];
    const int rin = t & 127;
    const uint8_t* s_tile = sf_in + static_cast<size_t>(t >> 7) * katoms * 512 + (rin & 31) * 16 + (rin >> 5) * 4;
    uint32_t* words = reinterpret_cast<uint32_t*>(rec + row_bytes);
    const int nwords = (wire_bytes - row_bytes) / 4;
    for (int a = lane; a < nwords; a += 32)
        words[a] = a < katoms ? *reinterpret_cast<const uint32_t*>(s_tile + static_cast<size_t>(a) * 512) : 0u;
}

// unpack: record r (expert ids[r] of this rank, position dest[r] in this rank's expert-sorted order) -> packed row
// dest[r] and its scale bytes in the ragged-group tile layout (every expert starts a fresh 128-row tile).
__global__ void __launch_bounds__(256)
moe_unpack_wire_fp4_kernel(const uint8_t* __restrict__ wire, const int* __restrict__ ids, const int* __restrict__ dest,
                           const int* __restrict__ offsets, const int* __restrict__ tile0, int rows, int row_bytes, int katoms,
                           int wire_bytes, uint8_t* __restrict__ q_out, uint8_t* __restrict__ sf_out) {
    const int r = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= rows) return;
    const int e = ids[r];
    const int d = dest[r];
    const uint8_t* rec = wire + static_cast<size_t>(r) * wire_bytes;
    const uint4* src = reinterpret_cast<const uint4*>(rec);
    uint4* dst = reinterpret_cast<uint4*>(q_out + static_cast<size_t>(d) * row_bytes);
    for (int j = lane; j < row_bytes / 16; j += 32) dst[j] = src[j];
    const int rg = d - offsets[e];
    const int tile_d = tile0[e] + (rg >> 7);
    const int rin = rg & 127;
    uint8_t* d_tile = sf_out + static_cast<size_t>(tile_d) * katoms * 512 + (rin & 31) * 16 + (rin >> 5) * 4;
    const uint32_t* words = reinterpret_cast<const uint32_t*>(rec + row_bytes);
    for (int a = lane; a < katoms; a += 32) *reinterpret_cast<uint32_t*>(d_tile + static_cast<size_t>(a) * 512) = words[a];
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
    if (experts <= 64) {
        if (dtype == DSL_F32)
            moe_route64_kernel<float><<<grid, 256, 0, st_of(stream)>>>(static_cast<const float*>(logits), tokens, experts, k, renorm, ids_out, weights_out);
        else
            moe_route64_kernel<__nv_bfloat16><<<grid, 256, 0, st_of(stream)>>>(static_cast<const __nv_bfloat16*>(logits), tokens, experts, k, renorm, ids_out, weights_out);
        return static_cast<int>(cudaGetLastError());
    }
    const size_t smem = 8 * static_cast<size_t>(experts) * sizeof(float);
    if (dtype == DSL_F32)
        moe_route_kernel<float><<<grid, 256, smem, st_of(stream)>>>(static_cast<const float*>(logits), tokens, experts, k, renorm, ids_out, weights_out);
    else
        moe_route_kernel<__nv_bfloat16><<<grid, 256, smem, st_of(stream)>>>(static_cast<const __nv_bfloat16*>(logits), tokens, experts, k, renorm, ids_out, weights_out);
    return static_cast<int>(cudaGetLastError());
}

extern "C" size_t dsl_moe_plan_scratch_bytes(int entries, int experts) {
    if (entries < 0 || experts < 1) return 0;
    return static_cast<size_t>((entries + kPlanBlock - 1) / kPlanBlock + 1) * static_cast<size_t>(experts) * sizeof(int);
}

extern "C" int dsl_moe_plan(const int* ids, int entries, int experts, int* scratch, int* offsets_out, int* tile0_out,
                            int* dest_out, void* stream) {
    if (ids == nullptr || scratch == nullptr || offsets_out == nullptr || tile0_out == nullptr || dest_out == nullptr) return DSL_ERR_NULL;
    if (entries < 0 || experts < 1 || experts > DSL_MAX_GROUPS) return DSL_ERR_SHAPE;
    const int blocks = (entries + kPlanBlock - 1) / kPlanBlock;
    const size_t smem = static_cast<size_t>(experts) * sizeof(int);
    if (blocks > 0) moe_count_kernel<<<blocks, 256, smem, st_of(stream)>>>(ids, entries, experts, scratch);
    moe_scan_kernel<<<1, 1024, 0, st_of(stream)>>>(scratch, blocks, experts, offsets_out, tile0_out);
    if (blocks > 0) moe_place_kernel<<<blocks, 256, smem, st_of(stream)>>>(ids, entries, experts, scratch, dest_out);
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

// ---- sum of the ranks' partial results over peer memory -----------------------------------------
// Every rank holds a partial result [total rows, D] in memory that its peers can address (mapped into this process by
// the caller, e.g. symmetric memory).  Rank r wants rows [row0, row0 + rows) of the sum: each thread takes one 16-byte
// vector, loads it from every rank's buffer (plain loads: the local one from HBM, the others over NVLink - no TMA, no
// multicast, nothing is written to a peer), adds in rank order in fp32 and stores the result locally.  The order is
// fixed, so the result does not depend on timing.  The caller orders the kernel after every rank's partial result is
// complete (a collective on the stream) and keeps a buffer untouched until every rank has read it.
struct PeerPtrs {
    const void* p[DSL_MAX_PEERS];
};
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
moe_reduce_pull_kernel(PeerPtrs ptrs, int world, size_t first_vec, size_t nvec, TO* __restrict__ out) {
    constexpr int VEC = 16 / sizeof(TI);
    for (size_t v = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; v < nvec; v += static_cast<size_t>(gridDim.x) * blockDim.x) {
        uint4 part[DSL_MAX_PEERS];
#pragma unroll
        for (int s = 0; s < DSL_MAX_PEERS; ++s)
            if (s < world) part[s] = __ldcg(reinterpret_cast<const uint4*>(ptrs.p[s]) + first_vec + v);   // all in flight together
        float acc[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
#pragma unroll
        for (int s = 0; s < DSL_MAX_PEERS; ++s) {
            if (s >= world) break;
            if (sizeof(TI) == 4) {
                const float* f = reinterpret_cast<const float*>(&part[s]);
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc[j] = __fadd_rn(acc[j], f[j]);
            } else {
                const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&part[s]);
#pragma unroll
                for (int j = 0; j < VEC / 2; ++j) {
                    const float2 f = __bfloat1622float2(h[j]);
                    acc[2 * j] = __fadd_rn(acc[2 * j], f.x);
                    acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], f.y);
                }
            }
        }
        if (sizeof(TO) == 4) {
            float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + v * VEC);
#pragma unroll
            for (int j = 0; j < VEC / 4; ++j) o[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
        } else if (VEC == 8) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(out) + v * VEC) = make_uint4(w[0], w[1], w[2], w[3]);
        } else {
            uint32_t w[2];
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(out) + v * VEC) = make_uint2(w[0], w[1]);
        }
    }
}

extern "C" int dsl_moe_reduce_pull(const void* const* part_ptrs, int world, long long row0, long long rows, int d_model,
                                   int in_dtype, void* out, int out_dtype, void* stream) {
    if (part_ptrs == nullptr || out == nullptr) return DSL_ERR_NULL;
    if (world < 1 || world > DSL_MAX_PEERS) return DSL_ERR_TOO_LARGE;
    if ((in_dtype != DSL_F32 && in_dtype != DSL_BF16) || (out_dtype != DSL_F32 && out_dtype != DSL_BF16)) return DSL_ERR_ENUM;
    if (row0 < 0 || rows < 0 || d_model < 1) return DSL_ERR_SHAPE;
    const int vec = in_dtype == DSL_F32 ? 4 : 8;
    if (d_model % vec != 0) return DSL_ERR_SHAPE;              // rows are whole 16-byte vectors
    PeerPtrs ptrs;
    for (int s = 0; s < DSL_MAX_PEERS; ++s) {
        ptrs.p[s] = s < world ? part_ptrs[s] : nullptr;
        if (s < world && ptrs.p[s] == nullptr) return DSL_ERR_NULL;
        if (s < world && (reinterpret_cast<uintptr_t>(ptrs.p[s]) & 15u) != 0) return DSL_ERR_ALIGN;
    }
    if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return DSL_ERR_ALIGN;
    if (rows == 0) return 0;
    const size_t per_row = static_cast<size_t>(d_model) / vec;
    const size_t nvec = static_cast<size_t>(rows) * per_row;
    const size_t first_vec = static_cast<size_t>(row0) * per_row;
    const size_t want = (nvec + 255) / 256;
    const unsigned grid = static_cast<unsigned>(want < 148u * 16u ? want : 148u * 16u);
    cudaStream_t st = st_of(stream);
    if (in_dtype == DSL_F32 && out_dtype == DSL_F32) moe_reduce_pull_kernel<float, float><<<grid, 256, 0, st>>>(ptrs, world, first_vec, nvec, static_cast<float*>(out));
    else if (in_dtype == DSL_F32) moe_reduce_pull_kernel<float, __nv_bfloat16><<<grid, 256, 0, st>>>(ptrs, world, first_vec, nvec, static_cast<__nv_bfloat16*>(out));
    else if (out_dtype == DSL_F32) moe_reduce_pull_kernel<__nv_bfloat16, float><<<grid, 256, 0, st>>>(ptrs, world, first_vec, nvec, static_cast<float*>(out));
    else moe_reduce_pull_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, 256, 0, st>>>(ptrs, world, first_vec, nvec, static_cast<__nv_bfloat16*>(out));
    return static_cast<int>(cudaGetLastError());
}

extern "C" size_t dsl_moe_wire_bytes(int K, int format) {
    if (K <= 0 || K % 32 != 0 || (format != DSL_FP4_NV && format != DSL_FP4_MX)) return 0;
    const int nblk = format == DSL_FP4_NV ? K / 16 : K / 32;
    const size_t raw = static_cast<size_t>(K) / 2 + 4u * static_cast<size_t>((nblk + 3) / 4);
    return (raw + 15) / 16 * 16;
}

extern "C" int dsl_moe_pack_wire_fp4(const uint8_t* q_in, const uint8_t* sf_in, const int* dest, int tokens, int k, int K,
                                     int format, uint8_t* wire_out, void* stream) {
    if (q_in == nullptr || sf_in == nullptr || dest == nullptr || wire_out == nullptr) return DSL_ERR_NULL;
    const size_t wb = dsl_moe_wire_bytes(K, format);
    if (wb == 0) return format != DSL_FP4_NV && format != DSL_FP4_MX ? DSL_ERR_ENUM : DSL_ERR_SHAPE;
    if (tokens < 0 || k < 1) return DSL_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(q_in) | reinterpret_cast<uintptr_t>(sf_in) | reinterpret_cast<uintptr_t>(wire_out)) & 15u)
        return DSL_ERR_ALIGN;
    const long long entries = static_cast<long long>(tokens) * k;
    if (entries == 0) return 0;
    if (entries > 0x7FFFFFFFll) return DSL_ERR_TOO_LARGE;
    const int nblk = format == DSL_FP4_NV ? K / 16 : K / 32;
    moe_pack_wire_fp4_kernel<<<static_cast<unsigned>((entries + 7) / 8), 256, 0, st_of(stream)>>>(
        q_in, sf_in, dest, static_cast<int>(entries), k, K / 2, (nblk + 3) / 4, static_cast<int>(wb), wire_out);
    return static_cast<int>(cudaGetLastError());
}

extern "C" int dsl_moe_unpack_wire_fp4(const uint8_t* wire_in, const int* ids, const int* dest, const int* offsets,
                                       const int* tile0, int rows, int K, int format, uint8_t* q_out, uint8_t* sf_out,
                                       void* stream) {
    if (wire_in == nullptr || ids == nullptr || dest == nullptr || offsets == nullptr || tile0 == nullptr || q_out == nullptr ||
        sf_out == nullptr)
        return DSL_ERR_NULL;
    const size_t wb = dsl_moe_wire_bytes(K, format);
    if (wb == 0) return format != DSL_FP4_NV && format != DSL_FP4_MX ? DSL_ERR_ENUM : DSL_ERR_SHAPE;
    if (rows < 0) return DSL_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(wire_in) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(sf_out)) & 15u)
        return DSL_ERR_ALIGN;
    if (rows == 0) return 0;
    const int nblk = format == DSL_FP4_NV ? K / 16 : K / 32;
    moe_unpack_wire_fp4_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, st_of(stream)>>>(
        wire_in, ids, dest, offsets, tile0, rows, K / 2, (nblk + 3) / 4, static_cast<int>(wb), q_out, sf_out);
    return static_cast<int>(cudaGetLastError());
}
