// Persistent, warp-specialised tcgen05 GEMM for sm_100a: dense and grouped (ragged row
// groups), FP8 E4M3 with per-tensor scales, block-scaled FP4 (NVFP4 / MXFP4) and plain BF16.
//
//   C[m, n] = (sum_k A[m, k] * B[g(m), n, k]) * scale_a * scale_b [* row_scale] [* col_scale]
//
// Data path per CTA (one CTA per SM, 192 threads):
//   warp 0   TMA producer: 128-byte-swizzled operand boxes (A: 128 rows, B: BLOCK_N rows,
//            128 bytes of K each) plus the scale-factor tiles of the stage (plain bulk
//            copies) into a NUM_STAGES-deep shared-memory ring, signalled by mbarriers.
//   warp 1   MMA issuer: copies the stage's scale tiles shared -> tensor memory
//            (tcgen05.cp), issues four K-steps of tcgen05.mma into an fp32 accumulator in
//            tensor memory, and releases the stage / publishes the accumulator with
//            tcgen05.commit.
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp owns one 32-lane quadrant),
//            apply the scales, convert, and store rows straight to global memory.
// Tiles are walked in the same order by all three roles; the device-side scheduler turns a
// linear tile index into (row group, row tile, column tile) from the group offsets, so ragged
// expert groups need no host-side knowledge of their sizes.  Every barrier wait is bounded.
#include <cuda_bf16.h>
#include <stdlib.h>
#include <string.h>

#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_tiles.cuh"
#include "ptx.cuh"

namespace dsl {

constexpr int SFA_COL = 256;            // scale-factor columns sit above the accumulators
constexpr int SFB_COL = 272;

template <int KIND, int BLOCK_N>
struct Cfg {
    static constexpr int A_STAGE = BLOCK_M * STAGE_KB;
    static constexpr int B_STAGE = BLOCK_N * STAGE_KB;
    // 512-byte scale tiles (128 rows x 4 K-blocks) along K per stage: NVFP4 4 (16 scales), MXFP4 2 (8)
    static constexpr int SF_ATOMS = KIND == KIND_NVF4 ? 4 : (KIND == KIND_MXF4 ? 2 : 0);
    static constexpr int N_TILES128 = BLOCK_N / 128;
    static constexpr int SFA_STAGE = SF_ATOMS * 512;
    static constexpr int SFB_STAGE = N_TILES128 * SF_ATOMS * 512;
    static constexpr int STAGE_BYTES = A_STAGE + B_STAGE + SFA_STAGE + SFB_STAGE;
    static constexpr int NUM_STAGES = BLOCK_N == 256 ? 4 : 6;
    static constexpr int ACC_STAGES = BLOCK_N == 256 ? 1 : 2;
    static constexpr int OFF_A = 0;
    static constexpr int OFF_B = OFF_A + NUM_STAGES * A_STAGE;
    static constexpr int OFF_SFA = OFF_B + NUM_STAGES * B_STAGE;
    static constexpr int OFF_SFB = OFF_SFA + NUM_STAGES * SFA_STAGE;
    static constexpr int OFF_BAR = OFF_SFB + NUM_STAGES * SFB_STAGE;        // 8-byte aligned
    static constexpr int NUM_BARS = 2 * NUM_STAGES + 2 * ACC_STAGES;
    static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;                 // tmem ptr, abort flag
    static constexpr int OFF_TABLE = OFF_MISC + 16;                         // offsets[G+1], tile0[G+1]
    static constexpr int SMEM_BYTES = OFF_TABLE + 2 * (DSL_MAX_GROUPS + 1) * 4 + 1024;   // + alignment slack
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
    static_assert(SMEM_BYTES > 116224, "two CTAs could share an SM and deadlock on tensor-memory allocation");
    static_assert(ACC_STAGES * BLOCK_N <= SFA_COL, "accumulators overlap the scale-factor columns");
};

template <int KIND, int BLOCK_N>
__global__ void __launch_bounds__(192, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const GemmArgs args) {
    using C = Cfg<KIND, BLOCK_N>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty_bar = full_bar + C::NUM_STAGES;
    uint64_t* acc_full = empty_bar + C::NUM_STAGES;
    uint64_t* acc_empty = acc_full + C::ACC_STAGES;
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC + 4);
    int* s_offs = reinterpret_cast<int*>(smem + C::OFF_TABLE);
    int* s_tile0 = s_offs + (DSL_MAX_GROUPS + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;

    // ---- set-up ------------------------------------------------------------------------
    if (threadIdx.x == 0) {
        for (int i = 0; i < C::NUM_STAGES; ++i) { mbar_init(full_bar + i, 1); mbar_init(empty_bar + i, 1); }
        for (int i = 0; i < C::ACC_STAGES; ++i) { mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 4); }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    load_group_offsets(s_offs, args.group_offsets, groups, args.m_total);
    if (C::SF_ATOMS > 0) {   // never let an uninitialised (possibly NaN) scale byte meet zero-filled data
        uint32_t* z = reinterpret_cast<uint32_t*>(smem + C::OFF_SFA);
        for (int i = threadIdx.x; i < C::NUM_STAGES * (C::SFA_STAGE + C::SFB_STAGE) / 4; i += blockDim.x) z[i] = 0u;
        fence_proxy_async_smem();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int g = 0; g < groups; ++g) {
            s_tile0[g] = t;
            const int rows = monotone_rows(s_offs, g);
            t += rows > 0 ? (rows + BLOCK_M - 1) / BLOCK_M : 0;
        }
        s_tile0[groups] = t;
    }
    if (warp == 1) tmem_alloc(tmem_ptr, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    TileWalker tw;
    tw.offs = s_offs;
    tw.tile0 = s_tile0;
    tw.groups = groups;
    tw.m_tiles = s_tile0[groups];
    tw.n_tiles = (args.n + BLOCK_N - 1) / BLOCK_N;
    tw.band = args.band < 1 ? 1 : args.band;
    tw.block_n = BLOCK_N;
    tw.total = static_cast<long long>(tw.m_tiles) * tw.n_tiles;
    const int num_kb = (args.k_bytes + STAGE_KB - 1) / STAGE_KB;
    // split-K: work item t = tile * split_k + slice; slice ks covers K-stages [ks*kb_per, ...)
    const int split_k = args.split_k > 1 ? args.split_k : 1;
    const int kb_per = (num_kb + split_k - 1) / split_k;
    const long long total_items = tw.total * split_k;

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < total_items && ok; t += gridDim.x) {
                const TileInfo ti = tw.decode(t / split_k);
                const int kb0 = static_cast<int>(t % split_k) * kb_per;
                const int kb1 = min(num_kb, kb0 + kb_per);
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    uint32_t bytes = C::A_STAGE + C::B_STAGE;
                    int atoms = 0;
                    bool sfb_valid[C::N_TILES128 > 0 ? C::N_TILES128 : 1];
                    if (C::SF_ATOMS > 0) {
                        atoms = min(C::SF_ATOMS, args.sf_katoms - kb * C::SF_ATOMS);
                        bytes += atoms * 512;
                        for (int j = 0; j < C::N_TILES128; ++j) {
                            sfb_valid[j] = ti.n0 / 128 + j < args.sfb_tiles_per_group;
                            if (sfb_valid[j]) bytes += atoms * 512;
                        }
                    }
                    mbar_arrive_expect_tx(full_bar + stage, bytes);
                    tma_load_2d(smem + C::OFF_A + stage * C::A_STAGE, &tmap_a, full_bar + stage, kb * STAGE_KB, ti.row0);
                    tma_load_3d(smem + C::OFF_B + stage * C::B_STAGE, &tmap_b, full_bar + stage, kb * STAGE_KB, ti.n0, ti.group);
                    if (C::SF_ATOMS > 0) {
                        const size_t katom0 = static_cast<size_t>(kb) * C::SF_ATOMS;
                        bulk_load(smem + C::OFF_SFA + stage * C::SFA_STAGE,
                                  args.sfa + (static_cast<size_t>(ti.mtile) * args.sf_katoms + katom0) * 512,
                                  atoms * 512, full_bar + stage);
                        for (int j = 0; j < C::N_TILES128; ++j) {
                            if (!sfb_valid[j]) continue;
                            const size_t rt = static_cast<size_t>(ti.group) * args.sfb_tiles_per_group + ti.n0 / 128 + j;
                            bulk_load(smem + C::OFF_SFB + stage * C::SFB_STAGE + j * C::SFA_STAGE,
                                      args.sfb + (rt * args.sf_katoms + katom0) * 512, atoms * 512, full_bar + stage);
                        }
                    }
                    if (++stage == C::NUM_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        {   // the warp stays converged; one elected lane issues (keeps operands warp-uniform)
            // instruction descriptor: M = 128, N = BLOCK_N, both operands K-major
            uint32_t idesc = (static_cast<uint32_t>(BLOCK_N >> 3) << 17) | (static_cast<uint32_t>(BLOCK_M >> 4) << 24);
            if (KIND == KIND_F8) idesc |= 1u << 4;                                  // fp32 accumulate, E4M3 x E4M3
            if (KIND == KIND_NVF4) idesc |= (1u << 7) | (1u << 10);                 // e2m1 x e2m1, UE4M3 scales
            if (KIND == KIND_MXF4) idesc |= (1u << 7) | (1u << 10) | (1u << 23);    // e2m1 x e2m1, UE8M0 scales
            if (KIND == KIND_BF16) idesc |= (1u << 4) | (1u << 7) | (1u << 10);     // fp32 accumulate, bf16 x bf16
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long iter = 0;
            for (long long t = blockIdx.x; t < total_items && ok; t += gridDim.x, ++iter) {
                const int kb0 = static_cast<int>(t % split_k) * kb_per;
                const int kb1 = min(num_kb, kb0 + kb_per);
                const int acc = static_cast<int>(iter % C::ACC_STAGES);
                const uint32_t acc_phase = static_cast<uint32_t>((iter / C::ACC_STAGES) & 1);
                if (!mbar_wait(acc_empty + acc, acc_phase ^ 1u, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BLOCK_N;
                for (int kb = kb0; kb < kb1; ++kb) {
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + C::OFF_A + stage * C::A_STAGE);
                    const uint32_t b_addr = smem_u32(smem + C::OFF_B + stage * C::B_STAGE);
                    if (elect_one()) {
                    if (C::SF_ATOMS > 0) {
                        const uint32_t sfa_addr = smem_u32(smem + C::OFF_SFA + stage * C::SFA_STAGE);
                        const uint32_t sfb_addr = smem_u32(smem + C::OFF_SFB + stage * C::SFB_STAGE);
#pragma unroll
                        for (int i = 0; i < C::SF_ATOMS; ++i) {
                            tc_cp_32x128b_warpx4(tmem_base + SFA_COL + i * 4, make_desc_sf(sfa_addr + i * 512));
#pragma unroll
                            for (int j = 0; j < C::N_TILES128; ++j)
                                tc_cp_32x128b_warpx4(tmem_base + SFB_COL + i * (BLOCK_N / 32) + j * 4,
                                                     make_desc_sf(sfb_addr + (j * C::SF_ATOMS + i) * 512));
                        }
                    }
                    const uint64_t adesc = make_desc_sw128(a_addr);
                    const uint64_t bdesc = make_desc_sw128(b_addr);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {   // 4 x 32 bytes of K per stage
                        const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
                        if (KIND == KIND_F8) {
                            mma_f8f6f4(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
                        } else if (KIND == KIND_BF16) {
                            mma_f16(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
                        } else if (KIND == KIND_NVF4) {
                            mma_nvf4(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, tmem_base + SFA_COL + k * 4,
                                     tmem_base + SFB_COL + k * (BLOCK_N / 32), accum);
                        } else {
                            const uint32_t sf_id = (k & 1) * 2;   // which byte pair of the 4-scale word
                            const uint32_t id = idesc | (sf_id << 29) | (sf_id << 4);
                            mma_mxf4(d_tmem, adesc + 2 * k, bdesc + 2 * k, id, tmem_base + SFA_COL + (k >> 1) * 4,
                                     tmem_base + SFB_COL + (k >> 1) * (BLOCK_N / 32), accum);
                        }
                    }
                    tc_commit(empty_bar + stage);
                    if (kb == kb1 - 1) tc_commit(acc_full + acc);
                    }
                    __syncwarp();
                    if (++stage == C::NUM_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
        // ================= epilogue =================
        const int quad = warp & 3;   // tensor-memory lanes [32*quad, 32*quad+32) belong to this warp
        float s1 = args.s1_dev != nullptr ? *args.s1_dev : args.s1;
        float s2 = args.s2_dev != nullptr ? *args.s2_dev : args.s2;
        if (args.scale_product) { s1 = s1 * s2; s2 = 1.0f; }
        const bool vec_ok = args.out_bf16 ? (args.ldc % 8 == 0) : (args.ldc % 4 == 0);
        bool ok = true;
        long long iter = 0;
        for (long long t = blockIdx.x; t < total_items && ok; t += gridDim.x, ++iter) {
            const TileInfo ti = tw.decode(t / split_k);
            const int ks = static_cast<int>(t % split_k);
            const int acc = static_cast<int>(iter % C::ACC_STAGES);
            const uint32_t acc_phase = static_cast<uint32_t>((iter / C::ACC_STAGES) & 1);
            if (!mbar_wait(acc_full + acc, acc_phase, abort_flag, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
            tc_fence_after();
            const int row = ti.row0 + quad * 32 + lane;
            const bool row_ok = row < ti.row_end;
            const float rs = (row_ok && args.row_scale != nullptr) ? args.row_scale[row] : 1.0f;
#pragma unroll 1
            for (int c = 0; c < BLOCK_N / 32; ++c) {
                uint32_t v[32];
                tmem_ld_32x32b_x32(tmem_base + acc * BLOCK_N + c * 32 + (static_cast<uint32_t>(quad * 32) << 16), v);
                tmem_ld_wait();
                const int col0 = ti.n0 + c * 32;
                if (!row_ok || col0 >= args.n) continue;
                if (split_k > 1) {
                    // raw fp32 partial sums of this K-slice; scales are applied by the reduction
                    float* dst = args.partial + (static_cast<size_t>(ks) * args.m_total + row) * args.n + col0;
                    if (args.n % 4 == 0 && col0 + 32 <= args.n) {
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            reinterpret_cast<float4*>(dst)[i] = make_float4(__uint_as_float(v[4 * i]), __uint_as_float(v[4 * i + 1]),
                                                                            __uint_as_float(v[4 * i + 2]), __uint_as_float(v[4 * i + 3]));
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (col0 + i < args.n) dst[i] = __uint_as_float(v[i]);
                    }
                } else {
                    store_chunk32(args, row, col0, ti.group, v, s1, s2, rs, vec_ok, ti.mtile, quad * 32 + lane);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty + acc);
        }
    }

    // ---- common exit -------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    const uint32_t aborted = *abort_flag;
    if (aborted != 0) {
        // let copies and MMAs that were already issued land before the CTA goes away
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(2000);
        if (threadIdx.x == 0 && args.status != nullptr) atomicOr(args.status, aborted);
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}


// Sums the split-K partial products in slice order (deterministic) and applies the epilogue.
// One thread per four consecutive columns of a row.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const GemmArgs args, int split_k) {
    const int n4 = (args.n + 3) / 4;
    const long long id = blockIdx.x * 256ll + threadIdx.x;
    if (id >= static_cast<long long>(args.m_total) * n4) return;
    const int row = static_cast<int>(id / n4);
    const int col0 = static_cast<int>(id - static_cast<long long>(row) * n4) * 4;
    float s1 = args.s1_dev != nullptr ? *args.s1_dev : args.s1;
    float s2 = args.s2_dev != nullptr ? *args.s2_dev : args.s2;
    if (args.scale_product) { s1 = s1 * s2; s2 = 1.0f; }
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const size_t slice = static_cast<size_t>(args.m_total) * args.n;
    const float* p = args.partial + static_cast<size_t>(row) * args.n + col0;
    const bool vec = args.n % 4 == 0;
    if (vec) {
        // all slices' loads are issued before the first addition (split_k <= 8): the partial sums are L2 hits
        // whose latency, one after the other, used to be most of this kernel's time
        float4 v[8];
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
            v[ks] = ks < split_k ? __ldcg(reinterpret_cast<const float4*>(p + ks * slice)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            if (ks < split_k) { acc[0] += v[ks].x; acc[1] += v[ks].y; acc[2] += v[ks].z; acc[3] += v[ks].w; }
        }
    } else {
        for (int ks = 0; ks < split_k; ++ks, p += slice)
            for (int i = 0; i < 4; ++i)
                if (col0 + i < args.n) acc[i] += p[i];
    }
    const float rs = args.row_scale != nullptr ? args.row_scale[row] : 1.0f;
    float x[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        x[i] = __fmul_rn(__fmul_rn(acc[i], s1), s2);
        if (args.row_scale != nullptr) x[i] = __fmul_rn(x[i], rs);
        if (args.col_scale != nullptr && col0 + i < args.n) x[i] = __fmul_rn(x[i], args.col_scale[col0 + i]);
    }
    const size_t off = static_cast<size_t>(row) * args.ldc + col0;
    if (vec && args.ldc % 4 == 0) {
        if (args.out_bf16) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(x[0], x[1]), hi = __floats2bfloat162_rn(x[2], x[3]);
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(args.c) + off) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
        } else {
            *reinterpret_cast<float4*>(static_cast<float*>(args.c) + off) = make_float4(x[0], x[1], x[2], x[3]);
        }
        return;
    }
    for (int i = 0; i < 4; ++i) {
        if (col0 + i >= args.n) break;
        if (args.out_bf16) static_cast<__nv_bfloat16*>(args.c)[off + i] = __float2bfloat16_rn(x[i]);
        else static_cast<float*>(args.c)[off + i] = x[i];
    }
}

// One bounded wait on a barrier that nothing signals: the give-up path, on purpose.
__global__ void bounded_wait_selftest_kernel(uint32_t* status, unsigned limit_us) {
    __shared__ uint64_t bar;
    __shared__ uint32_t flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        flag = 0;
        fence_mbar_init();
        const bool ok = mbar_wait(&bar, 0, &flag, ST_TIMEOUT_TEST, static_cast<uint64_t>(limit_us) * 1000ull);
        if (!ok && status != nullptr) atomicOr(status, flag);
    }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encoder() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
        if (q != cudaDriverEntryPointSuccess) return nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Byte tensor [d2][d1][d0] (d0 contiguous) with a box of box0 x box1 x 1 and the 128-byte swizzle.
// An encoded map is a pure function of these seven values, so each host thread keeps the last few it
// encoded (weights and reused activation buffers come back call after call) and skips the driver call.
bool make_tmap_u8(CUtensorMap* m, const void* base, uint64_t d0, uint64_t d1, uint64_t d2, uint32_t box0,
                  uint32_t box1) {
    struct Entry {
        const void* base;
        uint64_t d0, d1, d2;
        uint32_t box0, box1;
        bool valid;
        CUtensorMap map;
    };
    constexpr int kSlots = 64;
    thread_local Entry cache[kSlots] = {};
    uint64_t h = reinterpret_cast<uintptr_t>(base) >> 4;
    h = (h ^ (d0 * 0x9E3779B97F4A7C15ull) ^ (d1 * 0xC2B2AE3D27D4EB4Full) ^ (d2 << 7) ^ (static_cast<uint64_t>(box1) << 20) ^ box0) *
        0xD6E8FEB86659FD93ull;
    Entry& e = cache[(h >> 40) % kSlots];
    if (e.valid && e.base == base && e.d0 == d0 && e.d1 == d1 && e.d2 == d2 && e.box0 == box0 && e.box1 == box1) {
        *m = e.map;
        return true;
    }
    EncodeTiledFn enc = get_encoder();
    if (enc == nullptr) return false;
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {d0, d0 * d1};
    cuuint32_t box[3] = {box0, box1, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const cuuint32_t rank = d2 > 0 ? 3 : 2;
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, rank, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    e.base = base; e.d0 = d0; e.d1 = d1; e.d2 = d2; e.box0 = box0; e.box1 = box1;
    e.map = *m;
    e.valid = true;
    return true;
}

int sm_count() {
    static PerDeviceInt cache;   // 0 = not asked yet
    const int dev = current_device_slot();
    if (dev < 0) return 148;
    int n = cache.v[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        int v = 0;
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        n = v > 0 ? v : 148;
        cache.v[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

template <int KIND, int BLOCK_N>
static int launch_one(const void* A, const void* B, const GemmArgs& args, long long max_tiles, cudaStream_t st) {
    using C = Cfg<KIND, BLOCK_N>;
    CUtensorMap ta, tb;
    if (!make_tmap_u8(&ta, A, args.k_bytes, args.m_total, 0, STAGE_KB, BLOCK_M)) return DSL_ERR_DRIVER;
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;
    if (!make_tmap_u8(&tb, B, args.k_bytes, args.n, groups, STAGE_KB, BLOCK_N)) return DSL_ERR_DRIVER;
    static PerDeviceInt attr_set;   // per device; idempotent, a race here only repeats the same call
    const int dev = current_device_slot();
    if (dev < 0) return static_cast<int>(cudaErrorInvalidDevice);
    if (attr_set.v[dev].load(std::memory_order_acquire) == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_kernel<KIND, BLOCK_N>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return static_cast<int>(e);
        attr_set.v[dev].store(1, std::memory_order_release);
    }
    const long long items = max_tiles * (args.split_k > 1 ? args.split_k : 1);
    long long grid = items < sm_count() ? items : sm_count();
    if (grid < 1) grid = 1;
    gemm_kernel<KIND, BLOCK_N><<<static_cast<unsigned>(grid), 192, C::SMEM_BYTES, st>>>(ta, tb, args);
    if (args.split_k > 1) {
        const long long threads = static_cast<long long>(args.m_total) * ((args.n + 3) / 4);
        splitk_reduce_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, st>>>(args, args.split_k);
    }
    return static_cast<int>(cudaGetLastError());
}

// Which kernel serves a problem: the CTA-pair kernel (256x256 tiles) once there is more than
// one 128-row tile of work and the output is at least 256 wide; the 1-CTA kernel otherwise.
// Dense problems with at most DSL_DECODE_MAX_ROWS activation rows go to the weight-streaming kernel when it
// serves them (launch_gemm_decode says so).
// DSLGEMM_KERNEL=1cta|pair|decode overrides the choice (for measurements).
static int forced_kernel() {
    static int v = []() {
        const char* e = getenv("DSLGEMM_KERNEL");
        if (e == nullptr) return 0;
        return strcmp(e, "1cta") == 0 ? 1 : (strcmp(e, "pair") == 0 ? 2 : (strcmp(e, "decode") == 0 ? 3 : 0));
    }();
    return v;
}

int choose_split_k(const GemmArgs& args, long long tiles) {
    if (args.group_offsets != nullptr || args.partial == nullptr || tiles <= 0 || args.act != DSL_ACT_NONE || args.out_sf != nullptr) return 1;
    const int num_kb = (args.k_bytes + STAGE_KB - 1) / STAGE_KB;
    if (tiles * 2 > sm_count() || num_kb < 8) return 1;
    long long want = sm_count() / tiles;
    if (want > 8) want = 8;
    if (want > num_kb / 4) want = num_kb / 4;
    const size_t per_slice = static_cast<size_t>(args.m_total) * args.n * sizeof(float);
    while (want > 1 && per_slice * want > args.partial_bytes) --want;
    if (want < 2) return 1;
    const int kb_per = (num_kb + static_cast<int>(want) - 1) / static_cast<int>(want);
    return (num_kb + kb_per - 1) / kb_per;   // every slice non-empty
}

// Tile shape of the 1-CTA kernel for a problem: 128-wide tiles (two accumulator stages, more CTAs in
// flight) for narrow outputs and whenever 256-wide tiles would leave most SMs without work.
static bool one_cta_tiles(const GemmArgs& args, long long* max_tiles) {
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;
    const long long m_tiles_max = (args.m_total + BLOCK_M - 1) / BLOCK_M + groups - 1;
    const bool narrow = args.n <= 128 || (args.n % 256 != 0 && args.n % 256 <= 128 && args.n < 1024) ||
                        m_tiles_max * ((args.n + 255) / 256) * 2 <= sm_count();
    const int block_n = narrow ? 128 : 256;
    *max_tiles = m_tiles_max * ((args.n + block_n - 1) / block_n);
    return narrow;
}

// Bytes of caller workspace (header included) that launch_gemm would put to use for this problem on
// the current device; 0 when the kernels that serve it need none.  `args.partial` must be non-null
// with a generous `partial_bytes` so that the same decisions are taken as in a real launch.
size_t gemm_workspace_bytes(int kind, const GemmArgs& args) {
    if (args.m_total <= 0 || args.n <= 0) return 0;
    const int forced = forced_kernel();
    if (forced == 0 || forced == 3) {
        bool served = false;
        const size_t b = decode_scratch_bytes(kind, args, &served);
        if (served) return b > 0 ? b + DSL_WS_HEADER_BYTES : 0;
    }
    if (forced == 2 || (forced == 0 && args.m_total > 128 && args.n >= 256)) return 0;
    long long max_tiles = 0;
    one_cta_tiles(args, &max_tiles);
    const int split_k = choose_split_k(args, max_tiles);
    if (split_k <= 1) return 0;
    return DSL_WS_HEADER_BYTES + static_cast<size_t>(split_k) * args.m_total * args.n * sizeof(float);
}

int launch_gemm(int kind, const void* A, const void* B, GemmArgs args, cudaStream_t st) {
    if (args.m_total <= 0 || args.n <= 0) return 0;
    const int forced = forced_kernel();
    if (forced == 0 || forced == 3) {
        const int rc = launch_gemm_decode(kind, A, B, args, st);
        if (rc != DSL_NOT_SERVED) return rc;
    }
    if (forced == 2 || (forced == 0 && args.m_total > 128 && args.n >= 256)) return launch_gemm_pair(kind, A, B, args, st);
    long long max_tiles = 0;
    const bool narrow = one_cta_tiles(args, &max_tiles);
    if (args.band <= 0) args.band = 8;
    // Few tiles and a long K (decode shapes): cut K so that every SM streams part of the weight.
    // Dense problems only; needs caller scratch for the fp32 partial sums.
    args.split_k = choose_split_k(args, max_tiles);
    switch (kind) {
        case KIND_F8:
            return narrow ? launch_one<KIND_F8, 128>(A, B, args, max_tiles, st) : launch_one<KIND_F8, 256>(A, B, args, max_tiles, st);
        case KIND_NVF4:
            return narrow ? launch_one<KIND_NVF4, 128>(A, B, args, max_tiles, st) : launch_one<KIND_NVF4, 256>(A, B, args, max_tiles, st);
        case KIND_MXF4:
            return narrow ? launch_one<KIND_MXF4, 128>(A, B, args, max_tiles, st) : launch_one<KIND_MXF4, 256>(A, B, args, max_tiles, st);
        case KIND_BF16:
            return narrow ? launch_one<KIND_BF16, 128>(A, B, args, max_tiles, st) : launch_one<KIND_BF16, 256>(A, B, args, max_tiles, st);
        default:
            return DSL_ERR_ENUM;
    }
}

int launch_bounded_wait_selftest(uint32_t* status, unsigned limit_us, cudaStream_t st) {
    bounded_wait_selftest_kernel<<<1, 32, 0, st>>>(status, limit_us);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace dsl
