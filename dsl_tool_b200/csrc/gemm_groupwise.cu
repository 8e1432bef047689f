// FP8 E4M3 GEMM with fp32 scales per 128 K-elements (1x128 activation groups; per-column or
// 128x128-block weight scales), dense and grouped:
//
//   C[m, n] = sum_g ( sum_{k in group g} A[m,k] * B[n,k] ) * sa[m, g] * sb[g, n]
//
// which is what fp8_gemm_groupwise_kernel of the reference computes (cuda/gemm/fp8_gemm.cu:69-99),
// with the group size fixed at 128 = one shared-memory stage of K.
//
// fp32 scales cannot ride inside the tensor-core instruction, so every K-group's partial
// product is formed by four tcgen05.mma steps into one of two 128x256 fp32 buffers in tensor
// memory and promoted into register accumulators by eight epilogue warps
// (acc += partial * sa * sb) while the tensor core already fills the other buffer.
//
//   warp 0      TMA producer (as in gemm.cu)
//   warp 1      MMA issuer: per stage waits for a free partial buffer, issues 4 MMAs, commits
//               the stage back to the producer and the partial buffer to the epilogue
//   warps 2-9   epilogue: warp w owns tensor-memory lanes 32*(w%4).. and 128 of the 256 columns
#include <cuda_bf16.h>
#include <stdlib.h>
#include <string.h>

#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_tiles.cuh"
#include "ptx.cuh"

namespace dsl {

namespace gw {
constexpr int BLOCK_N = 256;
constexpr int A_STAGE = BLOCK_M * STAGE_KB;
constexpr int B_STAGE = BLOCK_N * STAGE_KB;
constexpr int NUM_STAGES = 4;
constexpr int OFF_A = 0;
constexpr int OFF_B = NUM_STAGES * A_STAGE;
constexpr int OFF_BAR = OFF_B + NUM_STAGES * B_STAGE;
constexpr int NUM_BARS = 2 * NUM_STAGES + 4;
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
constexpr int OFF_TABLE = OFF_MISC + 16;
constexpr int SMEM_BYTES = OFF_TABLE + 2 * (DSL_MAX_GROUPS + 1) * 4 + 1024;
constexpr int THREADS = 320;
static_assert(SMEM_BYTES > 116224 && SMEM_BYTES <= 232448, "one CTA per SM");
}  // namespace gw

template <bool SB_BLOCK, bool ACT>
__global__ void __launch_bounds__(gw::THREADS, 1)
gemm_fp8_groupwise_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const GemmArgs args) {
    using namespace gw;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* empty_bar = full_bar + NUM_STAGES;
    uint64_t* part_full = empty_bar + NUM_STAGES;   // [2] partial product ready in tensor memory
    uint64_t* part_empty = part_full + 2;           // [2] partial buffer drained by all 8 epilogue warps
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC + 4);
    int* s_offs = reinterpret_cast<int*>(smem + OFF_TABLE);
    int* s_tile0 = s_offs + (DSL_MAX_GROUPS + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < NUM_STAGES; ++i) { mbar_init(full_bar + i, 1); mbar_init(empty_bar + i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(part_full + i, 1); mbar_init(part_empty + i, 8); }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    build_tile_tables(s_offs, s_tile0, args.group_offsets, groups, args.m_total);
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
    const int num_kb = args.k_bytes / STAGE_KB;   // K % 128 == 0

    if (warp == 0) {
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long t = blockIdx.x; t < tw.total && ok; t += gridDim.x) {
                const TileInfo ti = tw.decode(t);
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    mbar_arrive_expect_tx(full_bar + stage, A_STAGE + B_STAGE);
                    tma_load_2d(smem + OFF_A + stage * A_STAGE, &tmap_a, full_bar + stage, kb * STAGE_KB, ti.row0);
                    tma_load_3d(smem + OFF_B + stage * B_STAGE, &tmap_b, full_bar + stage, kb * STAGE_KB, ti.n0, ti.group);
                    if (++stage == NUM_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(BLOCK_N >> 3) << 17) |
                                   (static_cast<uint32_t>(BLOCK_M >> 4) << 24);   // E4M3 x E4M3 -> fp32
            int stage = 0;
            uint32_t phase = 0;
            long long step = 0;   // K-groups issued so far by this CTA; buffer = step & 1
            bool ok = true;
            for (long long t = blockIdx.x; t < tw.total && ok; t += gridDim.x) {
                for (int kb = 0; kb < num_kb; ++kb, ++step) {
                    const int p = static_cast<int>(step & 1);
                    const uint32_t pphase = static_cast<uint32_t>((step >> 1) & 1);
                    if (!mbar_wait(part_empty + p, pphase ^ 1u, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t adesc = make_desc_sw128(smem_u32(smem + OFF_A + stage * A_STAGE));
                    const uint64_t bdesc = make_desc_sw128(smem_u32(smem + OFF_B + stage * B_STAGE));
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        mma_f8f6f4(tmem_base + p * BLOCK_N, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
                    tc_commit(empty_bar + stage);
                    tc_commit(part_full + p);
                    if (++stage == NUM_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
        const int quad = warp & 3;
        const int half = (warp - 2) >> 2;   // which 128 of the tile's 256 columns
        float s1 = args.s1_dev != nullptr ? *args.s1_dev : args.s1;
        float s2 = args.s2_dev != nullptr ? *args.s2_dev : args.s2;
        const bool vec_ok = args.out_bf16 ? (args.ldc % 8 == 0) : (args.ldc % 4 == 0);
        const int nb128 = (args.n + 127) / 128;
        long long step = 0;
        bool ok = true;
        for (long long t = blockIdx.x; t < tw.total && ok; t += gridDim.x) {
            const TileInfo ti = tw.decode(t);
            const int row = ti.row0 + quad * 32 + lane;
            const bool row_ok = row < ti.row_end;
            const int col_base = ti.n0 + half * 128;
            const float* sa_row = args.gsa + static_cast<size_t>(row_ok ? row : ti.row0) * num_kb;
            // block scales: one value per (128 columns, K-group); per-column: a row of n values per K-group
            const float* sb_ptr;
            if (SB_BLOCK) {
                const int nb = min(col_base / 128, nb128 - 1);
                sb_ptr = args.gsb + (static_cast<size_t>(ti.group) * nb128 + nb) * num_kb;
            } else {
                sb_ptr = args.gsb + static_cast<size_t>(ti.group) * num_kb * args.n;
            }
            float acc[128];
#pragma unroll
            for (int i = 0; i < 128; ++i) acc[i] = 0.f;
            float sa_next = sa_row[0];
            float sb_next = SB_BLOCK ? sb_ptr[0] : 0.f;
            for (int kb = 0; kb < num_kb; ++kb, ++step) {
                const float sa = sa_next;
                const float sbk = sb_next;
                if (kb + 1 < num_kb) {   // fetch the next group's scales while this one is promoted
                    sa_next = sa_row[kb + 1];
                    if (SB_BLOCK) sb_next = sb_ptr[kb + 1];
                }
                const int p = static_cast<int>(step & 1);
                const uint32_t pphase = static_cast<uint32_t>((step >> 1) & 1);
                if (!mbar_wait(part_full + p, pphase, abort_flag, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
                tc_fence_after();
                const uint32_t taddr = tmem_base + p * BLOCK_N + half * 128 + (static_cast<uint32_t>(quad * 32) << 16);
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32b_x32(taddr + c * 32, v);
                    tmem_ld_wait();
                    if (SB_BLOCK) {
                        const float s = __fmul_rn(sa, sbk);
#pragma unroll
                        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = fmaf(__uint_as_float(v[i]), s, acc[c * 32 + i]);
                    } else {
                        const float* sbrow = sb_ptr + static_cast<size_t>(kb) * args.n;
#pragma unroll
                        for (int i = 0; i < 32; ++i) {
                            const int col = col_base + c * 32 + i;
                            const float sb = col < args.n ? __ldg(sbrow + col) : 0.f;
                            acc[c * 32 + i] = fmaf(__fmul_rn(__uint_as_float(v[i]), sa), sb, acc[c * 32 + i]);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(part_empty + p);
            }
            if (!ok) break;
            if (!row_ok) continue;
            const float rs = args.row_scale != nullptr ? args.row_scale[row] : 1.0f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int col0 = col_base + c * 32;
                if (col0 >= args.n) continue;
                uint32_t v[32];
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(acc[c * 32 + i]);
                store_chunk32_t<ACT>(args, row, col0, ti.group, v, s1, s2, rs, vec_ok);
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    const uint32_t aborted = *abort_flag;
    if (aborted != 0) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(2000);
        if (threadIdx.x == 0 && args.status != nullptr) atomicOr(args.status, aborted);
    }
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <bool SB_BLOCK, bool ACT>
static int launch_gw(const void* A, const void* B, const GemmArgs& args, cudaStream_t st) {
    CUtensorMap ta, tb;
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;
    if (!make_tmap_u8(&ta, A, args.k_bytes, args.m_total, 0, STAGE_KB, BLOCK_M)) return DSL_ERR_DRIVER;
    if (!make_tmap_u8(&tb, B, args.k_bytes, args.n, groups, STAGE_KB, gw::BLOCK_N)) return DSL_ERR_DRIVER;
    static PerDeviceInt attr_set;   // per device
    const int dev = current_device_slot();
    if (dev < 0) return static_cast<int>(cudaErrorInvalidDevice);
    if (attr_set.v[dev].load(std::memory_order_acquire) == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_fp8_groupwise_kernel<SB_BLOCK, ACT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, gw::SMEM_BYTES);
        if (e != cudaSuccess) return static_cast<int>(e);
        attr_set.v[dev].store(1, std::memory_order_release);
    }
    const long long m_tiles_max = (args.m_total + BLOCK_M - 1) / BLOCK_M + groups - 1;
    const long long max_tiles = m_tiles_max * ((args.n + gw::BLOCK_N - 1) / gw::BLOCK_N);
    long long grid = max_tiles < sm_count() ? max_tiles : sm_count();
    if (grid < 1) grid = 1;
    gemm_fp8_groupwise_kernel<SB_BLOCK, ACT><<<static_cast<unsigned>(grid), gw::THREADS, gw::SMEM_BYTES, st>>>(ta, tb, args);
    return static_cast<int>(cudaGetLastError());
}

int launch_gemm_fp8_groupwise(const void* A, const void* B, GemmArgs args, cudaStream_t st) {
    if (args.m_total <= 0 || args.n <= 0) return 0;
    const char* forced = getenv("DSLGEMM_KERNEL");
    const bool force_1cta = forced != nullptr && strcmp(forced, "1cta") == 0;
    if (!force_1cta && args.m_total > 128 && args.n >= 256) return launch_gemm_fp8_groupwise_pair(A, B, args, st);
    if (args.band <= 0) args.band = 8;
    // two instantiations: the plain epilogue keeps the promotion loop free of spills, the activation one is larger
    if (args.act != DSL_ACT_NONE)
        return args.sb_block ? launch_gw<true, true>(A, B, args, st) : launch_gw<false, true>(A, B, args, st);
    return args.sb_block ? launch_gw<true, false>(A, B, args, st) : launch_gw<false, false>(A, B, args, st);
}

}  // namespace dsl
