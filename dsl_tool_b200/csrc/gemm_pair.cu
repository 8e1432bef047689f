// CTA-pair (cta_group::2) tcgen05 GEMM for sm_100a: two CTAs of a thread-block cluster share one
// 256x256 output tile.  CTA r of the pair loads A rows [128r, 128r+128) and B rows (output
// columns) [128r, 128r+128) of the tile with its own plain TMA loads (nothing is multicast);
// one tcgen05.mma.cta_group::2 issued by the leader CTA drives both SMs' tensor cores, each
// accumulating its 128 x 256 half in its own tensor memory.  Per SM this halves the weight
// bytes staged per MMA and lets one instruction carry twice the work of the 1-CTA kernel.
//
// Roles per CTA (192 threads):
//   warp 0     TMA producer for this CTA's operand halves and scale-factor tiles
//   warp 1     leader CTA: MMA issuer (scale tiles shared -> tensor memory in both CTAs, MMAs,
//              commits multicast to both CTAs' barriers); peer CTA: forwards "my stage has
//              landed" to the leader
//   warps 2-5  epilogue of this CTA's 128 rows
// Same formats, tile order and ragged-group scheduling as gemm.cu.  Every wait is bounded.
#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>

#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_tiles.cuh"
#include "ptx.cuh"

namespace dsl {
namespace pr {

constexpr int TILE_M = 256;
constexpr int TILE_N = 256;
// Tensor-memory columns.  Plain kinds: two 256-column accumulators.  Block-scaled kinds need 48
// columns for the scale factors, so their two accumulators overlap in columns [192, 256): tile i
// uses [0, 256) or [192, 448) in turn, and the epilogue reads the shared 64 columns first and
// releases them, so the next tile's MMAs start while the other 192 columns are still being read.
constexpr int SFA_COL = 448;
constexpr int SFB_COL = 464;
constexpr int OVERLAP_COL = 192;

template <int KIND>
struct Cfg {
    static constexpr int A_STAGE = 128 * STAGE_KB;
    static constexpr int B_STAGE = 128 * STAGE_KB;
    static constexpr int SF_ATOMS = KIND == KIND_NVF4 ? 4 : (KIND == KIND_MXF4 ? 2 : 0);
    static constexpr int SFA_STAGE = SF_ATOMS * 512;          // this CTA's 128 A rows
    static constexpr int SFB_STAGE = 2 * SF_ATOMS * 512;      // all 256 output columns
    static constexpr int NUM_STAGES = SF_ATOMS > 0 ? 5 : 6;
    static constexpr int ACC_STAGES = 2;
    static constexpr int ACC1_COL = SF_ATOMS > 0 ? OVERLAP_COL : TILE_N;
    static constexpr int OFF_A = 0;
    static constexpr int OFF_B = OFF_A + NUM_STAGES * A_STAGE;
    static constexpr int OFF_SFA = OFF_B + NUM_STAGES * B_STAGE;
    static constexpr int OFF_SFB = OFF_SFA + NUM_STAGES * SFA_STAGE;
    static constexpr int OFF_BAR = OFF_SFB + NUM_STAGES * SFB_STAGE;
    static constexpr int NUM_BARS = 3 * NUM_STAGES + 2 * ACC_STAGES + 1;
    static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
    static constexpr int OFF_TABLE = OFF_MISC + 16;                         // offs, tile0, sftile0
    static constexpr int OFF_EPI = (OFF_TABLE + 3 * (DSL_MAX_GROUPS + 1) * 4 + 15) & ~15;   // 4 epilogue warps x 2 KB exchange
    static constexpr int SMEM_BYTES = OFF_EPI + 4 * 2048 + 1024;
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
    static_assert(SMEM_BYTES > 116224, "two CTAs could share an SM and deadlock on tensor-memory allocation");
};

struct PairTile {
    int group, row0, row_end, n0, sf_tile;   // row0 / sf_tile are those of the pair's first 128 rows
};

struct PairWalker {
    const int* offs;
    const int* tile0;     // first 256-row tile of each group
    const int* sft0;      // first 128-row scale tile of each group
    int groups, m_tiles, n_tiles, band;
    long long total;
    __device__ __forceinline__ PairTile decode(long long t) const {
        const long long per_band = static_cast<long long>(m_tiles) * band;
        const int b = static_cast<int>(t / per_band);
        const int r = static_cast<int>(t - b * per_band);
        const int nb0 = b * band;
        const int wb = min(band, n_tiles - nb0);
        const int mt = r / wb;
        const int nt = nb0 + (r - mt * wb);
        int lo = 0, hi = groups;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (tile0[mid] <= mt) lo = mid; else hi = mid;
        }
        PairTile ti;
        ti.group = lo;
        ti.row0 = offs[lo] + (mt - tile0[lo]) * TILE_M;
        ti.row_end = offs[lo + 1];
        ti.n0 = nt * TILE_N;
        ti.sf_tile = sft0[lo] + (mt - tile0[lo]) * 2;
        return ti;
    }
};

}  // namespace pr

template <int KIND>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                 const GemmArgs args) {
    using C = pr::Cfg<KIND>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);   // this CTA's stage has landed
    uint64_t* peer_full = full_bar + C::NUM_STAGES;                        // leader only: the peer's stage has landed
    uint64_t* empty_bar = peer_full + C::NUM_STAGES;                       // MMAs reading the stage are done
    uint64_t* acc_full = empty_bar + C::NUM_STAGES;
    uint64_t* acc_empty = acc_full + C::ACC_STAGES;                        // leader only: both epilogues drained
    uint64_t* ovl_free = acc_empty + C::ACC_STAGES;                        // leader only: shared columns of the previous tile read
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC + 4);
    int* s_offs = reinterpret_cast<int*>(smem + C::OFF_TABLE);
    int* s_tile0 = s_offs + (DSL_MAX_GROUPS + 1);
    int* s_sft0 = s_tile0 + (DSL_MAX_GROUPS + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;
    const long long pair_id = blockIdx.x >> 1;
    const long long num_pairs = gridDim.x >> 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::NUM_STAGES; ++i) {
            mbar_init(full_bar + i, 1);
            mbar_init(peer_full + i, 1);
            mbar_init(empty_bar + i, 1);
        }
        for (int i = 0; i < C::ACC_STAGES; ++i) { mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 8); }
        mbar_init(ovl_free, 8);
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
    }
    if (C::SF_ATOMS > 0) {
        uint32_t* z = reinterpret_cast<uint32_t*>(smem + C::OFF_SFA);
        for (int i = threadIdx.x; i < C::NUM_STAGES * (C::SFA_STAGE + C::SFB_STAGE) / 4; i += blockDim.x) z[i] = 0u;
        fence_proxy_async_smem();
    }
    __syncthreads();
    cluster_sync_all();   // both CTAs' barriers exist before anything can signal them
    if (warp == 1) tmem_alloc_pair(tmem_ptr, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    // Everything above touches no global memory, so under programmatic stream serialisation it runs while the
    // preceding kernel of the stream (the activation quantiser) drains; from here on that kernel's results are
    // read (the row-group table first, then operands and scales).
    griddep_wait();
    load_group_offsets(s_offs, args.group_offsets, groups, args.m_total);
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0, st = 0;
        for (int g = 0; g < groups; ++g) {
            s_tile0[g] = t;
            s_sft0[g] = st;
            const int rows = monotone_rows(s_offs, g);
            if (rows > 0) {
                t += (rows + pr::TILE_M - 1) / pr::TILE_M;
                st += (rows + 127) / 128;
            }
        }
        s_tile0[groups] = t;
        s_sft0[groups] = st;
    }
    __syncthreads();

    pr::PairWalker tw;
    tw.offs = s_offs;
    tw.tile0 = s_tile0;
    tw.sft0 = s_sft0;
    tw.groups = groups;
    tw.m_tiles = s_tile0[groups];
    tw.n_tiles = (args.n + pr::TILE_N - 1) / pr::TILE_N;
    tw.band = args.band < 1 ? 1 : args.band;
    tw.total = static_cast<long long>(tw.m_tiles) * tw.n_tiles;
    const int num_kb = (args.k_bytes + STAGE_KB - 1) / STAGE_KB;
    const int sf_tiles_total = s_sft0[groups];

    if (warp == 0) {
        // ================= TMA producer (each CTA loads its own halves) =================
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (long long t = pair_id; t < tw.total && ok; t += num_pairs) {
            const pr::PairTile ti = tw.decode(t);
            const int my_sf_tile = ti.sf_tile + static_cast<int>(rank);
            const bool sfa_valid = C::SF_ATOMS > 0 && my_sf_tile < sf_tiles_total;
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_cluster(empty_bar + stage, phase ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                if (elect_one()) {
                    uint32_t bytes = C::A_STAGE + C::B_STAGE;
                    int atoms = 0;
                    bool sfb_valid[2] = {false, false};
                    if (C::SF_ATOMS > 0) {
                        atoms = min(C::SF_ATOMS, args.sf_katoms - kb * C::SF_ATOMS);
                        if (sfa_valid) bytes += atoms * 512;
                        for (int j = 0; j < 2; ++j) {
                            sfb_valid[j] = ti.n0 / 128 + j < args.sfb_tiles_per_group;
                            if (sfb_valid[j]) bytes += atoms * 512;
                        }
                    }
                    mbar_arrive_expect_tx(full_bar + stage, bytes);
                    tma_load_2d(smem + C::OFF_A + stage * C::A_STAGE, &tmap_a, full_bar + stage, kb * STAGE_KB,
                                ti.row0 + 128 * static_cast<int>(rank));
                    tma_load_3d(smem + C::OFF_B + stage * C::B_STAGE, &tmap_b, full_bar + stage, kb * STAGE_KB,
                                ti.n0 + 128 * static_cast<int>(rank), ti.group);
                    if (C::SF_ATOMS > 0) {
                        const size_t katom0 = static_cast<size_t>(kb) * C::SF_ATOMS;
                        if (sfa_valid)
                            bulk_load(smem + C::OFF_SFA + stage * C::SFA_STAGE,
                                      args.sfa + (static_cast<size_t>(my_sf_tile) * args.sf_katoms + katom0) * 512,
                                      atoms * 512, full_bar + stage);
                        for (int j = 0; j < 2; ++j) {
                            if (!sfb_valid[j]) continue;
                            const size_t rt = static_cast<size_t>(ti.group) * args.sfb_tiles_per_group + ti.n0 / 128 + j;
                            bulk_load(smem + C::OFF_SFB + stage * C::SFB_STAGE + j * C::SFA_STAGE,
                                      args.sfb + (rt * args.sf_katoms + katom0) * 512, atoms * 512, full_bar + stage);
                        }
                    }
                }
                __syncwarp();
                if (++stage == C::NUM_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            // ================= MMA issuer (leader CTA; the warp stays converged, one lane issues) =====
            uint32_t idesc = (static_cast<uint32_t>(pr::TILE_N >> 3) << 17) | (static_cast<uint32_t>(pr::TILE_M >> 4) << 24);
            if (KIND == KIND_F8) idesc |= 1u << 4;
            if (KIND == KIND_NVF4) idesc |= (1u << 7) | (1u << 10);
            if (KIND == KIND_MXF4) idesc |= (1u << 7) | (1u << 10) | (1u << 23);
            if (KIND == KIND_BF16) idesc |= (1u << 4) | (1u << 7) | (1u << 10);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            long long iter = 0;
            for (long long t = pair_id; t < tw.total && ok; t += num_pairs, ++iter) {
                const int acc = static_cast<int>(iter % C::ACC_STAGES);
                const uint32_t acc_phase = static_cast<uint32_t>((iter / C::ACC_STAGES) & 1);
                if (!mbar_wait_cluster(acc_empty + acc, acc_phase ^ 1u, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                if (C::SF_ATOMS > 0 && iter > 0 &&
                    !mbar_wait_cluster(ovl_free, static_cast<uint32_t>((iter - 1) & 1), abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * C::ACC1_COL;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    if (!mbar_wait_cluster(peer_full + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(smem + C::OFF_A + stage * C::A_STAGE);
                    const uint32_t b_addr = smem_u32(smem + C::OFF_B + stage * C::B_STAGE);
                    const uint32_t sfa_addr = smem_u32(smem + C::OFF_SFA + stage * C::SFA_STAGE);
                    const uint32_t sfb_addr = smem_u32(smem + C::OFF_SFB + stage * C::SFB_STAGE);
                    const uint64_t adesc = make_desc_sw128(a_addr);
                    const uint64_t bdesc = make_desc_sw128(b_addr);
                    if (elect_one()) {
                        if (C::SF_ATOMS > 0) {
#pragma unroll
                            for (int i = 0; i < C::SF_ATOMS; ++i) {
                                tc_cp_32x128b_warpx4_pair(tmem_base + pr::SFA_COL + i * 4, make_desc_sf(sfa_addr + i * 512));
#pragma unroll
                                for (int j = 0; j < 2; ++j)
                                    tc_cp_32x128b_warpx4_pair(tmem_base + pr::SFB_COL + i * 8 + j * 4,
                                                              make_desc_sf(sfb_addr + (j * C::SF_ATOMS + i) * 512));
                            }
                        }
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint32_t accum = (kb > 0 || k > 0) ? 1u : 0u;
                            if (KIND == KIND_F8) {
                                mma_f8f6f4_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
                            } else if (KIND == KIND_BF16) {
                                mma_f16_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, accum);
                            } else if (KIND == KIND_NVF4) {
                                mma_nvf4_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, tmem_base + pr::SFA_COL + k * 4,
                                              tmem_base + pr::SFB_COL + k * 8, accum);
                            } else {
                                const uint32_t sf_id = (k & 1) * 2;
                                const uint32_t id = idesc | (sf_id << 29) | (sf_id << 4);
                                mma_mxf4_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, id, tmem_base + pr::SFA_COL + (k >> 1) * 4,
                                              tmem_base + pr::SFB_COL + (k >> 1) * 8, accum);
                            }
                        }
                        tc_commit_pair(empty_bar + stage);
                        if (kb == num_kb - 1) tc_commit_pair(acc_full + acc);
                    }
                    __syncwarp();
                    if (++stage == C::NUM_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        } else {
            // ================= peer CTA: tell the leader when this CTA's stage has landed =================
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long t = pair_id; t < tw.total && ok; t += num_pairs) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    if (lane == 0) mbar_arrive_cluster(peer_full + stage, 0);
                    __syncwarp();
                    if (++stage == C::NUM_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
        // ================= epilogue (this CTA's 128 rows of the pair tile) =================
        const int quad = warp & 3;
        float s1 = args.s1_dev != nullptr ? *args.s1_dev : args.s1;
        float s2 = args.s2_dev != nullptr ? *args.s2_dev : args.s2;
        if (args.scale_product) { s1 = s1 * s2; s2 = 1.0f; }
        const bool vec_ok = args.out_bf16 ? (args.ldc % 8 == 0) : (args.ldc % 4 == 0);
        // plain bf16 results leave through the warp-wide store (rows exchanged in shared memory)
        const bool warp_store = args.out_bf16 && vec_ok && args.act == DSL_ACT_NONE && args.out_sf == nullptr;
        uint8_t* epi_scratch = smem + C::OFF_EPI + (warp - 2) * 2048;
        bool ok = true;
        long long iter = 0;
        for (long long t = pair_id; t < tw.total && ok; t += num_pairs, ++iter) {
            const pr::PairTile ti = tw.decode(t);
            const int acc = static_cast<int>(iter % C::ACC_STAGES);
            const uint32_t acc_phase = static_cast<uint32_t>((iter / C::ACC_STAGES) & 1);
            if (!mbar_wait_cluster(acc_full + acc, acc_phase, abort_flag, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
            tc_fence_after();
            const int row = ti.row0 + 128 * static_cast<int>(rank) + quad * 32 + lane;
            const bool row_ok = row < ti.row_end;
            const float rs = (row_ok && args.row_scale != nullptr) ? args.row_scale[row] : 1.0f;
            // Two chunk buffers: the tensor-memory load of the next 32 columns is in flight while the current
            // ones are scaled, converted and stored (a short-K tile's MMAs are no longer than its epilogue).
            // block-scaled kinds: the 64 columns shared with the other accumulator go first
            const uint32_t t_row = tmem_base + acc * C::ACC1_COL + (static_cast<uint32_t>(quad * 32) << 16);
            const int row_warp = ti.row0 + 128 * static_cast<int>(rank) + quad * 32;
            const bool rot = C::SF_ATOMS > 0 && acc == 0;
            uint32_t va[32], vb[32];
            tmem_ld_32x32b_x32(t_row + (rot ? 6 : 0) * 32, va);
#pragma unroll 1
            for (int j = 0; j < pr::TILE_N / 32; j += 2) {
                const int ca = rot ? ((j + 6) & 7) : j;
                const int cb = rot ? ((j + 7) & 7) : j + 1;
                tmem_ld_wait();
                tmem_ld_32x32b_x32(t_row + cb * 32, vb);
                if (C::SF_ATOMS > 0 && j == 0) {
                    // chunks 0 and 1 of this walk are the columns shared with the other accumulator: hand them back as
                    // soon as both are in registers, before any of the slower scale / convert / store work
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(ovl_free, 0);
                }
                if (warp_store && ti.n0 + ca * 32 + 32 <= args.n)
                    store_chunk32_bf16_warp(args, epi_scratch, row_warp, ti.row_end, ti.n0 + ca * 32, ti.group, va, s1, s2, rs, lane);
                else if (row_ok && ti.n0 + ca * 32 < args.n)
                    store_chunk32(args, row, ti.n0 + ca * 32, ti.group, va, s1, s2, rs, vec_ok, ti.sf_tile + static_cast<int>(rank), quad * 32 + lane);
                tmem_ld_wait();
                if (j + 2 < pr::TILE_N / 32) tmem_ld_32x32b_x32(t_row + (rot ? ((j + 8) & 7) : j + 2) * 32, va);
                if (warp_store && ti.n0 + cb * 32 + 32 <= args.n)
                    store_chunk32_bf16_warp(args, epi_scratch, row_warp, ti.row_end, ti.n0 + cb * 32, ti.group, vb, s1, s2, rs, lane);
                else if (row_ok && ti.n0 + cb * 32 < args.n)
                    store_chunk32(args, row, ti.n0 + cb * 32, ti.group, vb, s1, s2, rs, vec_ok, ti.sf_tile + static_cast<int>(rank), quad * 32 + lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(acc_empty + acc, 0);
        }
    }
    // ---- common exit -------------------------------------------------------------------
    tc_fence_before();
    __syncthreads();
    const uint32_t aborted = *abort_flag;
    if (aborted != 0) {
        const uint64_t t0 = globaltimer_ns();
        while (globaltimer_ns() - t0 < 200000ull) __nanosleep(2000);
        if (threadIdx.x == 0 && args.status != nullptr) atomicOr(args.status, aborted);
    }
    cluster_sync_all();   // the peer's shared memory and barriers stay alive until both CTAs are done
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---- host side ---------------------------------------------------------------------------
template <int KIND>
static int launch_pair_one(const void* A, const void* B, const GemmArgs& args, long long max_tiles, cudaStream_t st) {
    using C = pr::Cfg<KIND>;
    CUtensorMap ta, tb;
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;
    if (!make_tmap_u8(&ta, A, args.k_bytes, args.m_total, 0, STAGE_KB, 128)) return DSL_ERR_DRIVER;
    if (!make_tmap_u8(&tb, B, args.k_bytes, args.n, groups, STAGE_KB, 128)) return DSL_ERR_DRIVER;
    static PerDeviceInt clusters_of;   // per kernel instantiation and device; idempotent set-up
    const int dev = current_device_slot();
    if (dev < 0) return static_cast<int>(cudaErrorInvalidDevice);
    int max_clusters = clusters_of.v[dev].load(std::memory_order_acquire);
    if (max_clusters == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel<KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return static_cast<int>(e);
        const int sms = sm_count();
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(sms > 1 ? (sms / 2) * 2 : 2));
        cfg.blockDim = dim3(192);
        cfg.dynamicSmemBytes = C::SMEM_BYTES;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<KIND>, &cfg);
        max_clusters = (e == cudaSuccess && n > 0) ? n : (sms > 1 ? sms / 2 : 1);
        (void)cudaGetLastError();
        if (getenv("DSLGEMM_DEBUG") != nullptr) fprintf(stderr, "[dslgemm] pair kernel kind %d: %d resident clusters (occupancy query %s)\n", KIND, max_clusters, cudaGetErrorName(e));
        clusters_of.v[dev].store(max_clusters, std::memory_order_release);
    }
    long long clusters = max_tiles < max_clusters ? max_tiles : max_clusters;
    if (clusters < 1) clusters = 1;
    // Launched with programmatic stream serialisation: the grid's set-up (barriers, tensor-memory allocation)
    // overlaps the tail of the preceding kernel of the stream when that kernel allows it (the quantisers do);
    // the kernel's griddep_wait() guards every read of global memory.  DSLGEMM_PDL=0 launches it the plain way.
    static const bool pdl = [] { const char* e = getenv("DSLGEMM_PDL"); return !(e != nullptr && e[0] == '0'); }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<KIND>, ta, tb, args));
}

int launch_gemm_pair(int kind, const void* A, const void* B, GemmArgs args, cudaStream_t st) {
    if (args.m_total <= 0 || args.n <= 0) return 0;
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;
    const long long m_tiles_max = (args.m_total + pr::TILE_M - 1) / pr::TILE_M + groups - 1;
    const long long max_tiles = m_tiles_max * ((args.n + pr::TILE_N - 1) / pr::TILE_N);
    if (args.band <= 0) args.band = 8;
    switch (kind) {
        case KIND_F8: return launch_pair_one<KIND_F8>(A, B, args, max_tiles, st);
        case KIND_NVF4: return launch_pair_one<KIND_NVF4>(A, B, args, max_tiles, st);
        case KIND_MXF4: return launch_pair_one<KIND_MXF4>(A, B, args, max_tiles, st);
        case KIND_BF16: return launch_pair_one<KIND_BF16>(A, B, args, max_tiles, st);
        default: return DSL_ERR_ENUM;
    }
}

}  // namespace dsl
