// FP8 E4M3 GEMM with fp32 scales per 128 K-elements on a CTA pair (cta_group::2), dense and grouped:
//
//   C[m, n] = sum_g ( sum_{k in group g} A[m,k] * B[n,k] ) * sa[m, g] * sb[g, n]
//
// (fp8_gemm_groupwise_kernel of the reference, cuda/gemm/fp8_gemm.cu:69-99, group size 128 = one
// shared-memory stage of K).  Same pair structure as gemm_pair.cu: each CTA loads its own halves of
// the 256x256 tile, the leader issues tcgen05.mma.cta_group::2.  fp32 scales cannot ride in the
// MMA, so every K-group's 128x256 partial product (per CTA) lands in one of two tensor-memory
// buffers and eight epilogue warps promote it into register accumulators (acc += p * sa * sb)
// while the tensor cores fill the other buffer.  The promotion streams tensor memory in 16-column
// pieces, the next piece in flight while the current one is multiplied.
//
// Tiles are dealt to the CTA pairs round robin.  The tiles left over after the last full round are cut
// into four 64-column pieces each when all pieces fit into one round (Walker::plan): a piece is a
// pair's last item, multiplies with N = 64 from a tensor map with a 32-row box, and its partial
// products pass through four 64-column buffers with barriers of their own.  The K order per output
// element is unchanged, so the result is bit-identical to the uncut schedule.
//
//   warp 0     TMA producer          warp 1   leader: MMA issuer / peer: "stage landed" forwarder
//   warps 2-9  promotion + epilogue: warp w owns lanes 32*(w%4).. and 128 of the 256 columns (32 of a piece's 64)
#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>

#include "gemm.cuh"
#include "gemm_epilogue.cuh"
#include "gemm_tiles.cuh"
#include "ptx.cuh"

namespace dsl {
namespace gwp {

constexpr int TILE_M = 256;
constexpr int TILE_N = 256;
constexpr int A_STAGE = 128 * STAGE_KB;
constexpr int B_STAGE = 128 * STAGE_KB;
constexpr int NUM_STAGES = 6;
constexpr int OFF_A = 0;
constexpr int OFF_B = NUM_STAGES * A_STAGE;
constexpr int OFF_BAR = OFF_B + NUM_STAGES * B_STAGE;
constexpr int NARROW_RING = 4;                // accumulator buffers of a narrow piece (64 columns each)
constexpr int NUM_BARS = 3 * NUM_STAGES + 4 + 2 * NARROW_RING;
constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
constexpr int OFF_TABLE = OFF_MISC + 16;
constexpr int SMEM_BYTES = OFF_TABLE + 2 * (DSL_MAX_GROUPS + 1) * 4 + 1024;
// Promotion warps per CTA: 4 lane quarters x PARTS column parts.  Measured on 4096 x 4096 x 14336 (kernel alone, cool):
// 8 warps x 128 columns 1929 TFLOP/s, 16 warps x 64 columns (96 registers per thread) 1219 TFLOP/s - more warps
// polling tensor memory at once make every load slower, they do not hide its latency.  -DDSL_GWP_PARTS=4 rebuilds the
// 16-warp form.
#ifndef DSL_GWP_PARTS
#define DSL_GWP_PARTS 2
#endif
constexpr int PARTS = DSL_GWP_PARTS;            // 2: 8 warps x 128 columns, 4: 16 warps x 64 columns
constexpr int PROMO_WARPS = 4 * PARTS;
constexpr int THREADS = 64 + 32 * PROMO_WARPS;
static_assert(SMEM_BYTES > 116224 && SMEM_BYTES <= 232448, "one CTA per SM");

constexpr int NARROW_N = 64;                 // width of the pieces a last-round tile is cut into
constexpr int NARROW_PARTS = TILE_N / NARROW_N;
constexpr int B_NARROW = (NARROW_N / 2) * STAGE_KB;   // bytes of B each CTA loads per stage for a narrow piece

struct Tile {
    int group, row0, row_end, n0, width;
};

struct Walker {
    const int* offs;
    const int* tile0;
    int groups, m_tiles, n_tiles, band;
    int total;         // 256 x 256 tiles (the launcher refuses shapes with more than 2^29 of them)
    int full;          // tiles [0, full) run at full width; each tile of [full, total) as NARROW_PARTS pieces
    int items;         // work items of the whole launch
    // The tiles left over after the last full round of the grid would keep a few CTA pairs busy for a whole
    // tile time while the others idle; when all their 64-column pieces fit into one round they are cut up.
    // Every output element still sums the same K groups in the same order, so the result does not change.
    __host__ __device__ __forceinline__ void plan(int pairs) {
        const int rest = total % pairs;
        full = (total > pairs && rest > 0 && rest * NARROW_PARTS <= pairs) ? total - rest : total;
        items = full + (total - full) * NARROW_PARTS;
    }
    __host__ __device__ __forceinline__ Tile decode(int item) const {
        int t = item, part = 0, width = TILE_N;
        if (item >= full) {
            const int q = item - full;
            t = full + q / NARROW_PARTS;
            part = q % NARROW_PARTS;
            width = NARROW_N;
        }
        const int per_band = m_tiles * band;
        const int b = t / per_band;
        const int r = t - b * per_band;
        const int nb0 = b * band;
        const int wb = band < n_tiles - nb0 ? band : n_tiles - nb0;
        const int mt = r / wb;
        const int nt = nb0 + (r - mt * wb);
        int lo = 0, hi = groups;
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (tile0[mid] <= mt) lo = mid; else hi = mid;
        }
        Tile ti;
        ti.group = lo;
        ti.row0 = offs[lo] + (mt - tile0[lo]) * TILE_M;
        ti.row_end = offs[lo + 1];
        ti.n0 = nt * TILE_N + part * NARROW_N;
        ti.width = width;
        return ti;
    }
};

}  // namespace gwp

// One tile of the promotion warps' work: PIECES 16-column pieces of this warp's part of the tile, K group by K group.
// A warp's share is PIECES * 16 adjacent columns, part p starting right after part p - 1's.  The partial products arrive
// in a ring of RING tensor-memory buffers `buf_cols` columns apart; `step` counts the K groups this ring has carried.
// acc = p * s + acc on two adjacent columns with one packed instruction (fma.rn.f32x2: two IEEE fused multiply-adds,
// the same bits as two fmaf calls)
__device__ __forceinline__ void fma_pair(float& a0, float& a1, uint32_t p0, uint32_t p1, unsigned long long s2) {
    unsigned long long a, p;
    asm("mov.b64 %0, {%1, %2};" : "=l"(a) : "f"(a0), "f"(a1));
    asm("mov.b64 %0, {%1, %2};" : "=l"(p) : "r"(p0), "r"(p1));
    asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(a) : "l"(p), "l"(s2));
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a0), "=f"(a1) : "l"(a));
}

template <bool SB_BLOCK, bool ACT, int PIECES, int RING, bool FMA2 = true>
__device__ __forceinline__ bool promote_tile(const GemmArgs& args, const gwp::Tile& ti, int num_kb, int nb128, uint32_t tmem_base,
                                             uint64_t* part_full, uint64_t* part_empty, volatile uint32_t* abort_flag,
                                             uint32_t& step, int rank, int quad, int half, int lane, int buf_cols) {
    using namespace gwp;
    const int row = ti.row0 + 128 * rank + quad * 32 + lane;
    const bool row_ok = row < ti.row_end;
    const int col_base = ti.n0 + half * (PIECES * 16);
    const float* sa_row = args.gsa + static_cast<size_t>(row_ok ? row : ti.row0) * num_kb;
    const float* sb_ptr;
    if (SB_BLOCK) {
        const int nb = min(col_base / 128, nb128 - 1);
        sb_ptr = args.gsb + (static_cast<size_t>(ti.group) * nb128 + nb) * num_kb;
    } else {
        sb_ptr = args.gsb + static_cast<size_t>(ti.group) * num_kb * args.n;
    }
    float acc[PIECES * 16];
#pragma unroll
    for (int i = 0; i < PIECES * 16; ++i) acc[i] = 0.f;
    float sa_next = __ldg(sa_row);
    float sb_next = SB_BLOCK ? __ldg(sb_ptr) : 0.f;
    for (int kb = 0; kb < num_kb; ++kb, ++step) {
        const float sa = sa_next;
        const float s = SB_BLOCK ? __fmul_rn(sa, sb_next) : 0.f;
        if (kb + 1 < num_kb) {   // next group's scales are fetched while this one is promoted
            sa_next = __ldg(sa_row + kb + 1);
            if (SB_BLOCK) sb_next = __ldg(sb_ptr + kb + 1);
        }
        const int p = static_cast<int>(step % RING);
        const uint32_t pphase = (step / RING) & 1u;
        if (!mbar_wait_cluster(part_full + p, pphase, abort_flag, ST_TIMEOUT_EPILOGUE)) return false;
        tc_fence_after();
        const uint32_t taddr = tmem_base + p * buf_cols + half * (PIECES * 16) + (static_cast<uint32_t>(quad * 32) << 16);
        uint32_t buf[2][16];
        tmem_ld_32x32b_x16(taddr, buf[0]);
#pragma unroll
        for (int c = 0; c < PIECES; ++c) {
            tmem_ld_wait();
            if (c + 1 < PIECES) {
                tmem_ld_32x32b_x16(taddr + (c + 1) * 16, buf[(c + 1) & 1]);
            } else {   // the whole partial product is in registers: hand the buffer back now
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(part_empty + p, 0);
            }
            if (SB_BLOCK && FMA2) {
                unsigned long long s2;
                asm("mov.b64 %0, {%1, %1};" : "=l"(s2) : "f"(s));
#pragma unroll
                for (int i = 0; i < 16; i += 2)
                    fma_pair(acc[c * 16 + i], acc[c * 16 + i + 1], buf[c & 1][i], buf[c & 1][i + 1], s2);
            } else if (SB_BLOCK) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    acc[c * 16 + i] = fmaf(__uint_as_float(buf[c & 1][i]), s, acc[c * 16 + i]);
            } else {
                const float* sbrow = sb_ptr + static_cast<size_t>(kb) * args.n;
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    const int col = col_base + c * 16 + i;
                    const float sb = col < args.n ? __ldg(sbrow + col) : 0.f;
                    acc[c * 16 + i] = fmaf(__fmul_rn(__uint_as_float(buf[c & 1][i]), sa), sb, acc[c * 16 + i]);
                }
            }
        }
    }
    if (!row_ok) return true;
    // read here, once per tile, so that they hold no registers during the promotion
    const float s1 = args.s1_dev != nullptr ? *args.s1_dev : args.s1;
    const float s2 = args.s2_dev != nullptr ? *args.s2_dev : args.s2;
    const bool vec_ok = args.out_bf16 ? (args.ldc % 8 == 0) : (args.ldc % 4 == 0);
    const float rs = args.row_scale != nullptr ? args.row_scale[row] : 1.0f;
#pragma unroll
    for (int c = 0; c < PIECES / 2; ++c) {
        const int col0 = col_base + c * 32;
        if (col0 >= args.n) continue;
        uint32_t v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(acc[c * 32 + i]);
        store_chunk32_t<ACT>(args, row, col0, ti.group, v, s1, s2, rs, vec_ok);
    }
    return true;
}

template <bool SB_BLOCK, bool ACT, bool FMA2 = true>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gwp::THREADS, 1)
gemm_fp8_groupwise_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                               const __grid_constant__ CUtensorMap tmap_b_narrow, const GemmArgs args) {
    using namespace gwp;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + OFF_BAR);
    uint64_t* peer_full = full_bar + NUM_STAGES;      // leader only
    uint64_t* empty_bar = peer_full + NUM_STAGES;
    uint64_t* part_full = empty_bar + NUM_STAGES;     // [2] partial product complete (both CTAs)
    uint64_t* part_empty = part_full + 2;             // [2] leader only: all 16 promotion warps drained the buffer
    uint64_t* nar_full = part_empty + 2;              // [NARROW_RING] the same pair of rings for a narrow piece
    uint64_t* nar_empty = nar_full + NARROW_RING;     // [NARROW_RING]
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + OFF_MISC);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + OFF_MISC + 4);
    int* s_offs = reinterpret_cast<int*>(smem + OFF_TABLE);
    int* s_tile0 = s_offs + (DSL_MAX_GROUPS + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;
    const int pair_id = static_cast<int>(blockIdx.x >> 1);
    const int num_pairs = static_cast<int>(gridDim.x >> 1);

    if (threadIdx.x == 0) {
        for (int i = 0; i < NUM_STAGES; ++i) {
            mbar_init(full_bar + i, 1);
            mbar_init(peer_full + i, 1);
            mbar_init(empty_bar + i, 1);
        }
        for (int i = 0; i < 2; ++i) { mbar_init(part_full + i, 1); mbar_init(part_empty + i, 2 * PROMO_WARPS); }
        for (int i = 0; i < NARROW_RING; ++i) { mbar_init(nar_full + i, 1); mbar_init(nar_empty + i, 16); }
        *abort_flag = 0;
        fence_mbar_init();
        prefetch_tmap(&tmap_a);
        prefetch_tmap(&tmap_b);
        prefetch_tmap(&tmap_b_narrow);
    }
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) tmem_alloc_pair(tmem_ptr, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;

    // Everything above touches no global memory, so under programmatic stream serialisation it runs while the
    // preceding kernel of the stream (the activation quantiser) drains; from here on that kernel's results are read.
    griddep_wait();
    load_group_offsets(s_offs, args.group_offsets, groups, args.m_total);
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0;
        for (int g = 0; g < groups; ++g) {
            s_tile0[g] = t;
            const int rows = monotone_rows(s_offs, g);
            if (rows > 0) t += (rows + TILE_M - 1) / TILE_M;
        }
        s_tile0[groups] = t;
    }
    __syncthreads();

    Walker tw;
    tw.offs = s_offs;
    tw.tile0 = s_tile0;
    tw.groups = groups;
    tw.m_tiles = s_tile0[groups];
    tw.n_tiles = (args.n + TILE_N - 1) / TILE_N;
    tw.band = args.band < 1 ? 1 : args.band;
    tw.total = tw.m_tiles * tw.n_tiles;
    tw.plan(num_pairs);
    if (args.whole_tiles_only) { tw.full = tw.total; tw.items = tw.total; }
    const int num_kb = args.k_bytes / STAGE_KB;   // K % 128 == 0

    if (warp == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int t = pair_id; t < tw.items && ok; t += num_pairs) {
            const Tile ti = tw.decode(t);
            const bool narrow = ti.width != TILE_N;
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!mbar_wait_cluster(empty_bar + stage, phase ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                if (elect_one()) {
                    mbar_arrive_expect_tx(full_bar + stage, A_STAGE + (narrow ? B_NARROW : B_STAGE));
                    tma_load_2d(smem + OFF_A + stage * A_STAGE, &tmap_a, full_bar + stage, kb * STAGE_KB,
                                ti.row0 + 128 * static_cast<int>(rank));
                    if (narrow)
                        tma_load_3d(smem + OFF_B + stage * B_STAGE, &tmap_b_narrow, full_bar + stage, kb * STAGE_KB,
                                    ti.n0 + (NARROW_N / 2) * static_cast<int>(rank), ti.group);
                    else
                        tma_load_3d(smem + OFF_B + stage * B_STAGE, &tmap_b, full_bar + stage, kb * STAGE_KB,
                                    ti.n0 + 128 * static_cast<int>(rank), ti.group);
                }
                __syncwarp();
                if (++stage == NUM_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        if (rank == 0) {
            const uint32_t idesc_full = (1u << 4) | (static_cast<uint32_t>(TILE_N >> 3) << 17) |
                                        (static_cast<uint32_t>(TILE_M >> 4) << 24);   // E4M3 x E4M3 -> fp32
            const uint32_t idesc_narrow = (1u << 4) | (static_cast<uint32_t>(NARROW_N >> 3) << 17) |
                                          (static_cast<uint32_t>(TILE_M >> 4) << 24);
            int stage = 0;
            uint32_t phase = 0;
            uint32_t step = 0;   // only its two low bits matter (buffer and phase)
            bool ok = true;
            for (int t = pair_id; t < tw.items && ok; t += num_pairs) {
                // A narrow piece is always a pair's last item (there are at most as many as pairs).  Its partial products
                // go through a ring of four 64-column buffers of their own barriers: with the short MMA the round trip
                // MMA -> promotion -> "buffer free" would otherwise set the pace.  The four buffers lie in the columns
                // of full-width buffer 0, so its last reader must have finished first.
                const bool narrow = t >= tw.full;
                if (narrow) {
                    const uint32_t next0 = (step + 1u) & ~1u;   // the step that would use buffer 0 next
                    if (!mbar_wait_cluster(part_empty + 0, ((next0 >> 1) & 1u) ^ 1u, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    step = 0;
                }
                const uint32_t idesc = narrow ? idesc_narrow : idesc_full;
                uint64_t* acc_full = narrow ? nar_full : part_full;
                uint64_t* acc_empty = narrow ? nar_empty : part_empty;
                const uint32_t ring = narrow ? NARROW_RING : 2;
                const uint32_t ring_shift = narrow ? 2 : 1;
                const uint32_t buf_cols = narrow ? NARROW_N : TILE_N;
                for (int kb = 0; kb < num_kb; ++kb, ++step) {
                    const uint32_t p = step & (ring - 1u);
                    const uint32_t pphase = (step >> ring_shift) & 1u;
                    if (!mbar_wait_cluster(acc_empty + p, pphase ^ 1u, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    if (!mbar_wait_cluster(peer_full + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    tc_fence_after();
                    const uint64_t adesc = make_desc_sw128(smem_u32(smem + OFF_A + stage * A_STAGE));
                    const uint64_t bdesc = make_desc_sw128(smem_u32(smem + OFF_B + stage * B_STAGE));
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            mma_f8f6f4_pair(tmem_base + p * buf_cols, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0 ? 1u : 0u);
                        tc_commit_pair(empty_bar + stage);
                        tc_commit_pair(acc_full + p);
                    }
                    __syncwarp();
                    if (++stage == NUM_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        } else {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int t = pair_id; t < tw.items && ok; t += num_pairs) {
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!mbar_wait(full_bar + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                    if (lane == 0) mbar_arrive_cluster(peer_full + stage, 0);
                    __syncwarp();
                    if (++stage == NUM_STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else {
        // ================= promotion + epilogue =================
        const int quad = warp & 3;
        const int part = (warp - 2) >> 2;
        const int nb128 = (args.n + 127) / 128;
        uint32_t step = 0;
        bool ok = true;
        for (int t = pair_id; t < tw.items && ok; t += num_pairs) {
            const Tile ti = tw.decode(t);
            // full width: TILE_N / PARTS columns per warp, two buffers; a 64-column piece (a pair's last item) goes to the
            // warps of the first two parts, 32 columns each, through its own ring
            if (ti.width == TILE_N) {
                ok = promote_tile<SB_BLOCK, ACT, TILE_N / (16 * PARTS), 2, FMA2>(args, ti, num_kb, nb128, tmem_base, part_full, part_empty,
                                                                                 abort_flag, step, static_cast<int>(rank), quad, part, lane, TILE_N);
            } else if (part < 2) {
                uint32_t nstep = 0;
                ok = promote_tile<SB_BLOCK, ACT, NARROW_N / 32, NARROW_RING, FMA2>(args, ti, num_kb, nb128, tmem_base, nar_full, nar_empty,
                                                                             abort_flag, nstep, static_cast<int>(rank), quad, part, lane, NARROW_N);
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
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

template <bool SB_BLOCK, bool ACT, bool FMA2 = true>
static int launch_gw_pair(const void* A, const void* B, const GemmArgs& args, cudaStream_t st) {
    CUtensorMap ta, tb, tbn;
    const int groups = args.group_offsets != nullptr ? args.num_groups : 1;
    if (!make_tmap_u8(&ta, A, args.k_bytes, args.m_total, 0, STAGE_KB, 128)) return DSL_ERR_DRIVER;
    if (!make_tmap_u8(&tb, B, args.k_bytes, args.n, groups, STAGE_KB, 128)) return DSL_ERR_DRIVER;
    if (!make_tmap_u8(&tbn, B, args.k_bytes, args.n, groups, STAGE_KB, gwp::NARROW_N / 2)) return DSL_ERR_DRIVER;
    static PerDeviceInt clusters_of;   // per kernel instantiation and device; idempotent set-up
    const int dev = current_device_slot();
    if (dev < 0) return static_cast<int>(cudaErrorInvalidDevice);
    int max_clusters = clusters_of.v[dev].load(std::memory_order_acquire);
    if (max_clusters == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_fp8_groupwise_pair_kernel<SB_BLOCK, ACT, FMA2>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, gwp::SMEM_BYTES);
        if (e != cudaSuccess) return static_cast<int>(e);
        const int sms = sm_count();
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(static_cast<unsigned>(sms > 1 ? (sms / 2) * 2 : 2));
        cfg.blockDim = dim3(gwp::THREADS);
        cfg.dynamicSmemBytes = gwp::SMEM_BYTES;
        int n = 0;
        e = cudaOccupancyMaxActiveClusters(&n, gemm_fp8_groupwise_pair_kernel<SB_BLOCK, ACT, FMA2>, &cfg);
        max_clusters = (e == cudaSuccess && n > 0) ? n : (sms > 1 ? sms / 2 : 1);
        (void)cudaGetLastError();
        clusters_of.v[dev].store(max_clusters, std::memory_order_release);
    }
    const long long m_tiles_max = (args.m_total + gwp::TILE_M - 1) / gwp::TILE_M + groups - 1;
    const long long max_tiles = m_tiles_max * ((args.n + gwp::TILE_N - 1) / gwp::TILE_N);
    if (max_tiles > (1ll << 29)) return DSL_ERR_SHAPE;   // tile counters in the kernel are 32-bit
    long long clusters = max_tiles < max_clusters ? max_tiles : max_clusters;
    if (clusters < 1) clusters = 1;
    // Launched with programmatic stream serialisation: the grid's set-up overlaps the tail of the preceding kernel
    // of the stream when that kernel allows it (the quantisers do); the kernel's griddep_wait() guards the rest.
    // DSLGEMM_PDL=0 launches it the plain way (for measurements).
    static const bool pdl = [] { const char* e = getenv("DSLGEMM_PDL"); return !(e != nullptr && e[0] == '0'); }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(2 * clusters));
    cfg.blockDim = dim3(gwp::THREADS);
    cfg.dynamicSmemBytes = gwp::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_fp8_groupwise_pair_kernel<SB_BLOCK, ACT, FMA2>, ta, tb, tbn, args));
}

// The kernel's work list, computed on the host with the kernel's own Walker (no CUDA call): item i of the launch goes
// to CTA pair i % pairs and is written as six ints {pair, group, row0, row_end, n0, width}.  Returns the number of
// items, or -1 when `max_items` is too small.  For tests of the schedule (every output element covered exactly once).
int groupwise_pair_schedule_host(const int* group_offsets, int groups, int m_total, int n, int pairs, int band, int whole_tiles_only,
                                 int* out, int max_items) {
    using namespace gwp;
    if (group_offsets == nullptr) groups = 1;
    int* tile0 = static_cast<int*>(malloc(sizeof(int) * 2 * (groups + 1)));
    if (tile0 == nullptr) return -1;
    int* offs = tile0 + (groups + 1);   // the kernel's own sanitised copy of the offsets
    for (int g = 0; g <= groups; ++g)
        offs[g] = group_offsets != nullptr ? clamp_offset(group_offsets[g], m_total) : (g == 0 ? 0 : m_total);
    int t = 0;
    for (int g = 0; g < groups; ++g) {
        tile0[g] = t;
        const int rows = monotone_rows(offs, g);
        if (rows > 0) t += (rows + TILE_M - 1) / TILE_M;
    }
    tile0[groups] = t;
    Walker tw;
    tw.offs = offs;
    tw.tile0 = tile0;
    tw.groups = groups;
    tw.m_tiles = t;
    tw.n_tiles = (n + TILE_N - 1) / TILE_N;
    tw.band = band < 1 ? 8 : band;
    tw.total = tw.m_tiles * tw.n_tiles;
    tw.plan(pairs);
    if (whole_tiles_only) { tw.full = tw.total; tw.items = tw.total; }
    int count = tw.items;
    if (count > max_items) count = -1;
    for (int i = 0; i < count; ++i) {
        const Tile ti = tw.decode(i);
        int* o = out + 6 * i;
        o[0] = i % pairs; o[1] = ti.group; o[2] = ti.row0; o[3] = ti.row_end; o[4] = ti.n0; o[5] = ti.width;
    }
    free(tile0);
    return count;
}

int launch_gemm_fp8_groupwise_pair(const void* A, const void* B, GemmArgs args, cudaStream_t st) {
    if (args.m_total <= 0 || args.n <= 0) return 0;
    if (args.band <= 0) args.band = 8;
    {   // DSLGEMM_WHOLE_TILES=1 keeps every tile whole (for measurements)
        static const int whole = [] { const char* e = getenv("DSLGEMM_WHOLE_TILES"); return (e != nullptr && e[0] == '1') ? 1 : 0; }();
        args.whole_tiles_only = whole;
    }
    // two instantiations: the plain epilogue keeps the promotion loop free of spills, the activation one is larger
    if (args.act != DSL_ACT_NONE)
        return args.sb_block ? launch_gw_pair<true, true>(A, B, args, st) : launch_gw_pair<false, true>(A, B, args, st);
    // block scales: the promotion multiplies two columns per instruction (fma.rn.f32x2: 1864 -> 1929 TFLOP/s cool,
    // 1544 -> 1590 at the power cap on 4096 x 4096 x 14336); DSLGEMM_GW_FMA2=0 selects the scalar form (measurements)
    static const bool scalar_fma = [] { const char* e = getenv("DSLGEMM_GW_FMA2"); return e != nullptr && e[0] == '0'; }();
    if (args.sb_block && scalar_fma) return launch_gw_pair<true, false, false>(A, B, args, st);
    return args.sb_block ? launch_gw_pair<true, false>(A, B, args, st) : launch_gw_pair<false, false>(A, B, args, st);
}

}  // namespace dsl
