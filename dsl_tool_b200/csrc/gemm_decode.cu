// Weight-streaming GEMM for decode shapes (few activation rows, one row group): the problem is
// bound by reading the weight once from HBM, so the kernel is organised around that stream.
//
//   * Operand roles are swapped: the WEIGHT tile (128 rows of B, i.e. 128 output columns) is the
//     M = 128 side of tcgen05.mma and the activations (TOK = 16 ... 128 rows of A, zero-filled beyond
//     m_total by the TMA unit) are the N = TOK side.  The accumulator is 128 lanes x TOK columns,
//     so an MMA costs in proportion to the real token count instead of a padded 128-row tile.
//   * Work is cut along K so that every SM streams a share of the weight: the (column tile,
//     K stage) units are laid out end to end and every CTA takes one contiguous run of them.
//     With few column tiles every tile is cut into the same number of runs and the CTAs of a tile
//     form a thread-block cluster: the peers send their fp32 partial tiles straight into the
//     leader's shared memory (one bulk copy each, completing on the leader's mbarrier) and the
//     leader adds them in ascending K order and writes C - no trip through global memory.
//     Otherwise (more tiles than SMs, many tokens) runs may cross tile borders: a run that covers
//     a whole tile writes C directly; a partial one goes to scratch (at most two per CTA) and is
//     counted on the tile's arrival word, and the CTA that arrives last adds the tile's partials
//     in ascending K order.  Nobody waits for anybody.  The arrival words are the one part of the
//     scratch that is read before it is written: they live in the workspace's header, where no kernel
//     ever stores anything else, carry a per-launch epoch (a word of another epoch counts as empty) and
//     are zeroed by the CTA that finishes the tile, so scratch needs no initialisation.  Both ways the
//     result is identical from run to run.
//   * The kernel is launched with programmatic stream serialisation: set-up, and for a weight
//     the caller declares static also the first ring of weight tiles, overlap the tail of the
//     preceding kernel (the activation quantiser); everything else waits for it.
//
// Roles per CTA (192 threads) as in the other kernels: warp 0 TMA producer, warp 1 MMA issuer,
// warps 2-5 epilogue.  Every mbarrier wait is bounded.
#include <cuda_bf16.h>
#include <stdlib.h>

#include <atomic>
#include <chrono>

#include "gemm.cuh"
#include "gemm_tiles.cuh"
#include "ptx.cuh"

namespace dsl {

constexpr int DEC_SFW_COL = 256;        // weight scale factors (the M side)
constexpr int DEC_SFX_COL = 272;        // activation scale factors (the N side)
constexpr int DEC_MAX_CTAS = 256;       // grid size limit (one CTA per SM)

template <int KIND, int TOK>
struct DecCfg {
    static constexpr int W_STAGE = 128 * STAGE_KB;
    static constexpr int X_STAGE = TOK * STAGE_KB;
    static constexpr int SF_ATOMS = KIND == KIND_NVF4 ? 4 : (KIND == KIND_MXF4 ? 2 : 0);
    static constexpr int SF_STAGE = SF_ATOMS * 512;
    static constexpr int STAGE_BYTES = W_STAGE + X_STAGE + 2 * SF_STAGE;
    // cluster mode: room for this CTA's own fp32 partial tile ([TOK][128], slot 0) and those of up to
    // MAX_PEERS peers (slots 1..).  Up to 32 tokens it is a region of its own; beyond that the tiles are too
    // large for one and the drained operand ring is reused (the leader tells its peers when its ring is free).
    static constexpr int PART_BYTES = TOK * 128 * 4;
    static constexpr bool STAGE_IN_RING = TOK > 32;
    static constexpr int RECV_BYTES = STAGE_IN_RING ? 0 : 4 * PART_BYTES;
    static constexpr int RING_BUDGET = 200 * 1024 - RECV_BYTES;
    static constexpr int NUM_STAGES = RING_BUDGET / STAGE_BYTES > 10 ? 10 : RING_BUDGET / STAGE_BYTES;
    static constexpr int MAX_PEERS = STAGE_IN_RING ? ((NUM_STAGES * STAGE_BYTES) / PART_BYTES >= 4 ? 3 : 1) : 3;
    static_assert(!STAGE_IN_RING || (MAX_PEERS + 1) * PART_BYTES <= NUM_STAGES * STAGE_BYTES, "partial tiles must fit the ring");
    static constexpr int OFF_W = 0;
    static constexpr int OFF_X = OFF_W + NUM_STAGES * W_STAGE;
    static constexpr int OFF_SFW = OFF_X + NUM_STAGES * X_STAGE;
    static constexpr int OFF_SFX = OFF_SFW + NUM_STAGES * SF_STAGE;
    static constexpr int OFF_RECV = STAGE_IN_RING ? 0 : OFF_SFX + NUM_STAGES * SF_STAGE;          // 1024-byte aligned
    static constexpr int OFF_BAR = OFF_SFX + NUM_STAGES * SF_STAGE + RECV_BYTES;
    static constexpr int NUM_BARS = 2 * NUM_STAGES + 7;
    static constexpr int OFF_MISC = OFF_BAR + NUM_BARS * 8;
    static constexpr int OFF_TABLE = OFF_MISC + 16;                          // first unit of every CTA (+ the end)
    static constexpr int SMEM_BYTES = OFF_TABLE + (DEC_MAX_CTAS + 2) * 4 + 1024;
    static_assert(SMEM_BYTES <= 232448, "exceeds the 227 KB shared-memory limit");
    static_assert(SMEM_BYTES > 116224, "two CTAs could share an SM and deadlock on tensor-memory allocation");
    static_assert(NUM_STAGES >= 4, "pipeline too shallow");
};

struct DecPlan {
    int n_tiles;          // ceil(n / 128)
    int num_kb;           // K stages per tile
    long long units;      // n_tiles * num_kb
    int ctas;             // grid size; CTA c owns units [c*units/ctas, (c+1)*units/ctas)
    int cluster_runs;     // > 1: cluster mode, this many consecutive CTAs share one tile; 0: scratch mode
    unsigned long long* arrivals;   // scratch mode: one word per column tile in the workspace header,
                                    // (epoch << 16) | partials delivered
    unsigned long long epoch;       // differs from launch to launch (never 0), 48 bits
};

// First unit of CTA c.  Evaluated once per CTA index into a shared-memory table at kernel start.
__device__ __forceinline__ int dec_unit0(const DecPlan& p, int c) {
    return static_cast<int>((static_cast<long long>(c) * p.units) / p.ctas);
}

// scratch slot of the run that CTA c starts at unit seg_start: its first run uses slot 2c, a later one 2c+1
__device__ __forceinline__ int dec_slot(const int* u0, int c, int seg_start) { return seg_start == u0[c] ? 2 * c : 2 * c + 1; }

// Order in which a CTA visits the (column tile, K stage) units of its run.  Inside each tile the
// K stages are visited from a CTA-specific starting point, wrapping around: all CTAs need the
// same activation chunk for the same K stage, and without the offset they would all ask the same
// few L2 lines for it at the same moment (measured: 22 -> 17 us at 64 CTAs).  The order is a
// function of the grid only, so results stay identical from run to run.
struct UnitWalk {
    long long u, u_end;
    int S, tile, kb0, len, rot, i;
    __device__ __forceinline__ UnitWalk(long long u_begin, long long u_end_, int S_) : u(u_begin), u_end(u_end_), S(S_), len(0), i(0) {}
    // false when the run is exhausted; otherwise tile / kb describe the next unit
    __device__ __forceinline__ bool next(int& out_tile, int& out_kb) {
        if (i == len) {
            u += len;
            if (u >= u_end) return false;
            tile = static_cast<int>(u / S);
            kb0 = static_cast<int>(u - static_cast<long long>(tile) * S);
            len = static_cast<int>(min(static_cast<long long>(S - kb0), u_end - u));
            rot = static_cast<int>((blockIdx.x * 7u + static_cast<unsigned>(tile) * 3u) % static_cast<unsigned>(len));
            i = 0;
        }
        int k = i + rot;
        if (k >= len) k -= len;
        out_tile = tile;
        out_kb = kb0 + k;
        ++i;
        return true;
    }
};

// out = ((x * s1) * s2) [* row_scale[row]] [* col_scale[col]], the order of the tiled kernels' epilogue
__device__ __forceinline__ void store_out(const GemmArgs& args, int row, int col, float x, float s1, float s2, float cs) {
    x = __fmul_rn(__fmul_rn(x, s1), s2);
    if (args.row_scale != nullptr) x = __fmul_rn(x, args.row_scale[row]);
    if (args.col_scale != nullptr) x = __fmul_rn(x, cs);
    const size_t off = static_cast<size_t>(row) * args.ldc + col;
    if (args.out_bf16) static_cast<__nv_bfloat16*>(args.c)[off] = __float2bfloat16_rn(x);
    else static_cast<float*>(args.c)[off] = x;
}

// Bulk copy from this CTA's shared memory into the shared memory of CTA `rank` of the cluster (same
// offsets), completing `bytes` on that CTA's mbarrier.
__device__ __forceinline__ void bulk_send_to_cta(void* dst_local_equiv, const void* src, uint32_t bytes, uint64_t* bar_local_equiv,
                                                 uint32_t rank) {
    uint32_t dst, bar;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(dst) : "r"(smem_u32(dst_local_equiv)), "r"(rank));
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(bar) : "r"(smem_u32(bar_local_equiv)), "r"(rank));
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "r"(smem_u32(src)), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int KIND, int TOK>
__global__ void __launch_bounds__(192, 1)
gemm_decode_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_x,
                   const GemmArgs args, const DecPlan plan) {
    using C = DecCfg<KIND, TOK>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
    uint64_t* empty_bar = full_bar + C::NUM_STAGES;
    uint64_t* acc_full = empty_bar + C::NUM_STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint64_t* epi_bar = acc_empty + 2;     // meeting point of the four epilogue warps (bounded, like every wait here)
    uint64_t* recv_bar = epi_bar + 1;      // cluster mode, leader: completes when every peer's partial tile has landed
    uint64_t* go_bar = recv_bar + 1;       // cluster mode, peers, ring staging: the leader's ring is free to receive
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(smem + C::OFF_MISC);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC + 4);
    volatile uint32_t* last_flag = reinterpret_cast<volatile uint32_t*>(smem + C::OFF_MISC + 8);
    int* s_u0 = reinterpret_cast<int*>(smem + C::OFF_TABLE);
    float* recv = reinterpret_cast<float*>(smem + C::OFF_RECV);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const bool clustered = C::MAX_PEERS > 0 && plan.cluster_runs > 1;      // uniform over the grid
    const uint32_t crank = clustered ? cluster_ctarank() : 0u;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::NUM_STAGES; ++i) { mbar_init(full_bar + i, 1); mbar_init(empty_bar + i, 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(acc_full + i, 1); mbar_init(acc_empty + i, 4); }
        mbar_init(epi_bar, 4);
        mbar_init(recv_bar, 1);
        mbar_init(go_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
        if (clustered && crank == 0) mbar_arrive_expect_tx(recv_bar, static_cast<uint32_t>(plan.cluster_runs - 1) * C::PART_BYTES);
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_x);
    }
    for (int c = threadIdx.x; c <= plan.ctas; c += blockDim.x) s_u0[c] = dec_unit0(plan, c);
    if (C::SF_ATOMS > 0) {   // never let an uninitialised (possibly NaN) scale byte meet zero-filled data
        uint32_t* z = reinterpret_cast<uint32_t*>(smem + C::OFF_SFW);
        for (int i = threadIdx.x; i < C::NUM_STAGES * 2 * C::SF_STAGE / 4; i += blockDim.x) z[i] = 0u;
        fence_proxy_async_smem();
    }
    __syncthreads();
    // cluster mode: "my barriers are armed" (waited for below, before any role can send to a peer)
    if (clustered) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    if (warp == 1) tmem_alloc(tmem_ptr, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_ptr;
    if (clustered) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");

    const long long u_begin = s_u0[blockIdx.x];
    const long long u_end = s_u0[blockIdx.x + 1];
    const int S = plan.num_kb;

    if (warp == 0) {
        // ================= TMA producer =================
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            // The weight does not depend on the kernel that runs before this one: when the caller
            // vouches for that, the first ring of weight tiles is requested before waiting for it.
            const int ahead = args.b_static ? static_cast<int>(min(static_cast<long long>(C::NUM_STAGES), u_end - u_begin)) : 0;
            auto load_weight = [&](int tile, int kb, int st) {
                int atoms = 0;
                if (C::SF_ATOMS > 0) atoms = min(C::SF_ATOMS, args.sf_katoms - kb * C::SF_ATOMS);
                mbar_arrive_expect_tx(full_bar + st, C::W_STAGE + C::X_STAGE + 2 * atoms * 512);
                tma_load_2d(smem + C::OFF_W + st * C::W_STAGE, &tmap_w, full_bar + st, kb * STAGE_KB, tile * 128);
                if (C::SF_ATOMS > 0)
                    bulk_load(smem + C::OFF_SFW + st * C::SF_STAGE,
                              args.sfb + (static_cast<size_t>(tile) * args.sf_katoms + static_cast<size_t>(kb) * C::SF_ATOMS) * 512,
                              atoms * 512, full_bar + st);
            };
            {   // every stage is free at the start
                UnitWalk pre(u_begin, u_end, S);
                int tile, kb;
                for (int j = 0; j < ahead && pre.next(tile, kb); ++j) load_weight(tile, kb, j);
            }
            griddep_wait();
            UnitWalk walk(u_begin, u_end, S);
            int tile, kb;
            for (int j = 0; ok && walk.next(tile, kb); ++j) {
                if (j >= ahead) {
                    if (!mbar_wait(empty_bar + stage, phase ^ 1u, abort_flag, ST_TIMEOUT_PRODUCER)) { ok = false; break; }
                    load_weight(tile, kb, stage);
                }
                tma_load_2d(smem + C::OFF_X + stage * C::X_STAGE, &tmap_x, full_bar + stage, kb * STAGE_KB, 0);
                if (C::SF_ATOMS > 0) {
                    const int atoms = min(C::SF_ATOMS, args.sf_katoms - kb * C::SF_ATOMS);
                    bulk_load(smem + C::OFF_SFX + stage * C::SF_STAGE, args.sfa + static_cast<size_t>(kb) * C::SF_ATOMS * 512,
                              atoms * 512, full_bar + stage);
                }
                if (++stage == C::NUM_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else if (warp == 1) {
        // ================= MMA issuer =================
        griddep_wait();
        // instruction descriptor: M = 128 weight rows, N = TOK tokens, both operands K-major
        uint32_t idesc = (static_cast<uint32_t>(TOK >> 3) << 17) | (static_cast<uint32_t>(128 >> 4) << 24);
        if (KIND == KIND_F8) idesc |= 1u << 4;
        if (KIND == KIND_NVF4) idesc |= (1u << 7) | (1u << 10);
        if (KIND == KIND_MXF4) idesc |= (1u << 7) | (1u << 10) | (1u << 23);
        if (KIND == KIND_BF16) idesc |= (1u << 4) | (1u << 7) | (1u << 10);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int iter = 0;
        for (long long u = u_begin; u < u_end && ok; ++iter) {
            const int tile = static_cast<int>(u / S);
            const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * S);
            const int kb1 = static_cast<int>(min(static_cast<long long>(S), kb0 + (u_end - u)));
            const int acc = iter & 1;
            const uint32_t acc_phase = static_cast<uint32_t>((iter >> 1) & 1);
            if (!mbar_wait(acc_empty + acc, acc_phase ^ 1u, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * 128;
            for (int kb = kb0; kb < kb1; ++kb) {   // a count of stages; which K stage each one holds is the producer's business
                if (!mbar_wait(full_bar + stage, phase, abort_flag, ST_TIMEOUT_MMA)) { ok = false; break; }
                tc_fence_after();
                const uint32_t w_addr = smem_u32(smem + C::OFF_W + stage * C::W_STAGE);
                const uint32_t x_addr = smem_u32(smem + C::OFF_X + stage * C::X_STAGE);
                if (elect_one()) {
                    if (C::SF_ATOMS > 0) {
                        const uint32_t sfw_addr = smem_u32(smem + C::OFF_SFW + stage * C::SF_STAGE);
                        const uint32_t sfx_addr = smem_u32(smem + C::OFF_SFX + stage * C::SF_STAGE);
#pragma unroll
                        for (int i = 0; i < C::SF_ATOMS; ++i) {
                            tc_cp_32x128b_warpx4(tmem_base + DEC_SFW_COL + i * 4, make_desc_sf(sfw_addr + i * 512));
                            tc_cp_32x128b_warpx4(tmem_base + DEC_SFX_COL + i * 4, make_desc_sf(sfx_addr + i * 512));
                        }
                    }
                    const uint64_t wdesc = make_desc_sw128(w_addr);
                    const uint64_t xdesc = make_desc_sw128(x_addr);
#pragma unroll
                    for (int k = 0; k < 4; ++k) {   // 4 x 32 bytes of K per stage
                        const uint32_t accum = (kb > kb0 || k > 0) ? 1u : 0u;
                        if (KIND == KIND_F8) {
                            mma_f8f6f4(d_tmem, wdesc + 2 * k, xdesc + 2 * k, idesc, accum);
                        } else if (KIND == KIND_BF16) {
                            mma_f16(d_tmem, wdesc + 2 * k, xdesc + 2 * k, idesc, accum);
                        } else if (KIND == KIND_NVF4) {
                            mma_nvf4(d_tmem, wdesc + 2 * k, xdesc + 2 * k, idesc, tmem_base + DEC_SFW_COL + k * 4,
                                     tmem_base + DEC_SFX_COL + k * 4, accum);
                        } else {
                            const uint32_t sf_id = (k & 1) * 2;   // which byte pair of the 4-scale word
                            const uint32_t id = idesc | (sf_id << 29) | (sf_id << 4);
                            mma_mxf4(d_tmem, wdesc + 2 * k, xdesc + 2 * k, id, tmem_base + DEC_SFW_COL + (k >> 1) * 4,
                                     tmem_base + DEC_SFX_COL + (k >> 1) * 4, accum);
                        }
                    }
                    tc_commit(empty_bar + stage);
                    if (kb == kb1 - 1) tc_commit(acc_full + acc);
                }
                __syncwarp();
                if (++stage == C::NUM_STAGES) { stage = 0; phase ^= 1u; }
            }
            u += kb1 - kb0;
        }
    } else {
        // ================= epilogue =================
        griddep_wait();      // the scales read next and everything stored below depend on the predecessor
        const int quad = warp & 3;   // tensor-memory lanes [32*quad, 32*quad+32) belong to this warp
        const uint32_t lane_base = static_cast<uint32_t>(quad * 32) << 16;
        const int nl = quad * 32 + lane;
        float s1 = args.s1_dev != nullptr ? *args.s1_dev : args.s1;
        float s2 = args.s2_dev != nullptr ? *args.s2_dev : args.s2;
        if (args.scale_product) { s1 = s1 * s2; s2 = 1.0f; }
        bool ok = true;
        uint32_t epi_phase = 0;
        auto epilogue_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(epi_bar);
            const bool met = mbar_wait(epi_bar, epi_phase, abort_flag, ST_TIMEOUT_EPILOGUE);
            epi_phase ^= 1u;
            __syncwarp();
            return met;
        };
        if constexpr (C::MAX_PEERS > 0) {
            if (clustered && u_end > u_begin) {
                // ---- cluster mode: one run inside one tile; the leader (rank 0, lowest K) finishes the tile
                const int tile = static_cast<int>(u_begin / S);
                const int col = tile * 128 + nl;
                const bool col_ok = col < args.n;
                ok = mbar_wait(acc_full, 0, abort_flag, ST_TIMEOUT_EPILOGUE);
                tc_fence_after();
                // Everything below runs once per launch, i.e. from a cold instruction cache, where straight-line
                // code costs far more than its instruction count suggests (a fully unrolled 64-row finish took
                // 34 us).  So the accumulator goes to shared memory first and short rolled loops do the rest.
                if (ok) {
#pragma unroll 1
                    for (int c = 0; c < TOK / 16; ++c) {
                        uint32_t v[16];
                        tmem_ld_32x32b_x16(tmem_base + c * 16 + lane_base, v);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) recv[(c * 16 + i) * 128 + nl] = __uint_as_float(v[i]);
                    }
                    tc_fence_before();
                }
                if (C::STAGE_IN_RING && ok && crank == 0) {
                    // this CTA's MMAs are done (acc_full), so its operand ring can take the peers' tiles
                    __syncwarp();
                    if (warp == 2 && lane == 0)
                        for (int p = 1; p < plan.cluster_runs; ++p) mbar_arrive_cluster(go_bar, static_cast<uint32_t>(p));
                }
                if (ok && crank != 0) {
                    // peer: own partial tile (slot 0 here) -> the leader's slot for this rank, one bulk copy
                    fence_proxy_async_smem();
                    bool go = epilogue_sync();
                    if (C::STAGE_IN_RING && go) go = mbar_wait_cluster(go_bar, 0, abort_flag, ST_TIMEOUT_EPILOGUE);
                    if (go && warp == 2 && lane == 0)
                        bulk_send_to_cta(recv + static_cast<size_t>(crank) * (TOK * 128), recv, C::PART_BYTES, recv_bar, 0);
                } else if (ok) {
                    // leader: every thread finishes 8 consecutive columns of a row (16 threads per row, 8 rows per
                    // pass): 16-byte reads of the staged tiles and one 16-byte store per row piece instead of a
                    // 2-byte store per element, which is what the tail of this kernel used to wait for
                    const bool staged = epilogue_sync();                       // own tile is in shared memory
                    if (staged && mbar_wait(recv_bar, 0, abort_flag, ST_TIMEOUT_EPILOGUE)) {
                        const int runs = plan.cluster_runs;
                        const int et = (warp - 2) * 32 + lane;
                        const int g8 = (et & 15) * 8;
                        const int colg = tile * 128 + g8;
                        float cs8[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            cs8[j] = (args.col_scale != nullptr && colg + j < args.n) ? args.col_scale[colg + j] : 1.0f;
                        const bool vec = colg + 8 <= args.n && (args.out_bf16 ? args.ldc % 8 == 0 : args.ldc % 4 == 0);
#pragma unroll 1
                        for (int r = et >> 4; r < args.m_total; r += 8) {
                            const float4* src = reinterpret_cast<const float4*>(recv + r * 128 + g8);
                            float4 a = src[0], b = src[1];
#pragma unroll 1
                            for (int p = 1; p < runs; ++p) {                   // ascending K
                                const float4 pa = src[p * (TOK * 32)], pb = src[p * (TOK * 32) + 1];
                                a.x += pa.x; a.y += pa.y; a.z += pa.z; a.w += pa.w;
                                b.x += pb.x; b.y += pb.y; b.z += pb.z; b.w += pb.w;
                            }
                            float x[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                            const float rs = args.row_scale != nullptr ? args.row_scale[r] : 1.0f;
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                x[j] = __fmul_rn(__fmul_rn(x[j], s1), s2);
                                if (args.row_scale != nullptr) x[j] = __fmul_rn(x[j], rs);
                                if (args.col_scale != nullptr) x[j] = __fmul_rn(x[j], cs8[j]);
                            }
                            const size_t off = static_cast<size_t>(r) * args.ldc + colg;
                            if (vec && args.out_bf16) {
                                uint32_t w4[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * j], x[2 * j + 1]);
                                    w4[j] = *reinterpret_cast<uint32_t*>(&h);
                                }
                                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(args.c) + off) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                            } else if (vec) {
                                float4* dst = reinterpret_cast<float4*>(static_cast<float*>(args.c) + off);
                                dst[0] = make_float4(x[0], x[1], x[2], x[3]);
                                dst[1] = make_float4(x[4], x[5], x[6], x[7]);
                            } else {
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if (colg + j < args.n) {
                                        if (args.out_bf16) static_cast<__nv_bfloat16*>(args.c)[off + j] = __float2bfloat16_rn(x[j]);
                                        else static_cast<float*>(args.c)[off + j] = x[j];
                                    }
                                }
                            }
                        }
                    }
                }
            }
        }
        int iter = 0;
        for (long long u = u_begin; !clustered && u < u_end && ok; ++iter) {
            // ---- scratch mode
            const int tile = static_cast<int>(u / S);
            const int kb0 = static_cast<int>(u - static_cast<long long>(tile) * S);
            const int kb1 = static_cast<int>(min(static_cast<long long>(S), kb0 + (u_end - u)));
            const int acc = iter & 1;
            const uint32_t acc_phase = static_cast<uint32_t>((iter >> 1) & 1);
            if (!mbar_wait(acc_full + acc, acc_phase, abort_flag, ST_TIMEOUT_EPILOGUE)) { ok = false; break; }
            tc_fence_after();
            const int col = tile * 128 + nl;          // output column = weight row
            const bool col_ok = col < args.n;
            const bool whole = kb0 == 0 && kb1 == S;
            const float cs = (col_ok && args.col_scale != nullptr) ? args.col_scale[col] : 1.0f;
            if (whole) {
#pragma unroll 1
                for (int c = 0; c < TOK / 4; ++c) {      // short body: this code runs from a cold instruction cache
                    uint32_t v[4];
                    tmem_ld_32x32b_x4(tmem_base + acc * 128 + c * 4 + lane_base, v);
                    tmem_ld_wait();
                    if (!col_ok) continue;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = c * 4 + i;
                        if (row < args.m_total) store_out(args, row, col, __uint_as_float(v[i]), s1, s2, cs);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty + acc);
            } else {
                // deliver this run's partial tile, then count in; the last CTA to arrive finishes the tile
                float* pdst = args.partial + static_cast<size_t>(dec_slot(s_u0, blockIdx.x, static_cast<int>(u))) * (TOK * 128) + nl;
#pragma unroll 1
                for (int c = 0; c < TOK / 16; ++c) {
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(tmem_base + acc * 128 + c * 16 + lane_base, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        if (c * 16 + i < args.m_total) __stcg(pdst + (c * 16 + i) * 128, __uint_as_float(v[i]));
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty + acc);
                const int t0 = tile * S;
                const int t1 = t0 + S;
                // the CTAs that hold a piece of this tile: from the one whose run contains unit t0 to the
                // one whose run contains unit t1 - 1 (this CTA is one of them)
                int c_first = blockIdx.x, c_last = blockIdx.x;
                while (s_u0[c_first] > t0) --c_first;
                while (s_u0[c_last + 1] < t1) ++c_last;
                __threadfence();
                if (!epilogue_sync()) { ok = false; break; }
                if (warp == 2 && lane == 0) {
                    unsigned long long* word = plan.arrivals + tile;
                    // first guess: everybody else has arrived (right for the CTA on the critical path,
                    // which then needs one round trip; a wrong guess costs the others a second one)
                    unsigned long long old = (plan.epoch << 16) | static_cast<unsigned long long>(c_last - c_first);
                    unsigned long long want = 0;
                    for (int tries = 0; tries < 4096; ++tries) {   // lock-free: a retry means another CTA got in
                        want = (old >> 16) == plan.epoch ? old + 1 : ((plan.epoch << 16) | 1ull);
                        const unsigned long long seen = atomicCAS(word, old, want);
                        if (seen == old) break;
                        old = seen;
                        want = 0;
                    }
                    *last_flag = (want != 0 && static_cast<int>(want & 0xFFFFull) == c_last - c_first + 1) ? 1u : 0u;
                    if (want == 0) *abort_flag = ST_TIMEOUT_EPILOGUE;
                }
                if (!epilogue_sync()) { ok = false; break; }
                if (*last_flag != 0u) {
                    __threadfence();
                    if (col_ok) {
                        // Runs once per launch from a cold instruction cache: kept short.  Four rows in flight
                        // hide part of the L2 latency of the partial tiles.
#pragma unroll 1
                        for (int row0 = 0; row0 < args.m_total; row0 += 4) {
                            float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
                            for (int c = c_first; c <= c_last; ++c) {       // ascending K
                                const int a = max(s_u0[c], t0);
                                const float* src = args.partial + (static_cast<size_t>(dec_slot(s_u0, c, a)) * TOK + row0) * 128 + nl;
#pragma unroll
                                for (int j = 0; j < 4; ++j) sum[j] += row0 + j < args.m_total ? __ldcg(src + j * 128) : 0.f;
                            }
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (row0 + j < args.m_total) store_out(args, row0 + j, col, sum[j], s1, s2, cs);
                        }
                    }
                    if (warp == 2 && lane == 0) *reinterpret_cast<volatile unsigned long long*>(plan.arrivals + tile) = 0ull;
                }
            }
            u += kb1 - kb0;
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
    // cluster mode: nobody leaves while a peer's copy may still read from or write to its shared memory
    if (clustered) cluster_sync_all();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---- host side ---------------------------------------------------------------------------
// DSLGEMM_DECODE_CTAS=<n> forces scratch mode with that grid size, DSLGEMM_DECODE_CLUSTER=0 disables
// cluster mode (for measurements).
static int env_int(const char* name, int fallback) {
    const char* e = getenv(name);
    return e != nullptr ? atoi(e) : fallback;
}

// Arrival words carry a per-launch epoch in their upper 48 bits.  Epochs count up from a start value
// drawn once per process from the clock and the address-space layout, so that stale bytes a caller's
// workspace happens to hold (it need not be cleared) match the current epoch only by a 2^-48 accident,
// not because both are small integers.
static unsigned long long next_epoch() {
    static std::atomic<unsigned long long> source{[] {
        unsigned long long x = static_cast<unsigned long long>(std::chrono::steady_clock::now().time_since_epoch().count());
        x ^= static_cast<unsigned long long>(reinterpret_cast<uintptr_t>(&x)) << 17;
        x += 0x9E3779B97F4A7C15ull;                      // splitmix64 finaliser
        x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
        x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
        return x ^ (x >> 31);
    }()};
    unsigned long long e;
    do { e = source.fetch_add(1) & 0xFFFFFFFFFFFFull; } while (e == 0);
    return e;
}

// Grid, combine mode and scratch need of a problem.  Returns false when this kernel does not serve it.
// `scratch_needed` is what the plan would like to have behind the workspace header (0 in cluster mode);
// with less the grid shrinks (`plan.ctas`), with none the problem is not served.
template <int KIND, int TOK>
static bool plan_decode(const GemmArgs& args, DecPlan& plan, size_t* scratch_needed) {
    using C = DecCfg<KIND, TOK>;
    static const int forced_ctas = env_int("DSLGEMM_DECODE_CTAS", 0);
    static const int allow_cluster = env_int("DSLGEMM_DECODE_CLUSTER", 1);
    plan = DecPlan{};
    *scratch_needed = 0;
    plan.n_tiles = (args.n + 127) / 128;
    plan.num_kb = (args.k_bytes + STAGE_KB - 1) / STAGE_KB;
    plan.units = static_cast<long long>(plan.n_tiles) * plan.num_kb;
    if (plan.units > 0x7FFFFFFFll) return false;
    const int sms = sm_count();
    // Grid.  Few column tiles: every tile is cut into the same number of K runs (each CTA works inside one
    // tile); with 2 or 4 runs (and room for the peers' partial tiles) the CTAs of a tile form a cluster.
    // More tiles than SMs: one CTA per SM and the runs cross tile borders.  Every CTA streams at least four
    // stages.  Scratch mode keeps two partial tiles per CTA behind the workspace header and one arrival word
    // per column tile inside it.
    long long ctas = sms;
    int cluster_runs = 0;
    if (plan.n_tiles <= sms) {
        long long runs = sms / plan.n_tiles;
        if (runs > plan.num_kb / 4) runs = plan.num_kb / 4;
        if (runs < 1) runs = 1;
        if (allow_cluster && forced_ctas == 0 && runs >= 2 && C::MAX_PEERS >= 1) {
            cluster_runs = (runs >= 4 && C::MAX_PEERS >= 3) ? 4 : 2;
            runs = cluster_runs;
        }
        ctas = plan.n_tiles * runs;
    }
    if (ctas > plan.units / 4) { ctas = plan.units / 4; cluster_runs = 0; }
    if (forced_ctas > 0 && forced_ctas <= plan.units) ctas = forced_ctas;
    if (ctas > DEC_MAX_CTAS) { ctas = DEC_MAX_CTAS; cluster_runs = 0; }
    // More than 32 tokens: only the cluster combine is fast enough (the scratch combine walks the rows with
    // one L2 round trip after the other); otherwise the tiled split-K kernel takes the problem.
    if (TOK > 32 && cluster_runs == 0) return false;
    if (ctas < 1) return false;
    // every run a whole number of tiles (one CTA per tile, or fewer CTAs than tiles dividing them evenly):
    // each CTA writes C itself and nothing passes through scratch
    const bool whole_only = cluster_runs == 0 && plan.units % ctas == 0 && (plan.units / ctas) % plan.num_kb == 0;
    if (cluster_runs == 0 && !whole_only) {
        if (static_cast<size_t>(plan.n_tiles) * sizeof(unsigned long long) > DSL_WS_HEADER_BYTES) return false;
        const size_t per_cta = 2ull * TOK * 128 * sizeof(float);
        *scratch_needed = per_cta * static_cast<size_t>(ctas);
        const long long by_scratch = args.partial != nullptr ? static_cast<long long>(args.partial_bytes / per_cta) : 0;
        if (ctas > by_scratch) ctas = by_scratch;
        if (ctas < 1) return false;    // no scratch: the caller falls back to the tiled kernel
        plan.arrivals = args.ws_words;
    }
    plan.ctas = static_cast<int>(ctas);
    plan.cluster_runs = cluster_runs;
    return true;
}

template <int KIND, int TOK>
static int launch_decode_one(const void* A, const void* B, const GemmArgs& args, cudaStream_t st) {
    using C = DecCfg<KIND, TOK>;
    DecPlan plan;
    size_t wanted = 0;
    if (!plan_decode<KIND, TOK>(args, plan, &wanted)) return DSL_NOT_SERVED;
    plan.epoch = next_epoch();
    CUtensorMap tw, tx;
    if (!make_tmap_u8(&tw, B, args.k_bytes, args.n, 0, STAGE_KB, 128)) return DSL_ERR_DRIVER;
    if (!make_tmap_u8(&tx, A, args.k_bytes, args.m_total, 0, STAGE_KB, TOK)) return DSL_ERR_DRIVER;
    static PerDeviceInt attr_set;   // per device; idempotent, a race here only repeats the same call
    const int dev = current_device_slot();
    if (dev < 0) return static_cast<int>(cudaErrorInvalidDevice);
    if (attr_set.v[dev].load(std::memory_order_acquire) == 0) {
        cudaError_t e = cudaFuncSetAttribute(gemm_decode_kernel<KIND, TOK>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
        if (e != cudaSuccess) return static_cast<int>(e);
        attr_set.v[dev].store(1, std::memory_order_release);
    }
    // Programmatic stream serialisation: the grid may be set up (and, for a static weight, start its
    // weight stream) while the preceding kernel of the stream drains; griddep_wait() guards the rest.
    // DSLGEMM_PDL=0 launches it the plain way (for measurements).
    static const bool pdl = [] { const char* e = getenv("DSLGEMM_PDL"); return !(e != nullptr && e[0] == '0'); }();
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.ctas);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = C::SMEM_BYTES;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl ? 1 : 0;
    cfg.numAttrs = 1;
    if (plan.cluster_runs > 1) {
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = plan.cluster_runs;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    return static_cast<int>(cudaLaunchKernelEx(&cfg, gemm_decode_kernel<KIND, TOK>, tw, tx, args, plan));
}

template <int KIND>
static bool plan_decode_kind(const GemmArgs& args, size_t* wanted) {
    DecPlan plan;
    if (args.m_total <= 16) return plan_decode<KIND, 16>(args, plan, wanted);
    if (args.m_total <= 32) return plan_decode<KIND, 32>(args, plan, wanted);
    if (args.m_total <= 64) return plan_decode<KIND, 64>(args, plan, wanted);
    return plan_decode<KIND, 128>(args, plan, wanted);
}

static bool decode_domain(const GemmArgs& args) {
    return args.group_offsets == nullptr && args.m_total <= DSL_DECODE_MAX_ROWS && args.act == DSL_ACT_NONE &&
           args.out_sf == nullptr;
}

size_t decode_scratch_bytes(int kind, const GemmArgs& args, bool* served) {
    size_t wanted = 0;
    *served = false;
    if (!decode_domain(args)) return 0;
    switch (kind) {
        case KIND_F8: *served = plan_decode_kind<KIND_F8>(args, &wanted); break;
        case KIND_NVF4: *served = plan_decode_kind<KIND_NVF4>(args, &wanted); break;
        case KIND_MXF4: *served = plan_decode_kind<KIND_MXF4>(args, &wanted); break;
        case KIND_BF16: *served = plan_decode_kind<KIND_BF16>(args, &wanted); break;
        default: break;
    }
    return *served ? wanted : 0;
}

template <int KIND>
static int launch_decode_kind(const void* A, const void* B, const GemmArgs& args, cudaStream_t st) {
    static_assert(DSL_DECODE_MAX_ROWS == 128, "one instantiation per token bucket");
    if (args.m_total <= 16) return launch_decode_one<KIND, 16>(A, B, args, st);
    if (args.m_total <= 32) return launch_decode_one<KIND, 32>(A, B, args, st);
    if (args.m_total <= 64) return launch_decode_one<KIND, 64>(A, B, args, st);
    return launch_decode_one<KIND, 128>(A, B, args, st);
}

// Returns DSL_NOT_SERVED when the problem is not one this kernel serves (the caller then uses the tiled kernels).
int launch_gemm_decode(int kind, const void* A, const void* B, const GemmArgs& args, cudaStream_t st) {
    if (!decode_domain(args)) return DSL_NOT_SERVED;
    switch (kind) {
        case KIND_F8: return launch_decode_kind<KIND_F8>(A, B, args, st);
        case KIND_NVF4: return launch_decode_kind<KIND_NVF4>(A, B, args, st);
        case KIND_MXF4: return launch_decode_kind<KIND_MXF4>(A, B, args, st);
        case KIND_BF16: return launch_decode_kind<KIND_BF16>(A, B, args, st);
        default: return DSL_ERR_ENUM;
    }
}

}  // namespace dsl
