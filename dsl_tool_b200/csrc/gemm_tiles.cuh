// Device-side tile scheduler shared by the GEMM kernels: turns a linear tile index into
// (row group, row tile, column tile) from the row-group offsets held in shared memory.
#pragma once
#include <stdint.h>

namespace dsl {

constexpr int BLOCK_M = 128;
constexpr int STAGE_KB = 128;           // bytes of K per stage row = one 128-byte swizzle atom
constexpr int TMEM_COLS = 512;

struct TileInfo {
    int group, mtile, row0, row_end, n0;
};

struct TileWalker {
    const int* offs;
    const int* tile0;
    int groups, m_tiles, n_tiles, band, block_n;
    long long total;
    __device__ __forceinline__ TileInfo decode(long long t) const {
        const long long per_band = static_cast<long long>(m_tiles) * band;
        const int b = static_cast<int>(t / per_band);
        const int r = static_cast<int>(t - b * per_band);
        const int nb0 = b * band;
        const int wb = min(band, n_tiles - nb0);
        const int mt = r / wb;
        const int nt = nb0 + (r - mt * wb);
        int lo = 0, hi = groups;   // last g with tile0[g] <= mt
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (tile0[mid] <= mt) lo = mid; else hi = mid;
        }
        TileInfo ti;
        ti.group = lo;
        ti.mtile = mt;
        ti.row0 = offs[lo] + (mt - tile0[lo]) * BLOCK_M;
        ti.row_end = offs[lo + 1];
        ti.n0 = nt * block_n;
        return ti;
    }
};


// Row-group offsets live in the caller's device memory and are not trusted: an entry outside
// [0, m_total] or below its predecessor would send tiles, stores and scale-tile writes outside the
// operands.  Every kernel reads them through these two helpers: entries are clamped to [0, m_total] when
// they are loaded, and the (sequential) pass that builds the tile tables raises an entry to its
// predecessor, so the table every role works from is monotone inside [0, m_total] whatever was passed.
__host__ __device__ __forceinline__ int clamp_offset(int v, int m_total) { return v < 0 ? 0 : (v > m_total ? m_total : v); }

// All threads; the caller synchronises before the table is read.
__device__ __forceinline__ void load_group_offsets(int* s_offs, const int* group_offsets, int groups, int m_total) {
    for (int g = threadIdx.x; g <= groups; g += blockDim.x)
        s_offs[g] = group_offsets != nullptr ? clamp_offset(group_offsets[g], m_total) : (g == 0 ? 0 : m_total);
}

// One thread, ascending g: rows of group g after raising offs[g+1] to at least offs[g].
__host__ __device__ __forceinline__ int monotone_rows(int* offs, int g) {
    if (offs[g + 1] < offs[g]) offs[g + 1] = offs[g];
    return offs[g + 1] - offs[g];
}

// Fills offsets[0..groups] and the first-tile table tile0[0..groups] (shared memory).  Call
// from all threads; contains two __syncthreads().
__device__ __forceinline__ void build_tile_tables(int* s_offs, int* s_tile0, const int* group_offsets, int groups,
                                                  int m_total) {
    load_group_offsets(s_offs, group_offsets, groups, m_total);
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
    __syncthreads();
}

}  // namespace dsl
