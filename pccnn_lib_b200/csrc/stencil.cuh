// Candidate ranges of a grid cell: the 3^D cell stencil expressed as position ranges of the sorted
// point array (find_ranges_grid_ds.cu:65-166, 306-338 of phermosilla/pccnn_lib restated for a whole
// cell at once).  Shared by the neighbor search and the grid-based Poisson-disk sampling.
#pragma once

#include "common.cuh"

namespace pccnn {

template <int D>
struct Stencil {
    // Dimensions that receive a -1/0/+1 offset: all but the last one (whose +-1 window is a
    // contiguous key range), except in 2-D where the table is indexed by the full cell.
    static constexpr int kOffsetDims = (D == 2) ? 2 : D - 1;
    static constexpr int pow3(int e) { return e == 0 ? 1 : 3 * pow3(e - 1); }
    static constexpr int kRanges = pow3(kOffsetDims);
    // A staged candidate is D coordinates + its position, padded to whole float4s; the float4s
    // of one candidate live in separate planes so that every shared load has a 16-byte lane stride.
    static constexpr int kPlanes = (D + 1 + 3) / 4;
    static constexpr int kSlots = (kPlanes == 1) ? 256 : 96;  // candidates staged per round and warp (multiple of 32)
};

__device__ __forceinline__ int lower_bound_key(const int64_t* __restrict__ keys, int lo, int hi, long long v) {
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (__ldg(keys + mid) < v) lo = mid + 1; else hi = mid;
    }
    return lo;
}
__device__ __forceinline__ int upper_bound_key(const int64_t* __restrict__ keys, int lo, int hi, long long v) {
    while (lo < hi) {
        int mid = (lo + hi) >> 1;
        if (__ldg(keys + mid) <= v) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// Candidate ranges of the cell with key `key`, ascending in sorted position, computed by the
// whole warp: range starts go to lo[], the exclusive prefix of their lengths to pref[].
// Returns the number of candidates.
template <int D>
__device__ __forceinline__ int resolve_ranges(long long key, const GridDesc<D>& g,
                                              const int2* __restrict__ grid_ds,
                                              const int64_t* __restrict__ pt_keys, int num_pts,
                                              int* __restrict__ lo, int* __restrict__ pref) {
    using S = Stencil<D>;
    const int lane = lane_id();
    int c[D];
    const int b = key_to_cell<D>(key, g, c);
    int carry = 0;
    for (int o0 = 0; o0 < S::kRanges; o0 += 32) {
        const int o = o0 + lane;
        int2 r = make_int2(0, 0);
        if (o < S::kRanges) {
            int cc[D];
#pragma unroll
            for (int d = 0; d < D; ++d) cc[d] = c[d];
            int rem = o;
            bool inside = true;
#pragma unroll
            for (int d = S::kOffsetDims - 1; d >= 0; --d) {
                const int q = rem / 3;
                cc[d] += rem - q * 3 - 1;
                rem = q;
                inside = inside && cc[d] >= 0 && cc[d] < g.nc[d];
            }
            if (inside) {
                const long long ds = ((long long)b * g.nc[0] + cc[0]) * g.nc[1] + cc[1];
                int2 tube = __ldg(grid_ds + ds);
                tube.x = max(tube.x, 0);
                tube.y = min(tube.y, num_pts);
                if (D == 2) {
                    r = tube;
                } else if (tube.y > tube.x) {
                    const long long k = cell_key<D>(cc, g, b);
                    const long long klo = k - (c[D - 1] > 0 ? 1 : 0);
                    const long long khi = k + (c[D - 1] < g.nc[D - 1] - 1 ? 1 : 0);
                    r.x = lower_bound_key(pt_keys, tube.x, tube.y, klo);
                    r.y = upper_bound_key(pt_keys, r.x, tube.y, khi);
                }
            }
        }
        int len = max(r.y - r.x, 0);
        int incl = len;
#pragma unroll
        for (int s = 1; s < 32; s <<= 1) {
            const int v = __shfl_up_sync(kFullMask, incl, s);
            if (lane >= s) incl += v;
        }
        if (o < S::kRanges) {
            lo[o] = r.x;
            pref[o + 1] = carry + incl;
        }
        carry += __shfl_sync(kFullMask, incl, 31);
    }
    if (lane == 0) pref[0] = 0;
    __syncwarp();
    return carry;
}

}  // namespace pccnn
