// Cell-parallel greedy Poisson-disk sampling.
//
// Restates pccnn_lib_ops/poisson_disk_sampling/poisson_disk_sampling.cu:36-196 of
// phermosilla/pccnn_lib: the occupied cells are visited in 2^D passes, pass `c` handling the
// cells whose index parity in dimension d equals bit d of c.  Cells of one pass are at least
// one whole cell apart, so none of them appears in another one's neighbor lists and they can
// run in parallel; inside a cell the points are taken in ascending sorted position and a
// point is selected iff none of its radius neighbors has been selected before.
//
// Design: the reference spends one thread per cell and walks points x neighbors serially, each
// step waiting on dependent loads.  Here a warp owns a cell and takes 32 of its points at a time:
// the lanes scan their points' neighbor lists in parallel (all memory latency overlaps), and the
// order-dependent part (a point is rejected if an EARLIER point of the same group that is its
// neighbor was selected) runs on bit masks in registers.  Cell boundaries and the final index
// list come from device-wide stream compaction; nothing is copied from the host between passes.
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>

#include <mutex>

#include <cub/device/device_scan.cuh>

#include "common.cuh"
#include "stencil.cuh"

namespace pccnn {


__global__ void cell_flags_kernel(int n, const int64_t* __restrict__ keys, int32_t* __restrict__ flags) {
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        flags[i] = (i == 0 || keys[i] != keys[i - 1]) ? 1 : 0;
}

// Cells are routed once, before the passes: `code` holds the pass a cell belongs to (bit d = parity of
// its index in dimension d) and bit 7 marks a "crowded" cell, which also goes on the `crowded` list.
// Crowded = more than 32 points, or neighbor lists adding up to kCrowdedEntries or more: a single warp
// would be busy with such a cell long after the rest of the pass has finished.
constexpr int kCrowdedMaxPoints = 512;
constexpr int kCrowdedEntries = 1024;
constexpr int kPdsThreads = 512;
constexpr unsigned kCrowdedBit = 0x80u;

template <int D>
__global__ void cell_route_kernel(int n, const int64_t* __restrict__ keys, const int32_t* __restrict__ cell_starts,
                                  const int32_t* __restrict__ start_ids, const int32_t* __restrict__ grid_size,
                                  int32_t* counters, unsigned char* __restrict__ code, int32_t* __restrict__ crowded,
                                  int crowded_capacity) {
    const GridDesc<D> g = load_grid<D>(grid_size);
    const int num_cells = counters[0];
    const int stride = gridDim.x * blockDim.x;
    for (int cell = blockIdx.x * blockDim.x + threadIdx.x; cell < num_cells; cell += stride) {
        const int first = cell_starts[cell];
        const int last = (cell + 1 < num_cells) ? cell_starts[cell + 1] : n;
        int c[D];
        key_to_cell<D>(keys[first], g, c);
        unsigned v = 0;
#pragma unroll
        for (int d = 0; d < D; ++d) v |= (unsigned)(c[d] & 1) << d;
        const int count = last - first;
        const int entries = start_ids[last - 1] - (first > 0 ? start_ids[first - 1] : 0);
        if ((count > 32 || entries >= kCrowdedEntries) && count <= kCrowdedMaxPoints) {
            const int slot = atomicAdd(counters + 2, 1);
            if (slot < crowded_capacity) {
                crowded[slot] = cell;
                v |= kCrowdedBit;
            }
        }
        code[cell] = (unsigned char)v;
    }
}

// The in-order decisions of up to 32 consecutive points of one cell, [p0, group_end), given for the
// lane's point p = p0 + lane its `blocked` flag (a neighbor decided earlier is selected) and the mask
// of its neighbors inside the group.  Registers and shuffles only.  Returns the selected mask.
__device__ __forceinline__ unsigned decide_group(int count, bool blocked, unsigned in_group) {
    unsigned selected = 0u;
    for (int q = 0; q < count; ++q) {
        const bool take = !blocked && (in_group & selected) == 0u;  // meaningful in lane q
        selected |= __shfl_sync(kFullMask, take ? 1u : 0u, q) << q;
    }
    return selected;
}

// One group of up to 32 consecutive points of a cell, [p0, p0 + count): lane `slot0 + i` holds point
// p0 + i.  Scans the lane's neighbor list once, noting (a) whether a neighbor decided earlier (other
// cells, earlier passes, earlier groups of the cell) is selected and (b) which points of the group are
// its neighbors.  No early exit and no short-circuit: the loads of different neighbors stay
// independent of one another, so many are in flight at once.
__device__ __forceinline__ void scan_own_list(int p, int p0, int count, int slot0, const int2* __restrict__ neighbors,
                                              const int32_t* __restrict__ start_ids, volatile int32_t* vused,
                                              bool& blocked, unsigned& in_group) {
    const int lo = (p > 0) ? __ldg(start_ids + p - 1) : 0;
    const int hi = __ldg(start_ids + p);
#pragma unroll 4
    for (int t = lo; t < hi; ++t) {
        const int j = __ldg(&neighbors[t]).x;
        const bool same_group = j >= p0 && j < p0 + count;
        if (same_group) in_group |= 1u << (j - p0 + slot0);
        const int flag = vused[same_group ? p : j];  // own flag is still 0: a harmless read
        blocked = blocked | (flag != 0);
    }
}

// Warp role: cells of this pass that are not on the crowded list, 32 cells looked at at a time.  Most
// cells hold a handful of points, so the points of SEVERAL cells share the 32 lanes of a round: cells
// of one pass never interact, and inside a round a lane's in-group mask only covers its own cell.
__device__ void pds_sparse_cells(int pass, int n, int warp_index, int warps_total, int num_cells,
                                 const int32_t* __restrict__ cell_starts, const unsigned char* __restrict__ code,
                                 const int2* __restrict__ neighbors, const int32_t* __restrict__ start_ids,
                                 int32_t* used) {
    const int lane = lane_id();
    volatile int32_t* vused = used;
    // the 32 cells of a batch are taken num_batches apart: cells with long neighbor lists sit next to each
    // other in cell order (dense clouds) and spread like this they land in different warps
    const int num_batches = (num_cells + 31) / 32;
    for (int batch = warp_index; batch < num_batches; batch += warps_total) {
        const int cell = lane * num_batches + batch;
        const bool want = cell < num_cells && __ldg(code + cell) == (unsigned)pass;
        int my_first = 0, my_count = 0;
        if (want) {
            my_first = __ldg(cell_starts + cell);
            my_count = ((cell + 1 < num_cells) ? __ldg(cell_starts + cell + 1) : n) - my_first;
        }
        // Cells with more than 32 points (beyond the crowded kernel's capacity): alone, group after group.
        unsigned big = __ballot_sync(kFullMask, my_count > 32);
        while (big) {
            const int src = __ffs(big) - 1;
            big &= big - 1;
            const int first = __shfl_sync(kFullMask, my_first, src);
            const int last = first + __shfl_sync(kFullMask, my_count, src);
            for (int p0 = first; p0 < last; p0 += 32) {
                const int p = p0 + lane, count = min(32, last - p0);
                bool blocked = false;
                unsigned in_group = 0u;
                if (p < last) scan_own_list(p, p0, count, 0, neighbors, start_ids, vused, blocked, in_group);
                const unsigned selected = decide_group(count, blocked, in_group);
                if (p < last && ((selected >> lane) & 1u)) vused[p] = 1;
                __syncwarp();  // orders the stores before the next group's loads in this warp
            }
        }
        if (my_count > 32) my_count = 0;
        // Exclusive prefix sum of the remaining counts: lane i's cell would start at slot my_off.
        int my_off = my_count;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int v = __shfl_up_sync(kFullMask, my_off, d);
            if (lane >= d) my_off += v;
        }
        my_off -= my_count;
        unsigned todo = __ballot_sync(kFullMask, my_count > 0);
        while (todo) {
            // this round: the longest run of remaining cells whose points fit 32 slots
            const int lead = __ffs(todo) - 1;
            const int off0 = __shfl_sync(kFullMask, my_off, lead);
            const bool in_round = my_count > 0 && lane >= lead && my_off + my_count - off0 <= 32;
            const unsigned round = __ballot_sync(kFullMask, in_round);
            todo &= ~round;
            int p = -1, p0 = 0, count = 0, slot0 = 0;
            for (unsigned cells = round; cells; cells &= cells - 1) {
                const int src = __ffs(cells) - 1;
                const int o = __shfl_sync(kFullMask, my_off, src) - off0;
                const int c = __shfl_sync(kFullMask, my_count, src);
                const int f = __shfl_sync(kFullMask, my_first, src);
                if (lane >= o && lane < o + c) {
                    p = f + lane - o;
                    p0 = f;
                    count = c;
                    slot0 = o;
                }
            }
            bool blocked = true;  // lanes without a point never select
            unsigned in_group = 0u;
            if (p >= 0) {
                blocked = false;
                scan_own_list(p, p0, count, slot0, neighbors, start_ids, vused, blocked, in_group);
            }
            const unsigned selected = decide_group(32, blocked, in_group);
            if (p >= 0 && ((selected >> lane) & 1u)) vused[p] = 1;
        }
    }
}

// Block role: crowded cells, one thread block per cell.  Everything that does not depend on the order
// of the cell's points is done first, by all warps: a warp streams the neighbor list of a point with
// coalesced loads and records (a) whether a selected point outside the cell is among them and (b) the
// neighbors inside the cell, as one row of a bit matrix in shared memory.  The in-order decisions
// are then a walk of warp 0 over that matrix: lane w keeps word w of the selected set.
__device__ void pds_crowded_cells(int pass, int n, int block_index, int blocks_total, int num_cells, int num_crowded,
                                  const int32_t* __restrict__ cell_starts, const unsigned char* __restrict__ code,
                                  const int32_t* __restrict__ crowded, const int2* __restrict__ neighbors,
                                  const int32_t* __restrict__ start_ids, int32_t* used, unsigned* s_adj,
                                  unsigned char* s_blocked) {
    const int warp = threadIdx.x >> 5, lane = lane_id();
    for (int i = block_index; i < num_crowded; i += blocks_total) {
        const int cell = __ldg(crowded + i);
        if ((__ldg(code + cell) & ~kCrowdedBit) != (unsigned)pass) continue;  // uniform over the block
        const int first = __ldg(cell_starts + cell);
        const int last = (cell + 1 < num_cells) ? __ldg(cell_starts + cell + 1) : n;
        const int count = last - first, words = (count + 31) >> 5;
        for (int k = threadIdx.x; k < count * words; k += kPdsThreads) s_adj[k] = 0u;
        for (int k = threadIdx.x; k < count; k += kPdsThreads) s_blocked[k] = 0;
        __syncthreads();
        for (int q = warp; q < count; q += kPdsThreads / 32) {
            const int p = first + q;
            const int lo = (p > 0) ? __ldg(start_ids + p - 1) : 0;
            const int hi = __ldg(start_ids + p);
            bool flag = false;
#pragma unroll 8
            for (int t = lo + lane; t < hi; t += 32) {
                const int j = __ldg(&neighbors[t]).x;
                const bool inside = j >= first && j < last;
                if (inside) atomicOr(&s_adj[q * words + ((j - first) >> 5)], 1u << ((j - first) & 31));
                flag = flag | (used[inside ? p : j] != 0);  // points of this cell are all undecided: 0
            }
            if (__any_sync(kFullMask, flag) && lane == 0) s_blocked[q] = 1;
        }
        __syncthreads();
        if (warp == 0) {
            unsigned selected = 0u;  // lane w: points [32 w, 32 w + 32) of the cell
            for (int q = 0; q < count; ++q) {
                const unsigned row = (lane < words) ? s_adj[q * words + lane] : 0u;
                const bool hit = __any_sync(kFullMask, (row & selected) != 0u);
                if (!hit && !s_blocked[q] && lane == (q >> 5)) selected |= 1u << (q & 31);
            }
            while (selected) {
                used[first + lane * 32 + __ffs(selected) - 1] = 1;
                selected &= selected - 1;
            }
        }
        __syncthreads();
    }
}

// One launch per pass.  The first `crowded_blocks` blocks take the crowded cells, the others the rest;
// the two kinds of cell never interact inside a pass, so the roles overlap freely.
__global__ void __launch_bounds__(kPdsThreads)
pds_pass_kernel(int pass, int n, int crowded_blocks, const int32_t* __restrict__ cell_starts,
                const int32_t* __restrict__ counters, const unsigned char* __restrict__ code,
                const int32_t* __restrict__ crowded, int crowded_capacity, const int2* __restrict__ neighbors,
                const int32_t* __restrict__ start_ids, int32_t* used) {
    __shared__ unsigned s_adj[kCrowdedMaxPoints * (kCrowdedMaxPoints / 32)];
    __shared__ unsigned char s_blocked[kCrowdedMaxPoints];
    const int num_cells = counters[0];
    if ((int)blockIdx.x < crowded_blocks) {
        pds_crowded_cells(pass, n, blockIdx.x, crowded_blocks, num_cells, min(counters[2], crowded_capacity), cell_starts,
                          code, crowded, neighbors, start_ids, used, s_adj, s_blocked);
    } else {
        constexpr int kWarps = kPdsThreads / 32;
        pds_sparse_cells(pass, n, ((int)blockIdx.x - crowded_blocks) * kWarps + (threadIdx.x >> 5),
                         ((int)gridDim.x - crowded_blocks) * kWarps, num_cells, cell_starts, code, neighbors, start_ids,
                         used);
    }
}

struct PdsLayout {
    size_t flags_off, cells_off, used_off, counters_off, cub_off, cub_bytes, total;
};

static PdsLayout pds_layout(int64_t n) {
    PdsLayout L;
    const int nn = (int)(n > 0 ? n : 1);
    size_t a = 0, b = 0;
    cub::DeviceSelect::Flagged(nullptr, a, thrust::counting_iterator<int32_t>(0), (const int32_t*)nullptr,
                               (int32_t*)nullptr, (int32_t*)nullptr, nn);
    cub::DeviceSelect::Flagged(nullptr, b, thrust::counting_iterator<int64_t>(0), (const int32_t*)nullptr,
                               (int64_t*)nullptr, (int32_t*)nullptr, nn);
    L.cub_bytes = a > b ? a : b;
    L.flags_off = 0;
    L.cells_off = align_up((size_t)n * 4);
    L.used_off = L.cells_off + align_up((size_t)n * 4);
    L.counters_off = L.used_off + align_up((size_t)n * 4);
    L.cub_off = L.counters_off + 256;
    L.total = L.cub_off + align_up(L.cub_bytes) + 256;
    return L;
}

// ---- Poisson-disk sampling straight from the grid (no neighbor list) -------------------------------
// The list-based operator above needs the full self-neighborhood of the points, although a point is
// only ever compared with SELECTED points, of which a cell holds a handful.  Here the selected
// points of every cell are kept as a short list (stored in the cell's own slice of a point-sized
// array), and a cell being decided gathers the selected points of its 3^D stencil once, into shared
// memory, and tests its own points against them with the neighbor search's exact predicate
// (sample = the point being decided).  Same passes, same order inside a cell, hence the same
// selection as the list-based operator on the full radius-neighborhood.
constexpr int kGridPdsWarps = 4;
template <int D>
struct GridPds {
    // staged stencil candidates + room for the cell's own selections (2^D points pairwise a cell size
    // apart fit in one cell up to D = 3; the kernel falls back to the lists in memory beyond the buffer)
    static constexpr int kOwn = 1 << D;
    static constexpr int kCap = (D >= 5) ? 96 : 320;
};

template <int D>
__device__ __forceinline__ bool within_radius(const float (&s)[D], const float (&q)[D], const float (&inv)[D]) {
    float acc = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const float v = __fmul_rn(__fsub_rn(s[d], q[d]), inv[d]);
        acc = (d == 0) ? __fmul_rn(v, v) : __fmaf_rn(v, v, acc);
    }
    return acc < 1.0f;
}

template <int D>
__global__ void cell_parity_kernel(int n, const int64_t* __restrict__ keys, const int32_t* __restrict__ cell_starts,
                                   const int32_t* __restrict__ grid_size, const int32_t* __restrict__ counters,
                                   unsigned char* __restrict__ code) {
    const GridDesc<D> g = load_grid<D>(grid_size);
    const int num_cells = counters[0];
    const int stride = gridDim.x * blockDim.x;
    for (int cell = blockIdx.x * blockDim.x + threadIdx.x; cell < num_cells; cell += stride) {
        int c[D];
        key_to_cell<D>(keys[cell_starts[cell]], g, c);
        unsigned v = 0;
#pragma unroll
        for (int d = 0; d < D; ++d) v |= (unsigned)(c[d] & 1) << d;
        code[cell] = (unsigned char)v;
    }
}

// D <= 3: the stencil of a cell as cell indices, resolved once for all passes by one thread per
// (cell, range) - the binary searches of thousands of cells overlap here, whereas a pass kernel
// that resolves them itself pays their latency cell after cell.  Entry = first cell index * 4 +
// number of cells (0 ... 3) of the range.
template <int D>
__global__ void stencil_cells_kernel(int n, const int64_t* __restrict__ keys, const int32_t* __restrict__ cell_starts,
                                     const int32_t* __restrict__ counters, const int32_t* __restrict__ cell_of_point,
                                     const int2* __restrict__ grid_ds, const int32_t* __restrict__ grid_size,
                                     int32_t* __restrict__ table) {
    using S = Stencil<D>;
    const GridDesc<D> g = load_grid<D>(grid_size);
    const int num_cells = counters[0];
    const long long total = (long long)num_cells * S::kRanges;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += stride) {
        const int cell = (int)(i / S::kRanges), o = (int)(i - (long long)cell * S::kRanges);
        int c[D], cc[D];
        const int b = key_to_cell<D>(__ldg(keys + __ldg(cell_starts + cell)), g, c);
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
        int2 r = make_int2(0, 0);
        if (inside) {
            const long long ds = ((long long)b * g.nc[0] + cc[0]) * g.nc[1] + cc[1];
            int2 tube = __ldg(grid_ds + ds);
            tube.x = max(tube.x, 0);
            tube.y = min(tube.y, n);
            if (D == 2) {
                r = tube;
            } else if (tube.y > tube.x) {
                const long long k = cell_key<D>(cc, g, b);
                const long long klo = k - (c[D - 1] > 0 ? 1 : 0);
                const long long khi = k + (c[D - 1] < g.nc[D - 1] - 1 ? 1 : 0);
                r.x = lower_bound_key(keys, tube.x, tube.y, klo);
                r.y = upper_bound_key(keys, r.x, tube.y, khi);
            }
        }
        int entry = 0;
        if (r.y > r.x) {
            const int ca = __ldg(cell_of_point + r.x) - 1, cb = __ldg(cell_of_point + r.y - 1) - 1;
            entry = ca * 4 + min(cb - ca + 1, 3);
        }
        table[i] = entry;
    }
}

template <int D>
__global__ void __launch_bounds__(kGridPdsWarps * 32)
pds_grid_pass_kernel(int pass, int n, const float* __restrict__ pts, const int64_t* __restrict__ keys,
                     const int32_t* __restrict__ cell_starts, const int32_t* __restrict__ counters,
                     const unsigned char* __restrict__ code, const int32_t* __restrict__ cell_of_point,
                     const int2* __restrict__ grid_ds, const int32_t* __restrict__ grid_size,
                     const float* __restrict__ radii, const int32_t* __restrict__ table, int32_t* sel_list,
                     int32_t* sel_cnt, int32_t* __restrict__ used) {
    using S = Stencil<D>;
    constexpr int kCap = GridPds<D>::kCap, kOwn = GridPds<D>::kOwn;
    __shared__ int s_lo[kGridPdsWarps][S::kRanges];
    __shared__ int s_pref[kGridPdsWarps][S::kRanges + 1];
    __shared__ float s_cand[kGridPdsWarps][D][kCap];
    const int warp = threadIdx.x >> 5, lane = lane_id();
    const unsigned lt_mask = (1u << lane) - 1u;
    int* lo = s_lo[warp];
    int* pref = s_pref[warp];
    float (*cand)[kCap] = s_cand[warp];
    volatile int32_t* vsel_list = sel_list;
    const GridDesc<D> g = load_grid<D>(grid_size);
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = __frcp_rn(__ldg(radii + d));
    const int num_cells = counters[0];
    const int warps_total = gridDim.x * kGridPdsWarps;

    // A warp looks at 32 cells at a time.  The 32 are taken num_batches apart rather than next to each other:
    // crowded cells sit next to each other in cell order (dense clouds), and spread like this they land in
    // different warps instead of queueing up in one.
    const int num_batches = (num_cells + 31) / 32;
    for (int batch = blockIdx.x * kGridPdsWarps + warp; batch < num_batches; batch += warps_total) {
        const int my_cell = lane * num_batches + batch;
        const bool want = my_cell < num_cells && __ldg(code + my_cell) == (unsigned)pass;
        unsigned todo = __ballot_sync(kFullMask, want);
        while (todo) {
            const int ci = (__ffs(todo) - 1) * num_batches + batch;
            todo &= todo - 1;
            const int first = __ldg(cell_starts + ci);
            const int last = (ci + 1 < num_cells) ? __ldg(cell_starts + ci + 1) : n;
            if (!table) resolve_ranges<D>(__ldg(keys + first), g, grid_ds, keys, n, lo, pref);

            // Selected points of the stencil cells -> shared memory.  A range holds at most three cells
            // (one in 2-D); every lane fetches the short lists of its own range, all loads in flight at once.
            int staged = 0;
            bool staged_all = true;
            for (int o0 = 0; o0 < S::kRanges && staged_all; o0 += 32) {
                const int o = o0 + lane;
                int cf[3] = {0, 0, 0}, cn[3] = {0, 0, 0};
                if (o < S::kRanges) {
                    int ca = 0, cells_here = 0;
                    if (table) {
                        const int entry = __ldg(table + (int64_t)ci * S::kRanges + o);
                        ca = entry >> 2;
                        cells_here = entry & 3;
                    } else {
                        const int len = pref[o + 1] - pref[o];
                        if (len > 0) {
                            ca = __ldg(cell_of_point + lo[o]) - 1;
                            cells_here = __ldg(cell_of_point + lo[o] + len - 1) - ca;
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 3; ++j) {
                        if (j < cells_here) {
                            cn[j] = sel_cnt[ca + j];
                            cf[j] = __ldg(cell_starts + ca + j);
                        }
                    }
                }
                const int mine = cn[0] + cn[1] + cn[2];
                int incl = mine;
#pragma unroll
                for (int sft = 1; sft < 32; sft <<= 1) {
                    const int v = __shfl_up_sync(kFullMask, incl, sft);
                    if (lane >= sft) incl += v;
                }
                const int batch = __shfl_sync(kFullMask, incl, 31);
                if (staged + batch > kCap - kOwn) {
                    staged_all = false;  // too many for the buffer: this cell reads the lists from memory instead
                    break;
                }
                int pos = staged + incl - mine;
#pragma unroll
                for (int j = 0; j < 3; ++j) {
                    for (int k = 0; k < cn[j]; ++k) {
                        const int q = sel_list[cf[j] + k];
#pragma unroll
                        for (int d = 0; d < D; ++d) cand[d][pos] = __ldg(pts + (int64_t)q * D + d);
                        ++pos;
                    }
                }
                staged += batch;
            }
            __syncwarp();

            int own = 0;  // points of this cell selected so far
            for (int p0 = first; p0 < last; p0 += 32) {
                const int p = p0 + lane, count = min(32, last - p0);
                const bool has = p < last;
                float x[D];
#pragma unroll
                for (int d = 0; d < D; ++d) x[d] = has ? __ldg(pts + (int64_t)p * D + d) : 0.f;
                bool blocked = !has;
                if (staged_all) {
                    // staged stencil selections followed by this cell's own earlier selections
                    for (int i = 0; i < staged; ++i) {
                        float q[D];
#pragma unroll
                        for (int d = 0; d < D; ++d) q[d] = cand[d][i];
                        blocked = blocked | within_radius<D>(x, q, inv);
                    }
                } else {
                    for (int o = 0; o < S::kRanges; ++o) {
                        int ca, cb;
                        if (table) {
                            const int entry = __ldg(table + (int64_t)ci * S::kRanges + o);
                            ca = entry >> 2;
                            cb = ca + (entry & 3) - 1;
                        } else {
                            const int len = pref[o + 1] - pref[o];
                            if (len <= 0) continue;
                            ca = __ldg(cell_of_point + lo[o]) - 1;
                            cb = __ldg(cell_of_point + lo[o] + len - 1) - 1;
                        }
                        for (int c = ca; c <= cb; ++c) {
                            if (c == ci) continue;  // own selections are taken from the list below
                            const int cnt = sel_cnt[c], cfirst = __ldg(cell_starts + c);
                            for (int k = 0; k < cnt; ++k) {
                                const int qi = sel_list[cfirst + k];
                                float q[D];
#pragma unroll
                                for (int d = 0; d < D; ++d) q[d] = __ldg(pts + (int64_t)qi * D + d);
                                blocked = blocked | within_radius<D>(x, q, inv);
                            }
                        }
                    }
                    for (int k = 0; k < own; ++k) {
                        const int qi = vsel_list[first + k];
                        float q[D];
#pragma unroll
                        for (int d = 0; d < D; ++d) q[d] = __ldg(pts + (int64_t)qi * D + d);
                        blocked = blocked | within_radius<D>(x, q, inv);
                    }
                }
                // earlier points of the same group that are this point's neighbors
                unsigned in_group = 0u;
                for (int qi = 0; qi < count; ++qi) {
                    float q[D];
#pragma unroll
                    for (int d = 0; d < D; ++d) q[d] = __shfl_sync(kFullMask, x[d], qi);
                    if (qi != lane && within_radius<D>(x, q, inv)) in_group |= 1u << qi;
                }
                const unsigned selected = decide_group(count, blocked, in_group);
                const int rank = __popc(selected & lt_mask);
                if (has && ((selected >> lane) & 1u)) {
                    used[p] = 1;
                    vsel_list[first + own + rank] = p;
                    if (staged_all && staged + rank < kCap) {
#pragma unroll
                        for (int d = 0; d < D; ++d) cand[d][staged + rank] = x[d];
                    }
                }
                const int fresh = __popc(selected);
                own += fresh;
                if (staged_all) {
                    // more selections than the buffer holds (possible in five or more dimensions, where a
                    // cell can host more than 2^D points a cell size apart): the remaining groups of this
                    // cell read the lists from memory, which are complete
                    if (staged + fresh > kCap) staged_all = false;
                    else staged += fresh;
                }
                __syncwarp();
            }
            if (lane == 0) sel_cnt[ci] = own;
            __syncwarp();
        }
    }
}

struct GridPdsLayout {
    size_t flags_off, cells_off, used_off, cell_of_point_off, sel_list_off, sel_cnt_off, counters_off, cub_off, cub_bytes,
        table_off, total;
};

static GridPdsLayout grid_pds_layout(int64_t n) {
    GridPdsLayout L;
    const int nn = (int)(n > 0 ? n : 1);
    size_t a = 0, b = 0, c = 0;
    cub::DeviceSelect::Flagged(nullptr, a, thrust::counting_iterator<int32_t>(0), (const int32_t*)nullptr,
                               (int32_t*)nullptr, (int32_t*)nullptr, nn);
    cub::DeviceSelect::Flagged(nullptr, b, thrust::counting_iterator<int64_t>(0), (const int32_t*)nullptr,
                               (int64_t*)nullptr, (int32_t*)nullptr, nn);
    cub::DeviceScan::InclusiveSum(nullptr, c, (const int32_t*)nullptr, (int32_t*)nullptr, nn);
    L.cub_bytes = a > b ? a : b;
    if (c > L.cub_bytes) L.cub_bytes = c;
    const size_t slice = align_up((size_t)n * 4);
    L.flags_off = 0;
    L.cells_off = slice;
    L.used_off = 2 * slice;
    L.cell_of_point_off = 3 * slice;
    L.sel_list_off = 4 * slice;
    L.sel_cnt_off = 5 * slice;
    L.counters_off = 6 * slice;
    L.cub_off = L.counters_off + 256;
    // stencil table of the D <= 3 path: 9 entries per cell (higher dimensions resolve the ranges in the pass kernel)
    L.table_off = L.cub_off + align_up(L.cub_bytes) + 256;
    L.total = L.table_off + align_up((size_t)n * 9 * 4);
    return L;
}

}  // namespace pccnn

using namespace pccnn;

extern "C" {

size_t pccnn_poisson_disk_sampling_workspace_bytes(int64_t n) { return pds_layout(n < 0 ? 0 : n).total; }

int pccnn_poisson_disk_sampling(int D, int64_t n, const int64_t* sorted_keys, const int32_t* neighbors,
                                const int32_t* start_ids, const int32_t* grid_size, int64_t* out_selected,
                                int64_t* out_count_host, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims, "poisson_disk_sampling: point dimension %d outside [2, 6]", D);
    PCCNN_CHECK_ARG(n >= 0 && n < 0x7fffffffLL, "poisson_disk_sampling: %lld points outside [0, 2^31)", (long long)n);
    PCCNN_CHECK_ARG(out_count_host, "poisson_disk_sampling: null out_count_host");
    *out_count_host = 0;
    if (n == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(sorted_keys && start_ids && grid_size && out_selected, "poisson_disk_sampling: null pointer");
    const PdsLayout L = pds_layout(n);
    if (!workspace || workspace_bytes < L.total) {
        set_error("poisson_disk_sampling: workspace of %zu bytes, need %zu", workspace_bytes, L.total);
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    int32_t* flags = (int32_t*)(ws + L.flags_off);
    int32_t* cells = (int32_t*)(ws + L.cells_off);
    int32_t* used = (int32_t*)(ws + L.used_off);
    int32_t* counters = (int32_t*)(ws + L.counters_off);  // [0] = occupied cells, [1] = selected points, [2] = crowded cells
    // The cell-boundary flags are dead once the cell list exists; their 4 n bytes then hold one routing
    // byte per cell (at most n cells) and, behind those, the crowded-cell list.  A cell that finds the
    // list full stays with the warp-per-cell kernel, which handles any cell.
    unsigned char* code = (unsigned char*)flags;
    const size_t code_bytes = align_up((size_t)n);
    int32_t* crowded = (int32_t*)(ws + L.flags_off + code_bytes);
    const int crowded_capacity = (int)((L.cells_off - L.flags_off > code_bytes ? L.cells_off - L.flags_off - code_bytes : 0) / 4);
    const int nn = (int)n;

    cell_flags_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>(nn, sorted_keys, flags);
    PCCNN_LAUNCH_CHECK();
    size_t cub_bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceSelect::Flagged(ws + L.cub_off, cub_bytes, thrust::counting_iterator<int32_t>(0), flags,
                                          cells, counters, nn, s));
    PCCNN_CUDA(cudaMemsetAsync(used, 0, (size_t)n * 4, s));
    PCCNN_CUDA(cudaMemsetAsync(counters + 2, 0, 4, s));
    PCCNN_DISPATCH_DIM(D, (cell_route_kernel<DIM><<<grid_for(n, 256, 8), 256, 0, s>>>(
                              nn, sorted_keys, cells, start_ids, grid_size, counters, code, crowded, crowded_capacity)));
    PCCNN_LAUNCH_CHECK();
    // two blocks of each role per SM: 2048 threads and 4 x 33 KB of shared memory, all resident at once
    const int crowded_blocks = 2 * sm_count();
    const unsigned sparse_blocks = grid_for((n + 31) / 32 * 32, kPdsThreads, 2);
    for (int pass = 0; pass < (1 << D); ++pass) {
        pds_pass_kernel<<<crowded_blocks + sparse_blocks, kPdsThreads, 0, s>>>(
            pass, nn, crowded_blocks, cells, counters, code, crowded, crowded_capacity, (const int2*)neighbors, start_ids,
            used);
        PCCNN_LAUNCH_CHECK();
    }
    cub_bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceSelect::Flagged(ws + L.cub_off, cub_bytes, thrust::counting_iterator<int64_t>(0), used,
                                          out_selected, counters + 1, nn, s));
    int32_t count = 0;
    PCCNN_CUDA(cudaMemcpyAsync(&count, counters + 1, 4, cudaMemcpyDeviceToHost, s));
    PCCNN_CUDA(cudaStreamSynchronize(s));
    *out_count_host = count;
    return PCCNN_OK;
}

size_t pccnn_poisson_disk_sampling_grid_workspace_bytes(int64_t n) { return grid_pds_layout(n < 0 ? 0 : n).total; }

int pccnn_poisson_disk_sampling_grid(int D, int64_t n, const float* sorted_pts, const int64_t* sorted_keys,
                                     const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                                     int64_t* out_selected, int64_t* out_count_host, void* workspace,
                                     size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims, "poisson_disk_sampling_grid: point dimension %d outside [2, 6]", D);
    PCCNN_CHECK_ARG(n >= 0 && n < 0x7fffffffLL, "poisson_disk_sampling_grid: %lld points outside [0, 2^31)", (long long)n);
    PCCNN_CHECK_ARG(out_count_host, "poisson_disk_sampling_grid: null out_count_host");
    *out_count_host = 0;
    if (n == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(sorted_pts && sorted_keys && grid_ds && grid_size && radii && out_selected,
                    "poisson_disk_sampling_grid: null pointer");
    const GridPdsLayout L = grid_pds_layout(n);
    if (!workspace || workspace_bytes < L.total) {
        set_error("poisson_disk_sampling_grid: workspace of %zu bytes, need %zu", workspace_bytes, L.total);
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    int32_t* flags = (int32_t*)(ws + L.flags_off);
    int32_t* cells = (int32_t*)(ws + L.cells_off);
    int32_t* used = (int32_t*)(ws + L.used_off);
    int32_t* cell_of_point = (int32_t*)(ws + L.cell_of_point_off);  // 1-based index of the point's cell
    int32_t* sel_list = (int32_t*)(ws + L.sel_list_off);
    int32_t* sel_cnt = (int32_t*)(ws + L.sel_cnt_off);
    int32_t* counters = (int32_t*)(ws + L.counters_off);  // [0] = occupied cells, [1] = selected points
    const int nn = (int)n;

    cell_flags_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>(nn, sorted_keys, flags);
    PCCNN_LAUNCH_CHECK();
    size_t cub_bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceSelect::Flagged(ws + L.cub_off, cub_bytes, thrust::counting_iterator<int32_t>(0), flags,
                                          cells, counters, nn, s));
    cub_bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceScan::InclusiveSum(ws + L.cub_off, cub_bytes, flags, cell_of_point, nn, s));
    // used and the per-cell counts start at zero; the flags are dead now and their space takes the routing bytes
    PCCNN_CUDA(cudaMemsetAsync(used, 0, (size_t)n * 4, s));
    PCCNN_CUDA(cudaMemsetAsync(sel_cnt, 0, (size_t)n * 4, s));
    unsigned char* code = (unsigned char*)flags;
    PCCNN_DISPATCH_DIM(D, (cell_parity_kernel<DIM><<<grid_for(n, 256, 8), 256, 0, s>>>(nn, sorted_keys, cells, grid_size,
                                                                                  counters, code)));
    PCCNN_LAUNCH_CHECK();
    int32_t* table = nullptr;
    if (D <= 3) {
        table = (int32_t*)(ws + L.table_off);
        if (D == 2) {
            stencil_cells_kernel<2><<<grid_for(n * 9, 256, 8), 256, 0, s>>>(nn, sorted_keys, cells, counters, cell_of_point,
                                                                           (const int2*)grid_ds, grid_size, table);
        } else {
            stencil_cells_kernel<3><<<grid_for(n * 9, 256, 8), 256, 0, s>>>(nn, sorted_keys, cells, counters, cell_of_point,
                                                                           (const int2*)grid_ds, grid_size, table);
        }
        PCCNN_LAUNCH_CHECK();
    }
    const unsigned grid = grid_for(n, kGridPdsWarps * 32, 16);
    for (int pass = 0; pass < (1 << D); ++pass) {
        PCCNN_DISPATCH_DIM(D, (pds_grid_pass_kernel<DIM><<<grid, kGridPdsWarps * 32, 0, s>>>(
                                  pass, nn, sorted_pts, sorted_keys, cells, counters, code, cell_of_point,
                                  (const int2*)grid_ds, grid_size, radii, table, sel_list, sel_cnt, used)));
        PCCNN_LAUNCH_CHECK();
    }
    cub_bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceSelect::Flagged(ws + L.cub_off, cub_bytes, thrust::counting_iterator<int64_t>(0), used,
                                          out_selected, counters + 1, nn, s));
    int32_t count = 0;
    PCCNN_CUDA(cudaMemcpyAsync(&count, counters + 1, 4, cudaMemcpyDeviceToHost, s));
    PCCNN_CUDA(cudaStreamSynchronize(s));
    *out_count_host = count;
    return PCCNN_OK;
}

// ---- variant for callers that cannot allocate device memory ---------------------------------
// Scratch of the variant below: a fixed array inside the library image.  Every GPU that loads the
// library keeps these bytes until the process exits.
constexpr int64_t kStaticPdsMaxPoints = 1 << 20;
constexpr size_t kStaticPdsBytes = (size_t)14 << 20;
static __device__ __align__(256) unsigned char g_pds_static_scratch[kStaticPdsBytes];

int64_t pccnn_poisson_disk_sampling_static_max_points(void) { return kStaticPdsMaxPoints; }

int pccnn_poisson_disk_sampling_static(int D, int64_t n, const int64_t* sorted_keys, const int32_t* neighbors,
                                       const int32_t* start_ids, const int32_t* grid_size, int64_t* out_selected,
                                       int64_t* out_count_host, void* stream) {
    PCCNN_CHECK_ARG(out_count_host, "poisson_disk_sampling_static: null out_count_host");
    *out_count_host = 0;
    if (n > kStaticPdsMaxPoints || pds_layout(n < 0 ? 0 : n).total > kStaticPdsBytes) {
        set_error("poisson_disk_sampling_static: %lld points exceed the built-in scratch (at most %lld points); "
                  "use pccnn_poisson_disk_sampling with a caller-provided workspace",
                  (long long)n, (long long)kStaticPdsMaxPoints);
        return PCCNN_ERR_INVALID;
    }
    // In host code the array's name is only a handle; the device address has to be asked for, once
    // per device, with that device current.
    static void* device_ptr[64];
    static std::mutex mu;
    int dev = 0;
    PCCNN_CUDA(cudaGetDevice(&dev));
    PCCNN_CHECK_ARG(dev >= 0 && dev < 64, "poisson_disk_sampling_static: device index %d not supported", dev);
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!device_ptr[dev]) {
            void* p = nullptr;
            PCCNN_CUDA(cudaGetSymbolAddress(&p, g_pds_static_scratch));
            device_ptr[dev] = p;
        }
        scratch = device_ptr[dev];
    }
    // Same implementation as the workspace variant; it zeroes the selection flags and re-initialises
    // the compaction state itself, so nothing of the previous call's contents is read.
    return pccnn_poisson_disk_sampling(D, n, sorted_keys, neighbors, start_ids, grid_size, out_selected,
                                       out_count_host, scratch, kStaticPdsBytes, stream);
}

}  // extern "C"
