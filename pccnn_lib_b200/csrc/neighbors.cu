// Radius neighbor search on the uniform grid, emitting int32 CSR lists.
//
// Semantics follow pccnn_lib_ops/find_neighbors/{find_ranges_grid_ds,count_neighbors,
// store_neighbors}.cu of phermosilla/pccnn_lib: candidates are the points of the 3^D cell
// stencil of the sample's cell inside the sample's cloud; a candidate p is kept iff
// sqrtf(sum_d ((s_d - p_d) * (1/r_d))^2) < 1.0f with the sum taken as an FMA chain in
// ascending d (nvcc contracts math_helper.cuh:309-313 that way).  sqrtf is monotone and
// correctly rounded, and the largest float below 1 has a square root that still rounds below
// 1, so the predicate equals `sum < 1.0f`; the kernels test that and skip the square root.
//
// Design: one warp per sample.  The lanes first resolve the 3^(D-1) candidate ranges in
// parallel (cell-range table lookup + binary search for the three consecutive last-dimension
// cells, which are contiguous in the sorted array), park them in shared memory, then sweep
// each range 32 candidates at a time with coalesced loads.  __ballot_sync + popc give every
// hit its rank, so rows come out in ascending point index without atomics and the result is
// deterministic.  A count pass, a device-wide scan and a store pass replace the reference's
// three kernels + cumsum; the candidate ranges never travel through HBM.
#include <cub/device/device_scan.cuh>

#include "common.cuh"

namespace pccnn {

template <int D>
struct Stencil {
    // Dimensions that receive a -1/0/+1 offset: all but the last one (whose +-1 window is a
    // contiguous key range), except in 2-D where the table is indexed by the full cell.
    static constexpr int kOffsetDims = (D == 2) ? 2 : D - 1;
    static constexpr int pow3(int e) { return e == 0 ? 1 : 3 * pow3(e - 1); }
    static constexpr int kRanges = pow3(kOffsetDims);
};

constexpr int kWarpsPerBlock = 4;

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

// Candidate ranges of one sample, ascending in sorted position; computed by the whole warp.
template <int D>
__device__ __forceinline__ void resolve_ranges(long long key, const GridDesc<D>& g,
                                               const int2* __restrict__ grid_ds,
                                               const int64_t* __restrict__ pt_keys, int num_pts,
                                               int2* __restrict__ ranges) {
    using S = Stencil<D>;
    int c[D];
    const int b = key_to_cell<D>(key, g, c);
    for (int o = lane_id(); o < S::kRanges; o += 32) {
        int2 r = make_int2(0, 0);
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
        if (r.y < r.x) r.y = r.x;
        ranges[o] = r;
    }
    __syncwarp();
}

template <int D>
__device__ __forceinline__ bool in_radius(const float (&s)[D], const float* __restrict__ p,
                                          const float (&inv)[D]) {
    float acc = 0.f;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        const float v = __fmul_rn(__fsub_rn(s[d], __ldg(p + d)), inv[d]);
        acc = (d == 0) ? __fmul_rn(v, v) : __fmaf_rn(v, v, acc);
    }
    return acc < 1.0f;
}

enum : int { kCount = 0, kStore = 1, kStoreLimited = 2 };

template <int D, int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
neighbors_kernel(int num_pts, const float* __restrict__ pts, const int64_t* __restrict__ pt_keys,
                 int num_samples, const float* __restrict__ samples, const int64_t* __restrict__ sample_keys,
                 const int2* __restrict__ grid_ds, const int32_t* __restrict__ grid_size,
                 const float* __restrict__ radii, int max_neighbors,
                 int32_t* __restrict__ counts,             // kCount: out; kStoreLimited: raw counts in
                 const int32_t* __restrict__ start_ids,    // stores: inclusive ends
                 const int64_t* __restrict__ pt_index_map, int2* __restrict__ out) {
    using S = Stencil<D>;
    __shared__ int2 s_ranges[kWarpsPerBlock][S::kRanges];
    const int warp = threadIdx.x >> 5, lane = lane_id();
    const unsigned lt_mask = (1u << lane) - 1u;
    const GridDesc<D> g = load_grid<D>(grid_size);
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = __frcp_rn(__ldg(radii + d));

    const int warps_total = gridDim.x * kWarpsPerBlock;
    for (int m = blockIdx.x * kWarpsPerBlock + warp; m < num_samples; m += warps_total) {
        resolve_ranges<D>(__ldg(sample_keys + m), g, grid_ds, pt_keys, num_pts, s_ranges[warp]);
        float s[D];
#pragma unroll
        for (int d = 0; d < D; ++d) s[d] = __ldg(samples + (int64_t)m * D + d);

        int found = 0;
        int base = 0, total = 0;
        if (MODE != kCount) base = (m > 0) ? __ldg(start_ids + m - 1) : 0;
        if (MODE == kStoreLimited) total = __ldg(counts + m);
        const bool thin = (MODE == kStoreLimited) && total > max_neighbors;

        for (int r = 0; r < S::kRanges; ++r) {
            const int2 rg = s_ranges[warp][r];
            for (int j0 = rg.x; j0 < rg.y; j0 += 32) {
                const int j = j0 + lane;
                const bool hit = (j < rg.y) && in_radius<D>(s, pts + (int64_t)j * D, inv);
                const unsigned bal = __ballot_sync(kFullMask, hit);
                if (MODE != kCount && hit) {
                    const int rank = found + __popc(bal & lt_mask);
                    const int id = pt_index_map ? (int)__ldg(pt_index_map + j) : j;
                    if (!thin) {
                        out[base + rank] = make_int2(id, m);
                    } else {
                        // Even-stride thinning: hit `rank` of `total` is kept iff it starts a new
                        // one of the max_neighbors equal slices of the list.
                        const long long a = (long long)rank * max_neighbors / total;
                        const long long bnext = (long long)(rank + 1) * max_neighbors / total;
                        if (bnext > a) out[base + (int)a] = make_int2(id, m);
                    }
                }
                found += __popc(bal);
            }
        }
        if (MODE == kCount && lane == 0) counts[m] = found;
        __syncwarp();
    }
}

__global__ void clamp_counts_kernel(int n, const int32_t* __restrict__ counts, int max_neighbors,
                                    int32_t* __restrict__ out, unsigned long long* __restrict__ total) {
    unsigned long long local = 0;
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int c = counts[i];
        if (max_neighbors > 0) c = min(c, max_neighbors);
        out[i] = c;
        local += (unsigned long long)c;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(kFullMask, local, o);
    if (lane_id() == 0 && local) atomicAdd(total, local);
}

struct NeighborLayout {
    size_t counts_off, total_off, cub_off, cub_bytes, total;
};

static NeighborLayout neighbor_layout(int64_t m) {
    NeighborLayout L;
    size_t cub_bytes = 0;
    cub::DeviceScan::InclusiveSum(nullptr, cub_bytes, (const int32_t*)nullptr, (int32_t*)nullptr,
                                  (int)(m > 0 ? m : 1));
    L.counts_off = 0;
    L.total_off = align_up((size_t)m * 4);
    L.cub_off = L.total_off + 256;
    L.cub_bytes = cub_bytes;
    L.total = L.cub_off + align_up(cub_bytes) + 256;
    return L;
}

static int check_common(const char* who, int D, int64_t num_pts, int64_t num_samples) {
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims, "%s: point dimension %d outside [2, 6]", who, D);
    PCCNN_CHECK_ARG(num_pts >= 0 && num_pts < 0x7fffffffLL, "%s: %lld points outside [0, 2^31)", who,
                    (long long)num_pts);
    PCCNN_CHECK_ARG(num_samples >= 0 && num_samples < 0x7fffffffLL, "%s: %lld samples outside [0, 2^31)", who,
                    (long long)num_samples);
    return PCCNN_OK;
}

}  // namespace pccnn

using namespace pccnn;

extern "C" {

size_t pccnn_find_neighbors_workspace_bytes(int D, int64_t num_samples) {
    (void)D;
    return neighbor_layout(num_samples < 0 ? 0 : num_samples).total;
}

int pccnn_find_neighbors_count(int D, int64_t num_pts, const float* pts, const int64_t* pt_keys,
                               int64_t num_samples, const float* samples, const int64_t* sample_keys,
                               const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                               int32_t max_neighbors, int32_t* out_start_ids, int64_t* out_total_host,
                               void* workspace, size_t workspace_bytes, void* stream) {
    if (int rc = check_common("find_neighbors_count", D, num_pts, num_samples)) return rc;
    PCCNN_CHECK_ARG(out_total_host, "find_neighbors_count: null out_total_host");
    PCCNN_CHECK_ARG(max_neighbors >= 0, "find_neighbors_count: negative max_neighbors");
    *out_total_host = 0;
    if (num_samples == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(samples && sample_keys && grid_ds && grid_size && radii && out_start_ids,
                    "find_neighbors_count: null pointer");
    PCCNN_CHECK_ARG(num_pts == 0 || (pts && pt_keys), "find_neighbors_count: null points");
    const NeighborLayout L = neighbor_layout(num_samples);
    if (!workspace || workspace_bytes < L.total) {
        set_error("find_neighbors_count: workspace of %zu bytes, need %zu", workspace_bytes, L.total);
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    int32_t* counts = (int32_t*)(ws + L.counts_off);
    unsigned long long* total_dev = (unsigned long long*)(ws + L.total_off);
    PCCNN_CUDA(cudaMemsetAsync(total_dev, 0, 8, s));
    const unsigned grid = grid_for(num_samples * 32, kWarpsPerBlock * 32, 16);
    PCCNN_DISPATCH_DIM(D, (neighbors_kernel<DIM, kCount><<<grid, kWarpsPerBlock * 32, 0, s>>>(
                              (int)num_pts, pts, pt_keys, (int)num_samples, samples, sample_keys,
                              (const int2*)grid_ds, grid_size, radii, max_neighbors, counts, nullptr, nullptr,
                              nullptr)));
    PCCNN_LAUNCH_CHECK();
    clamp_counts_kernel<<<grid_for(num_samples, 256, 8), 256, 0, s>>>((int)num_samples, counts, max_neighbors,
                                                                     out_start_ids, total_dev);
    PCCNN_LAUNCH_CHECK();
    size_t cub_bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceScan::InclusiveSum(ws + L.cub_off, cub_bytes, out_start_ids, out_start_ids,
                                             (int)num_samples, s));
    unsigned long long total = 0;
    PCCNN_CUDA(cudaMemcpyAsync(&total, total_dev, 8, cudaMemcpyDeviceToHost, s));
    PCCNN_CUDA(cudaStreamSynchronize(s));
    *out_total_host = (int64_t)total;
    if (total >= 0x80000000ULL) {
        set_error("find_neighbors_count: %llu neighbor pairs do not fit the int32 CSR offsets; split the batch",
                  total);
        return PCCNN_ERR_OVERFLOW;
    }
    return PCCNN_OK;
}

int pccnn_find_neighbors_store(int D, int64_t num_pts, const float* pts, const int64_t* pt_keys,
                               int64_t num_samples, const float* samples, const int64_t* sample_keys,
                               const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                               int32_t max_neighbors, const int32_t* start_ids, const int64_t* pt_index_map,
                               int32_t* out_neighbors, void* workspace, size_t workspace_bytes, void* stream) {
    if (int rc = check_common("find_neighbors_store", D, num_pts, num_samples)) return rc;
    PCCNN_CHECK_ARG(max_neighbors >= 0, "find_neighbors_store: negative max_neighbors");
    if (num_samples == 0 || num_pts == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(pts && pt_keys && samples && sample_keys && grid_ds && grid_size && radii && start_ids,
                    "find_neighbors_store: null pointer");
    const NeighborLayout L = neighbor_layout(num_samples);
    if (!workspace || workspace_bytes < L.total) {
        set_error("find_neighbors_store: workspace of %zu bytes, need %zu", workspace_bytes, L.total);
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    int32_t* counts = (int32_t*)((char*)workspace + L.counts_off);
    const unsigned grid = grid_for(num_samples * 32, kWarpsPerBlock * 32, 16);
    if (max_neighbors > 0) {
        PCCNN_DISPATCH_DIM(D, (neighbors_kernel<DIM, kStoreLimited><<<grid, kWarpsPerBlock * 32, 0, s>>>(
                                  (int)num_pts, pts, pt_keys, (int)num_samples, samples, sample_keys,
                                  (const int2*)grid_ds, grid_size, radii, max_neighbors, counts, start_ids,
                                  pt_index_map, (int2*)out_neighbors)));
    } else {
        PCCNN_DISPATCH_DIM(D, (neighbors_kernel<DIM, kStore><<<grid, kWarpsPerBlock * 32, 0, s>>>(
                                  (int)num_pts, pts, pt_keys, (int)num_samples, samples, sample_keys,
                                  (const int2*)grid_ds, grid_size, radii, max_neighbors, counts, start_ids,
                                  pt_index_map, (int2*)out_neighbors)));
    }
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

}  // extern "C"
