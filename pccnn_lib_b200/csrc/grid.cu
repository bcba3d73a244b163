// Uniform-grid front end: bounding boxes, grid sizing, cell keys, stable key sort with the
// gathers that follow it, and the (batch, c0, c1) cell-range table.
//
// All of these are streaming kernels bound by HBM bandwidth: one thread per point, fully
// coalesced loads/stores, grid sized as a multiple of the SM count.  The arithmetic restates
// pccnn_lib_ops/compute_keys/compute_keys.cu:35-74, shared/grid_utils.cuh:57-137 and
// build_grid/build_grid_ds.cu:32-68 of phermosilla/pccnn_lib operation for operation so that
// keys and tables are bit-identical.
#include <cub/device/device_radix_sort.cuh>
#include <stdarg.h>

#include <mutex>

#include "common.cuh"

namespace pccnn {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static int cached[64];
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

// ---- bounding box -------------------------------------------------------------------------
// Floats are mapped to ints whose signed order equals the float order, so the exact min/max
// can be taken with integer atomics.
__device__ __forceinline__ int float_to_ordered(float f) {
    int i = __float_as_int(f);
    return i >= 0 ? i : i ^ 0x7fffffff;
}
__device__ __forceinline__ float ordered_to_float(int i) {
    return __int_as_float(i >= 0 ? i : i ^ 0x7fffffff);
}

__global__ void bbox_init_kernel(int64_t count, int* mn, int* mx) {
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < count) {
        mn[i] = float_to_ordered(__int_as_float(0x7f800000));  // +inf
        mx[i] = float_to_ordered(__int_as_float(0xff800000));  // -inf
    }
}

constexpr int kBboxItems = 16;  // points per thread

template <int D>
__device__ __forceinline__ void bbox_flush(int b, const float (&lo)[D], const float (&hi)[D], int* mn, int* mx) {
#pragma unroll
    for (int d = 0; d < D; ++d) {
        atomicMin(mn + (int64_t)b * D + d, float_to_ordered(lo[d]));
        atomicMax(mx + (int64_t)b * D + d, float_to_ordered(hi[d]));
    }
}

template <int D>
__global__ void __launch_bounds__(256)
bbox_accum_kernel(int64_t n, const float* __restrict__ pts, const int32_t* __restrict__ batch_ids,
                  int64_t num_batches, int* mn, int* mx) {
    // A block owns 256 * kBboxItems consecutive points; a thread strides through them by 256 so
    // loads stay coalesced.  Clouds are stored contiguously, so a thread almost always sees one
    // cloud: it keeps a running min/max in registers and only touches memory when the cloud
    // changes.  Warps that hold a single cloud then reduce with shuffles: one atomic pair per
    // dimension and warp instead of one per point.
    const float inf = __int_as_float(0x7f800000);
    const int64_t base = (int64_t)blockIdx.x * (256 * kBboxItems);
    int cur = -1;
    float lo[D], hi[D];
#pragma unroll
    for (int d = 0; d < D; ++d) { lo[d] = inf; hi[d] = -inf; }
#pragma unroll 4
    for (int it = 0; it < kBboxItems; ++it) {
        const int64_t i = base + it * 256 + threadIdx.x;
        if (i >= n) break;
        const int b = batch_ids[i];
        if (b < 0 || b >= num_batches) continue;
        if (b != cur) {
            if (cur >= 0) bbox_flush<D>(cur, lo, hi, mn, mx);
            cur = b;
#pragma unroll
            for (int d = 0; d < D; ++d) { lo[d] = inf; hi[d] = -inf; }
        }
#pragma unroll
        for (int d = 0; d < D; ++d) {
            const float v = pts[i * D + d];
            lo[d] = fminf(lo[d], v);
            hi[d] = fmaxf(hi[d], v);
        }
    }
    const int c0 = __shfl_sync(kFullMask, cur, 0);
    const bool uniform = __all_sync(kFullMask, cur == c0 || cur < 0) && c0 >= 0;
    if (uniform) {
#pragma unroll
        for (int d = 0; d < D; ++d) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                lo[d] = fminf(lo[d], __shfl_xor_sync(kFullMask, lo[d], o));
                hi[d] = fmaxf(hi[d], __shfl_xor_sync(kFullMask, hi[d], o));
            }
        }
        if (lane_id() == 0) bbox_flush<D>(c0, lo, hi, mn, mx);
    } else if (cur >= 0) {
        bbox_flush<D>(cur, lo, hi, mn, mx);
    }
}

__global__ void bbox_finish_kernel(int64_t count, int* mn, int* mx) {
    int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x;
    if (i < count) {
        float lo = ordered_to_float(mn[i]);
        float hi = ordered_to_float(mx[i]);
        reinterpret_cast<float*>(mn)[i] = __fsub_rn(lo, 1e-6f);
        reinterpret_cast<float*>(mx)[i] = __fadd_rn(hi, 1e-6f);
    }
}

template <int D>
__global__ void num_cells_kernel(int64_t num_batches, const float* __restrict__ mn,
                                 const float* __restrict__ mx, const float* __restrict__ cell,
                                 int32_t* __restrict__ out) {
    // One warp per dimension; a single small block.
    const int d = threadIdx.x >> 5;
    if (d >= D) return;
    const float c = cell[d];
    int best = INT_MIN;
    for (int64_t b = lane_id(); b < num_batches; b += 32) {
        float q = __fdiv_rn(__fsub_rn(mx[b * D + d], mn[b * D + d]), c);
        int v = (int)q + 1;  // truncation toward zero, as Tensor.to(int32)
        best = max(best, v);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(kFullMask, best, o));
    if (lane_id() == 0) out[d] = best;
}

// ---- keys ---------------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256)
compute_keys_kernel(int64_t n, const float* __restrict__ pts, const int32_t* __restrict__ batch_ids,
                    const float* __restrict__ aabb_min, const int32_t* __restrict__ grid_size,
                    const float* __restrict__ cell_size, int64_t* __restrict__ out_keys) {
    const GridDesc<D> g = load_grid<D>(grid_size);
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = __frcp_rn(__ldg(cell_size + d));  // == torch::reciprocal
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += stride) {
        const int b = batch_ids[i];
        int c[D];
#pragma unroll
        for (int d = 0; d < D; ++d) {
            // (p - min) * inv in two separately rounded steps, then floor, then clamp.
            float rel = __fmul_rn(__fsub_rn(pts[i * D + d], __ldg(aabb_min + (int64_t)b * D + d)), inv[d]);
            int ci = (int)floorf(rel);
            c[d] = min(max(ci, 0), g.nc[d] - 1);
        }
        out_keys[i] = cell_key<D>(c, g, b);
    }
}

// ---- sort ---------------------------------------------------------------------------------
__global__ void iota_kernel(int64_t n, int32_t* out) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += stride) out[i] = (int32_t)i;
}

template <int D>
__global__ void __launch_bounds__(256)
gather_sorted_kernel(int64_t n, const int32_t* __restrict__ ids, const float* __restrict__ pts,
                     int64_t* __restrict__ out_ids, float* __restrict__ out_pts) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += stride) {
        const int32_t id = ids[i];
        out_ids[i] = id;
        if constexpr (D > 0) {
#pragma unroll
            for (int d = 0; d < D; ++d) out_pts[i * D + d] = __ldg(pts + (int64_t)id * D + d);
        }
    }
}

struct SortLayout {
    size_t iota_off, ids_off, cub_off, cub_bytes, total;
};

static SortLayout sort_layout(int64_t n) {
    SortLayout L;
    size_t cub_bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, cub_bytes, (const int64_t*)nullptr, (int64_t*)nullptr,
                                    (const int32_t*)nullptr, (int32_t*)nullptr, (int64_t)(n > 0 ? n : 1), 0, 64);
    L.iota_off = 0;
    L.ids_off = align_up((size_t)n * 4);
    L.cub_off = L.ids_off + align_up((size_t)n * 4);
    L.cub_bytes = cub_bytes;
    L.total = L.cub_off + align_up(cub_bytes) + 256;
    return L;
}

// ---- cell-range table ---------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256)
build_grid_kernel(int64_t n, const int64_t* __restrict__ keys, const int32_t* __restrict__ grid_size,
                  int64_t num_entries, int2* __restrict__ out) {
    long long div = 1;
#pragma unroll
    for (int d = 2; d < D; ++d) div *= __ldg(grid_size + d);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = blockIdx.x * (int64_t)blockDim.x + threadIdx.x; i < n; i += stride) {
        const long long cur = keys[i] / div;
        if (cur < 0 || cur >= num_entries) continue;  // keys outside the table are ignored
        if (i > 0 && keys[i - 1] / div != cur) out[cur].x = (int)i;
        if (i + 1 == n) out[cur].y = (int)n;
        else if (keys[i + 1] / div != cur) out[cur].y = (int)(i + 1);
    }
}

}  // namespace pccnn

using namespace pccnn;

extern "C" {

const char* pccnn_last_error(void) { return g_error; }
const char* pccnn_version(void) { return "pccnn_lib_b200 0.1 (sm_100a)"; }

int pccnn_bounding_box(int D, int64_t n, const float* pts, const int32_t* batch_ids, int64_t num_batches,
                       float* out_min, float* out_max, void* stream) {
    PCCNN_CHECK_ARG(n >= 0 && num_batches >= 0, "bounding_box: negative size");
    PCCNN_CHECK_ARG(out_min && out_max, "bounding_box: null output");
    if (num_batches == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(n == 0 || (pts && batch_ids), "bounding_box: null input");
    cudaStream_t s = (cudaStream_t)stream;
    const int64_t count = num_batches * D;
    const unsigned cb = (unsigned)((count + 255) / 256);
    bbox_init_kernel<<<cb, 256, 0, s>>>(count, (int*)out_min, (int*)out_max);
    PCCNN_LAUNCH_CHECK();
    if (n > 0) {
        PCCNN_DISPATCH_DIM(D, (bbox_accum_kernel<DIM><<<(unsigned)((n + 256 * kBboxItems - 1) / (256 * kBboxItems)), 256, 0, s>>>(
                                  n, pts, batch_ids, num_batches, (int*)out_min, (int*)out_max)));
        PCCNN_LAUNCH_CHECK();
    }
    bbox_finish_kernel<<<cb, 256, 0, s>>>(count, (int*)out_min, (int*)out_max);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int pccnn_grid_num_cells(int D, int64_t num_batches, const float* aabb_min, const float* aabb_max,
                         const float* cell_size, int32_t* out_grid_size, void* stream) {
    PCCNN_CHECK_ARG(num_batches > 0, "grid_num_cells: needs at least one cloud");
    PCCNN_CHECK_ARG(aabb_min && aabb_max && cell_size && out_grid_size, "grid_num_cells: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    PCCNN_DISPATCH_DIM(D, (num_cells_kernel<DIM><<<1, 32 * kMaxDims, 0, s>>>(num_batches, aabb_min, aabb_max,
                                                                            cell_size, out_grid_size)));
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

int pccnn_compute_keys(int D, int64_t n, const float* pts, const int32_t* batch_ids, const float* aabb_min,
                       const int32_t* grid_size, const float* cell_size, int64_t* out_keys, void* stream) {
    PCCNN_CHECK_ARG(n >= 0, "compute_keys: negative size");
    if (n == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(pts && batch_ids && aabb_min && grid_size && cell_size && out_keys,
                    "compute_keys: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    PCCNN_DISPATCH_DIM(D, (compute_keys_kernel<DIM><<<grid_for(n, 256, 8), 256, 0, s>>>(
                              n, pts, batch_ids, aabb_min, grid_size, cell_size, out_keys)));
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

size_t pccnn_sort_keys_workspace_bytes(int64_t n) { return sort_layout(n < 0 ? 0 : n).total; }

int pccnn_sort_keys(int64_t n, const int64_t* keys, int key_bits, int64_t* out_sorted_keys,
                    int64_t* out_sorted_ids, int D, const float* pts, float* out_sorted_pts, void* workspace,
                    size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(n >= 0 && n < 0x7fffffffLL, "sort_keys: size %lld outside [0, 2^31)", (long long)n);
    PCCNN_CHECK_ARG(key_bits >= 1 && key_bits <= 64, "sort_keys: key_bits %d outside [1, 64]", key_bits);
    if (n == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(keys && out_sorted_keys && out_sorted_ids, "sort_keys: null pointer");
    PCCNN_CHECK_ARG(!out_sorted_pts || (pts && D >= kMinDims && D <= kMaxDims),
                    "sort_keys: gathering points needs pts and D in [2, 6]");
    const SortLayout L = sort_layout(n);
    if (!workspace || workspace_bytes < L.total) {
        set_error("sort_keys: workspace of %zu bytes, need %zu", workspace_bytes, L.total);
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    int32_t* iota = (int32_t*)(ws + L.iota_off);
    int32_t* ids = (int32_t*)(ws + L.ids_off);
    iota_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>(n, iota);
    PCCNN_LAUNCH_CHECK();
    size_t cub_bytes = L.cub_bytes;
    // LSD radix sort is stable: equal keys keep ascending original index.
    PCCNN_CUDA(cub::DeviceRadixSort::SortPairs(ws + L.cub_off, cub_bytes, keys, out_sorted_keys, iota, ids, n, 0,
                                               key_bits, s));
    if (out_sorted_pts) {
        PCCNN_DISPATCH_DIM(D, (gather_sorted_kernel<DIM><<<grid_for(n, 256, 8), 256, 0, s>>>(n, ids, pts, out_sorted_ids,
                                                                                      out_sorted_pts)));
    } else {
        gather_sorted_kernel<0><<<grid_for(n, 256, 8), 256, 0, s>>>(n, ids, nullptr, out_sorted_ids, nullptr);
    }
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

size_t pccnn_grid_front_end_workspace_bytes(int64_t n) { return sort_layout(n < 0 ? 0 : n).total; }

int pccnn_grid_front_end(int D, int64_t n, const float* pts, const int32_t* batch_ids, int64_t num_batches,
                         const float* cell_size, float* out_aabb_min, float* out_aabb_max, int32_t* out_grid_size,
                         int32_t* out_grid_size_host, int64_t* out_keys, int64_t* out_sorted_keys,
                         int64_t* out_sorted_ids, float* out_sorted_pts, void* workspace, size_t workspace_bytes,
                         void* stream) {
    PCCNN_CHECK_ARG(D >= kMinDims && D <= kMaxDims, "grid_front_end: point dimension %d outside [2, 6]", D);
    PCCNN_CHECK_ARG(n >= 0 && n < 0x7fffffffLL && num_batches > 0, "grid_front_end: bad sizes");
    PCCNN_CHECK_ARG(out_grid_size && out_grid_size_host && cell_size, "grid_front_end: null pointer");
    cudaStream_t s = (cudaStream_t)stream;
    if (int rc = pccnn_bounding_box(D, n, pts, batch_ids, num_batches, out_aabb_min, out_aabb_max, stream)) return rc;
    if (int rc = pccnn_grid_num_cells(D, num_batches, out_aabb_min, out_aabb_max, cell_size, out_grid_size, stream))
        return rc;
    // The one host round trip: the cells per axis size the caller's table and bound the key bits.  The
    // key kernel does not need it and is queued first.
    if (int rc = pccnn_compute_keys(D, n, pts, batch_ids, out_aabb_min, out_grid_size, cell_size, out_keys, stream))
        return rc;
    PCCNN_CUDA(cudaMemcpyAsync(out_grid_size_host, out_grid_size, (size_t)D * 4, cudaMemcpyDeviceToHost, s));
    PCCNN_CUDA(cudaStreamSynchronize(s));
    double span = (double)num_batches;
    for (int d = 0; d < D; ++d) span *= (double)out_grid_size_host[d];
    int key_bits = 1;
    while (key_bits < 64 && (double)(1ull << key_bits) < span + 1.0) ++key_bits;
    return pccnn_sort_keys(n, out_keys, key_bits, out_sorted_keys, out_sorted_ids, D, pts, out_sorted_pts, workspace,
                           workspace_bytes, stream);
}

int pccnn_build_grid_ds(int D, int64_t n, const int64_t* sorted_keys, const int32_t* grid_size,
                        int64_t num_entries, int32_t* out_grid_ds, void* stream) {
    PCCNN_CHECK_ARG(n >= 0 && num_entries >= 0, "build_grid_ds: negative size");
    PCCNN_CHECK_ARG(n < 0x7fffffffLL, "build_grid_ds: %lld points do not fit int32 positions", (long long)n);
    cudaStream_t s = (cudaStream_t)stream;
    if (num_entries > 0) {
        PCCNN_CHECK_ARG(out_grid_ds, "build_grid_ds: null output");
        PCCNN_CUDA(cudaMemsetAsync(out_grid_ds, 0, (size_t)num_entries * 8, s));
    }
    if (n == 0 || num_entries == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(sorted_keys && grid_size, "build_grid_ds: null pointer");
    PCCNN_DISPATCH_DIM(D, (build_grid_kernel<DIM><<<grid_for(n, 256, 8), 256, 0, s>>>(
                              n, sorted_keys, grid_size, num_entries, (int2*)out_grid_ds)));
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

}  // extern "C"
