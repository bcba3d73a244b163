// Cell-parallel greedy Poisson-disk sampling.
//
// Restates pccnn_lib_ops/poisson_disk_sampling/poisson_disk_sampling.cu:36-196 of
// phermosilla/pccnn_lib: the occupied cells are visited in 2^D passes, pass `c` handling the
// cells whose index parity in dimension d equals bit d of c.  Cells of one pass are at least
// one whole cell apart, so none of them appears in another one's neighbor lists and they can
// run in parallel; inside a cell the points are taken in ascending sorted position and a
// point is selected iff none of its radius neighbors has been selected before.
//
// Design: the reference spends one thread per cell and walks points x neighbors serially.
// Here a warp owns a cell: the points stay sequential (that is the algorithm) but the lanes
// scan a point's neighbor rows 32 at a time with coalesced loads and stop at the first
// selected neighbor.  Cell boundaries and the final index list come from device-wide stream
// compaction; nothing is copied from the host between passes.
#include <cub/device/device_select.cuh>
#include <thrust/iterator/counting_iterator.h>

#include <mutex>

#include "common.cuh"

namespace pccnn {

constexpr int kPdsWarps = 4;

__global__ void cell_flags_kernel(int n, const int64_t* __restrict__ keys, int32_t* __restrict__ flags) {
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        flags[i] = (i == 0 || keys[i] != keys[i - 1]) ? 1 : 0;
}

template <int D>
__global__ void __launch_bounds__(kPdsWarps * 32)
pds_pass_kernel(int pass, int n, const int64_t* __restrict__ keys, const int32_t* __restrict__ cell_starts,
                const int32_t* __restrict__ num_cells_ptr, const int2* __restrict__ neighbors,
                const int32_t* __restrict__ start_ids, const int32_t* __restrict__ grid_size, int32_t* used) {
    const GridDesc<D> g = load_grid<D>(grid_size);
    const int num_cells = *num_cells_ptr;
    const int lane = lane_id();
    volatile int32_t* vused = used;
    const int warps_total = gridDim.x * kPdsWarps;
    for (int cell = blockIdx.x * kPdsWarps + (threadIdx.x >> 5); cell < num_cells; cell += warps_total) {
        const int first = __ldg(cell_starts + cell);
        const int last = (cell + 1 < num_cells) ? __ldg(cell_starts + cell + 1) : n;
        int c[D];
        key_to_cell<D>(__ldg(keys + first), g, c);
        bool mine = true;
#pragma unroll
        for (int d = 0; d < D; ++d) mine = mine && ((c[d] & 1) == ((pass >> d) & 1));
        if (!mine) continue;
        for (int p = first; p < last; ++p) {
            const int lo = (p > 0) ? __ldg(start_ids + p - 1) : 0;
            const int hi = __ldg(start_ids + p);
            bool blocked = false;
            for (int t0 = lo; t0 < hi; t0 += 32) {
                const int t = t0 + lane;
                bool b = false;
                if (t < hi) b = vused[__ldg(&neighbors[t]).x] != 0;
                if (__any_sync(kFullMask, b)) {
                    blocked = true;
                    break;
                }
            }
            if (!blocked && lane == 0) vused[p] = 1;
            __syncwarp();  // orders the store before the next point's loads in this warp
        }
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
    int32_t* counters = (int32_t*)(ws + L.counters_off);  // [0] = occupied cells, [1] = selected points
    const int nn = (int)n;

    cell_flags_kernel<<<grid_for(n, 256, 8), 256, 0, s>>>(nn, sorted_keys, flags);
    PCCNN_LAUNCH_CHECK();
    size_t cub_bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceSelect::Flagged(ws + L.cub_off, cub_bytes, thrust::counting_iterator<int32_t>(0), flags,
                                          cells, counters, nn, s));
    PCCNN_CUDA(cudaMemsetAsync(used, 0, (size_t)n * 4, s));
    const unsigned grid = grid_for(n * 32, kPdsWarps * 32, 16);
    for (int pass = 0; pass < (1 << D); ++pass) {
        PCCNN_DISPATCH_DIM(D, (pds_pass_kernel<DIM><<<grid, kPdsWarps * 32, 0, s>>>(
                                  pass, nn, sorted_keys, cells, counters, (const int2*)neighbors, start_ids,
                                  grid_size, used)));
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
