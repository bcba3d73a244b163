// Failure reporting of kernels that cannot return a value, and validation of caller-supplied neighbor lists.
//
// The reference checks nothing (no TORCH_CHECK, no cudaGetLastError anywhere in pccnn_lib_ops); a neighbor list
// with a bad index is a memory fault there.  Here:
//   * a kernel whose bounded wait ran out records a status word in the caller's workspace; the operator that
//     launched it ends with publish_status_kernel, which copies a non-zero word into one int of pinned, mapped
//     host memory.  The host reads that int without synchronising: at the start of the next convolution call and
//     in pccnn_check_status, which can also synchronise the stream first.  The word is sticky until it is read.
//   * pccnn_validate_neighbors checks a [T, 2] list and its end offsets on the device and reports the first bad
//     row as an error code instead of letting a later kernel fault on it.
#include <mutex>

#include "common.cuh"
#include "status.cuh"

namespace pccnn {

static int* g_status_host = nullptr;  // one int, pinned + mapped + portable: visible to every device of the process
static std::once_flag g_status_once;
static cudaError_t g_status_err = cudaSuccess;

int* sticky_status_word() {
    std::call_once(g_status_once, [] {
        g_status_err = cudaHostAlloc((void**)&g_status_host, 64, cudaHostAllocPortable | cudaHostAllocMapped);
        if (g_status_err == cudaSuccess) {
            for (int i = 0; i < 16; ++i) g_status_host[i] = 0;
        } else {
            g_status_host = nullptr;
        }
    });
    return g_status_host;
}

__global__ void publish_status_kernel(const int* __restrict__ status, int* __restrict__ sticky, int origin) {
    const int v = *status;
    if (v != 0) {
        atomicCAS_system(sticky, 0, (origin << 8) | (v & 0xff));  // the first failure stays
        __threadfence_system();
    }
}

int publish_status(const int* status_dev, int origin, cudaStream_t s) {
    int* sticky = sticky_status_word();
    if (!sticky) {
        set_error("cudaHostAlloc of the status word failed: %s", cudaGetErrorString(g_status_err));
        return PCCNN_ERR_CUDA;
    }
    int* sticky_dev = nullptr;
    PCCNN_CUDA(cudaHostGetDevicePointer((void**)&sticky_dev, sticky, 0));
    publish_status_kernel<<<1, 1, 0, s>>>(status_dev, sticky_dev, origin);
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

static const char* origin_name(int origin) {
    switch (origin) {
        case kOriginConvForward: return "convolution forward";
        case kOriginConvBackward: return "convolution backward";
        case kOriginWeightVar: return "weight-variance operator";
        default: return "kernel";
    }
}

int take_sticky_status(const char* who) {
    int* sticky = sticky_status_word();
    if (!sticky) return PCCNN_OK;
    const int v = *(volatile int*)sticky;
    if (v == 0) return PCCNN_OK;
    *(volatile int*)sticky = 0;
    set_error("%s: an earlier %s on this process gave up on a bounded wait inside a tensor-core kernel (status %d); "
              "its outputs are incomplete", who, origin_name(v >> 8), v & 0xff);
    return PCCNN_ERR_DEVICE;
}

// ---- neighbor-list validation ---------------------------------------------------------------
struct ListReport {
    int code;            // 0 ok; 1 point index out of range; 2 sample index does not match its segment;
                         // 3 end offsets decrease; 4 last end offset != T; 5 negative end offset
    long long where;     // row or sample of the first problem seen
    int value;
};

__global__ void validate_list_kernel(long long num_pts, int num_samples, const int2* __restrict__ neighbors,
                                     const int32_t* __restrict__ start_ids, long long total, ListReport* report) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
    auto fail = [&](int code, long long where, int value) {
        if (atomicCAS(&report->code, 0, code) == 0) {
            report->where = where;
            report->value = value;
        }
    };
    for (long long m = tid; m < num_samples; m += stride) {
        const int hi = start_ids[m], lo = m > 0 ? start_ids[m - 1] : 0;
        if (hi < 0) fail(5, m, hi);
        else if (hi < lo) fail(3, m, hi);
        else if (m == num_samples - 1 && hi != total) fail(4, m, hi);
    }
    if (report->code != 0) return;  // offsets are broken: rows cannot be attributed to samples
    for (long long m = tid; m < num_samples; m += stride) {
        const long long hi = min((long long)start_ids[m], total);
        const long long lo = max((long long)(m > 0 ? start_ids[m - 1] : 0), 0LL);
        // every thread owns whole segments: rows of sample m must carry m in .y
        for (long long t = lo; t < hi; ++t) {
            const int2 row = neighbors[t];
            if (row.x < 0 || row.x >= num_pts) fail(1, t, row.x);
            else if (row.y != (int)m) fail(2, t, row.y);
        }
    }
}

}  // namespace pccnn

using namespace pccnn;

extern "C" {

int pccnn_check_status(int synchronize, void* stream) {
    if (synchronize) PCCNN_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    return take_sticky_status("check_status");
}

size_t pccnn_validate_neighbors_workspace_bytes(void) { return 256; }

int pccnn_validate_neighbors(int64_t num_pts, int64_t num_samples, const int32_t* neighbors, const int32_t* start_ids,
                             int64_t total, void* workspace, size_t workspace_bytes, void* stream) {
    PCCNN_CHECK_ARG(num_pts >= 0 && num_samples >= 0 && num_samples < 0x7fffffffLL && total >= 0 && total < 0x80000000LL,
                    "validate_neighbors: bad sizes");
    if (num_samples == 0) {
        PCCNN_CHECK_ARG(total == 0, "validate_neighbors: %lld rows but no sample", (long long)total);
        return PCCNN_OK;
    }
    PCCNN_CHECK_ARG(start_ids && (neighbors || total == 0), "validate_neighbors: null pointer");
    if (!workspace || workspace_bytes < sizeof(ListReport)) {
        set_error("validate_neighbors: workspace of %zu bytes, need %zu", workspace_bytes, (size_t)256);
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    ListReport* report = (ListReport*)workspace;
    PCCNN_CUDA(cudaMemsetAsync(report, 0, sizeof(ListReport), s));
    validate_list_kernel<<<grid_for(num_samples, 256, 8), 256, 0, s>>>(num_pts, (int)num_samples, (const int2*)neighbors,
                                                                       start_ids, total, report);
    PCCNN_LAUNCH_CHECK();
    ListReport host;
    PCCNN_CUDA(cudaMemcpyAsync(&host, report, sizeof(ListReport), cudaMemcpyDeviceToHost, s));
    PCCNN_CUDA(cudaStreamSynchronize(s));
    if (host.code == 0) return PCCNN_OK;
    static const char* what[] = {"", "point index outside [0, num_pts)", "sample index differs from the segment it is stored in",
                                 "end offsets decrease", "last end offset differs from the number of rows",
                                 "negative end offset"};
    set_error("validate_neighbors: %s (at %s %lld, value %d)", what[host.code], host.code <= 2 ? "row" : "sample",
              host.where, host.value);
    return PCCNN_ERR_INVALID;
}

}  // extern "C"
