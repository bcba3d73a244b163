// Shared host/device helpers of libpccnn_b200: error reporting, launch sizing,
// warp primitives, grid-parameter loading and the key arithmetic of the reference
// (shared/grid_utils.cuh:57-137 of phermosilla/pccnn_lib) restated for sm_100a.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/pccnn_b200.h"

namespace pccnn {

constexpr int kMaxDims = 6;
constexpr int kMinDims = 2;
constexpr unsigned kFullMask = 0xffffffffu;

// ---- host-side error plumbing -------------------------------------------------------------
void set_error(const char* fmt, ...);

#define PCCNN_CHECK_ARG(cond, ...)          \
    do {                                    \
        if (!(cond)) {                      \
            pccnn::set_error(__VA_ARGS__);  \
            return PCCNN_ERR_INVALID;       \
        }                                   \
    } while (0)

#define PCCNN_CUDA(call)                                                                  \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            pccnn::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(e_),      \
                             __FILE__, __LINE__);                                         \
            return PCCNN_ERR_CUDA;                                                        \
        }                                                                                 \
    } while (0)

#define PCCNN_LAUNCH_CHECK() PCCNN_CUDA(cudaGetLastError())

// Number of SMs of the current device (cached per device).
int sm_count();

inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// Grid size for a grid-stride kernel: enough blocks to cover `work_items` but no more than
// `blocks_per_sm` resident blocks on every SM, so the grid is a multiple of the SM count
// whenever the work is large.
inline unsigned grid_for(int64_t work_items, int block, int blocks_per_sm) {
    int64_t need = (work_items + block - 1) / block;
    int64_t cap = (int64_t)sm_count() * blocks_per_sm;
    if (need < 1) need = 1;
    return (unsigned)(need < cap ? need : cap);
}

// ---- device helpers -----------------------------------------------------------------------
#ifdef __CUDACC__

// Grid of a grid-stride kernel whose blocks all get the same share of the work: exactly the blocks that are resident
// at once (registers decide how many), so that no partial second wave runs alone at a fraction of the occupancy.
template <class Kernel>
inline unsigned resident_grid(Kernel kernel, int64_t work_items, int block) {
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, block, 0) != cudaSuccess || per_sm < 1) per_sm = 1;
    return grid_for(work_items, block, per_sm);
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }

// Packed fp32x2 arithmetic (sm_100): both halves are rounded to nearest, as by the scalar
// __fsub_rn / __fmul_rn / __fmaf_rn.
__device__ __forceinline__ unsigned long long pack_f32x2(float a, float b) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ unsigned long long sub_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long mul_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(kFullMask, v, o);
    return v;
}

// Grid description read from the device tensors the reference passes around.
template <int D>
struct GridDesc {
    int nc[D];          // cells per dimension
    long long total;    // cells per cloud
};

template <int D>
__device__ __forceinline__ GridDesc<D> load_grid(const int32_t* __restrict__ grid_size) {
    GridDesc<D> g;
    g.total = 1;
#pragma unroll
    for (int d = 0; d < D; ++d) {
        g.nc[d] = __ldg(grid_size + d);
        g.total *= g.nc[d];
    }
    return g;
}

// key = row-major index over (batch, c0..c_{D-1}); shared/grid_utils.cuh:80-94 of the reference.
template <int D>
__device__ __forceinline__ long long cell_key(const int (&c)[D], const GridDesc<D>& g, int batch) {
    long long key = 0, acc = 1;
#pragma unroll
    for (int d = D - 1; d >= 0; --d) {
        key += c[d] * acc;
        acc *= g.nc[d];
    }
    return key + acc * batch;
}

// Inverse of cell_key; shared/grid_utils.cuh:103-117 of the reference.
template <int D>
__device__ __forceinline__ int key_to_cell(long long key, const GridDesc<D>& g, int (&c)[D]) {
    long long batch = key / g.total;
    if (g.total <= 0x7fffffffLL) {
        unsigned rem = (unsigned)(key - batch * g.total);
#pragma unroll
        for (int d = D - 1; d >= 0; --d) {
            unsigned q = rem / (unsigned)g.nc[d];
            c[d] = (int)(rem - q * (unsigned)g.nc[d]);
            rem = q;
        }
    } else {
        long long rem = key - batch * g.total;
#pragma unroll
        for (int d = D - 1; d >= 0; --d) {
            long long q = rem / g.nc[d];
            c[d] = (int)(rem - q * g.nc[d]);
            rem = q;
        }
    }
    return (int)batch;
}

#endif  // __CUDACC__

// Dispatch a templated launcher over the point dimension.
#define PCCNN_DISPATCH_DIM(D, EXPR_WITH_DIM)                                            \
    switch (D) {                                                                        \
        case 2: { constexpr int DIM = 2; EXPR_WITH_DIM; } break;                        \
        case 3: { constexpr int DIM = 3; EXPR_WITH_DIM; } break;                        \
        case 4: { constexpr int DIM = 4; EXPR_WITH_DIM; } break;                        \
        case 5: { constexpr int DIM = 5; EXPR_WITH_DIM; } break;                        \
        case 6: { constexpr int DIM = 6; EXPR_WITH_DIM; } break;                        \
        default:                                                                        \
            pccnn::set_error("point dimension %d outside [2, 6]", (int)(D));            \
            return PCCNN_ERR_INVALID;                                                   \
    }

}  // namespace pccnn
