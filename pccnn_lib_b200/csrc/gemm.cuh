// Internal interface of the tensor-core contraction (gemm.cu).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace pccnn {

// A bf16 matrix with K contiguous, rows padded with zeros to `ld` elements (a multiple of 64),
// optionally split into hi + lo parts for fp32 accuracy.
struct GemmOperand {
    void* hi;
    void* lo;  // null: single bf16 pass
    int64_t ld;
    // Columns that exist from `hi` / `lo` to the end of the row (0: all `ld` of them).  An operand that is a column
    // slice of a wider matrix starts inside a row; what a tile reads past the end of that row is filled with zeros
    // by the TMA unit instead of running into the next row.
    int64_t cols = 0;
};

// C[M, N] (fp32, row stride ldc) = A[M, K] * B[N, K]^T.  Three passes when both operands carry a
// lo part, one otherwise.  `status` is a device int the kernel sets non-zero if a bounded wait
// ran out.
// c_is_bf16 != 0: C points to a bf16 matrix (ldc in elements) and the result is rounded to bf16.
int gemm_bf16_nt(const GemmOperand& a, const GemmOperand& b, float* C, int64_t M, int N, int K_padded, int ldc,
                 int* status, cudaStream_t s, int c_is_bf16 = 0);

// dst[c, r] = src[r, c] for bf16 matrices, destination rows zero-padded to ld_dst elements.
int transpose_bf16(int rows, int cols, const void* src, int64_t ld_src, int ld_dst, void* dst, cudaStream_t s);

// C[I, N] (fp32, zeroed by the caller or holding a running sum) += A[rows, I]^T * B[rows, N];
// operand rows padded to a multiple of 64 elements.  Partial sums are added with float reductions.
int gemm_bf16_tn_accumulate(const GemmOperand& a, const GemmOperand& b, float* C, int64_t rows, int I, int N, int ldc,
                            int* status, cudaStream_t s);

// hi = bf16(src), lo = bf16(src - hi); destination rows padded with zeros to ld_dst.  lo may be null.
int split_bf16(int64_t rows, int cols, const float* src, int64_t ld_src, int ld_dst, void* hi, void* lo,
               cudaStream_t s);
// Same, but writes the transpose: destination row c holds source column c.
int split_bf16_transpose(int rows, int cols, const float* src, int64_t ld_src, int ld_dst, void* hi, void* lo,
                         cudaStream_t s);

}  // namespace pccnn
