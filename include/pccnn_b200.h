/*
 * pccnn_b200.h -- C ABI of libpccnn_b200.so, the sm_100a implementation of the
 * point-convolution hot path of phermosilla/pccnn_lib.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer unless its name ends in `_host`.
 *   - Arrays are contiguous row-major.  Points are [n, D] float32, batch ids
 *     int32, grid keys int64, neighbor lists [T, 2] int32 rows
 *     (point index, sample index) grouped by ascending sample index, and
 *     `start_ids[m]` is the INCLUSIVE END offset of sample m in that list
 *     (the reference's naming; see compute_pdf/compute_pdf.cu:51-52 there).
 *   - D is the point dimension, 2 <= D <= 6 (shared/defines.cuh:41-58 of the
 *     reference dispatches the same range).
 *   - `grid_size` [D] int32, `cell_size` / `radii` / `bandwidth` [D] float32 live
 *     on the device, as the reference's tensors do.
 *   - `stream` is a cudaStream_t passed as void*.  Calls enqueue on it and
 *     return without synchronising, except where a host result is documented.
 *   - Scratch memory is supplied by the caller: ask the matching
 *     *_workspace_bytes() function, allocate at least that much (256-byte
 *     aligned), and pass it in.  The library itself never allocates device
 *     memory.
 *   - Every function returns PCCNN_OK (0) or an error code; the text of the last
 *     error of the calling thread is available from pccnn_last_error().
 *   - There is no CPU fallback: without a CUDA device every compute entry point
 *     returns PCCNN_ERR_CUDA.
 *
 * File:line citations name the reference interface each entry point replaces,
 * relative to the root of phermosilla/pccnn_lib.
 */
#ifndef PCCNN_B200_H_
#define PCCNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define PCCNN_OK 0
#define PCCNN_ERR_INVALID 1   /* bad argument (dimension, size, null pointer, alignment) */
#define PCCNN_ERR_CUDA 2      /* CUDA runtime error; message holds cudaGetErrorString */
#define PCCNN_ERR_WORKSPACE 3 /* workspace too small */
#define PCCNN_ERR_OVERFLOW 4  /* neighbor count does not fit the int32 CSR of the reference */
#define PCCNN_ERR_DEVICE 5    /* a kernel reported a failed internal check (bounded wait ran out, bad index) */

/* Text of the last error raised on the calling thread ("" if none). */
const char* pccnn_last_error(void);
/* Library version string. */
const char* pccnn_version(void);

/* ------------------------------------------------------------------------- */
/* Failure reporting and input validation                                     */
/* ------------------------------------------------------------------------- */

/* The reference checks nothing (no TORCH_CHECK, no cudaGetLastError in pccnn_lib_ops); these two entry points
 * have no counterpart there.
 *
 * Kernels of this library never wait without a limit.  When a wait inside a tensor-core kernel of a convolution
 * runs out, the kernel records it, releases what it holds and returns; the operator ends with a one-thread
 * kernel that copies the record into one int of pinned host memory.  That int is sticky: the next convolution
 * entry point of the process finds it, clears it and returns PCCNN_ERR_DEVICE before doing anything, and
 * pccnn_check_status does the same on request -- with synchronize != 0 it first waits for `stream`, so that a
 * failure of the calls enqueued so far cannot be missed; with synchronize == 0 it only reports what has already
 * reached the host. */
int pccnn_check_status(int synchronize, void* stream);

/* Checks a caller-built neighbor list before it is handed to pccnn_compute_pdf*, pccnn_poisson_disk_sampling or the
 * convolutions, which index points, features and samples with its entries unchecked: every row.x in
 * [0, num_pts), every row.y equal to the sample whose segment holds the row, end offsets non-negative and
 * non-decreasing, last end offset == total.  Synchronises the stream; returns PCCNN_ERR_INVALID with the first
 * offending row or sample in the message.  Workspace: pccnn_validate_neighbors_workspace_bytes(). */
size_t pccnn_validate_neighbors_workspace_bytes(void);
int pccnn_validate_neighbors(int64_t num_pts, int64_t num_samples, const int32_t* neighbors, const int32_t* start_ids,
                             int64_t total, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* Bounding box and grid sizing (caller-side code of the reference)           */
/* ------------------------------------------------------------------------- */

/* Per-cloud axis-aligned bounding box, exact float min/max then -/+ 1e-6f.
 * Replaces pccnn_lib/pc/BoundingBox.py:17-18 (torch_scatter scatter_min/max).
 * out_min, out_max: [num_batches, D] float32.  Clouds without points get
 * +inf / -inf before the epsilon is applied. */
int pccnn_bounding_box(int D, int64_t n, const float* pts, const int32_t* batch_ids,
                       int64_t num_batches, float* out_min, float* out_max, void* stream);

/* num_cells[d] = max_b( (int32)((max[b,d] - min[b,d]) / cell_size[d]) + 1 ).
 * Replaces pccnn_lib/pc/Grid.py:27-28.  out_grid_size: [D] int32 on device. */
int pccnn_grid_num_cells(int D, int64_t num_batches, const float* aabb_min, const float* aabb_max,
                         const float* cell_size, int32_t* out_grid_size, void* stream);

/* ------------------------------------------------------------------------- */
/* Keys, sort, cell-range table                                               */
/* ------------------------------------------------------------------------- */

/* Grid key of every point:  cell = clamp((int)floorf((p - min_b) * (1/cell)), 0, nc-1),
 * key = row-major index over (batch, cell_0, ..., cell_{D-1}), last dimension fastest.
 * Replaces compute_keys()  pccnn_lib_ops/compute_keys/compute_keys.cu:78-128
 * (kernel :35-74, cell/key math shared/grid_utils.cuh:57-94).  Bit-exact. */
int pccnn_compute_keys(int D, int64_t n, const float* pts, const int32_t* batch_ids,
                       const float* aabb_min, const int32_t* grid_size, const float* cell_size,
                       int64_t* out_keys, void* stream);

/* Stable ascending sort of the keys; out_sorted_ids is the permutation (ties keep
 * ascending original index).  Replaces torch.argsort in pccnn_lib/pc/Grid.py:52
 * and the gather of the keys in Grid.py:68-70.  `key_bits` = number of low key bits
 * that can be non-zero (1..64; 64 is always safe).  out_sorted_pts may be NULL;
 * otherwise the points are gathered into sorted order too (D and pts required),
 * replacing the index_select of pccnn_lib/pc/Neighborhood.py:27-29. */
size_t pccnn_sort_keys_workspace_bytes(int64_t n);
int pccnn_sort_keys(int64_t n, const int64_t* keys, int key_bits, int64_t* out_sorted_keys,
                    int64_t* out_sorted_ids, int D, const float* pts, float* out_sorted_pts,
                    void* workspace, size_t workspace_bytes, void* stream);

/* Fused grid front end: bounding boxes, cells per axis, keys, stable sort and the sorted copies
 * in one call with ONE host synchronisation (the cells per axis are also returned on the host,
 * because the caller sizes the cell table with them).  Equivalent to pccnn_bounding_box +
 * pccnn_grid_num_cells + pccnn_compute_keys + pccnn_sort_keys with the key bits derived from the
 * grid size; replaces the caller-side sequence BoundingBox.__init__ (pccnn_lib/pc/BoundingBox.py:
 * 10-18), Grid.__init__ and Grid.compute_cell_ids (pc/Grid.py:10-52) and the gathers of
 * pc/Grid.py:68-70 / pc/Neighborhood.py:27-32 of the reference.  All outputs as in those calls;
 * out_grid_size_host: D int32 values in host memory. */
size_t pccnn_grid_front_end_workspace_bytes(int64_t n);
int pccnn_grid_front_end(int D, int64_t n, const float* pts, const int32_t* batch_ids,
                         int64_t num_batches, const float* cell_size, float* out_aabb_min,
                         float* out_aabb_max, int32_t* out_grid_size, int32_t* out_grid_size_host,
                         int64_t* out_keys, int64_t* out_sorted_keys, int64_t* out_sorted_ids,
                         float* out_sorted_pts, void* workspace, size_t workspace_bytes, void* stream);

/* Cell-range table over SORTED keys: entry (b, c0, c1) = [first, last+1) positions of
 * the points whose cell starts with (c0, c1); untouched entries stay (0, 0).
 * out_grid_ds: [num_entries, 2] int32, num_entries = B*nc0*nc1; zero-filled here.
 * Replaces build_grid_ds()  pccnn_lib_ops/build_grid/build_grid_ds.cu:72-114
 * (kernel :32-68, index math shared/grid_utils.cuh:127-137).  Bit-exact. */
int pccnn_build_grid_ds(int D, int64_t n, const int64_t* sorted_keys, const int32_t* grid_size,
                        int64_t num_entries, int32_t* out_grid_ds, void* stream);

/* ------------------------------------------------------------------------- */
/* Radius neighbor search                                                     */
/* ------------------------------------------------------------------------- */

/* Two calls replace find_neighbors()  pccnn_lib_ops/find_neighbors/find_neighbors.cu:27-66
 * (find_ranges_grid_ds.cu:41-167,306-338; count_neighbors.cu:37-104;
 * store_neighbors.cu:45-282): the first counts and scans, the second writes the list
 * once the caller has allocated it.
 *
 * A point p of the sorted array `pts` is a neighbor of sample s iff both are in the
 * same cloud and sqrtf(sum_d ((s_d - p_d) * (1/radii_d))^2) < 1.0f, evaluated with the
 * reference's float operation order.  The radius must equal the grid cell size.
 * Within a sample the rows are in ascending order of the point index (the
 * reference's order is the nondeterministic order of its atomic tickets).
 *
 * max_neighbors > 0: a sample with more than max_neighbors hits keeps exactly
 * max_neighbors of them, chosen at even strides through the ascending list (the
 * reference keeps a random subset of that size, store_neighbors.cu:45-113).
 *
 * pccnn_find_neighbors_count writes out_start_ids[num_samples] (inclusive ends) and,
 * after synchronising the stream, *out_total_host = T.  The workspace keeps the raw
 * per-sample counts for the store call and must be passed to it unchanged.
 * Returns PCCNN_ERR_OVERFLOW if T >= 2^31.
 *
 * Workspace: pccnn_find_neighbors_workspace_bytes is the recommended size.  Beyond the fixed
 * part (pccnn_find_neighbors_min_workspace_bytes) it holds a pool in which the count pass keeps
 * one bit per tested candidate so that the store pass need not test again; samples whose bits
 * no longer fit are simply tested twice.  Any size >= the minimum gives the same result.
 * sample_key_bits: number of low key bits that can be set (0 = unknown, all 64); samples that are not
 * the sorted points themselves are ordered by key with that many radix passes' worth of bits. */
size_t pccnn_find_neighbors_workspace_bytes(int D, int64_t num_samples);
size_t pccnn_find_neighbors_min_workspace_bytes(int D, int64_t num_samples);
int pccnn_find_neighbors_count(int D, int64_t num_pts, const float* pts, const int64_t* pt_keys,
                               int64_t num_samples, const float* samples, const int64_t* sample_keys,
                               const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                               int32_t max_neighbors, int32_t sample_key_bits, int32_t* out_start_ids,
                               int64_t* out_total_host, void* workspace, size_t workspace_bytes,
                               void* stream);
/* pt_index_map may be NULL; otherwise row.x = (int32)pt_index_map[point index], which
 * replaces the mapping through sorted_ids in pccnn_lib/pc/Neighborhood.py:47-53. */
int pccnn_find_neighbors_store(int D, int64_t num_pts, const float* pts, const int64_t* pt_keys,
                               int64_t num_samples, const float* samples, const int64_t* sample_keys,
                               const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                               int32_t max_neighbors, const int32_t* start_ids,
                               const int64_t* pt_index_map, int32_t* out_neighbors,
                               void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* Kernel density estimation                                                  */
/* ------------------------------------------------------------------------- */

/* pdf_i = sum_{j in seg(i)} prod_d(1/bw_d) * (2*3.1415)^(-manifold_dims/2)
 *                           * expf(-0.5 * |(p_j - p_i) * (1/bw)|^2).
 * Replaces compute_pdf()  pccnn_lib_ops/compute_pdf/compute_pdf.cu:153-203 (kernel :24-77).
 * float32, summation order differs from the reference: tolerance-matched.
 * The workspace is optional (null / 0 allowed): with pccnn_compute_pdf_workspace_bytes(D, n) bytes,
 * 3-D points are gathered from a 16-byte padded copy (one load per neighbor instead of three). */
size_t pccnn_compute_pdf_workspace_bytes(int D, int64_t n);
int pccnn_compute_pdf(int D, int manifold_dims, const float* bandwidth, int64_t n, const float* pts,
                      const int32_t* neighbors, const int32_t* start_ids, float* out_pdf,
                      void* workspace, size_t workspace_bytes, void* stream);

/* Gradient of sum_i in_grads[i] * pdf_i with respect to the points.
 * Replaces compute_pdf_grads()  compute_pdf.cu:206-257 (kernel :80-149).
 * out_pt_grads: [n, D] float32, zero-filled here. */
int pccnn_compute_pdf_grads(int D, int manifold_dims, const float* bandwidth, int64_t n, const float* pts,
                            const int32_t* neighbors, const int32_t* start_ids, const float* in_grads,
                            float* out_pt_grads, void* stream);

/* The same gradient for a list that is the FULL self-neighborhood of the points: samples = points, no cap on the
 * neighbor count, so that every pair (i, j) sits in the row of i and in the row of j (what pccnn_lib/pc/Pointcloud.py:88-97
 * builds when its cap of 300 does not bite).  One pass over the row of each point, no reductions into other rows:
 *     grad_i = scale * sum_{j in row(i)} (in_grads[i] + in_grads[j]) * w_ij * (p_j - p_i) / bw^2.
 * The caller vouches for the symmetry; on any other list the result is wrong, not undefined.  No counterpart in the
 * reference, whose one operator serves both cases.  out_pt_grads: [n, D], written, not accumulated.  The workspace is
 * optional as for pccnn_compute_pdf (same size). */
int pccnn_compute_pdf_grads_symmetric(int D, int manifold_dims, const float* bandwidth, int64_t n, const float* pts,
                                      const int32_t* neighbors, const int32_t* start_ids, const float* in_grads,
                                      float* out_pt_grads, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* Poisson-disk sampling                                                      */
/* ------------------------------------------------------------------------- */

/* Cell-parallel greedy Poisson-disk selection over points in SORTED order with a
 * self-neighborhood in sorted index space: 2^D passes by cell parity, cells of one
 * pass in parallel, points of a cell in ascending position, a point is selected iff
 * none of its neighbors is selected yet.
 * Replaces poisson_disk_sampling()
 * pccnn_lib_ops/poisson_disk_sampling/poisson_disk_sampling.cu:110-196 (kernel :36-106).
 * out_selected: capacity n int64, ascending positions; *out_count_host = how many
 * (written after synchronising the stream). */
size_t pccnn_poisson_disk_sampling_workspace_bytes(int64_t n);
int pccnn_poisson_disk_sampling(int D, int64_t n, const int64_t* sorted_keys, const int32_t* neighbors,
                                const int32_t* start_ids, const int32_t* grid_size, int64_t* out_selected,
                                int64_t* out_count_host, void* workspace, size_t workspace_bytes,
                                void* stream);

/* Poisson-disk sampling straight from the grid: the same selection as
 * pccnn_poisson_disk_sampling on the full radius-neighborhood of the points (radius = cell
 * size, max_neighbors = 0), without that neighbor list ever being built.  Replaces the pair
 * find_neighbors + poisson_disk_sampling of pccnn_lib/pc/PointPooling.py:39-69 of the
 * reference (kernel poisson_disk_sampling.cu:36-106: pass order, in-cell order and rejection
 * rule unchanged; the radius test is the one of count_neighbors.cu:87).
 * sorted_pts [n, D] and sorted_keys [n] in cell order, grid_ds / grid_size as for the search,
 * radii [D] = the cell size.  out_selected: room for n int64 positions (ascending). */
size_t pccnn_poisson_disk_sampling_grid_workspace_bytes(int64_t n);
int pccnn_poisson_disk_sampling_grid(int D, int64_t n, const float* sorted_pts,
                                     const int64_t* sorted_keys, const int32_t* grid_ds,
                                     const int32_t* grid_size, const float* radii,
                                     int64_t* out_selected, int64_t* out_count_host,
                                     void* workspace, size_t workspace_bytes, void* stream);

/* Poisson-disk sampling for callers that cannot allocate device memory.  No counterpart in the
 * reference (every op there allocates its own temporaries through torch).
 *
 * Some hosts may not call cudaMalloc while this library runs: a serving process that hands all
 * device memory to a pool of its own at start-up, so that a later cudaMalloc would simply fail;
 * a plugin whose execute callback is forbidden to allocate by the host's contract; a control
 * loop with a latency budget, for which the device-wide synchronisation and driver locks of
 * cudaMalloc / cudaFree are unacceptable.  This variant takes inputs and outputs only;
 * its scratch is a fixed array inside the library (14 MiB per GPU that loads the library, held
 * until the process exits), enough for n <= pccnn_poisson_disk_sampling_static_max_points()
 * = 1 048 576 points.  Larger n is rejected with PCCNN_ERR_INVALID and a message that names the
 * limit.  It calls neither cudaMalloc / cudaFree nor any allocating library routine.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call before starting any stream capture.  All calls share the one array, which
 * keeps the previous call's contents: the function clears what it needs itself, but two calls
 * that overlap on the GPU (different streams or threads) race on it -- run them one after another.
 * Result and arguments are those of pccnn_poisson_disk_sampling. */
int64_t pccnn_poisson_disk_sampling_static_max_points(void);
int pccnn_poisson_disk_sampling_static(int D, int64_t n, const int64_t* sorted_keys, const int32_t* neighbors,
                                       const int32_t* start_ids, const int32_t* grid_size,
                                       int64_t* out_selected, int64_t* out_count_host, void* stream);

/* ------------------------------------------------------------------------- */
/* Point convolutions                                                         */
/* ------------------------------------------------------------------------- */

/* Shared conventions: feats [num_pts, cin] float32; neighbors / start_ids as produced by the
 * neighbor search (row.x indexes pts and feats, row.y indexes samples); radii [D] on the device;
 * out [num_samples, cout] float32.  The contraction runs on the tensor cores with a bf16 hi/lo
 * split (three passes), which keeps the result within 1e-4 relative of an fp32 evaluation.
 * Scratch: pccnn_conv_workspace_bytes(num_pts, num_samples, cin, basis_size, cout) (it holds, besides the projected
 * features of one chunk of samples and the weights, bf16 hi / lo copies of the feature rows for the tensor-core pair
 * kernels, hence num_pts). */
size_t pccnn_conv_workspace_bytes(int64_t num_pts, int64_t num_samples, int cin, int basis_size, int cout);

/* Which kernels do the per-pair work of every convolution entry point below (no counterpart in the reference): 0, the
 * default, uses tcgen05 pair kernels for 3-D points with at least 32 input channels and CUDA-core kernels otherwise;
 * 1 uses the CUDA-core kernels everywhere.  Both give the same results within the stated tolerances; the switch
 * exists so that they can be compared.  Process-wide. */
int pccnn_conv_set_path(int path);

/* KPConv forward: basis b[t,k] = clamp(1 - |kernel_pts[k] - d_t| / sigma, 0, 1), weights
 * [num_kernel_pts * cin, cout] with row index c * num_kernel_pts + k.
 * Replaces kpconv()  pccnn_lib_ops/pcconvs/kpconv.cu:32-60 (stages shared/pt_diff.cu:27-49,
 * shared/kernel_pts_basis.cu:23-39, shared/feat_basis_proj.cu:133-191).  Any 1 <= num_kernel_pts
 * <= 64 is accepted (the reference only instantiates 8, 16, 32 and 64). */
int pccnn_kp_conv(int D, int64_t num_pts, const float* pts, const float* feats, int cin,
                  int64_t num_samples, const float* samples, const int32_t* neighbors,
                  const int32_t* start_ids, const float* radii, const float* kernel_pts,
                  int num_kernel_pts, float sigma, const float* weights, int cout, float* out,
                  void* workspace, size_t workspace_bytes, void* stream);

/* KPConv forward for bf16 features, bf16 weights and bf16 output (3-D points): one bf16 tensor-core
 * pass with fp32 accumulation; the projected operand is rounded to bf16 once.  Matches an fp32
 * evaluation within 1e-2 relative.  No counterpart in the reference, which dispatches float and
 * double only (pcconvs/shared/feat_basis_utils.cuh:41). */
int pccnn_kp_conv_bf16(int D, int64_t num_pts, const float* pts, const void* feats_bf16, int cin,
                       int64_t num_samples, const float* samples, const int32_t* neighbors,
                       const int32_t* start_ids, const float* radii, const float* kernel_pts,
                       int num_kernel_pts, float sigma, const void* weights_bf16, int cout, void* out_bf16,
                       void* workspace, size_t workspace_bytes, void* stream);

/* KPConv forward WITHOUT a neighbor list (3-D points): the projection kernel finds the neighbors of every sample on
 * the grid itself -- the 27-cell stencil and the exact radius predicate of the search -- so the [T, 2] list of
 * find_neighbors is neither written nor read.  Same result as pccnn_find_neighbors_* followed by pccnn_kp_conv(_bf16)
 * (rows in the same ascending order).  Replaces the sequence __create_neighborhood__ + kp_conv of
 * pccnn_lib/pc/layers/KPConv.py:127-146,118-123 of the reference for inference.
 * sorted_pts / sorted_keys [num_pts]: the points in grid order with their keys (pccnn_sort_keys); grid_ds, grid_size,
 * radii (= cell size) as for the search; samples [num_samples, 3] with their keys on the same grid, any order.
 * feats [num_pts, cin] are in the CALLER's order: pt_index_map[j] (the sort permutation; NULL = identity) is the
 * feature row of sorted position j.  feats_are_bf16 != 0: features, weights and output are bf16 (one tensor-core
 * pass, as pccnn_kp_conv_bf16), otherwise fp32.  Scratch: pccnn_kp_conv_grid_workspace_bytes. */
size_t pccnn_kp_conv_grid_workspace_bytes(int64_t num_pts, int64_t num_samples, int cin, int num_kernel_pts, int cout);
int pccnn_kp_conv_grid(int64_t num_pts, const float* sorted_pts, const int64_t* sorted_keys, const int64_t* pt_index_map,
                       const void* feats, int feats_are_bf16, int cin, int64_t num_samples, const float* samples,
                       const int64_t* sample_keys, const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                       const float* kernel_pts, int num_kernel_pts, float sigma, const void* weights, int cout, void* out,
                       void* workspace, size_t workspace_bytes, void* stream);

/* MCConv forward: basis b[t,:] = leaky_relu_{0.2}(d_t . axis + bias) / pdf[n0(t)], axis [D, hidden],
 * bias [hidden], weights [num_mlps, hidden / num_mlps * cin, cout / num_mlps] (hidden counts the
 * units of all MLPs together, as the reference's proj_axis_ does).
 * Replaces mcconv()  pccnn_lib_ops/pcconvs/mcconv.cu:32-71 (stages shared/mlp_basis.cu:27-48).
 * With num_mlps > 1 the slices of the operands must start on 16-byte boundaries: hidden / num_mlps * cin a multiple
 * of 8 here, and cout / num_mlps a multiple of 8 as well in pccnn_mc_conv_grads; other shapes are refused with
 * PCCNN_ERR_INVALID before anything is launched.  num_mlps == 1 has no such restriction. */
int pccnn_mc_conv(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                  int64_t num_samples, const float* samples, const int32_t* neighbors,
                  const int32_t* start_ids, const float* radii, const float* axis, const float* bias,
                  int hidden, int num_mlps, const float* weights, int cout, float* out,
                  void* workspace, size_t workspace_bytes, void* stream);

/* Gradients of the two convolutions for an upstream gradient in_grads [num_samples, cout].
 * Every output is zero-filled here and accumulated with float reductions (like the reference,
 * whose scatter steps use atomics), so results are reproducible only up to summation order.
 * Scratch: pccnn_conv_grads_workspace_bytes(num_pts, num_samples, cin, basis_size, cout).
 *
 * pccnn_kp_conv_grads replaces kpconv_grads()  pccnn_lib_ops/pcconvs/kpconv.cu:63-112
 * (shared/feat_basis_proj_grads.cu:158-223, shared/kernel_pts_basis.cu:41-70, shared/pt_diff.cu:51-80);
 * outputs: weights [K*cin, cout], features [num_pts, cin], kernel points [K, D], points [num_pts, D],
 * samples [num_samples, D].
 * pccnn_mc_conv_grads replaces mcconv_grads()  pccnn_lib_ops/pcconvs/mcconv.cu:73-143
 * (shared/mlp_basis.cu:50-96); outputs: weights (shape of the weights), features, axis [D, hidden],
 * bias [hidden], pdf [num_pts], points, samples. */
size_t pccnn_conv_grads_workspace_bytes(int64_t num_pts, int64_t num_samples, int cin, int basis_size, int cout);
/* Data parallelism (no counterpart in the reference, which is single-process): `event` (a cudaEvent_t) is recorded
 * on the stream of the NEXT pccnn_kp_conv_grads / pccnn_mc_conv_grads call of this thread at the point where
 * out_weight_grads is final, i.e. before the last per-pair kernel of the call; a communication stream that waits
 * for it can sum the weight gradient over the ranks while the feature / point gradients are still computed.
 * One shot: the call consumes it.  NULL cancels. */
int pccnn_conv_grads_set_weight_grads_event(void* event);
int pccnn_kp_conv_grads(int D, int64_t num_pts, const float* pts, const float* feats, int cin,
                        int64_t num_samples, const float* samples, const int32_t* neighbors,
                        const int32_t* start_ids, const float* radii, const float* kernel_pts,
                        int num_kernel_pts, float sigma, const float* weights, int cout,
                        const float* in_grads, float* out_weight_grads, float* out_feat_grads,
                        float* out_kernel_pt_grads, float* out_pt_grads, float* out_sample_grads,
                        void* workspace, size_t workspace_bytes, void* stream);
int pccnn_mc_conv_grads(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                        int64_t num_samples, const float* samples, const int32_t* neighbors,
                        const int32_t* start_ids, const float* radii, const float* axis, const float* bias,
                        int hidden, int num_mlps, const float* weights, int cout, const float* in_grads,
                        float* out_weight_grads, float* out_feat_grads, float* out_axis_grads,
                        float* out_bias_grads, float* out_pdf_grads, float* out_pt_grads,
                        float* out_sample_grads, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* Weight variance (variance-aware initialisation)                            */
/* ------------------------------------------------------------------------- */

/* out_variance[0] (device float) = 1 / mean_m( sum_{i, j in seg(m)} (b_i . b_j) (f_i . f_j) ), the quantity the
 * layers of the reference accumulate during their warm-up passes to scale their weight initialisation
 * (pccnn_lib/pc/layers/KPConv.py:103-116, MCConv.py:97-110).  The double sum over the neighbors of a sample is
 * the squared norm of the sample's projected features, so it is computed in O(n) per sample, not O(n^2).
 * Replace kpconv_compute_weight_variance()  pccnn_lib_ops/pcconvs/kpconv.cu:115-135 and
 * mcconv_compute_weight_variance()  mcconv.cu:146-171 (kernel shared/compute_variance_weights.cu:24-170).
 * Scratch: pccnn_conv_weight_var_workspace_bytes(num_pts, num_samples, cin, basis_size).  num_samples >= 1. */
size_t pccnn_conv_weight_var_workspace_bytes(int64_t num_pts, int64_t num_samples, int cin, int basis_size);
int pccnn_kp_conv_weight_var(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                             const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                             const float* kernel_pts, int num_kernel_pts, float sigma, float* out_variance,
                             void* workspace, size_t workspace_bytes, void* stream);
int pccnn_mc_conv_weight_var(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                             int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                             const float* radii, const float* axis, const float* bias, int hidden, float* out_variance,
                             void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* The other convolutions of the reference                                    */
/* ------------------------------------------------------------------------- */

/* Same projection + tensor-core contraction as KPConv with another basis; workspaces from
 * pccnn_conv_workspace_bytes / pccnn_conv_grads_workspace_bytes / pccnn_conv_weight_var_workspace_bytes with
 * basis_size = the number of basis functions.  Weights [basis_size * cin, cout], row index c * basis_size + k.
 *
 * KPConvN: b[t, k] = clamp(1 - |kp_k - d_t| / sigma, 0, 1) / pdf[n0(t)].  Replaces kpconvn(), kpconvn_grads(),
 * kpconvn_compute_weight_variance()  pccnn_lib_ops/pcconvs/kpconvn.cu:32-155.  Gradient outputs: weights, features,
 * kernel points [K, D], points, samples (the reference returns no density gradient). */
int pccnn_kp_conv_n(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                    int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                    const float* radii, const float* kernel_pts, int num_kernel_pts, float sigma, const float* weights,
                    int cout, float* out, void* workspace, size_t workspace_bytes, void* stream);
int pccnn_kp_conv_n_grads(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                          int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                          const float* radii, const float* kernel_pts, int num_kernel_pts, float sigma,
                          const float* weights, int cout, const float* in_grads, float* out_weight_grads,
                          float* out_feat_grads, float* out_kernel_pt_grads, float* out_pt_grads, float* out_sample_grads,
                          void* workspace, size_t workspace_bytes, void* stream);
int pccnn_kp_conv_n_weight_var(int D, int64_t num_pts, const float* pts, const float* pdf, const float* feats, int cin,
                               int64_t num_samples, const float* samples, const int32_t* neighbors,
                               const int32_t* start_ids, const float* radii, const float* kernel_pts, int num_kernel_pts,
                               float sigma, float* out_variance, void* workspace, size_t workspace_bytes, void* stream);

/* PCCNN: b[t, k] = exp(-|kp_k - d_t|^2 / (2 sigma^2)) / pdf[n0(t)].  Replaces pccnn(), pccnn_grads(),
 * pccnn_compute_weight_variance()  pccnn_lib_ops/pcconvs/pccnn.cu:32-165 (basis shared/kernel_pts_basis.cu:72-111).
 * Argument order as there (features before the density).  Gradient outputs: weights, features, kernel points,
 * density [num_pts], points, samples. */
int pccnn_pccnn_conv(int D, int64_t num_pts, const float* pts, const float* feats, int cin, const float* pdf,
                     int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                     const float* radii, const float* kernel_pts, int num_kernel_pts, float sigma, const float* weights,
                     int cout, float* out, void* workspace, size_t workspace_bytes, void* stream);
int pccnn_pccnn_conv_grads(int D, int64_t num_pts, const float* pts, const float* feats, int cin, const float* pdf,
                           int64_t num_samples, const float* samples, const int32_t* neighbors, const int32_t* start_ids,
                           const float* radii, const float* kernel_pts, int num_kernel_pts, float sigma,
                           const float* weights, int cout, const float* in_grads, float* out_weight_grads,
                           float* out_feat_grads, float* out_kernel_pt_grads, float* out_pdf_grads, float* out_pt_grads,
                           float* out_sample_grads, void* workspace, size_t workspace_bytes, void* stream);
int pccnn_pccnn_conv_weight_var(int D, int64_t num_pts, const float* pts, const float* feats, int cin, const float* pdf,
                                int64_t num_samples, const float* samples, const int32_t* neighbors,
                                const int32_t* start_ids, const float* radii, const float* kernel_pts, int num_kernel_pts,
                                float sigma, float* out_variance, void* workspace, size_t workspace_bytes, void* stream);

/* SPHConv (3-D points only): one-hot basis over radial x azimuth x polar bins (+ one bin for offsets shorter than
 * 1e-4), bin edges ascending on the device, at most 64 edges and 64 basis functions; the output of a sample is
 * divided by its neighbor count + 1e-6.  Replaces sphconv(), sphconv_grads(), sphconv_compute_weight_variance()
 * pccnn_lib_ops/pcconvs/sphconv.cu:32-146 (basis shared/spherical_basis.cu:24-168).  Gradient outputs: weights and
 * features only, as in the reference (the bins are not differentiable). */
int pccnn_sph_conv(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                   const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                   const float* radial_bins, int num_radial, const float* azimuth_bins, int num_azimuth,
                   const float* polar_bins, int num_polar, const float* weights, int cout, float* out, void* workspace,
                   size_t workspace_bytes, void* stream);
int pccnn_sph_conv_grads(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                         const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                         const float* radial_bins, int num_radial, const float* azimuth_bins, int num_azimuth,
                         const float* polar_bins, int num_polar, const float* weights, int cout, const float* in_grads,
                         float* out_weight_grads, float* out_feat_grads, void* workspace, size_t workspace_bytes,
                         void* stream);
int pccnn_sph_conv_weight_var(int D, int64_t num_pts, const float* pts, const float* feats, int cin, int64_t num_samples,
                              const float* samples, const int32_t* neighbors, const int32_t* start_ids, const float* radii,
                              const float* radial_bins, int num_radial, const float* azimuth_bins, int num_azimuth,
                              const float* polar_bins, int num_polar, float* out_variance, void* workspace,
                              size_t workspace_bytes, void* stream);

/* PointConv.  pccnn_point_conv_basis: out_basis[t, :] = ((pts[n0(t)] - samples[n1(t)]) / radii) . axis + bias, a
 * [num_pairs, hidden] tensor that the layer post-processes in Python; its gradients: points [num_pts, D], samples
 * [num_samples, D], axis [D, hidden], bias [hidden] (all zero-filled here).  Replace pointconv_basis() and
 * pointconv_basis_grads()  pccnn_lib_ops/pcconvs/pointconv.cu:32-86.
 * pccnn_point_conv* take the basis [num_pairs, hidden] (hidden <= 64) as an input; gradient outputs: weights,
 * features, basis [num_pairs, hidden].  Replace pointconv(), pointconv_grads(), pointconv_compute_weight_variance()
 * pointconv.cu:89-139. */
int pccnn_point_conv_basis(int D, int64_t num_pairs, const float* pts, const float* radii, const float* samples,
                           const int32_t* neighbors, const float* axis, const float* bias, int hidden, float* out_basis,
                           void* stream);
int pccnn_point_conv_basis_grads(int D, int64_t num_pts, int64_t num_samples, int64_t num_pairs, const float* pts,
                                 const float* radii, const float* samples, const int32_t* neighbors, const float* axis,
                                 int hidden, const float* in_grads, float* out_pt_grads, float* out_sample_grads,
                                 float* out_axis_grads, float* out_bias_grads, void* stream);
int pccnn_point_conv(int64_t num_pts, const float* basis, int hidden, const float* feats, int cin, int64_t num_samples,
                     const int32_t* neighbors, const int32_t* start_ids, const float* weights, int cout, float* out,
                     void* workspace, size_t workspace_bytes, void* stream);
int pccnn_point_conv_grads(int64_t num_pts, const float* basis, int hidden, const float* feats, int cin,
                           int64_t num_samples, int64_t num_pairs, const int32_t* neighbors, const int32_t* start_ids,
                           const float* weights, int cout, const float* in_grads, float* out_weight_grads,
                           float* out_feat_grads, float* out_basis_grads, void* workspace, size_t workspace_bytes,
                           void* stream);
int pccnn_point_conv_weight_var(int64_t num_pts, const float* basis, int hidden, const float* feats, int cin,
                                int64_t num_samples, const int32_t* neighbors, const int32_t* start_ids,
                                float* out_variance, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------- */
/* Dense contraction on the tensor cores                                      */
/* ------------------------------------------------------------------------- */

/* C[M, N] = A[M, K] * B[N, K]^T, fp32 in and out, row strides lda / ldb / ldc in elements.
 * Replaces the torch::matmul (cuBLAS SGEMM) calls of pccnn_lib_ops/pcconvs/kpconv.cu:56-57,95-96
 * and mcconv.cu:64-68,111-120.  split != 0: operands are split into bf16 hi + lo parts and three
 * tcgen05 passes give fp32-level accuracy (relative error of a product below 2^-16);
 * split == 0: one bf16 pass.  Synchronises the stream to read the kernel's status word. */
size_t pccnn_gemm_workspace_bytes(int64_t M, int N, int K);

/* Test hooks of the tensor-core kernels on the current device (no counterpart in the reference): the poll limit of
 * their bounded waits (<= 0 restores the default of 2^21 polls) and a producer that issues no load from K block
 * `withhold_from` on (< 0: off), so that a test can let the consumers' waits run out with no copy in flight and
 * check that the kernel returns, the status is reported and the next call works.  Not for production use. */
int pccnn_gemm_set_test_hooks(int poll_limit, int withhold_from);
int pccnn_gemm_f32(int64_t M, int N, int K, const float* A, int64_t lda, const float* B, int64_t ldb,
                   float* C, int64_t ldc, int split, void* workspace, size_t workspace_bytes, void* stream);

/* The tensor-core kernel alone, on operands that are already bf16: A [M, lda], B [N, ldb] with K
 * contiguous, K a multiple of 64 and lda, ldb >= K multiples of 64; a_lo / b_lo are the optional
 * low parts of the split (both or neither).  Asynchronous; *status_dev (device int, zeroed by the
 * caller) becomes non-zero if a bounded wait inside the kernel ran out. */
int pccnn_gemm_bf16(int64_t M, int N, int K, const void* a_hi, const void* a_lo, int64_t lda, const void* b_hi,
                    const void* b_lo, int64_t ldb, float* C, int64_t ldc, int* status_dev, void* stream);

/* C[I, N] = A[rows, I]^T * B[rows, N] (the weight-gradient contraction dW = P^T g of
 * pccnn_lib_ops/pcconvs/kpconv.cu:90-93): the reduction runs over the rows, split across CTAs,
 * partial tiles are summed with float reductions (the order of the partial sums is not fixed). */
size_t pccnn_gemm_tn_workspace_bytes(int64_t rows, int I, int N);
int pccnn_gemm_tn_f32(int64_t rows, int I, int N, const float* A, int64_t lda, const float* B, int64_t ldb,
                      float* C, int64_t ldc, int split, void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* PCCNN_B200_H_ */
