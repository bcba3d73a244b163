/*
 * pccnn_oracle.c -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * CPU restatement (plain C + OpenMP) of the integer/grid/KDE part of the point-convolution
 * hot path of phermosilla/pccnn_lib, used only as the checker in tests/, in the smoke test and
 * as the timed CPU baseline of bench.py.  Nothing in the pccnn_lib_b200 package may call it.
 *
 * Every function names the reference lines it follows (paths relative to the reference root).
 * The reference itself has no CPU implementation (all of its ops launch CUDA kernels), so this
 * file restates the kernels' arithmetic; it is pinned by the NumPy / scikit-learn expectations
 * that the reference's own unit tests compute (unit_test/test_cell_ids.py, test_grid_ds.py,
 * test_find_neighs.py, test_pdf.py, test_pd_pooling.py), which tests/test_oracle_pins.py replays.
 *
 * Build: gcc -O3 -fopenmp -ffp-contract=off -shared -fPIC (see oracle/Makefile).
 * -ffp-contract=off matters: the GPU code fuses exactly the multiply-adds written as fmaf
 * below and nothing else.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define MAXD 6

/* ---- pccnn_lib/pc/BoundingBox.py:17-18: exact per-cloud min/max, then -/+ 1e-6 in float ---- */
void orc_bounding_box(int D, int64_t n, const float* pts, const int32_t* batch_ids, int64_t B,
                      float* out_min, float* out_max) {
    for (int64_t i = 0; i < B * D; ++i) { out_min[i] = INFINITY; out_max[i] = -INFINITY; }
    for (int64_t i = 0; i < n; ++i) {
        int b = batch_ids[i];
        for (int d = 0; d < D; ++d) {
            float v = pts[i * D + d];
            if (v < out_min[b * D + d]) out_min[b * D + d] = v;
            if (v > out_max[b * D + d]) out_max[b * D + d] = v;
        }
    }
    for (int64_t i = 0; i < B * D; ++i) { out_min[i] = out_min[i] - 1e-6f; out_max[i] = out_max[i] + 1e-6f; }
}

/* ---- pccnn_lib/pc/Grid.py:27-28: num_cells = max_b(int32((max-min)/cell) + 1) ---- */
void orc_grid_num_cells(int D, int64_t B, const float* mn, const float* mx, const float* cell, int32_t* out) {
    for (int d = 0; d < D; ++d) {
        int best = INT32_MIN;
        for (int64_t b = 0; b < B; ++b) {
            float q = (mx[b * D + d] - mn[b * D + d]) / cell[d];
            int v = (int)q + 1;
            if (v > best) best = v;
        }
        out[d] = best;
    }
}

/* ---- compute_keys/compute_keys.cu:56-73, shared/grid_utils.cuh:57-94 ---- */
void orc_compute_keys(int D, int64_t n, const float* pts, const int32_t* batch_ids, const float* aabb_min,
                      const int32_t* grid_size, const float* cell_size, int64_t* out_keys) {
    float inv[MAXD];
    for (int d = 0; d < D; ++d) inv[d] = 1.0f / cell_size[d]; /* torch::reciprocal, compute_keys.cu:114 */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) {
        int b = batch_ids[i];
        int64_t key = 0, acc = 1;
        for (int d = D - 1; d >= 0; --d) {
            float rel = (pts[i * D + d] - aabb_min[b * D + d]); /* rounded subtraction ...        */
            rel = rel * inv[d];                                 /* ... then rounded multiply      */
            int c = (int)floorf(rel);
            if (c < 0) c = 0;
            if (c > grid_size[d] - 1) c = grid_size[d] - 1;
            key += (int64_t)c * acc;
            acc *= grid_size[d];
        }
        out_keys[i] = key + acc * b;
    }
}

/* ---- stable ascending argsort (canonical form of torch.argsort in pccnn_lib/pc/Grid.py:52) ---- */
void orc_stable_argsort(int64_t n, const int64_t* keys, int64_t* out_ids) {
    int64_t* ka = (int64_t*)malloc(sizeof(int64_t) * (n ? n : 1));
    int64_t* kb = (int64_t*)malloc(sizeof(int64_t) * (n ? n : 1));
    int64_t* ia = (int64_t*)malloc(sizeof(int64_t) * (n ? n : 1));
    int64_t* ib = (int64_t*)malloc(sizeof(int64_t) * (n ? n : 1));
    for (int64_t i = 0; i < n; ++i) { ka[i] = keys[i]; ia[i] = i; }
    for (int shift = 0; shift < 64; shift += 8) { /* LSD radix, 8 bits a pass, keys are non-negative */
        int64_t hist[257] = {0};
        for (int64_t i = 0; i < n; ++i) hist[((uint64_t)ka[i] >> shift & 255) + 1]++;
        if (hist[1] == n) continue; /* every digit zero */
        for (int k = 0; k < 256; ++k) hist[k + 1] += hist[k];
        for (int64_t i = 0; i < n; ++i) {
            int64_t p = hist[(uint64_t)ka[i] >> shift & 255]++;
            kb[p] = ka[i]; ib[p] = ia[i];
        }
        int64_t* t = ka; ka = kb; kb = t; t = ia; ia = ib; ib = t;
    }
    memcpy(out_ids, ia, sizeof(int64_t) * n);
    free(ka); free(kb); free(ia); free(ib);
}

/* ---- build_grid/build_grid_ds.cu:44-67, shared/grid_utils.cuh:127-137 ---- */
void orc_build_grid_ds(int D, int64_t n, const int64_t* keys, const int32_t* grid_size, int64_t num_entries,
                       int32_t* out) {
    int64_t div = 1;
    for (int d = 2; d < D; ++d) div *= grid_size[d];
    memset(out, 0, sizeof(int32_t) * 2 * num_entries);
    for (int64_t i = 0; i < n; ++i) {
        int64_t cur = keys[i] / div;
        if (i > 0 && keys[i - 1] / div != cur) out[2 * cur] = (int32_t)i;
        if (i + 1 == n) out[2 * cur + 1] = (int32_t)n;
        else if (keys[i + 1] / div != cur) out[2 * cur + 1] = (int32_t)(i + 1);
    }
}

/* ---- neighbor search ----
 * Stencil and key window: find_neighbors/find_ranges_grid_ds.cu:65-166 and :306-338; the
 * predicate: count_neighbors.cu:87 / store_neighbors.cu:168 with shared/math_helper.cuh:306-321
 * (dot product accumulated as an FMA chain, as nvcc contracts it).
 * Deviations, both stated in the header of the C ABI: rows of a sample are in ascending point
 * index (the reference's order is that of its atomic tickets), and the last-dimension window
 * is clamped to the grid instead of wrapping into the neighboring row (the reference's wrap
 * only adds far-away candidates that the distance test rejects; with fewer than three cells
 * in the last dimension and D > 3 it would list a neighbor twice). */
static int64_t lower_bound64(const int64_t* k, int64_t lo, int64_t hi, int64_t v) {
    while (lo < hi) { int64_t m = (lo + hi) >> 1; if (k[m] < v) lo = m + 1; else hi = m; }
    return lo;
}
static int64_t upper_bound64(const int64_t* k, int64_t lo, int64_t hi, int64_t v) {
    while (lo < hi) { int64_t m = (lo + hi) >> 1; if (k[m] <= v) lo = m + 1; else hi = m; }
    return lo;
}

static int in_radius(int D, const float* s, const float* p, const float* inv) {
    float acc = 0.0f;
    for (int d = 0; d < D; ++d) {
        float v = (s[d] - p[d]);
        v = v * inv[d];
        acc = fmaf(v, v, acc);
    }
    return sqrtf(acc) < 1.0f;
}

/* Visits the neighbors of sample m in ascending point index.  If out == NULL only counts. */
static int visit_sample(int D, const float* pts, const int64_t* pt_keys, int64_t num_pts, const float* s, int64_t key,
                        const int32_t* grid_ds, const int32_t* nc, const float* inv, int32_t* out_pt_ids) {
    int64_t total = 1;
    for (int d = 0; d < D; ++d) total *= nc[d];
    int c[MAXD];
    int64_t rem = key % total;
    int b = (int)(key / total);
    for (int d = D - 1; d >= 0; --d) { c[d] = (int)(rem % nc[d]); rem /= nc[d]; }
    const int off_dims = (D == 2) ? 2 : D - 1;
    int n_off = 1;
    for (int d = 0; d < off_dims; ++d) n_off *= 3;
    int found = 0;
    for (int o = 0; o < n_off; ++o) {
        int cc[MAXD];
        for (int d = 0; d < D; ++d) cc[d] = c[d];
        int r = o, inside = 1;
        for (int d = off_dims - 1; d >= 0; --d) {
            cc[d] += r % 3 - 1; r /= 3;
            inside = inside && cc[d] >= 0 && cc[d] < nc[d];
        }
        if (!inside) continue;
        int64_t ds = ((int64_t)b * nc[0] + cc[0]) * nc[1] + cc[1];
        int64_t lo = grid_ds[2 * ds], hi = grid_ds[2 * ds + 1];
        if (hi > num_pts) hi = num_pts;
        if (hi <= lo) continue;
        if (D != 2) {
            int64_t k = 0, acc = 1;
            for (int d = D - 1; d >= 0; --d) { k += (int64_t)cc[d] * acc; acc *= nc[d]; }
            k += acc * b;
            int64_t klo = k - (c[D - 1] > 0 ? 1 : 0), khi = k + (c[D - 1] < nc[D - 1] - 1 ? 1 : 0);
            lo = lower_bound64(pt_keys, lo, hi, klo);
            hi = upper_bound64(pt_keys, lo, hi, khi);
        }
        for (int64_t j = lo; j < hi; ++j) {
            if (in_radius(D, s, pts + j * D, inv)) {
                if (out_pt_ids) out_pt_ids[found] = (int32_t)j;
                ++found;
            }
        }
    }
    return found;
}

/* Count pass + inclusive scan.  counts_raw[m] = all hits; start_ids = inclusive scan of
 * min(count, max_neighbors) (store_neighbors.cu:219-258).  Returns T. */
int64_t orc_find_neighbors_count(int D, int64_t num_pts, const float* pts, const int64_t* pt_keys,
                                 int64_t num_samples, const float* samples, const int64_t* sample_keys,
                                 const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                                 int32_t max_neighbors, int32_t* counts_raw, int32_t* start_ids) {
    float inv[MAXD];
    for (int d = 0; d < D; ++d) inv[d] = 1.0f / radii[d]; /* find_neighbors.cu:59 */
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t m = 0; m < num_samples; ++m)
        counts_raw[m] = visit_sample(D, pts, pt_keys, num_pts, samples + m * D, sample_keys[m], grid_ds, grid_size,
                                     inv, NULL);
    int64_t run = 0;
    for (int64_t m = 0; m < num_samples; ++m) {
        int c = counts_raw[m];
        if (max_neighbors > 0 && c > max_neighbors) c = max_neighbors;
        run += c;
        start_ids[m] = (int32_t)run;
    }
    return run;
}

/* Store pass: rows (point index, sample index).  With max_neighbors > 0 a sample with more
 * hits keeps hit `rank` iff floor((rank+1)*max/count) > floor(rank*max/count). */
void orc_find_neighbors_store(int D, int64_t num_pts, const float* pts, const int64_t* pt_keys,
                              int64_t num_samples, const float* samples, const int64_t* sample_keys,
                              const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                              int32_t max_neighbors, const int32_t* counts_raw, const int32_t* start_ids,
                              int32_t* out_neighbors) {
    float inv[MAXD];
    for (int d = 0; d < D; ++d) inv[d] = 1.0f / radii[d];
#pragma omp parallel
    {
        int32_t* tmp = NULL;
        int64_t cap = 0;
#pragma omp for schedule(dynamic, 256)
        for (int64_t m = 0; m < num_samples; ++m) {
            int total = counts_raw[m];
            if (total > cap) { cap = total * 2 + 64; tmp = (int32_t*)realloc(tmp, sizeof(int32_t) * cap); }
            visit_sample(D, pts, pt_keys, num_pts, samples + m * D, sample_keys[m], grid_ds, grid_size, inv, tmp);
            int64_t base = m > 0 ? start_ids[m - 1] : 0;
            if (max_neighbors > 0 && total > max_neighbors) {
                for (int64_t r = 0; r < total; ++r) {
                    int64_t a = r * max_neighbors / total, bn = (r + 1) * max_neighbors / total;
                    if (bn > a) { out_neighbors[2 * (base + a)] = tmp[r]; out_neighbors[2 * (base + a) + 1] = (int32_t)m; }
                }
            } else {
                for (int64_t r = 0; r < total; ++r) {
                    out_neighbors[2 * (base + r)] = tmp[r]; out_neighbors[2 * (base + r) + 1] = (int32_t)m;
                }
            }
        }
        free(tmp);
    }
}

/* ---- compute_pdf/compute_pdf.cu:42-76: sequential float accumulation of double-scaled terms ---- */
void orc_compute_pdf(int D, int manifold_dims, const float* bandwidth, int64_t n, const float* pts,
                     const int32_t* neighbors, const int32_t* start_ids, float* out_pdf) {
    float ibw[MAXD];
    for (int d = 0; d < D; ++d) ibw[d] = 1.0f / bandwidth[d]; /* compute_pdf.cu:190 */
    const double cst = 1.0 / pow(2.0 * 3.1415, (double)(float)manifold_dims / 2.0);
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t i = 0; i < n; ++i) {
        int64_t lo = i > 0 ? start_ids[i - 1] : 0, hi = start_ids[i];
        float acc = 0.0f;
        for (int64_t t = lo; t < hi; ++t) {
            int64_t j = neighbors[2 * t];
            float dot = 0.0f;
            for (int d = 0; d < D; ++d) {
                float v = (pts[j * D + d] - pts[i * D + d]);
                v = v * ibw[d];
                dot = fmaf(v, v, dot);
            }
            float e = expf(dot * -0.5f);
            float local = 1.0f;
            for (int d = 0; d < D; ++d) local *= ibw[d];
            acc = (float)((double)acc + (double)local * cst * (double)e);
        }
        out_pdf[i] = acc;
    }
}

/* ---- compute_pdf/compute_pdf.cu:98-147; accumulated in double so the result is order-free ---- */
void orc_compute_pdf_grads(int D, int manifold_dims, const float* bandwidth, int64_t n, const float* pts,
                           const int32_t* neighbors, const int32_t* start_ids, const float* in_grads,
                           double* out_grads /* [n, D] double */) {
    float ibw[MAXD];
    for (int d = 0; d < D; ++d) ibw[d] = 1.0f / bandwidth[d];
    const double cst = 1.0 / pow(2.0 * 3.1415, (double)(float)manifold_dims / 2.0);
    memset(out_grads, 0, sizeof(double) * n * D);
    for (int64_t i = 0; i < n; ++i) {
        int64_t lo = i > 0 ? start_ids[i - 1] : 0, hi = start_ids[i];
        for (int64_t t = lo; t < hi; ++t) {
            int64_t j = neighbors[2 * t];
            float v[MAXD], dot = 0.0f;
            for (int d = 0; d < D; ++d) {
                v[d] = (pts[j * D + d] - pts[i * D + d]);
                v[d] = v[d] * ibw[d];
                dot = fmaf(v[d], v[d], dot);
            }
            float local = 1.0f;
            for (int d = 0; d < D; ++d) local *= ibw[d];
            double w = (double)local * cst * (double)expf(dot * -0.5f);
            for (int d = 0; d < D; ++d) {
                double g = (double)v[d] * ibw[d] * in_grads[i] * w;
                out_grads[i * D + d] += g;
                out_grads[j * D + d] -= g;
            }
        }
    }
}

/* ---- poisson_disk_sampling/poisson_disk_sampling.cu:56-105 (kernel) and :155-192 (passes) ----
 * Sequential emulation of the 2^D parity passes.  Returns the number selected. */
int64_t orc_poisson_disk_sampling(int D, int64_t n, const int64_t* sorted_keys, const int32_t* neighbors,
                                  const int32_t* start_ids, const int32_t* grid_size, int64_t* out_selected) {
    int32_t* used = (int32_t*)calloc(n ? n : 1, sizeof(int32_t));
    int64_t total = 1;
    for (int d = 0; d < D; ++d) total *= grid_size[d];
    for (int pass = 0; pass < (1 << D); ++pass) {
        int64_t i = 0;
        while (i < n) {
            int64_t e = i + 1;
            while (e < n && sorted_keys[e] == sorted_keys[i]) ++e; /* one occupied cell = [i, e) */
            int64_t rem = sorted_keys[i] % total;
            int mine = 1;
            for (int d = D - 1; d >= 0; --d) {
                int c = (int)(rem % grid_size[d]); rem /= grid_size[d];
                mine = mine && ((c % 2) == ((pass >> d) & 1));
            }
            if (mine) {
                for (int64_t p = i; p < e; ++p) {
                    int64_t lo = p > 0 ? start_ids[p - 1] : 0, hi = start_ids[p];
                    int valid = 1;
                    for (int64_t t = lo; t < hi && valid; ++t) valid = used[neighbors[2 * t]] == 0;
                    if (valid) used[p] = 1;
                }
            }
            i = e;
        }
    }
    int64_t k = 0;
    for (int64_t i = 0; i < n; ++i) if (used[i]) out_selected[k++] = i;
    free(used);
    return k;
}

/* Thread control for the timed CPU baseline: a launcher may have capped OMP_NUM_THREADS (torchrun sets it
 * to 1 per rank); the bench asks for all the cores it is allowed to use and reports what it got. */
int orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}
