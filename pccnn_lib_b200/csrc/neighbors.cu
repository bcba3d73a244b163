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
// Design.  The reference re-reads every candidate from global memory for every sample, twice
// (count and store), through three kernels and a [M, 9, 2] range tensor.  Here the samples are
// visited in cell order (their own order when they are the sorted points themselves, a sorted
// permutation otherwise), and one warp owns 32 consecutive samples.  Samples of the same cell
// share their candidate ranges, so the warp resolves the 3^(D-1) ranges once per cell (table
// lookup + binary search for the three consecutive last-dimension cells, which are contiguous
// in the sorted array), copies the candidates (coordinates + position) once into its private
// shared-memory buffer with coalesced loads, and then sweeps that buffer for each of its
// samples: one conflict-free 16-byte shared load per test instead of three L2 loads.
// __ballot_sync + popc rank the hits, so rows come out in ascending point index without
// atomics and the result is deterministic.  A count pass, a device-wide scan and a store pass
// replace the reference's three kernels + cumsum.  Everything is warp-synchronous: no block
// barrier, no wait on another warp.
#include <cub/device/device_radix_sort.cuh>
#include <cub/device/device_scan.cuh>

#include "common.cuh"
#include "stencil.cuh"

namespace pccnn {

constexpr int kWarpsPerBlock = 4;

enum : int { kCount = 0, kStore = 1, kStoreLimited = 2 };

constexpr unsigned kNoMask = 0xffffffffu;

// Hit-mask cache.  The count pass keeps the ballot of every 32-candidate group it tests
// (1 bit per test) in a pool inside the workspace; the store pass then only replays the bits
// instead of reloading coordinates and repeating the arithmetic.  Space is reserved per run of
// same-cell samples with one atomic add; a run that no longer fits is marked kNoMask and the
// store pass recomputes it, so any pool size is correct and a larger one is merely faster.
struct MaskCache {
    unsigned* sample_off;             // [M] first mask word of the sample, or kNoMask
    unsigned* pool;                   // mask words
    unsigned long long* cursor;       // words handed out so far (count pass)
    unsigned long long pool_words;
};

template <int D>
__device__ __forceinline__ int chunks_per_sample(int num_cand) {
    using S = Stencil<D>;
    return (num_cand / S::kSlots) * (S::kSlots / 32) + ((num_cand % S::kSlots) + 31) / 32;
}

template <int MODE>
__device__ __forceinline__ void emit_row(int2* __restrict__ out, int base, int rank, int id, int m, int total,
                                         int max_neighbors) {
    if (MODE == kStore || total <= max_neighbors) {
        out[base + rank] = make_int2(id, m);
    } else {
        // Even-stride thinning: hit `rank` of `total` is kept iff it starts a new one of the
        // max_neighbors equal slices of the list, i.e. iff floor((rank + 1) * max / total) exceeds
        // a = floor(rank * max / total), which is the case iff (rank * max) mod total + max >= total.
        // One 32-bit division when the product fits, the 64-bit form otherwise.
        if ((unsigned long long)rank * (unsigned)max_neighbors < 0x80000000ull) {
            const unsigned prod = (unsigned)rank * (unsigned)max_neighbors;
            const unsigned a = prod / (unsigned)total, rem = prod - a * (unsigned)total;
            if (rem + (unsigned)max_neighbors >= (unsigned)total) out[base + (int)a] = make_int2(id, m);
        } else {
            const long long a = (long long)rank * max_neighbors / total;
            const long long bnext = (long long)(rank + 1) * max_neighbors / total;
            if (bnext > a) out[base + (int)a] = make_int2(id, m);
        }
    }
}

// MIN_BLOCKS: resident blocks per SM the register allocation has to leave room for (the 3-D count pass gains 4 %
// from 8 blocks of 64 registers against 7 of 72 and 3 % more from 9 blocks of 56, which spills four words).  0 leaves the choice to the compiler, which is not the same as 1:
// told that one block is enough, it gives the 3-D store pass 96 registers instead of 56 and the pass loses 7 %.
template <int D, int MODE, int MIN_BLOCKS = 0>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, MIN_BLOCKS)
neighbors_kernel(int num_pts, const float* __restrict__ pts, const int64_t* __restrict__ pt_keys,
                 int num_samples, const float* __restrict__ samples, const int64_t* __restrict__ sample_keys,
                 const int32_t* __restrict__ sample_order,  // samples in cell order, or null = identity
                 const int2* __restrict__ grid_ds, const int32_t* __restrict__ grid_size,
                 const float* __restrict__ radii, int max_neighbors,
                 int32_t* __restrict__ counts,             // kCount: out; kStoreLimited: raw counts in
                 const int32_t* __restrict__ start_ids,    // stores: inclusive ends
                 const int64_t* __restrict__ pt_index_map, int2* __restrict__ out, MaskCache cache,
                 const int32_t* __restrict__ tile_order, int num_tiles) {
    using S = Stencil<D>;
    constexpr int kChunks = S::kSlots / 32;
    __shared__ float4 s_slots[kWarpsPerBlock][S::kPlanes * S::kSlots];
    __shared__ int s_lo[kWarpsPerBlock][S::kRanges];
    __shared__ int s_pref[kWarpsPerBlock][S::kRanges + 1];
    const int warp = threadIdx.x >> 5, lane = lane_id();
    const unsigned lane_bit = 1u << lane, lt_mask = lane_bit - 1u;
    float4* slots = s_slots[warp];
    int* slot_ids = reinterpret_cast<int*>(s_slots[warp]);  // masked store pass: positions only
    int* lo = s_lo[warp];
    int* pref = s_pref[warp];

    // Tiles of 32 samples; with tile_order the heaviest come first, so that no SM is left alone with one of them
    // at the end of the launch.
    const int slot = blockIdx.x * kWarpsPerBlock + warp;
    if (slot >= num_tiles) return;
    const int i0 = (tile_order ? __ldg(tile_order + slot) : slot) * 32;
    if (i0 >= num_samples) return;
    const int n_here = min(32, num_samples - i0);
    const GridDesc<D> g = load_grid<D>(grid_size);
    float inv[D];
#pragma unroll
    for (int d = 0; d < D; ++d) inv[d] = __frcp_rn(__ldg(radii + d));

    // Lane k owns the k-th sample of this warp's tile.
    int my_sample = -1, my_found = 0, my_base = 0, my_total = 0;
    unsigned my_mask = kNoMask;
    long long my_key = -1;
    float my_s[D];
#pragma unroll
    for (int d = 0; d < D; ++d) my_s[d] = 0.f;
    if (lane < n_here) {
        my_sample = sample_order ? __ldg(sample_order + i0 + lane) : i0 + lane;
        my_key = __ldg(sample_keys + my_sample);
#pragma unroll
        for (int d = 0; d < D; ++d) my_s[d] = __ldg(samples + (int64_t)my_sample * D + d);
        if (MODE != kCount) {
            my_base = (my_sample > 0) ? __ldg(start_ids + my_sample - 1) : 0;
            my_mask = cache.sample_off[my_sample];
        }
        if (MODE == kStoreLimited) my_total = __ldg(counts + my_sample);
    }

    int k0 = 0;
    while (k0 < n_here) {
        // Run of samples [k0, k1) that share the cell of sample k0.
        const long long key0 = __shfl_sync(kFullMask, my_key, k0);
        const unsigned same = __ballot_sync(kFullMask, lane < n_here && my_key == key0) >> k0;
        const int k1 = k0 + (same == 0xffffffffu ? 32 : __ffs(~same) - 1);
        const int num_cand = resolve_ranges<D>(key0, g, grid_ds, pt_keys, num_pts, lo, pref);
        const int cps = chunks_per_sample<D>(num_cand);

        // Mask space of this run.
        unsigned run_mask = kNoMask;
        if (MODE == kCount) {
            unsigned long long got = 0;
            const unsigned long long need = (unsigned long long)(k1 - k0) * cps;
            if (lane == 0) got = atomicAdd(cache.cursor, need);
            got = __shfl_sync(kFullMask, got, 0);
            if (got + need <= cache.pool_words) run_mask = (unsigned)got;
            if (lane >= k0 && lane < k1 && run_mask != kNoMask) my_mask = run_mask + (unsigned)(lane - k0) * cps;
        } else {
            run_mask = __shfl_sync(kFullMask, my_mask, k0);
        }
        const bool replay = (MODE != kCount) && run_mask != kNoMask;

        int r = 0;  // range that holds this lane's next candidate; only ever moves forward
        for (int round0 = 0; round0 < num_cand; round0 += S::kSlots) {
            const int n_slots = min(S::kSlots, num_cand - round0);
            const int n_padded = (n_slots + 31) & ~31;
            const int n_chunks = n_padded >> 5;
            const int chunk_base = (round0 / S::kSlots) * kChunks;
            // Stage: consecutive lanes take consecutive candidates (contiguous in memory inside a
            // range).  The last 32-group is padded with candidates at +inf, which never pass the
            // test, so the sweep below needs no bounds check.  A replaying store pass only needs
            // the positions.
            for (int sl = lane; sl < n_padded; sl += 32) {
                float w[4 * S::kPlanes];
#pragma unroll
                for (int d = 0; d < 4 * S::kPlanes; ++d) w[d] = __int_as_float(0x7f800000);
                int j = 0;
                if (sl < n_slots) {
                    const int gidx = round0 + sl;
                    while (gidx >= pref[r + 1]) ++r;
                    j = lo[r] + gidx - pref[r];
                    if (!replay) {
#pragma unroll
                        for (int d = 0; d < D; ++d) w[d] = __ldg(pts + (int64_t)j * D + d);
                        w[D] = __int_as_float(j);
                    }
                }
                if (replay) {
                    // final ids, mapped once per staged candidate instead of once per hit
                    slot_ids[sl] = (pt_index_map && sl < n_slots) ? (int)__ldg(pt_index_map + j) : j;
                } else {
#pragma unroll
                    for (int q = 0; q < S::kPlanes; ++q)
                        slots[q * S::kSlots + sl] = make_float4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
                }
            }
            __syncwarp();

            if (replay) {
                // Store pass, bits known.  One load fetches the mask words of kReplay samples
                // (lane = sample-in-group * kChunks + group-of-32 index), and the load for the next
                // samples is issued before the current ones are replayed, so the memory latency
                // is paid once per run instead of once per sample.
                constexpr int kReplay = (32 / kChunks) < 8 ? (32 / kChunks) : 8;
                const int sub = lane / kChunks, cidx = lane - sub * kChunks;
                auto load_words = [&](int k) -> unsigned {
                    const int kk = k + sub;
                    const unsigned off = __shfl_sync(kFullMask, my_mask, min(kk, 31));
                    const bool want = sub < kReplay && kk < k1 && cidx < n_chunks;
                    return want ? __ldcs(cache.pool + off + chunk_base + cidx) : 0u;
                };
                unsigned words = load_words(k0);
                for (int k = k0; k < k1; k += kReplay) {
                    const unsigned cur = words;
                    if (k + kReplay < k1) words = load_words(k + kReplay);
                    const int n_sub = min(kReplay, k1 - k);
                    // Both loops are unrolled so that every shuffle has a constant source lane; groups
                    // past the end of a short round hold zero words and emit nothing.
#pragma unroll
                    for (int gi = 0; gi < kReplay; ++gi) {
                        if (gi >= n_sub) break;
                        const int kk = k + gi;
                        int found = __shfl_sync(kFullMask, my_found, kk);
                        const int m = __shfl_sync(kFullMask, my_sample, kk);
                        const int base = __shfl_sync(kFullMask, my_base, kk);
                        const int total = (MODE == kStoreLimited) ? __shfl_sync(kFullMask, my_total, kk) : 0;
#pragma unroll
                        for (int ci = 0; ci < kChunks; ++ci) {
                            const unsigned bal = __shfl_sync(kFullMask, cur, gi * kChunks + ci);
                            // The id is read and the slot computed by every lane, so that the hit itself is
                            // a single predicated store instead of a divergent block.
                            const int id = slot_ids[ci * 32 + lane];
                            const int rank = found + __popc(bal & lt_mask);
                            if (MODE == kStore) {
                                if (bal & lane_bit) out[base + rank] = make_int2(id, m);
                            } else if (bal & lane_bit) {
                                emit_row<MODE>(out, base, rank, id, m, total, max_neighbors);
                            }
                            found += __popc(bal);
                        }
                        if (lane == kk) my_found = found;
                    }
                }
            } else {
                // Sweep with arithmetic: kGroup samples share every candidate load.
                constexpr int kGroup = (MODE == kCount) ? 4 : 2;
                for (int k = k0; k < k1; k += kGroup) {
                    float s[kGroup][D];
                    int found[kGroup], m[kGroup], base[kGroup], total[kGroup];
                    unsigned word[kGroup];
#pragma unroll
                    for (int gi = 0; gi < kGroup; ++gi) {
                        const int kk = min(k + gi, k1 - 1);  // the tail of a run repeats its last sample
#pragma unroll
                        for (int d = 0; d < D; ++d) s[gi][d] = __shfl_sync(kFullMask, my_s[d], kk);
                        found[gi] = (MODE == kCount) ? 0 : __shfl_sync(kFullMask, my_found, kk);
                        m[gi] = (MODE == kCount) ? 0 : __shfl_sync(kFullMask, my_sample, kk);
                        base[gi] = (MODE == kCount) ? 0 : __shfl_sync(kFullMask, my_base, kk);
                        total[gi] = (MODE == kStoreLimited) ? __shfl_sync(kFullMask, my_total, kk) : 0;
                        word[gi] = 0u;
                    }
                    for (int ci = 0; ci < n_chunks; ++ci) {
                        float w[4 * S::kPlanes];
#pragma unroll
                        for (int q = 0; q < S::kPlanes; ++q) {
                            const float4 v = slots[q * S::kSlots + ci * 32 + lane];
                            w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z; w[4 * q + 3] = v.w;
                        }
                        // Two samples per instruction: the packed fp32x2 forms round each half exactly like
                        // the scalar operation (round to nearest, no flush), so the predicate keeps its bits,
                        // and they take one issue slot instead of two in a loop that is bound by issue.
                        float dist2[kGroup];
#pragma unroll
                        for (int gi = 0; gi < kGroup; gi += 2) {
                            if (MODE != kCount) {  // the rarely used recomputing store keeps its register budget
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    float acc = 0.f;
#pragma unroll
                                    for (int d = 0; d < D; ++d) {
                                        const float v = __fmul_rn(__fsub_rn(s[gi + h][d], w[d]), inv[d]);
                                        acc = (d == 0) ? __fmul_rn(v, v) : __fmaf_rn(v, v, acc);
                                    }
                                    dist2[gi + h] = acc;
                                }
                                continue;
                            }
                            unsigned long long acc2 = 0ull;
#pragma unroll
                            for (int d = 0; d < D; ++d) {
                                const unsigned long long v =
                                    mul_f32x2(sub_f32x2(pack_f32x2(s[gi][d], s[gi + 1][d]), pack_f32x2(w[d], w[d])),
                                              pack_f32x2(inv[d], inv[d]));
                                acc2 = (d == 0) ? mul_f32x2(v, v) : fma_f32x2(v, v, acc2);
                            }
                            unpack_f32x2(acc2, dist2[gi], dist2[gi + 1]);
                        }
#pragma unroll
                        for (int gi = 0; gi < kGroup; ++gi) {
                            const bool hit = dist2[gi] < 1.0f;
                            const unsigned bal = __ballot_sync(kFullMask, hit);
                            if (MODE == kCount) {
                                if (lane == ci) word[gi] = bal;  // lane ci keeps the bits of group ci
                            } else {
                                if (hit && (gi == 0 || k + gi < k1)) {
                                    const int j = __float_as_int(w[D]);
                                    const int id = pt_index_map ? (int)__ldg(pt_index_map + j) : j;
                                    emit_row<MODE>(out, base[gi], found[gi] + __popc(bal & lt_mask), id, m[gi],
                                                   total[gi], max_neighbors);
                                }
                                found[gi] += __popc(bal);
                            }
                        }
                    }
#pragma unroll
                    for (int gi = 0; gi < kGroup; ++gi) {
                        const bool live = k + gi < k1;
                        if (MODE == kCount) {
                            const int sum = __reduce_add_sync(kFullMask, __popc(word[gi]));
                            if (lane == k + gi && live) my_found += sum;
                            if (run_mask != kNoMask && live && lane < n_chunks)
                                cache.pool[run_mask + (unsigned)(k + gi - k0) * cps + chunk_base + lane] = word[gi];
                        } else if (lane == k + gi && live) {
                            my_found = found[gi];
                        }
                    }
                }
            }
            __syncwarp();  // everyone is done with the buffer before the next round overwrites it
        }
        k0 = k1;
    }
    if (MODE == kCount && lane < n_here) {
        counts[my_sample] = my_found;
        cache.sample_off[my_sample] = my_mask;
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

// Work estimates per tile of 32 samples (in the order the search visits them), for the heaviest-first order.
// Before anything is counted: the points in the three cells around the tile's first sample along the last
// axis (two binary searches in the sorted keys), a measure of the local density.
__global__ void tile_density_kernel(int num_tiles, const int64_t* __restrict__ sample_keys,
                                    const int32_t* __restrict__ order, const int64_t* __restrict__ pt_keys, int num_pts,
                                    uint32_t* __restrict__ est) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= num_tiles) return;
    const int i = t * 32;
    const long long key = __ldg(sample_keys + (order ? __ldg(order + i) : i));
    const int lo = lower_bound_key(pt_keys, 0, num_pts, key - 1);
    const int hi = upper_bound_key(pt_keys, lo, num_pts, key + 1);
    // its class: the power of two and the bit below it (half octaves; see tile_order)
    const int v = hi - lo, c = 32 - __clz(v);
    est[t] = (uint32_t)(2 * c + (c >= 2 ? ((v >> (c - 2)) & 1) : 0));
}

// Once the counts are known: the pairs of the tile.
__global__ void tile_pairs_kernel(int num_tiles, int num_samples, const int32_t* __restrict__ order,
                                  const int32_t* __restrict__ counts, uint32_t* __restrict__ est) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= num_tiles) return;
    uint32_t sum = 0;
    for (int i = t * 32; i < min(num_samples, t * 32 + 32); ++i) sum += (uint32_t)__ldg(counts + (order ? __ldg(order + i) : i));
    est[t] = (uint32_t)(2 * (32 - __clz((int)min(sum, 0x7fffffffu))));  // whole octaves, on the scale of the density classes
}

__global__ void iota32_kernel(int n, int32_t* out) {
    const int stride = gridDim.x * blockDim.x;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = i;
}

struct NeighborLayout {
    size_t counts_off, total_off, order_off, iota_off, keys_off, cub_off, cub_bytes, mask_off_off, tiles_off, pool_off, total;
    int num_tiles;
    size_t tile_sort_bytes;
};

// Launches of at least this many tiles visit them heaviest first (below, the few extra launches cost more than an
// uneven end of the search).
constexpr int kMinTilesForOrdering = 8192;

// Hit-mask pool requested by default: 256 bytes (2048 tested candidates) per sample.
constexpr size_t kMaskBytesPerSample = 256;

static NeighborLayout neighbor_layout(int64_t m) {
    NeighborLayout L;
    const int mm = (int)(m > 0 ? m : 1);
    size_t scan_bytes = 0, sort_bytes = 0;
    cub::DeviceScan::InclusiveSum(nullptr, scan_bytes, (const int32_t*)nullptr, (int32_t*)nullptr, mm);
    cub::DeviceRadixSort::SortPairs(nullptr, sort_bytes, (const int64_t*)nullptr, (int64_t*)nullptr,
                                    (const int32_t*)nullptr, (int32_t*)nullptr, mm, 0, 64);
    L.cub_bytes = scan_bytes > sort_bytes ? scan_bytes : sort_bytes;
    L.counts_off = 0;
    L.total_off = align_up((size_t)m * 4);
    L.order_off = L.total_off + 256;
    L.iota_off = L.order_off + align_up((size_t)m * 4);
    L.keys_off = L.iota_off + align_up((size_t)m * 4);
    L.cub_off = L.keys_off + align_up((size_t)m * 8);
    L.num_tiles = (mm + 31) / 32;
    L.tile_sort_bytes = 0;
    cub::DeviceRadixSort::SortPairsDescending(nullptr, L.tile_sort_bytes, (const uint32_t*)nullptr, (uint32_t*)nullptr,
                                              (const int32_t*)nullptr, (int32_t*)nullptr, L.num_tiles, 0, 7);
    if (L.tile_sort_bytes > L.cub_bytes) L.cub_bytes = L.tile_sort_bytes;
    L.mask_off_off = L.cub_off + align_up(L.cub_bytes) + 256;
    L.tiles_off = L.mask_off_off + align_up((size_t)m * 4);
    L.pool_off = L.tiles_off + 4 * align_up((size_t)L.num_tiles * 4);  // estimates, sorted estimates, tile ids, order
    size_t pool = (size_t)m * kMaskBytesPerSample;
    if (pool < (1u << 20)) pool = 1u << 20;
    if (pool > ((size_t)8 << 30)) pool = (size_t)8 << 30;
    L.total = L.pool_off + pool;
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

// Samples that ARE the sorted points (same arrays) are already in cell order.
static bool samples_are_sorted_points(const float* pts, const int64_t* pt_keys, const float* samples,
                                      const int64_t* sample_keys) {
    return samples == pts && sample_keys == pt_keys;
}

// The pool is whatever the caller's workspace holds beyond the fixed part.
static MaskCache mask_cache(char* ws, const NeighborLayout& L, size_t workspace_bytes) {
    MaskCache c;
    c.sample_off = (unsigned*)(ws + L.mask_off_off);
    c.pool = (unsigned*)(ws + L.pool_off);
    c.cursor = (unsigned long long*)(ws + L.total_off + 8);
    size_t words = workspace_bytes > L.pool_off ? (workspace_bytes - L.pool_off) / 4 : 0;
    if (words > 0xfffffff0ull) words = 0xfffffff0ull;
    c.pool_words = words;
    return c;
}

static unsigned neighbor_grid(int64_t num_samples) {
    return (unsigned)((num_samples + kWarpsPerBlock * 32 - 1) / (kWarpsPerBlock * 32));
}

// Heaviest-first order of the tiles; null when the launch is too small for it to pay.  `counts` null = before the
// count pass (density estimate).  The tiles are ordered by a coarse class of their estimate only (half octaves of
// the density, whole octaves of the pair count: what measured best for each pass), with a stable sort: the classes
// go from heavy to light, and inside a class the tiles keep their cell order, so that tiles running at the same
// time still share candidates in the caches.
static int tile_order(char* ws, const NeighborLayout& L, int m, const int64_t* sample_keys, const int32_t* order,
                      const int64_t* pt_keys, int num_pts, const int32_t* counts, cudaStream_t s, const int32_t** out) {
    *out = nullptr;
    if (L.num_tiles < kMinTilesForOrdering || num_pts == 0) return PCCNN_OK;
    const size_t stride = align_up((size_t)L.num_tiles * 4);
    uint32_t* est = (uint32_t*)(ws + L.tiles_off);
    uint32_t* est_sorted = (uint32_t*)(ws + L.tiles_off + stride);
    int32_t* ids = (int32_t*)(ws + L.tiles_off + 2 * stride);
    int32_t* sorted_ids = (int32_t*)(ws + L.tiles_off + 3 * stride);
    const unsigned grid = (unsigned)((L.num_tiles + 255) / 256);
    if (counts)
        tile_pairs_kernel<<<grid, 256, 0, s>>>(L.num_tiles, m, order, counts, est);
    else
        tile_density_kernel<<<grid, 256, 0, s>>>(L.num_tiles, sample_keys, order, pt_keys, num_pts, est);
    PCCNN_LAUNCH_CHECK();
    iota32_kernel<<<grid, 256, 0, s>>>(L.num_tiles, ids);
    PCCNN_LAUNCH_CHECK();
    size_t bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceRadixSort::SortPairsDescending(ws + L.cub_off, bytes, (const uint32_t*)est, est_sorted,
                                                         (const int32_t*)ids, sorted_ids, L.num_tiles, 0, 7, s));
    *out = sorted_ids;
    return PCCNN_OK;
}

}  // namespace pccnn

using namespace pccnn;

extern "C" {

size_t pccnn_find_neighbors_workspace_bytes(int D, int64_t num_samples) {
    (void)D;
    return neighbor_layout(num_samples < 0 ? 0 : num_samples).total;
}

size_t pccnn_find_neighbors_min_workspace_bytes(int D, int64_t num_samples) {
    (void)D;
    return neighbor_layout(num_samples < 0 ? 0 : num_samples).pool_off;
}

int pccnn_find_neighbors_count(int D, int64_t num_pts, const float* pts, const int64_t* pt_keys,
                               int64_t num_samples, const float* samples, const int64_t* sample_keys,
                               const int32_t* grid_ds, const int32_t* grid_size, const float* radii,
                               int32_t max_neighbors, int32_t sample_key_bits, int32_t* out_start_ids,
                               int64_t* out_total_host, void* workspace, size_t workspace_bytes, void* stream) {
    if (int rc = check_common("find_neighbors_count", D, num_pts, num_samples)) return rc;
    PCCNN_CHECK_ARG(sample_key_bits >= 0 && sample_key_bits <= 64, "find_neighbors_count: sample_key_bits outside [0, 64]");
    PCCNN_CHECK_ARG(out_total_host, "find_neighbors_count: null out_total_host");
    PCCNN_CHECK_ARG(max_neighbors >= 0, "find_neighbors_count: negative max_neighbors");
    *out_total_host = 0;
    if (num_samples == 0) return PCCNN_OK;
    PCCNN_CHECK_ARG(samples && sample_keys && grid_ds && grid_size && radii && out_start_ids,
                    "find_neighbors_count: null pointer");
    PCCNN_CHECK_ARG(num_pts == 0 || (pts && pt_keys), "find_neighbors_count: null points");
    const NeighborLayout L = neighbor_layout(num_samples);
    if (!workspace || workspace_bytes < L.pool_off) {
        set_error("find_neighbors_count: workspace of %zu bytes, need at least %zu", workspace_bytes, L.pool_off);
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    int32_t* counts = (int32_t*)(ws + L.counts_off);
    unsigned long long* total_dev = (unsigned long long*)(ws + L.total_off);
    const int m = (int)num_samples;
    PCCNN_CUDA(cudaMemsetAsync(total_dev, 0, 16, s));  // pair total + mask cursor
    const MaskCache cache = mask_cache(ws, L, workspace_bytes);

    const int32_t* order = nullptr;
    if (!samples_are_sorted_points(pts, pt_keys, samples, sample_keys)) {
        // Visit the samples in cell order: stable sort of (key, index).
        int32_t* iota = (int32_t*)(ws + L.iota_off);
        iota32_kernel<<<grid_for(m, 256, 8), 256, 0, s>>>(m, iota);
        PCCNN_LAUNCH_CHECK();
        size_t cub_bytes = L.cub_bytes;
        PCCNN_CUDA(cub::DeviceRadixSort::SortPairs(ws + L.cub_off, cub_bytes, sample_keys, (int64_t*)(ws + L.keys_off),
                                                   (const int32_t*)iota, (int32_t*)(ws + L.order_off), m, 0,
                                                   sample_key_bits > 0 ? sample_key_bits : 64, s));
        order = (const int32_t*)(ws + L.order_off);
    }
    const int32_t* tiles = nullptr;
    if (int rc = tile_order(ws, L, m, sample_keys, order, pt_keys, (int)num_pts, nullptr, s, &tiles)) return rc;
    PCCNN_DISPATCH_DIM(D, (neighbors_kernel<DIM, kCount, (DIM == 3 ? 9 : 0)><<<neighbor_grid(m), kWarpsPerBlock * 32, 0, s>>>(
                              (int)num_pts, pts, pt_keys, m, samples, sample_keys, order, (const int2*)grid_ds,
                              grid_size, radii, max_neighbors, counts, nullptr, nullptr, nullptr, cache, tiles,
                              L.num_tiles)));
    PCCNN_LAUNCH_CHECK();
    clamp_counts_kernel<<<grid_for(m, 256, 8), 256, 0, s>>>(m, counts, max_neighbors, out_start_ids, total_dev);
    PCCNN_LAUNCH_CHECK();
    size_t cub_bytes = L.cub_bytes;
    PCCNN_CUDA(cub::DeviceScan::InclusiveSum(ws + L.cub_off, cub_bytes, out_start_ids, out_start_ids, m, s));
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
    if (!workspace || workspace_bytes < L.pool_off) {
        set_error("find_neighbors_store: workspace of %zu bytes, need at least %zu", workspace_bytes, L.pool_off);
        return PCCNN_ERR_WORKSPACE;
    }
    cudaStream_t s = (cudaStream_t)stream;
    char* ws = (char*)workspace;
    int32_t* counts = (int32_t*)(ws + L.counts_off);
    const int32_t* order =
        samples_are_sorted_points(pts, pt_keys, samples, sample_keys) ? nullptr : (const int32_t*)(ws + L.order_off);
    const int m = (int)num_samples;
    const MaskCache cache = mask_cache(ws, L, workspace_bytes);
    const int32_t* tiles = nullptr;
    if (int rc = tile_order(ws, L, m, sample_keys, order, pt_keys, (int)num_pts, counts, s, &tiles)) return rc;
    if (max_neighbors > 0) {
        PCCNN_DISPATCH_DIM(D, (neighbors_kernel<DIM, kStoreLimited><<<neighbor_grid(m), kWarpsPerBlock * 32, 0, s>>>(
                                  (int)num_pts, pts, pt_keys, m, samples, sample_keys, order, (const int2*)grid_ds,
                                  grid_size, radii, max_neighbors, counts, start_ids, pt_index_map,
                                  (int2*)out_neighbors, cache, tiles, L.num_tiles)));
    } else {
        PCCNN_DISPATCH_DIM(D, (neighbors_kernel<DIM, kStore><<<neighbor_grid(m), kWarpsPerBlock * 32, 0, s>>>(
                                  (int)num_pts, pts, pt_keys, m, samples, sample_keys, order, (const int2*)grid_ds,
                                  grid_size, radii, max_neighbors, counts, start_ids, pt_index_map,
                                  (int2*)out_neighbors, cache, tiles, L.num_tiles)));
    }
    PCCNN_LAUNCH_CHECK();
    return PCCNN_OK;
}

}  // extern "C"
