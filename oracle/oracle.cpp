// CPU oracle for the bits-knn hot path.  TEST INFRASTRUCTURE ONLY.
//
// This file restates, in plain host C++, what the reference package
// (jiriklepl/bits-knn-jpdc2024) computes on the path the CUDA library
// accelerates.  It is the checker the tests and the benchmark's CPU-baseline leg
// compare against; no product code path may call into it.
//
// Parity status: PINNED.  The generator + distance + selection + checksum chain
// below reproduces the `Checksum:` lines the reference published for its
// selection runs (data/kselection-hopper01-108424.err; see tests/golden/).
//
// Every function cites the reference file:line it follows.  The generator uses
// libstdc++'s <random> because the reference's data are defined by it
// (`std::default_random_engine` is `minstd_rand0` there).
#include <algorithm>
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <limits>
#include <numeric>
#include <random>
#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace
{

struct pair_t
{
    float distance;
    std::int32_t index;
};

// Total order used by the engine and the oracle: ascending distance, ties broken by the
// lowest index.  The reference compares distances only (src/topk/serial_knn.cpp:40,
// src/topk/parallel_knn.cpp:37-39), which leaves the label among equal distances
// unspecified; the index is the tie-break the replacement promises.
inline bool pair_less(const pair_t& a, const pair_t& b)
{
    return a.distance < b.distance || (a.distance == b.distance && a.index < b.index);
}

} // namespace

extern "C"
{

// Number of host threads the OpenMP loops below will use.
int oracle_num_threads()
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

// ---------------------------------------------------------------------------------------
// Data generators.
// include/bits/generator/uniform_generator.hpp:42-59: one engine seeded once, discard(4096),
// then element-by-element draws from std::uniform_real_distribution<float>{min,max}.
// src/main.cpp:291-298: points are generated first, queries second, from the SAME engine.
// A seed of 0 means "non-deterministic" in the reference (uniform_generator.hpp:57); the
// oracle rejects it (returns 1) because a checker must be repeatable.
// ---------------------------------------------------------------------------------------
int oracle_generate_uniform(std::uint64_t seed, float min, float max, std::size_t point_count,
                            std::size_t query_count, std::size_t dim, float* points,
                            float* queries)
{
    if (seed == 0 || !(min < max))
    {
        return 1;
    }
    std::default_random_engine engine{static_cast<std::default_random_engine::result_type>(seed)};
    engine.discard(1U << 12U);
    {
        std::uniform_real_distribution<float> dist{min, max};
        for (std::size_t i = 0; i < point_count * dim; ++i)
        {
            points[i] = dist(engine);
        }
    }
    {
        // generate() constructs a fresh distribution object per call (uniform_generator.hpp:44)
        std::uniform_real_distribution<float> dist{min, max};
        for (std::size_t i = 0; i < query_count * dim; ++i)
        {
            queries[i] = dist(engine);
        }
    }
    return 0;
}

// include/bits/generator/normal_generator.hpp:42-59 (same engine protocol, fresh
// std::normal_distribution<float>{mean,std_dev} per generate() call, so a cached second
// Box-Muller value never crosses from the points into the queries).
int oracle_generate_normal(std::uint64_t seed, float mean, float std_dev, std::size_t point_count,
                           std::size_t query_count, std::size_t dim, float* points,
                           float* queries)
{
    if (seed == 0 || !(std_dev > 0))
    {
        return 1;
    }
    std::default_random_engine engine{static_cast<std::default_random_engine::result_type>(seed)};
    engine.discard(1U << 12U);
    {
        std::normal_distribution<float> dist{mean, std_dev};
        for (std::size_t i = 0; i < point_count * dim; ++i)
        {
            points[i] = dist(engine);
        }
    }
    {
        std::normal_distribution<float> dist{mean, std_dev};
        for (std::size_t i = 0; i < query_count * dim; ++i)
        {
            queries[i] = dist(engine);
        }
    }
    return 0;
}

// include/bits/preprocessor/ordering_preprocessor.hpp:36-42: sort the FLAT coordinate array
// (not vectors) and zero every query.  descending != 0 -> std::greater, else std::less.
void oracle_preprocess_ordering(float* points, std::size_t point_floats, float* queries,
                                std::size_t query_floats, int descending)
{
    std::fill(queries, queries + query_floats, 0.0F);
    if (descending != 0)
    {
        std::sort(points, points + point_floats, std::greater<>{});
    }
    else
    {
        std::sort(points, points + point_floats, std::less<>{});
    }
}

// ---------------------------------------------------------------------------------------
// Distances.  Row-major points[n][dim], queries[q][dim]; out[q][ld] row-major.
// ---------------------------------------------------------------------------------------

// include/bits/distance/abstract_gemm.cuh:79-93 (l2_ops::run): one accumulator per
// (query, point), `diff = query - point; acc = fmaf(diff, diff, acc)`, dimensions in
// increasing order (the K loop of abstract_gemm.cuh:600-680 never splits or reorders K;
// its zero padding of K to a multiple of 16 adds fmaf(0,0,acc) == acc).
void oracle_l2(const float* points, const float* queries, std::size_t n, std::size_t q,
               std::size_t dim, float* out, std::size_t ld)
{
#pragma omp parallel for schedule(static)
    for (std::size_t i = 0; i < q; ++i)
    {
        const float* qv = queries + i * dim;
        for (std::size_t j = 0; j < n; ++j)
        {
            const float* pv = points + j * dim;
            float acc = 0.0F;
            for (std::size_t d = 0; d < dim; ++d)
            {
                const float diff = qv[d] - pv[d];
                acc = std::fmaf(diff, diff, acc);
            }
            out[i * ld + j] = acc;
        }
    }
}

// include/bits/distance/abstract_gemm.cuh:139-169 (partial_l2_ops) and
// include/bits/topk/singlepass/fused_cache_kernel_structs.cuh:496-519,622-630:
// `dot = fmaf(query, point, dot); norm = fmaf(point, point, norm)` in increasing dimension
// order, result `norm - 2*dot`.  The query norm is NOT added.  (`a += b*c` is contracted
// to an FMA by nvcc's default -fmad=true; `2*dot` is exact, so whether the final
// subtraction is fused does not change the bits.)
void oracle_l2_partial(const float* points, const float* queries, std::size_t n, std::size_t q,
                       std::size_t dim, float* out, std::size_t ld)
{
#pragma omp parallel for schedule(static)
    for (std::size_t i = 0; i < q; ++i)
    {
        const float* qv = queries + i * dim;
        for (std::size_t j = 0; j < n; ++j)
        {
            const float* pv = points + j * dim;
            float dot = 0.0F;
            float nrm = 0.0F;
            for (std::size_t d = 0; d < dim; ++d)
            {
                dot = std::fmaf(qv[d], pv[d], dot);
                nrm = std::fmaf(pv[d], pv[d], nrm);
            }
            out[i * ld + j] = nrm - 2.0F * dot;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Selection.
// ---------------------------------------------------------------------------------------

// src/topk/serial_knn.cpp:35-53: sort each row of (distance, column) pairs, report the first
// k.  The comparator is extended with the index (see pair_less).  `labels` (nullable) gives
// explicit labels per matrix element and `label_offsets` (nullable) one offset per row added
// to the implicit column index -- the two optional inputs of the reference kernel
// (include/bits/topk/singlepass/bits_kernel.hpp:22-27, detail/bits_kernel.cuh:235-243).
// Rows shorter than k are padded with (+inf, position) like the reference's first block load
// (detail/bits_kernel.cuh:340-358).
void oracle_select(const float* dist, std::size_t ld, const std::int32_t* labels,
                   std::size_t ld_labels, const std::int32_t* label_offsets, std::size_t q,
                   std::size_t n, std::size_t k, float* out_dist, std::int32_t* out_idx)
{
#pragma omp parallel
    {
        std::vector<pair_t> row(n);
#pragma omp for schedule(dynamic, 1)
        for (std::size_t i = 0; i < q; ++i)
        {
            const std::int32_t off = label_offsets != nullptr ? label_offsets[i] : 0;
            for (std::size_t j = 0; j < n; ++j)
            {
                row[j].distance = dist[i * ld + j];
                row[j].index = labels != nullptr ? labels[i * ld_labels + j]
                                                 : static_cast<std::int32_t>(j) + off;
            }
            const std::size_t kk = std::min(k, n);
            std::partial_sort(row.begin(), row.begin() + kk, row.end(), pair_less);
            for (std::size_t j = 0; j < kk; ++j)
            {
                out_dist[i * k + j] = row[j].distance;
                out_idx[i * k + j] = row[j].index;
            }
            for (std::size_t j = kk; j < k; ++j)
            {
                out_dist[i * k + j] = std::numeric_limits<float>::infinity();
                out_idx[i * k + j] = static_cast<std::int32_t>(j);
            }
        }
    }
}

// src/topk/parallel_knn.cpp:30-65: OpenMP loop over queries; a max-heap of the first k
// elements, every later element replaces the top when `top.distance > d` (strict), final
// sort of the k survivors.  Restated with the (distance, index) order so its result is the
// same as oracle_select's; this is the routine the benchmark times as the CPU baseline.
// Requires k <= n.
void oracle_select_heap(const float* dist, std::size_t ld, std::size_t q, std::size_t n,
                        std::size_t k, float* out_dist, std::int32_t* out_idx)
{
#pragma omp parallel
    {
        std::vector<pair_t> heap(k);
#pragma omp for schedule(static)
        for (std::size_t i = 0; i < q; ++i)
        {
            const float* row = dist + i * ld;
            for (std::size_t j = 0; j < k; ++j)
            {
                heap[j] = pair_t{row[j], static_cast<std::int32_t>(j)};
            }
            std::make_heap(heap.begin(), heap.end(), pair_less);
            for (std::size_t j = k; j < n; ++j)
            {
                // columns arrive in increasing order, so an equal distance never displaces
                // the incumbent: the strict test of parallel_knn.cpp:54 is also the
                // lowest-index rule.
                if (heap.front().distance > row[j])
                {
                    std::pop_heap(heap.begin(), heap.end(), pair_less);
                    heap.back() = pair_t{row[j], static_cast<std::int32_t>(j)};
                    std::push_heap(heap.begin(), heap.end(), pair_less);
                }
            }
            std::sort(heap.begin(), heap.end(), pair_less);
            for (std::size_t j = 0; j < k; ++j)
            {
                out_dist[i * k + j] = heap[j].distance;
                out_idx[i * k + j] = heap[j].index;
            }
        }
    }
}

// Brute-force k-NN without materialising the matrix: per query the partial (mode 1) or full
// (mode 0) squared distance to every point, then the k smallest pairs.  Distance arithmetic
// as in oracle_l2 / oracle_l2_partial; labels are `index_base + point`, the role
// `label_offsets` plays for a database shard (src/topk/singlepass/bits_knn.cu:67-76).
void oracle_knn(const float* points, const float* queries, std::size_t n, std::size_t q,
                std::size_t dim, std::size_t k, int partial, std::int32_t index_base,
                float* out_dist, std::int32_t* out_idx)
{
#pragma omp parallel
    {
        std::vector<pair_t> row(n);
#pragma omp for schedule(dynamic, 1)
        for (std::size_t i = 0; i < q; ++i)
        {
            const float* qv = queries + i * dim;
            for (std::size_t j = 0; j < n; ++j)
            {
                const float* pv = points + j * dim;
                float d;
                if (partial != 0)
                {
                    float dot = 0.0F;
                    float nrm = 0.0F;
                    for (std::size_t c = 0; c < dim; ++c)
                    {
                        dot = std::fmaf(qv[c], pv[c], dot);
                        nrm = std::fmaf(pv[c], pv[c], nrm);
                    }
                    d = nrm - 2.0F * dot;
                }
                else
                {
                    float acc = 0.0F;
                    for (std::size_t c = 0; c < dim; ++c)
                    {
                        const float diff = qv[c] - pv[c];
                        acc = std::fmaf(diff, diff, acc);
                    }
                    d = acc;
                }
                row[j] = pair_t{d, static_cast<std::int32_t>(j) + index_base};
            }
            const std::size_t kk = std::min(k, n);
            std::partial_sort(row.begin(), row.begin() + kk, row.end(), pair_less);
            for (std::size_t j = 0; j < kk; ++j)
            {
                out_dist[i * k + j] = row[j].distance;
                out_idx[i * k + j] = row[j].index;
            }
            for (std::size_t j = kk; j < k; ++j)
            {
                out_dist[i * k + j] = std::numeric_limits<float>::infinity();
                out_idx[i * k + j] = static_cast<std::int32_t>(j);
            }
        }
    }
}

// The CPU k-NN flow as the reference's `parallel` algorithm runs it, without the matrix in between:
// per query (OpenMP) the distance to every point -- the FMA chains of partial_l2_ops
// (include/bits/distance/abstract_gemm.cuh:139-169; its CPU distance, src/distance/eigen_distance.cpp:39-43,
// computes the same partial form) or of l2_ops (:79-93) -- fed into the max-heap of
// src/topk/parallel_knn.cpp:30-65 (`top > d` replaces the top), final sort of the k survivors.
// This is the routine the benchmark times as the CPU baseline of the k-NN paths.  Requires k <= n.
void oracle_knn_heap(const float* points, const float* queries, std::size_t n, std::size_t q,
                     std::size_t dim, std::size_t k, int partial, float* out_dist, std::int32_t* out_idx)
{
#pragma omp parallel
    {
        std::vector<pair_t> heap(k);
#pragma omp for schedule(dynamic, 1)
        for (std::size_t i = 0; i < q; ++i)
        {
            const float* qv = queries + i * dim;
            auto distance = [&](std::size_t j) {
                const float* pv = points + j * dim;
                if (partial != 0)
                {
                    float dot = 0.0F;
                    float nrm = 0.0F;
                    for (std::size_t c = 0; c < dim; ++c)
                    {
                        dot = std::fmaf(qv[c], pv[c], dot);
                        nrm = std::fmaf(pv[c], pv[c], nrm);
                    }
                    return nrm - 2.0F * dot;
                }
                float acc = 0.0F;
                for (std::size_t c = 0; c < dim; ++c)
                {
                    const float diff = qv[c] - pv[c];
                    acc = std::fmaf(diff, diff, acc);
                }
                return acc;
            };
            for (std::size_t j = 0; j < k; ++j)
            {
                heap[j] = pair_t{distance(j), static_cast<std::int32_t>(j)};
            }
            std::make_heap(heap.begin(), heap.end(), pair_less);
            for (std::size_t j = k; j < n; ++j)
            {
                const float d = distance(j);
                if (heap.front().distance > d)
                {
                    std::pop_heap(heap.begin(), heap.end(), pair_less);
                    heap.back() = pair_t{d, static_cast<std::int32_t>(j)};
                    std::push_heap(heap.begin(), heap.end(), pair_less);
                }
            }
            std::sort(heap.begin(), heap.end(), pair_less);
            for (std::size_t j = 0; j < k; ++j)
            {
                out_dist[i * k + j] = heap[j].distance;
                out_idx[i * k + j] = heap[j].index;
            }
        }
    }
}

// Merge `lists` candidate lists of k pairs per query into the k smallest pairs.
// Candidates are addressed as cand[list * list_stride + query * query_stride + j]; this
// is pass 2 of the reference's split-row scheme (src/topk/singlepass/bits_knn.cu:170-183:
// a selection over q x (k*deg) candidates with explicit labels).
void oracle_merge(const float* cand_dist, const std::int32_t* cand_idx, std::size_t list_stride,
                  std::size_t query_stride, std::size_t q, std::size_t lists, std::size_t k,
                  float* out_dist, std::int32_t* out_idx)
{
#pragma omp parallel
    {
        std::vector<pair_t> row(lists * k);
#pragma omp for schedule(static)
        for (std::size_t i = 0; i < q; ++i)
        {
            for (std::size_t l = 0; l < lists; ++l)
            {
                for (std::size_t j = 0; j < k; ++j)
                {
                    const std::size_t at = l * list_stride + i * query_stride + j;
                    row[l * k + j] = pair_t{cand_dist[at], cand_idx[at]};
                }
            }
            std::partial_sort(row.begin(), row.begin() + k, row.end(), pair_less);
            for (std::size_t j = 0; j < k; ++j)
            {
                out_dist[i * k + j] = row[j].distance;
                out_idx[i * k + j] = row[j].index;
            }
        }
    }
}

// src/main.cpp:410-416: the stderr checksum is the sum of the k indices of QUERY 0 only,
// accumulated in an unsigned 32-bit integer (wraps modulo 2^32).
std::uint32_t oracle_checksum(const std::int32_t* out_idx_query0, std::size_t k)
{
    std::uint32_t sink = 0;
    for (std::size_t j = 0; j < k; ++j)
    {
        sink += static_cast<std::uint32_t>(out_idx_query0[j]);
    }
    return sink;
}

// src/verify.cpp:16-35 approx_equal: relative difference |a-b| / min(|a|+|b|, FLT_MAX) below
// epsilon, with the special cases for exact equality and values at or near zero.
static bool approx_equal(float a, float b, float epsilon)
{
    if (a == b)
    {
        return true;
    }
    const float mag = std::fabs(a) + std::fabs(b);
    const float diff = std::fabs(a - b);
    const float tiny = std::numeric_limits<float>::min();
    if (a == 0 || b == 0 || mag < tiny)
    {
        return diff < epsilon * tiny;
    }
    return diff / std::min(mag, std::numeric_limits<float>::max()) < epsilon;
}

// src/verify.cpp:37-51 normalize: an insertion pass over the WHOLE flattened result that
// moves an element left while its distance is approximately equal to its left neighbour's
// and its index is larger (so runs of near-equal distances end up in descending index
// order in both results before labels are compared).
static void normalize_pairs(std::vector<pair_t>& data)
{
    for (std::ptrdiff_t i = 1; i < static_cast<std::ptrdiff_t>(data.size()); ++i)
    {
        std::ptrdiff_t j = i;
        while (j > 0 && approx_equal(data[j].distance, data[j - 1].distance, 1e-3F) &&
               data[j].index > data[j - 1].index)
        {
            std::swap(data[j], data[j - 1]);
            --j;
        }
    }
}

// src/verify.cpp:55-74 is_distance_same: every neighbouring pair in [begin, end) is
// approximately equal; an empty range counts as "not the same".
static bool tail_is_one_tie(const std::vector<pair_t>& data, std::size_t begin, std::size_t end)
{
    if (begin == end)
    {
        return false;
    }
    for (std::size_t i = begin + 1; i < end; ++i)
    {
        if (!approx_equal(data[i - 1].distance, data[i].distance, 1e-3F))
        {
            return false;
        }
    }
    return true;
}

// src/verify.cpp:78-112 verify: after normalising both results, a slot whose labels differ is
// forgiven only when the rest of that query's row is a single tie group in both results and
// the two distances at the slot agree.  Returns the number of unforgiven slots (0 = the
// reference's `true`).
std::size_t oracle_verify(const float* dist_a, const std::int32_t* idx_a, const float* dist_b,
                          const std::int32_t* idx_b, std::size_t q, std::size_t k)
{
    std::vector<pair_t> expected(q * k);
    std::vector<pair_t> actual(q * k);
    for (std::size_t i = 0; i < q * k; ++i)
    {
        expected[i] = pair_t{dist_a[i], idx_a[i]};
        actual[i] = pair_t{dist_b[i], idx_b[i]};
    }
    normalize_pairs(expected);
    normalize_pairs(actual);
    std::size_t bad = 0;
    for (std::size_t i = 0; i < expected.size(); ++i)
    {
        if (expected[i].index == actual[i].index)
        {
            continue;
        }
        const std::size_t last = i + (k - (i % k));
        if (tail_is_one_tie(expected, i, last) && tail_is_one_tie(actual, i, last) &&
            approx_equal(expected[i].distance, actual[i].distance, 1e-3F))
        {
            continue;
        }
        ++bad;
    }
    return bad;
}

} // extern "C"
