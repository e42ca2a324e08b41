// C entry points around the REFERENCE's own algorithm objects, for the checker library
// oracle/_ref/libref_knn.so (test infrastructure; built by `make -C oracle ref` from the
// reference sources where they lie, never copied into this repository).
//
// Everything that computes here is the reference's code: serial_knn / parallel_knn (CPU
// selection), bits_knn / bits_prefetch_knn (its `bits` kernel), fused_cache_knn, magma_distance.
// This file only feeds them a caller-provided distance matrix or point set and times
// selection() the way the reference's main loop does (src/main.cpp:387-391).
// The reference's objects create CUDA events in their constructors, so a GPU must be present.
#include <chrono>
#include <cstdint>
#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "bits/cuda_stream.hpp"
#include "bits/distance/cuda_distance.hpp"
#include "bits/distance/magma_distance.hpp"
#include "bits/knn.hpp"
#include "bits/topk/parallel_knn.hpp"
#include "bits/topk/serial_knn.hpp"
#include "bits/topk/singlepass/bits_knn.hpp"
#include "bits/topk/singlepass/fused_cache_knn.hpp"

namespace
{

// Distance object whose matrix is given by the caller (host memory) instead of computed.
class given_matrix : public cuda_distance
{
public:
    given_matrix(const float* host, std::size_t q, std::size_t n) : host_(host), q_(q), n_(n) {}
    std::string name() const override { return "given"; }
    void prepare(const knn_args& args) override
    {
        args_ = args;
        dist_gpu_.release();
        dist_gpu_ = cuda_array<float, 2>{{q_, n_}};
        cuda_stream::make_default().copy_to_gpu_async(dist_gpu_.view(), host_).sync();
    }
    void compute() override {}
    array_view<float, 2> matrix_cpu() override
    {
        return array_view<float, 2>{const_cast<float*>(host_), {q_, n_}, {n_, 1}};
    }

private:
    const float* host_;
    std::size_t q_, n_;
};

thread_local std::string g_error;

std::unique_ptr<knn> make_selection(const std::string& alg)
{
    if (alg == "serial")
        return std::make_unique<serial_knn>();
    if (alg == "parallel")
        return std::make_unique<parallel_knn>();
    if (alg == "bits")
        return std::make_unique<bits_knn>();
    if (alg == "bits-prefetch")
        return std::make_unique<bits_prefetch_knn>();
    return nullptr;
}

} // namespace

extern "C" const char* ref_last_error() { return g_error.c_str(); }

// Runs the reference selection algorithm `alg` on a host matrix (q x n, row major).  `repeats`
// timed calls of selection() after one untimed call; *seconds = the fastest.  Returns 0 on success.
extern "C" int ref_select(const char* alg, const float* dist, std::size_t q, std::size_t n, std::size_t k,
                          std::size_t block_size, std::size_t batch, int repeats, float* out_dist,
                          std::int32_t* out_idx, double* seconds)
try
{
    auto algo = make_selection(alg);
    if (!algo)
    {
        g_error = std::string("unknown reference algorithm: ") + alg;
        return 1;
    }
    static const float dummy = 0.0F;
    knn_args args{};
    args.points = &dummy;
    args.queries = &dummy;
    args.point_count = n;
    args.query_count = q;
    args.dim = 1;
    args.points_layout = matrix_layout::row_major;
    args.queries_layout = matrix_layout::row_major;
    args.dist_layout = matrix_layout::row_major;
    args.dist_block_size = block_size;
    args.selection_block_size = block_size;
    args.k = k;
    args.items_per_thread = {batch, 1, 1};
    args.deg = 1;
    algo->set_dist_impl(std::make_unique<given_matrix>(dist, q, n));
    algo->initialize(args);
    double best = 1e30;
    for (int i = 0; i <= repeats; ++i)
    {
        algo->prepare();
        algo->distances();
        const auto start = std::chrono::steady_clock::now();
        algo->selection();
        const std::chrono::duration<double> d = std::chrono::steady_clock::now() - start;
        if (i > 0 || repeats == 0)
        {
            best = d.count() < best ? d.count() : best;
        }
    }
    const auto result = algo->finish();
    for (std::size_t i = 0; i < q * k; ++i)
    {
        out_dist[i] = result[i].distance;
        out_idx[i] = result[i].index;
    }
    if (seconds != nullptr)
    {
        *seconds = best;
    }
    return 0;
}
catch (std::exception& e)
{
    g_error = e.what();
    return 2;
}

// The reference's fused-cache algorithm on host points (n x dim) and queries (q x dim), row major.
// items = {QUERY_REG, DB_REG, DIM_REG}, block_size = BLOCK_QUERY_DIM, deg = DIM_MULT
// (src/topk/singlepass/fused_cache_knn.cu:202-216).
extern "C" int ref_fused_cache(const float* points, const float* queries, std::size_t n, std::size_t q, std::size_t dim,
                               std::size_t k, std::size_t block_query_dim, std::size_t dim_mult, int repeats,
                               float* out_dist, std::int32_t* out_idx, double* seconds)
try
{
    fused_cache_knn algo;
    knn_args args{};
    args.points = points;
    args.queries = queries;
    args.point_count = n;
    args.query_count = q;
    args.dim = dim;
    args.points_layout = matrix_layout::row_major;
    args.queries_layout = matrix_layout::row_major;
    args.dist_layout = matrix_layout::row_major;
    args.dist_block_size = block_query_dim;
    args.selection_block_size = block_query_dim;
    args.k = k;
    args.items_per_thread = {8, 4, 2};
    args.deg = dim_mult;
    algo.initialize(args);
    double best = 1e30;
    for (int i = 0; i <= repeats; ++i)
    {
        algo.prepare();
        algo.distances();
        const auto start = std::chrono::steady_clock::now();
        algo.selection();
        const std::chrono::duration<double> d = std::chrono::steady_clock::now() - start;
        if (i > 0 || repeats == 0)
        {
            best = d.count() < best ? d.count() : best;
        }
    }
    const auto result = algo.finish();
    for (std::size_t i = 0; i < q * k; ++i)
    {
        out_dist[i] = result[i].distance;
        out_idx[i] = result[i].index;
    }
    if (seconds != nullptr)
    {
        *seconds = best;
    }
    return 0;
}
catch (std::exception& e)
{
    g_error = e.what();
    return 2;
}

// The reference's GEMM-form distance (magma-dist / magma-part-dist) -> host matrix q x n.
extern "C" int ref_l2(const float* points, const float* queries, std::size_t n, std::size_t q, std::size_t dim,
                      int partial, int repeats, float* out, double* seconds)
try
{
    std::unique_ptr<magma_distance> dist;
    if (partial != 0)
        dist = std::make_unique<magma_partial_distance>();
    else
        dist = std::make_unique<magma_distance>();
    knn_args args{};
    args.points = points;
    args.queries = queries;
    args.point_count = n;
    args.query_count = q;
    args.dim = dim;
    args.points_layout = matrix_layout::row_major;
    args.queries_layout = matrix_layout::row_major;
    args.dist_layout = matrix_layout::row_major;
    args.dist_block_size = 256;
    args.selection_block_size = 256;
    args.k = 1;
    args.items_per_thread = {1, 1, 1};
    args.deg = 1;
    dist->prepare(args);
    double best = 1e30;
    for (int i = 0; i <= repeats; ++i)
    {
        const auto start = std::chrono::steady_clock::now();
        dist->compute();
        cuda_stream::make_default().sync();
        const std::chrono::duration<double> d = std::chrono::steady_clock::now() - start;
        if (i > 0 || repeats == 0)
        {
            best = d.count() < best ? d.count() : best;
        }
    }
    const auto view = dist->matrix_cpu();
    for (std::size_t i = 0; i < q; ++i)
    {
        std::memcpy(out + i * n, &view(i, 0), n * sizeof(float));
    }
    if (seconds != nullptr)
    {
        *seconds = best;
    }
    return 0;
}
catch (std::exception& e)
{
    g_error = e.what();
    return 2;
}
