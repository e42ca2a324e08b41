// Algorithm objects of the registry: thin adapters from the reference's plug-in API to the
// C ABI.  Each phase ends with a stream synchronisation so that host timers around the
// phases measure what the reference's do (src/main.cpp:366-408, src/knn.cpp:24-29,
// src/topk/singlepass/bits_knn.cu:95,113).
#include <algorithm>
#include <cmath>
#include <cstdio>
#include <exception>
#include <iostream>
#include <thread>

#include "bitsknn/knn.hpp"

namespace bits
{

void cuda_check(cudaError_t status, const char* what, const char* file, int line)
{
    if (status != cudaSuccess)
    {
        std::cerr << file << ":" << line << " " << cudaGetErrorName(status) << ": " << cudaGetErrorString(status)
                  << "\n\t" << what << '\n';
        throw std::runtime_error{"CUDA error."};
    }
}

void abi_check(int status)
{
    if (status != BITSKNN_OK)
    {
        throw std::runtime_error{bitsknn_last_error_string()};
    }
}

// End of a device phase: the stream is idle (host timers around the phase measure the kernels,
// as the reference's do: src/topk/singlepass/bits_knn.cu:95,113) and no kernel of the phase gave
// up a bounded wait -- an expired wait leaves the outputs incomplete, so it is an error like any
// other ("a kernel gave up a bounded wait"), not a result.
void end_phase()
{
    BITS_CUCH(cudaStreamSynchronize(nullptr));
    abi_check(bitsknn_device_status(nullptr));
}

// events are created on first use, so that building the registry needs no device
transfer_timer::transfer_timer() = default;

transfer_timer::~transfer_timer()
{
    if (begin_ != nullptr)
    {
        cudaEventDestroy(begin_);
    }
    if (end_ != nullptr)
    {
        cudaEventDestroy(end_);
    }
}

void transfer_timer::begin(cudaStream_t stream)
{
    if (begin_ == nullptr)
    {
        BITS_CUCH(cudaEventCreate(&begin_));
        BITS_CUCH(cudaEventCreate(&end_));
    }
    BITS_CUCH(cudaEventRecord(begin_, stream));
}

void transfer_timer::end(cudaStream_t stream, bool wait)
{
    BITS_CUCH(cudaEventRecord(end_, stream));
    if (wait)
    {
        BITS_CUCH(cudaEventSynchronize(end_));
    }
    measured_ = true;
}

float transfer_timer::seconds() const
{
    if (!measured_)
    {
        return 0;
    }
    BITS_CUCH(cudaEventSynchronize(end_));
    float ms = 0;
    BITS_CUCH(cudaEventElapsedTime(&ms, begin_, end_));
    return ms / 1e3F;
}

namespace
{

// host transpose of a cols x rows (column-major view of rows x cols) matrix to row major
std::vector<float> to_row_major(const float* src, std::size_t rows, std::size_t cols)
{
    std::vector<float> out(rows * cols);
    for (std::size_t c = 0; c < cols; ++c)
    {
        for (std::size_t r = 0; r < rows; ++r)
        {
            out[r * cols + c] = src[c * rows + r];
        }
    }
    return out;
}

inline bool pair_less(const distance_pair& a, const distance_pair& b)
{
    return a.distance < b.distance || (a.distance == b.distance && a.index < b.index);
}

} // namespace

cuda_distance::~cuda_distance()
{
    release_pieces();
    if (copy_stream_ != nullptr)
    {
        cudaStreamDestroy(copy_stream_);
    }
}

void cuda_distance::release_pieces()
{
    for (auto& p : pieces_)
    {
        cudaEventDestroy(p.arrived);
    }
    pieces_.clear();
    pieces_fresh_ = false;
}

void cuda_distance::prepare(const knn_args& args)
{
    args_ = args;
    release_pieces();
    dist_gpu_.release();
    points_gpu_.release();
    queries_gpu_.release();
    staging_.release();
    points_gpu_ = device_buffer<float>{args_.point_count * args_.dim};
    queries_gpu_ = device_buffer<float>{args_.query_count * args_.dim};
    if (needs_matrix_)
    {
        dist_gpu_ = device_buffer<float>{args_.query_count * args_.point_count};
    }
    if (copy_stream_ == nullptr)
    {
        BITS_CUCH(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
    }
    const std::size_t n = args_.point_count;
    const std::size_t q = args_.query_count;
    const std::size_t dim = args_.dim;
    const bool points_cm = args_.points_layout == matrix_layout::column_major;
    const bool queries_cm = args_.queries_layout == matrix_layout::column_major;
    // the device always holds row-major inputs; a column-major host matrix is uploaded as it is
    // and transposed by a kernel on the copy stream
    if (points_cm || queries_cm)
    {
        staging_ = device_buffer<float>{(points_cm ? n * dim : 0) + (queries_cm ? q * dim : 0)};
    }
    timer_.begin(copy_stream_);
    if (queries_cm)
    {
        float* raw = staging_.data() + (points_cm ? n * dim : 0);
        BITS_CUCH(cudaMemcpyAsync(raw, args_.queries, q * dim * sizeof(float), cudaMemcpyHostToDevice, copy_stream_));
        abi_check(bitsknn_transpose(raw, static_cast<std::int64_t>(dim), static_cast<std::int64_t>(q), queries_gpu_.data(),
                                    copy_stream_));
    }
    else
    {
        BITS_CUCH(cudaMemcpyAsync(queries_gpu_.data(), args_.queries, q * dim * sizeof(float), cudaMemcpyHostToDevice,
                                  copy_stream_));
    }
    // pieces of at least 16 MiB, four at most: the distance kernel of a piece can start while
    // the next one is still on the bus
    const std::size_t bytes = n * dim * sizeof(float);
    const std::size_t count = points_cm ? 1 : std::min<std::size_t>(4, std::max<std::size_t>(1, bytes >> 24));
    for (std::size_t i = 0; i < count; ++i)
    {
        piece p{i * n / count, (i + 1) * n / count, nullptr};
        if (points_cm)
        {
            BITS_CUCH(cudaMemcpyAsync(staging_.data(), args_.points, bytes, cudaMemcpyHostToDevice, copy_stream_));
            abi_check(bitsknn_transpose(staging_.data(), static_cast<std::int64_t>(dim), static_cast<std::int64_t>(n),
                                        points_gpu_.data(), copy_stream_));
        }
        else
        {
            BITS_CUCH(cudaMemcpyAsync(points_gpu_.data() + p.begin * dim, args_.points + p.begin * dim,
                                      (p.end - p.begin) * dim * sizeof(float), cudaMemcpyHostToDevice, copy_stream_));
        }
        BITS_CUCH(cudaEventCreateWithFlags(&p.arrived, cudaEventDisableTiming));
        BITS_CUCH(cudaEventRecord(p.arrived, copy_stream_));
        pieces_.push_back(p);
    }
    timer_.end(copy_stream_, /*wait*/ false);
    pieces_fresh_ = true;
}

void cuda_distance::wait_inputs()
{
    for (const auto& p : pieces_)
    {
        BITS_CUCH(cudaStreamWaitEvent(nullptr, p.arrived, 0));
    }
    pieces_fresh_ = false;
}

const std::vector<float>& cuda_distance::matrix_cpu()
{
    dist_cpu_.resize(args_.query_count * args_.point_count);
    BITS_CUCH(cudaMemcpy(dist_cpu_.data(), dist_gpu_.data(), dist_cpu_.size() * sizeof(float),
                         cudaMemcpyDeviceToHost));
    return dist_cpu_;
}

void gemm_distance::compute()
{
    const auto n = static_cast<std::int64_t>(args_.point_count);
    const auto q = static_cast<std::int64_t>(args_.query_count);
    const int dim = static_cast<int>(args_.dim);
    const std::size_t need = bitsknn_l2_workspace_bytes(n, q, dim, mode_);
    if (need > workspace_.size())
    {
        workspace_ = device_buffer<unsigned char>{need};
    }
    if (pieces_fresh_ && pieces_.size() > 1)
    {
        // first computation after the upload: the columns of every piece as soon as it has arrived
        pieces_fresh_ = false;
        for (const auto& p : pieces_)
        {
            BITS_CUCH(cudaStreamWaitEvent(nullptr, p.arrived, 0));
            abi_check(bitsknn_l2(points_gpu_.data() + p.begin * args_.dim, queries_gpu_.data(),
                                 static_cast<std::int64_t>(p.end - p.begin), q, dim, mode_, dist_gpu_.data() + p.begin, n,
                                 workspace_.data(), workspace_.size(), nullptr));
        }
        return;
    }
    wait_inputs();
    abi_check(bitsknn_l2(points_gpu_.data(), queries_gpu_.data(), n, q, dim, mode_, dist_gpu_.data(), n,
                         workspace_.data(), workspace_.size(), nullptr));
}

std::unique_ptr<cuda_distance> knn::default_distance() const
{
    // the reference's default for every algorithm is its full-L2 GEMM-form distance
    // (src/knn.cpp:16-20)
    return std::make_unique<gemm_distance>(BITSKNN_L2_EXACT, "magma-dist");
}

void knn::initialize(const knn_args& args)
{
    args_ = args;
    args_.dist_layout = matrix_layout::row_major;
    if (dist_impl_ == nullptr)
    {
        dist_impl_ = default_distance();
    }
    dist_impl_->prepare(args_);
}

void knn::distances()
{
    dist_impl_->compute();
    end_phase();
}

void cuda_knn::initialize(const knn_args& args)
{
    knn::initialize(args);
    out_dist_gpu_ = device_buffer<float>{query_count() * k()};
    out_label_gpu_ = device_buffer<std::int32_t>{query_count() * k()};
}

std::vector<distance_pair> cuda_knn::finish()
{
    if (no_output_)
    {
        out_timer_.begin();
        out_timer_.end();
        return {};
    }
    const std::size_t count = query_count() * k();
    std::vector<float> dist(count);
    std::vector<std::int32_t> label(count);
    out_timer_.begin();
    BITS_CUCH(cudaMemcpyAsync(dist.data(), out_dist_gpu_.data(), count * sizeof(float), cudaMemcpyDeviceToHost, nullptr));
    BITS_CUCH(cudaMemcpyAsync(label.data(), out_label_gpu_.data(), count * sizeof(std::int32_t),
                              cudaMemcpyDeviceToHost, nullptr));
    out_timer_.end();
    std::vector<distance_pair> result(count);
    for (std::size_t i = 0; i < count; ++i)
    {
        result[i] = distance_pair{dist[i], label[i]};
    }
    return result;
}

void bits_knn::initialize(const knn_args& args)
{
    cuda_knn::initialize(args);
    // few, long rows: the library cuts them into slices (what the reference's `bits-sq --deg` does
    // by hand) so that every SM has a block to run
    splits_ = bitsknn_select_auto_splits(static_cast<std::int64_t>(query_count()),
                                         static_cast<std::int64_t>(point_count()), static_cast<int>(k()));
    workspace_.release();
    if (splits_ > 1)
    {
        workspace_ = device_buffer<unsigned char>{bitsknn_select_split_workspace_bytes(
            static_cast<std::int64_t>(query_count()), static_cast<int>(k()), splits_)};
    }
}

void bits_knn::selection()
{
    const auto n = static_cast<std::int64_t>(point_count());
    if (splits_ > 1)
    {
        abi_check(bitsknn_select_split(in_dist_gpu(), n, nullptr, static_cast<std::int64_t>(query_count()), n,
                                       static_cast<int>(k()), splits_, workspace_.data(), workspace_.size(),
                                       out_dist_gpu(), out_label_gpu(), nullptr));
    }
    else
    {
        abi_check(bitsknn_select(in_dist_gpu(), n, nullptr, 0, nullptr, static_cast<std::int64_t>(query_count()), n,
                                 static_cast<int>(k()), out_dist_gpu(), out_label_gpu(), nullptr));
    }
    end_phase();
}

void ablation_knn::selection()
{
    const auto n = static_cast<std::int64_t>(point_count());
    abi_check(bitsknn_select_ablation(in_dist_gpu(), n, static_cast<std::int64_t>(query_count()), n, static_cast<int>(k()),
                                      variant_, out_dist_gpu(), out_label_gpu(), nullptr));
    end_phase();
}

void bits_sq_knn::initialize(const knn_args& args)
{
    cuda_knn::initialize(args);
    const int deg = static_cast<int>(std::max<std::size_t>(args_.deg, 1));
    workspace_ = device_buffer<unsigned char>{bitsknn_select_split_workspace_bytes(
        static_cast<std::int64_t>(query_count()), static_cast<int>(k()), deg)};
}

void bits_sq_knn::selection()
{
    const auto n = static_cast<std::int64_t>(point_count());
    const int deg = static_cast<int>(std::max<std::size_t>(args_.deg, 1));
    abi_check(bitsknn_select_split(in_dist_gpu(), n, nullptr, static_cast<std::int64_t>(query_count()), n,
                                   static_cast<int>(k()), deg, workspace_.data(), workspace_.size(), out_dist_gpu(),
                                   out_label_gpu(), nullptr));
    end_phase();
}

void fused_knn::initialize(const knn_args& args)
{
    cuda_knn::initialize(args);
    workspace_ = device_buffer<unsigned char>{bitsknn_fused_workspace_bytes(
        static_cast<std::int64_t>(point_count()), static_cast<std::int64_t>(query_count()), static_cast<int>(dim()),
        static_cast<int>(k()), mode_)};
}

void fused_knn::selection()
{
    dist_impl_->wait_inputs();
    abi_check(bitsknn_fused(dist_impl_->points_gpu(), dist_impl_->queries_gpu(), static_cast<std::int64_t>(point_count()),
                            static_cast<std::int64_t>(query_count()), static_cast<int>(dim()), static_cast<int>(k()),
                            mode_, 0, out_dist_gpu(), out_label_gpu(), workspace_.data(), workspace_.size(), nullptr));
    end_phase();
}

// ---- bits-sharded: the database split over the visible GPUs, one host thread per GPU ------------

namespace
{

// Runs fn(g) on one host thread per shard and rethrows the first failure.
template <class Fn>
void for_each_shard(std::size_t shards, Fn fn)
{
    std::vector<std::thread> threads;
    std::vector<std::exception_ptr> errors(shards);
    for (std::size_t g = 0; g < shards; ++g)
    {
        threads.emplace_back([&, g] {
            try
            {
                fn(g);
            }
            catch (...)
            {
                errors[g] = std::current_exception();
            }
        });
    }
    for (auto& t : threads)
    {
        t.join();
    }
    for (auto& e : errors)
    {
        if (e)
        {
            std::rethrow_exception(e);
        }
    }
}

} // namespace

sharded_knn::~sharded_knn()
{
    for (std::size_t g = 0; g < shards_.size(); ++g)
    {
        cudaSetDevice(shards_[g].device);
        bitsknn_sharded_destroy(shards_[g].handle);
        shards_[g] = shard{};
    }
    cudaSetDevice(0);
}

void sharded_knn::initialize(const knn_args& args)
{
    args_ = args;
    int visible = 0;
    BITS_CUCH(cudaGetDeviceCount(&visible));
    // `--deg G` limits the search to G GPUs (the reference's `--deg` cuts a row into G slices for
    // `bits-sq`, src/topk/singlepass/bits_knn.cu:132-186; here it cuts the database into G shards);
    // the default of 1 means "all visible GPUs"
    std::size_t world = static_cast<std::size_t>(std::max(visible, 1));
    if (args_.deg > 1)
    {
        world = std::min<std::size_t>(world, args_.deg);
    }
    world = std::min<std::size_t>(world, std::max<std::size_t>(point_count(), 1));
    for (auto& old : shards_)
    {
        cudaSetDevice(old.device);
        bitsknn_sharded_destroy(old.handle);
    }
    shards_.clear();
    shards_.resize(world);

    // row-major host inputs (a column-major host matrix is transposed once, here)
    std::vector<float> tmp_points;
    std::vector<float> tmp_queries;
    const float* points = args_.points;
    const float* queries = args_.queries;
    if (args_.points_layout == matrix_layout::column_major)
    {
        tmp_points = to_row_major(points, point_count(), dim());
        points = tmp_points.data();
    }
    if (args_.queries_layout == matrix_layout::column_major)
    {
        tmp_queries = to_row_major(queries, query_count(), dim());
        queries = tmp_queries.data();
    }
    unsigned char id[BITSKNN_SHARDED_ID_BYTES] = {};
    if (world > 1)
    {
        abi_check(bitsknn_sharded_unique_id(id));
    }
    const auto n = point_count();
    const auto q = static_cast<std::int64_t>(query_count());
    const int kk = static_cast<int>(k());
    const int d = static_cast<int>(dim());
    for_each_shard(world, [&](std::size_t g) {
        shard& s = shards_[g];
        s.device = static_cast<int>(g);
        BITS_CUCH(cudaSetDevice(s.device));
        // contiguous, nearly equal shards: the first n % world shards hold one point more
        const std::size_t base = n / world;
        const std::size_t extra = n % world;
        s.begin = g * base + std::min(g, extra);
        s.count = base + (g < extra ? 1 : 0);
        s.points = device_buffer<float>{s.count * dim()};
        s.queries = device_buffer<float>{query_count() * dim()};
        s.out_dist = device_buffer<float>{query_count() * k()};
        s.out_label = device_buffer<std::int32_t>{query_count() * k()};
        transfer_timer timer;
        timer.begin();
        BITS_CUCH(cudaMemcpyAsync(s.points.data(), points + s.begin * dim(), s.count * dim() * sizeof(float),
                                  cudaMemcpyHostToDevice, nullptr));
        BITS_CUCH(cudaMemcpyAsync(s.queries.data(), queries, query_count() * dim() * sizeof(float), cudaMemcpyHostToDevice,
                                  nullptr));
        timer.end();
        s.transfer_seconds = timer.seconds();
        abi_check(bitsknn_sharded_create(&s.handle, id, static_cast<int>(g), static_cast<int>(world)));
        s.fused_ws = device_buffer<unsigned char>{
            bitsknn_fused_workspace_bytes(static_cast<std::int64_t>(s.count), q, d, kk, mode_)};
        s.exchange_ws = device_buffer<unsigned char>{bitsknn_sharded_workspace_bytes(s.handle, q, kk)};
    });
    BITS_CUCH(cudaSetDevice(0));
}

void sharded_knn::selection()
{
    for_each_shard(shards_.size(), [&](std::size_t g) {
        shard& s = shards_[g];
        BITS_CUCH(cudaSetDevice(s.device));
        abi_check(bitsknn_sharded_search_fused(s.handle, s.points.data(), s.queries.data(),
                                               static_cast<std::int64_t>(s.count),
                                               static_cast<std::int64_t>(query_count()), static_cast<int>(dim()),
                                               static_cast<int>(k()), mode_, static_cast<std::int32_t>(s.begin),
                                               s.out_dist.data(), s.out_label.data(), s.fused_ws.data(),
                                               s.fused_ws.size(), s.exchange_ws.data(), s.exchange_ws.size(), nullptr));
        end_phase();
    });
    BITS_CUCH(cudaSetDevice(0));
}

std::vector<distance_pair> sharded_knn::finish()
{
    // every shard ends with the full result; shard 0's copy is the one downloaded
    const shard& s = shards_.front();
    BITS_CUCH(cudaSetDevice(s.device));
    if (no_output_)
    {
        out_timer_.begin();
        out_timer_.end();
        return {};
    }
    const std::size_t count = query_count() * k();
    std::vector<float> dist(count);
    std::vector<std::int32_t> label(count);
    out_timer_.begin();
    BITS_CUCH(cudaMemcpyAsync(dist.data(), s.out_dist.data(), count * sizeof(float), cudaMemcpyDeviceToHost, nullptr));
    BITS_CUCH(cudaMemcpyAsync(label.data(), s.out_label.data(), count * sizeof(std::int32_t), cudaMemcpyDeviceToHost,
                              nullptr));
    out_timer_.end();
    std::vector<distance_pair> result(count);
    for (std::size_t i = 0; i < count; ++i)
    {
        result[i] = distance_pair{dist[i], label[i]};
    }
    return result;
}

float sharded_knn::transfer_in_seconds() const
{
    float longest = 0;
    for (const auto& s : shards_)
    {
        longest = std::max(longest, s.transfer_seconds);
    }
    return longest;
}

void serial_knn::distances()
{
    knn::distances();
    const auto& matrix = dist_impl_->matrix_cpu();
    dist_.resize(matrix.size());
    for (std::size_t i = 0; i < query_count(); ++i)
    {
        for (std::size_t j = 0; j < point_count(); ++j)
        {
            dist_[i * point_count() + j] = distance_pair{matrix[i * point_count() + j], static_cast<std::int32_t>(j)};
        }
    }
}

void serial_knn::selection()
{
    for (std::size_t i = 0; i < query_count(); ++i)
    {
        const auto begin = dist_.begin() + static_cast<std::ptrdiff_t>(i * point_count());
        std::sort(begin, begin + static_cast<std::ptrdiff_t>(point_count()), pair_less);
    }
}

std::vector<distance_pair> serial_knn::finish()
{
    std::vector<distance_pair> result(query_count() * k());
    for (std::size_t i = 0; i < query_count(); ++i)
    {
        for (std::size_t j = 0; j < k(); ++j)
        {
            result[i * k() + j] = j < point_count()
                                      ? dist_[i * point_count() + j]
                                      : distance_pair{INFINITY, static_cast<std::int32_t>(j)};
        }
    }
    return result;
}

void parallel_knn::distances()
{
    knn::distances();
    matrix_ = &dist_impl_->matrix_cpu();
}

void parallel_knn::selection()
{
    const std::size_t n = point_count();
    const std::size_t kk = std::min(k(), n);
    result_.assign(query_count() * k(), distance_pair{INFINITY, 0});
#pragma omp parallel for
    for (std::size_t i = 0; i < query_count(); ++i)
    {
        const float* row = matrix_->data() + i * n;
        const auto begin = result_.begin() + static_cast<std::ptrdiff_t>(i * k());
        const auto end = begin + static_cast<std::ptrdiff_t>(kk);
        for (std::size_t j = 0; j < kk; ++j)
        {
            begin[static_cast<std::ptrdiff_t>(j)] = distance_pair{row[j], static_cast<std::int32_t>(j)};
        }
        std::make_heap(begin, end, pair_less);
        for (std::size_t j = kk; j < n; ++j)
        {
            if (begin->distance > row[j])
            {
                std::pop_heap(begin, end, pair_less);
                *(end - 1) = distance_pair{row[j], static_cast<std::int32_t>(j)};
                std::push_heap(begin, end, pair_less);
            }
        }
        std::sort(begin, end, pair_less);
        for (std::size_t j = kk; j < k(); ++j)
        {
            begin[static_cast<std::ptrdiff_t>(j)] = distance_pair{INFINITY, static_cast<std::int32_t>(j)};
        }
    }
}

std::vector<std::unique_ptr<knn>> make_registry()
{
    std::vector<std::unique_ptr<knn>> algorithms;
    algorithms.push_back(std::make_unique<serial_knn>());
    algorithms.push_back(std::make_unique<parallel_knn>());
    algorithms.push_back(std::make_unique<ablation_knn>("partial-bitonic-regs", BITSKNN_ABLATION_NO_BUFFER));
    algorithms.push_back(std::make_unique<ablation_knn>("partial-bitonic-buffered-static", BITSKNN_ABLATION_SHARED_LIST));
    algorithms.push_back(std::make_unique<bits_knn>("bits"));
    algorithms.push_back(std::make_unique<bits_knn>("bits-prefetch"));
    algorithms.push_back(std::make_unique<bits_sq_knn>());
    algorithms.push_back(std::make_unique<fused_knn>("fused-cache"));
    algorithms.push_back(std::make_unique<fused_knn>("bits-fused"));
    algorithms.push_back(std::make_unique<fused_knn>("bits-fused-tf32", BITSKNN_L2_TF32));
    algorithms.push_back(std::make_unique<fused_knn>("bits-fused-bf16", BITSKNN_L2_BF16));
    algorithms.push_back(std::make_unique<sharded_knn>("bits-sharded", BITSKNN_L2_EXACT));
    algorithms.push_back(std::make_unique<sharded_knn>("bits-sharded-bf16", BITSKNN_L2_BF16));
    algorithms.push_back(std::make_unique<dist_runner>(BITSKNN_L2_EXACT, "magma-dist"));
    algorithms.push_back(std::make_unique<dist_runner>(BITSKNN_L2_PARTIAL, "magma-part-dist"));
    algorithms.push_back(std::make_unique<dist_runner>(BITSKNN_L2_TF32, "tc-dist-tf32"));
    algorithms.push_back(std::make_unique<dist_runner>(BITSKNN_L2_BF16, "tc-dist-bf16"));
    return algorithms;
}

} // namespace bits
