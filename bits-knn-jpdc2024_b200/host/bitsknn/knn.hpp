// Host-side plug-in interface of the k-NN engine: the same algorithm-object API as the
// reference (`class knn` with the phases initialize / prepare / distances / selection /
// postprocessing / finish, include/bits/knn.hpp:19-129; `cuda_knn`, include/bits/cuda_knn.hpp:15-56;
// `cuda_distance`, include/bits/distance/cuda_distance.hpp:12-70; `knn_args`,
// include/bits/knn_args.hpp:9-37), so that code written against the reference's registry can
// drive these objects unchanged.  All device work goes through the C ABI of bitsknn.h.
#ifndef BITSKNN_HOST_KNN_HPP_
#define BITSKNN_HOST_KNN_HPP_

#include <array>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include <cuda_runtime_api.h>

#include "bitsknn.h"

namespace bits
{

enum class matrix_layout
{
    row_major,
    column_major
};

// (distance, index) pair of a result, 8 bytes, as the reference returns from finish()
struct distance_pair
{
    float distance;
    std::int32_t index;
};

struct knn_args
{
    const float* points;  // host, point_count x dim (row major) or dim x point_count
    const float* queries; // host, query_count x dim (row major) or dim x query_count
    std::size_t point_count;
    std::size_t query_count;
    std::size_t dim;
    matrix_layout points_layout;
    matrix_layout queries_layout;
    matrix_layout dist_layout;
    std::size_t dist_block_size;
    std::size_t selection_block_size;
    std::size_t k;
    std::array<std::size_t, 3> items_per_thread;
    std::size_t deg;
};

// Throws the reference's "CUDA error." after printing where it happened (include/bits/cuch.hpp:11-19).
void cuda_check(cudaError_t status, const char* what, const char* file, int line);
#define BITS_CUCH(expr) ::bits::cuda_check((expr), #expr, __FILE__, __LINE__)

// Throws std::runtime_error with the library's message for a non-zero C-ABI status; the texts
// match the reference's ("Unsupported k value: ...", "CUDA error.").
void abi_check(int status);

// Owning device allocation (cudaFree in the destructor), movable, not copyable.
template <class T>
class device_buffer
{
public:
    device_buffer() = default;
    explicit device_buffer(std::size_t count) : count_(count)
    {
        if (count_ > 0)
        {
            BITS_CUCH(cudaMalloc(reinterpret_cast<void**>(&ptr_), count_ * sizeof(T)));
        }
    }
    device_buffer(const device_buffer&) = delete;
    device_buffer& operator=(const device_buffer&) = delete;
    device_buffer(device_buffer&& other) noexcept : ptr_(other.ptr_), count_(other.count_)
    {
        other.ptr_ = nullptr;
        other.count_ = 0;
    }
    device_buffer& operator=(device_buffer&& other) noexcept
    {
        if (this != &other)
        {
            release();
            ptr_ = other.ptr_;
            count_ = other.count_;
            other.ptr_ = nullptr;
            other.count_ = 0;
        }
        return *this;
    }
    ~device_buffer() { release(); }

    void release() noexcept
    {
        if (ptr_ != nullptr)
        {
            cudaFree(ptr_);
            ptr_ = nullptr;
            count_ = 0;
        }
    }
    T* data() const { return ptr_; }
    std::size_t size() const { return count_; }

private:
    T* ptr_ = nullptr;
    std::size_t count_ = 0;
};

// Pair of CUDA events that times one transfer (role of the reference's cuda_event members).
class transfer_timer
{
public:
    transfer_timer();
    transfer_timer(const transfer_timer&) = delete;
    transfer_timer& operator=(const transfer_timer&) = delete;
    ~transfer_timer();
    // records on `stream`; end() waits for the region unless `wait` is false (then seconds() does)
    void begin(cudaStream_t stream = nullptr);
    void end(cudaStream_t stream = nullptr, bool wait = true);
    float seconds() const;

private:
    cudaEvent_t begin_ = nullptr;
    cudaEvent_t end_ = nullptr;
    bool measured_ = false;
};

// Distance plug-in: owns the device copies of the inputs and the q x n matrix.
class cuda_distance
{
public:
    virtual ~cuda_distance();
    cuda_distance() = default;
    cuda_distance(const cuda_distance&) = delete;
    cuda_distance& operator=(const cuda_distance&) = delete;

    // Allocates device memory and uploads the inputs (timed).  The points travel in pieces on a
    // copy stream of their own; a column-major host matrix is uploaded as it is and transposed on
    // the device.  With page-locked host memory prepare() returns while copies are still in
    // flight: compute() then starts on each piece as it arrives, and every other reader calls
    // wait_inputs() first.  (The reference transposes on the host and uploads with two blocking
    // copies, src/distance/magma_distance.cu:32-70.)
    virtual void prepare(const knn_args& args);
    // Makes the legacy default stream wait for the uploads of prepare().
    void wait_inputs();
    virtual void compute() = 0;
    virtual float transfer_seconds() const { return timer_.seconds(); }
    // Row-major q x n matrix on the device / downloaded to the host.
    virtual float* matrix_gpu() const { return dist_gpu_.data(); }
    virtual const std::vector<float>& matrix_cpu();
    virtual std::string name() const = 0;

    const float* points_gpu() const { return points_gpu_.data(); }
    const float* queries_gpu() const { return queries_gpu_.data(); }

protected:
    struct piece
    {
        std::size_t begin; // first point of the piece
        std::size_t end;
        cudaEvent_t arrived;
    };
    void release_pieces();

    std::vector<piece> pieces_;   // upload pieces of the points, in order
    bool pieces_fresh_ = false;   // prepare() ran and no compute() has consumed the pieces yet
    cudaStream_t copy_stream_ = nullptr;
    device_buffer<float> staging_; // column-major inputs before their device transpose
    knn_args args_{};
    device_buffer<float> points_gpu_;  // always point_count x dim row major on the device
    device_buffer<float> queries_gpu_; // always query_count x dim row major on the device
    device_buffer<float> dist_gpu_;
    std::vector<float> dist_cpu_;
    transfer_timer timer_;
    bool needs_matrix_ = true;
};

// GEMM-form distance on the device (ids magma-dist / magma-part-dist / tc-dist-*).
class gemm_distance : public cuda_distance
{
public:
    explicit gemm_distance(int mode, std::string name) : mode_(mode), name_(std::move(name)) {}
    void compute() override;
    std::string name() const override { return name_; }

private:
    int mode_;
    std::string name_;
    device_buffer<unsigned char> workspace_;
};

// Keeps the inputs on the device but computes no matrix (for fused algorithms).
class no_distance : public cuda_distance
{
public:
    no_distance() { needs_matrix_ = false; }
    void compute() override {}
    std::string name() const override { return "none"; }
};

class knn
{
public:
    using pair_t = distance_pair;
    knn() = default;
    knn(const knn&) = delete;
    knn& operator=(const knn&) = delete;
    virtual ~knn() = default;

    virtual void initialize(const knn_args& args);
    virtual std::string id() const = 0;
    virtual void prepare() {}
    virtual void distances();
    virtual void selection() {}
    virtual void postprocessing() {}
    virtual std::vector<distance_pair> finish() { return {}; }
    virtual float transfer_in_seconds() const { return 0; }
    virtual float transfer_out_seconds() const { return 0; }
    virtual void set_dist_impl(std::unique_ptr<cuda_distance>&& impl) { dist_impl_ = std::move(impl); }

    std::size_t dim() const { return args_.dim; }
    std::size_t k() const { return args_.k; }
    std::size_t point_count() const { return args_.point_count; }
    std::size_t query_count() const { return args_.query_count; }
    std::size_t selection_block_size() const { return args_.selection_block_size; }
    void no_output() { no_output_ = true; }

protected:
    virtual std::unique_ptr<cuda_distance> default_distance() const;

    bool no_output_ = false;
    knn_args args_{};
    std::unique_ptr<cuda_distance> dist_impl_;
};

// Base of the device algorithms: owns the q x k outputs, downloads them in finish().
class cuda_knn : public knn
{
public:
    void initialize(const knn_args& args) override;
    std::vector<distance_pair> finish() override;
    float transfer_in_seconds() const override { return dist_impl_->transfer_seconds(); }
    float transfer_out_seconds() const override { return out_timer_.seconds(); }

protected:
    float* in_dist_gpu() const { return dist_impl_->matrix_gpu(); }
    float* out_dist_gpu() const { return out_dist_gpu_.data(); }
    std::int32_t* out_label_gpu() const { return out_label_gpu_.data(); }

private:
    device_buffer<float> out_dist_gpu_;
    device_buffer<std::int32_t> out_label_gpu_;
    transfer_timer out_timer_;
};

// `bits` / `bits-prefetch`: selection over the distance matrix (one kernel for both ids; the
// bulk-copy ring replaces the reference's optional L2 prefetch).
class bits_knn : public cuda_knn
{
public:
    explicit bits_knn(std::string id = "bits") : id_(std::move(id)) {}
    std::string id() const override { return id_; }
    void initialize(const knn_args& args) override;
    void selection() override;

private:
    std::string id_;
    int splits_ = 1;                         // slices per row chosen by the library for this shape
    device_buffer<unsigned char> workspace_; // candidates of the slices (only when splits_ > 1)
};

// `partial-bitonic-regs` (the selection kernel without its radius filter: every value is sorted
// and merged) and `partial-bitonic-buffered-static` (filtered buffer, but list and networks in
// shared memory).  Kept, like in the reference (partial_bitonic.cu:217-294,
// partial_bitonic_buffered.cu:216-337), to show what the buffer and the register list buy.
class ablation_knn : public cuda_knn
{
public:
    ablation_knn(std::string id, int variant) : id_(std::move(id)), variant_(variant) {}
    std::string id() const override { return id_; }
    void selection() override;

private:
    std::string id_;
    int variant_;
};

// `bits-sq`: rows cut into `deg` slices, then merged (reference: single_query_bits).
class bits_sq_knn : public cuda_knn
{
public:
    std::string id() const override { return "bits-sq"; }
    void initialize(const knn_args& args) override;
    void selection() override;

private:
    device_buffer<unsigned char> workspace_;
};

// `fused-cache` (alias `bits-fused`): distances and selection in one kernel, no matrix.
class fused_knn : public cuda_knn
{
public:
    explicit fused_knn(std::string id = "fused-cache", int mode = BITSKNN_L2_PARTIAL) : id_(std::move(id)), mode_(mode) {}
    std::string id() const override { return id_; }
    void initialize(const knn_args& args) override;
    void distances() override {}
    void selection() override;

protected:
    std::unique_ptr<cuda_distance> default_distance() const override { return std::make_unique<no_distance>(); }

private:
    std::string id_;
    int mode_;
    device_buffer<unsigned char> workspace_; // tensor-core modes only
};

// `bits-sharded`: the database cut into contiguous shards over the visible GPUs (`--deg G` limits
// their number), one host thread and one stream per GPU; every shard runs the fused search of its
// points with global indices, the library all-gathers the candidates (NCCL) and merges them.  The
// reference is single-GPU; the closest thing it has is `bits-sq`, which cuts rows into slices
// and merges their candidates (src/topk/singlepass/bits_knn.cu:116-186).
class sharded_knn : public knn
{
public:
    explicit sharded_knn(std::string id = "bits-sharded", int mode = BITSKNN_L2_EXACT) : id_(std::move(id)), mode_(mode) {}
    ~sharded_knn() override;
    std::string id() const override { return id_; }
    void initialize(const knn_args& args) override;
    void distances() override {}
    void selection() override;
    std::vector<distance_pair> finish() override;
    float transfer_in_seconds() const override;
    float transfer_out_seconds() const override { return out_timer_.seconds(); }
    std::size_t shard_count() const { return shards_.size(); }

private:
    struct shard
    {
        int device = 0;
        std::size_t begin = 0; // first point of the shard
        std::size_t count = 0;
        bitsknn_sharded_t* handle = nullptr;
        device_buffer<float> points;
        device_buffer<float> queries;
        device_buffer<float> out_dist;
        device_buffer<std::int32_t> out_label;
        device_buffer<unsigned char> fused_ws;
        device_buffer<unsigned char> exchange_ws;
        float transfer_seconds = 0;
    };
    std::string id_;
    int mode_;
    std::vector<shard> shards_;
    transfer_timer out_timer_;
};

// Distance-only registry entries (reference: dist_runner<D>, include/bits/distance/dist_runner.hpp:8-15).
class dist_runner : public knn
{
public:
    dist_runner(int mode, std::string id) : mode_(mode), id_(std::move(id)) {}
    std::string id() const override { return id_; }
    float transfer_in_seconds() const override { return dist_impl_->transfer_seconds(); }

protected:
    std::unique_ptr<cuda_distance> default_distance() const override
    {
        return std::make_unique<gemm_distance>(mode_, id_);
    }

private:
    int mode_;
    std::string id_;
};

// CPU comparators of the registry, selected explicitly with `-a serial|parallel` or
// `--verify`: full sort of every row / OpenMP heap (reference: src/topk/serial_knn.cpp:9-54,
// src/topk/parallel_knn.cpp:12-67).  They read the matrix the distance plug-in computed on
// the device, exactly like the reference's `serial`.  Pairs are ordered by (distance, index).
class serial_knn : public knn
{
public:
    std::string id() const override { return "serial"; }
    void distances() override;
    void selection() override;
    std::vector<distance_pair> finish() override;
    float transfer_in_seconds() const override { return dist_impl_->transfer_seconds(); }

private:
    std::vector<distance_pair> dist_;
};

class parallel_knn : public knn
{
public:
    std::string id() const override { return "parallel"; }
    void distances() override;
    void selection() override;
    std::vector<distance_pair> finish() override { return result_; }
    float transfer_in_seconds() const override { return dist_impl_->transfer_seconds(); }

private:
    const std::vector<float>* matrix_ = nullptr;
    std::vector<distance_pair> result_;
};

// Tolerant comparison of two results (reference: src/verify.cpp:78-112); prints differences
// to stderr like the reference and returns true when they agree.
bool verify(const std::vector<distance_pair>& expected, const std::vector<distance_pair>& actual, std::size_t k);

// All registered algorithms, in the reference's registration order where they exist there.
std::vector<std::unique_ptr<knn>> make_registry();

} // namespace bits

#endif // BITSKNN_HOST_KNN_HPP_
