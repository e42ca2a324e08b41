// Database-sharded search: every GPU holds a contiguous shard of the database and all queries.
//
// A search is the local top-k of the shard with global labels (label base / index base = the
// shard's first global index -- the mechanism the reference uses for row slices,
// src/topk/singlepass/bits_knn.cu:67-76), one NCCL all-gather of the q x k candidate pairs of
// every shard (packed as [2][q][k] 32-bit words: distances, then labels) and the merge kernel over
// the `world` sorted lists of each query.  The reference is single-GPU; its split-row two-pass
// scheme (bits_knn.cu:116-186) is the template.
//
// Streams: the local kernel runs on the caller's stream; the exchange and the merge run on a
// stream owned by the handle, ordered by events.  The `submit` form returns as soon as those are
// queued, so the all-gather and merge of search i overlap the local kernel of search i + 1 (two
// buffer slots); `drain` makes the caller's stream wait for everything submitted.  No kernel of
// this library waits on a peer: the only inter-GPU dependency is inside NCCL.
//
// NCCL is bound at run time (dlopen of libnccl.so.2: the copy already loaded in the process, e.g.
// by a framework, else the system's), so the library itself loads where NCCL is absent and only
// the multi-GPU entry points need it.
#include <dlfcn.h>

#include <cstdint>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace bitsknn
{

namespace
{

// the few NCCL declarations used here (stable since NCCL 2.0)
using nccl_comm_t = void*;
struct nccl_unique_id
{
    char internal[BITSKNN_SHARDED_ID_BYTES];
};
constexpr int NCCL_FLOAT32 = 7;
using get_unique_id_fn = int (*)(nccl_unique_id*);
using comm_init_rank_fn = int (*)(nccl_comm_t*, int, nccl_unique_id, int);
using comm_destroy_fn = int (*)(nccl_comm_t);
using all_gather_fn = int (*)(const void*, void*, size_t, int, nccl_comm_t, cudaStream_t);
using error_string_fn = const char* (*)(int);

struct nccl_api
{
    get_unique_id_fn get_unique_id = nullptr;
    comm_init_rank_fn comm_init_rank = nullptr;
    comm_destroy_fn comm_destroy = nullptr;
    all_gather_fn all_gather = nullptr;
    error_string_fn error_string = nullptr;
    bool ok = false;
};

const nccl_api& nccl()
{
    static nccl_api api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
        if (handle == nullptr)
        {
            handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        }
        if (handle == nullptr)
        {
            handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        }
        if (handle == nullptr)
        {
            return;
        }
        api.get_unique_id = reinterpret_cast<get_unique_id_fn>(dlsym(handle, "ncclGetUniqueId"));
        api.comm_init_rank = reinterpret_cast<comm_init_rank_fn>(dlsym(handle, "ncclCommInitRank"));
        api.comm_destroy = reinterpret_cast<comm_destroy_fn>(dlsym(handle, "ncclCommDestroy"));
        api.all_gather = reinterpret_cast<all_gather_fn>(dlsym(handle, "ncclAllGather"));
        api.error_string = reinterpret_cast<error_string_fn>(dlsym(handle, "ncclGetErrorString"));
        api.ok = api.get_unique_id != nullptr && api.comm_init_rank != nullptr && api.comm_destroy != nullptr &&
                 api.all_gather != nullptr && api.error_string != nullptr;
    });
    return api;
}

int nccl_missing()
{
    const char* why = dlerror();
    return fail(BITSKNN_ERR_COMM, "NCCL error. libnccl.so.2 cannot be loaded: %s", why != nullptr ? why : "not found");
}

int nccl_fail(int rc, const char* what)
{
    return fail(BITSKNN_ERR_COMM, "NCCL error. %s: %s", what, nccl().error_string(rc));
}

#define BITSKNN_NCCL_TRY(expr)                                                                     \
    do                                                                                             \
    {                                                                                              \
        const int bitsknn_nccl_rc_ = (expr);                                                       \
        if (bitsknn_nccl_rc_ != 0)                                                                 \
        {                                                                                          \
            return nccl_fail(bitsknn_nccl_rc_, #expr);                                             \
        }                                                                                          \
    } while (0)

constexpr int SLOTS = 2;

} // namespace

} // namespace bitsknn

// One rank of a sharded search.
struct bitsknn_sharded
{
    void* comm = nullptr;
    bool own_comm = false;
    int rank = 0;
    int world = 1;
    int device = 0;
    cudaStream_t side = nullptr;           // exchange + merge
    cudaEvent_t local_done[2] = {};        // the local kernel of the slot's search has finished
    cudaEvent_t search_done[2] = {};       // ... and its merge
    bool slot_used[2] = {false, false};
    uint64_t submitted = 0;
};

namespace bitsknn
{

namespace
{

int make_handle(bitsknn_sharded** out, void* comm, bool own, int rank, int world)
{
    auto* h = new (std::nothrow) bitsknn_sharded{};
    if (h == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "out of host memory");
    }
    h->comm = comm;
    h->own_comm = own;
    h->rank = rank;
    h->world = world;
    cudaError_t err = cudaGetDevice(&h->device);
    if (err == cudaSuccess)
    {
        // lowest priority: the exchange and merge of one search run beside the next search's kernels
        // and should only take the SMs those leave free
        int least = 0;
        int greatest = 0;
        err = cudaDeviceGetStreamPriorityRange(&least, &greatest);
        if (err == cudaSuccess)
        {
            err = cudaStreamCreateWithPriority(&h->side, cudaStreamNonBlocking, least);
        }
    }
    for (int s = 0; s < SLOTS && err == cudaSuccess; ++s)
    {
        err = cudaEventCreateWithFlags(&h->local_done[s], cudaEventDisableTiming);
        if (err == cudaSuccess)
        {
            err = cudaEventCreateWithFlags(&h->search_done[s], cudaEventDisableTiming);
        }
    }
    if (err != cudaSuccess)
    {
        const int rc = cuda_fail(err, "creating the stream and events of a sharded-search handle", __FILE__, __LINE__);
        bitsknn_sharded_destroy(h);
        return rc;
    }
    *out = h;
    return BITSKNN_OK;
}

int check_rank(int rank, int world)
{
    if (world < 1 || rank < 0 || rank >= world)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid rank %d of %d", rank, world);
    }
    return BITSKNN_OK;
}

struct slot_buffers
{
    float* local;    // [2][q][k]
    float* gathered; // [world][2][q][k]
};

size_t slot_words(int world, int64_t q, int k) { return static_cast<size_t>(1 + world) * 2U * q * k; }

slot_buffers slot_of(const bitsknn_sharded* h, void* ws, int slot, int64_t q, int k)
{
    float* base = static_cast<float*>(ws) + static_cast<size_t>(slot) * slot_words(h->world, q, k);
    return {base, base + 2U * static_cast<size_t>(q) * k};
}

int check_search(const bitsknn_sharded* h, int64_t q, int k, const void* out_d, const void* out_x, const void* ws,
                 size_t ws_bytes)
{
    if (h == nullptr || out_d == nullptr || out_x == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (q < 0 || k < 1)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "invalid sizes: q=%lld k=%d", static_cast<long long>(q), k);
    }
    if (h->world > 1)
    {
        const size_t need = bitsknn_sharded_workspace_bytes(h, q, k);
        if (ws == nullptr || ws_bytes < need || (reinterpret_cast<uintptr_t>(ws) & 15U) != 0)
        {
            return fail(BITSKNN_ERR_WORKSPACE, "exchange workspace of %zu bytes (16-byte aligned) needed, %zu given", need,
                        ws_bytes);
        }
        if (static_cast<int64_t>(h->world) * k > 65536)
        {
            return fail(BITSKNN_ERR_INVALID_ARGUMENT, "shards * k = %lld exceeds 65536",
                        static_cast<long long>(h->world) * k);
        }
    }
    return BITSKNN_OK;
}

// Where the local kernel of the next search writes: the caller's output (one shard) or the local
// plane of the next slot, once that slot's previous search no longer reads it.
int begin_search(bitsknn_sharded* h, void* ws, int64_t q, int k, float* out_d, int32_t* out_x, cudaStream_t stream,
                 int* slot, float** loc_d, int32_t** loc_x)
{
    if (h->world == 1)
    {
        *slot = 0;
        *loc_d = out_d;
        *loc_x = out_x;
        return BITSKNN_OK;
    }
    *slot = static_cast<int>(h->submitted & 1U);
    if (h->slot_used[*slot])
    {
        BITSKNN_CUDA_TRY(cudaStreamWaitEvent(stream, h->search_done[*slot], 0));
    }
    const slot_buffers b = slot_of(h, ws, *slot, q, k);
    *loc_d = b.local;
    *loc_x = reinterpret_cast<int32_t*>(b.local + static_cast<size_t>(q) * k);
    return BITSKNN_OK;
}

// Queues the all-gather and the merge of the slot behind the local kernel.
int finish_search(bitsknn_sharded* h, void* ws, int slot, int64_t q, int k, float* out_d, int32_t* out_x,
                  cudaStream_t stream, bool wait)
{
    if (h->world == 1 || q == 0)
    {
        return BITSKNN_OK;
    }
    const slot_buffers b = slot_of(h, ws, slot, q, k);
    const size_t words = 2U * static_cast<size_t>(q) * k;
    BITSKNN_CUDA_TRY(cudaEventRecord(h->local_done[slot], stream));
    BITSKNN_CUDA_TRY(cudaStreamWaitEvent(h->side, h->local_done[slot], 0));
    BITSKNN_NCCL_TRY(nccl().all_gather(b.local, b.gathered, words, NCCL_FLOAT32, h->comm, h->side));
    const int rc = merge_lists(b.gathered, reinterpret_cast<const int32_t*>(b.gathered) + static_cast<size_t>(q) * k,
                               static_cast<int64_t>(words), k, q, h->world, k, k, nullptr, out_d, out_x,
                               merge_input::sorted, h->side);
    if (rc != BITSKNN_OK)
    {
        return rc;
    }
    BITSKNN_CUDA_TRY(cudaEventRecord(h->search_done[slot], h->side));
    h->slot_used[slot] = true;
    ++h->submitted;
    if (wait)
    {
        BITSKNN_CUDA_TRY(cudaStreamWaitEvent(stream, h->search_done[slot], 0));
    }
    return BITSKNN_OK;
}

int search_select(bitsknn_sharded* h, const float* d_dist, int64_t ld, int64_t q, int64_t n_local, int k,
                  int32_t shard_begin, float* out_d, int32_t* out_x, void* ws, size_t ws_bytes, cudaStream_t stream,
                  bool wait)
{
    if (const int rc = check_search(h, q, k, out_d, out_x, ws, ws_bytes); rc != BITSKNN_OK)
    {
        return rc;
    }
    int slot = 0;
    float* loc_d = nullptr;
    int32_t* loc_x = nullptr;
    if (const int rc = begin_search(h, ws, q, k, out_d, out_x, stream, &slot, &loc_d, &loc_x); rc != BITSKNN_OK)
    {
        return rc;
    }
    if (const int rc = select_rows(d_dist, ld, nullptr, 0, nullptr, shard_begin, q, n_local, k, loc_d, loc_x, stream);
        rc != BITSKNN_OK)
    {
        return rc;
    }
    return finish_search(h, ws, slot, q, k, out_d, out_x, stream, wait);
}

int search_fused(bitsknn_sharded* h, const float* d_points, const float* d_queries, int64_t n_local, int64_t q, int dim,
                 int k, int mode, int32_t shard_begin, float* out_d, int32_t* out_x, void* fused_ws, size_t fused_ws_bytes,
                 void* ws, size_t ws_bytes, cudaStream_t stream, bool wait)
{
    if (const int rc = check_search(h, q, k, out_d, out_x, ws, ws_bytes); rc != BITSKNN_OK)
    {
        return rc;
    }
    int slot = 0;
    float* loc_d = nullptr;
    int32_t* loc_x = nullptr;
    if (const int rc = begin_search(h, ws, q, k, out_d, out_x, stream, &slot, &loc_d, &loc_x); rc != BITSKNN_OK)
    {
        return rc;
    }
    if (const int rc = bitsknn_fused(d_points, d_queries, n_local, q, dim, k, mode, shard_begin, loc_d, loc_x, fused_ws,
                                     fused_ws_bytes, stream);
        rc != BITSKNN_OK)
    {
        return rc;
    }
    return finish_search(h, ws, slot, q, k, out_d, out_x, stream, wait);
}

} // namespace

} // namespace bitsknn

using namespace bitsknn;

extern "C" int bitsknn_sharded_unique_id(void* id)
{
    if (id == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (!nccl().ok)
    {
        return nccl_missing();
    }
    nccl_unique_id uid{};
    BITSKNN_NCCL_TRY(nccl().get_unique_id(&uid));
    std::memcpy(id, uid.internal, BITSKNN_SHARDED_ID_BYTES);
    return BITSKNN_OK;
}

extern "C" int bitsknn_sharded_create(bitsknn_sharded** handle, const void* id, int rank, int world)
{
    if (handle == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (const int rc = check_rank(rank, world); rc != BITSKNN_OK)
    {
        return rc;
    }
    void* comm = nullptr;
    if (world > 1)
    {
        if (id == nullptr)
        {
            return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
        }
        if (!nccl().ok)
        {
            return nccl_missing();
        }
        nccl_unique_id uid{};
        std::memcpy(uid.internal, id, BITSKNN_SHARDED_ID_BYTES);
        BITSKNN_NCCL_TRY(nccl().comm_init_rank(&comm, world, uid, rank));
    }
    return make_handle(handle, comm, true, rank, world);
}

extern "C" int bitsknn_sharded_init(bitsknn_sharded** handle, void* nccl_comm, int rank, int world)
{
    if (handle == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    if (const int rc = check_rank(rank, world); rc != BITSKNN_OK)
    {
        return rc;
    }
    if (world > 1)
    {
        if (nccl_comm == nullptr)
        {
            return fail(BITSKNN_ERR_INVALID_ARGUMENT, "a communicator is needed for more than one shard");
        }
        if (!nccl().ok)
        {
            return nccl_missing();
        }
    }
    return make_handle(handle, nccl_comm, false, rank, world);
}

extern "C" int bitsknn_sharded_destroy(bitsknn_sharded* h)
{
    if (h == nullptr)
    {
        return BITSKNN_OK;
    }
    int rc = BITSKNN_OK;
    if (h->side != nullptr)
    {
        cudaStreamSynchronize(h->side);
    }
    if (h->own_comm && h->comm != nullptr && nccl().ok)
    {
        if (const int nrc = nccl().comm_destroy(h->comm); nrc != 0)
        {
            rc = nccl_fail(nrc, "ncclCommDestroy");
        }
    }
    for (int s = 0; s < SLOTS; ++s)
    {
        if (h->local_done[s] != nullptr)
        {
            cudaEventDestroy(h->local_done[s]);
        }
        if (h->search_done[s] != nullptr)
        {
            cudaEventDestroy(h->search_done[s]);
        }
    }
    if (h->side != nullptr)
    {
        cudaStreamDestroy(h->side);
    }
    delete h;
    return rc;
}

extern "C" size_t bitsknn_sharded_workspace_bytes(const bitsknn_sharded* h, int64_t q, int k)
{
    if (h == nullptr || q <= 0 || k <= 0 || h->world == 1)
    {
        return 0;
    }
    return static_cast<size_t>(SLOTS) * slot_words(h->world, q, k) * sizeof(float);
}

extern "C" int bitsknn_sharded_search_select(bitsknn_sharded* h, const float* d_dist, int64_t ld, int64_t q,
                                             int64_t n_local, int k, int32_t shard_begin, float* d_out_dist,
                                             int32_t* d_out_idx, void* d_workspace, size_t workspace_bytes,
                                             bitsknn_stream_t stream)
{
    return search_select(h, d_dist, ld, q, n_local, k, shard_begin, d_out_dist, d_out_idx, d_workspace, workspace_bytes,
                         static_cast<cudaStream_t>(stream), true);
}

extern "C" int bitsknn_sharded_submit_select(bitsknn_sharded* h, const float* d_dist, int64_t ld, int64_t q,
                                             int64_t n_local, int k, int32_t shard_begin, float* d_out_dist,
                                             int32_t* d_out_idx, void* d_workspace, size_t workspace_bytes,
                                             bitsknn_stream_t stream)
{
    return search_select(h, d_dist, ld, q, n_local, k, shard_begin, d_out_dist, d_out_idx, d_workspace, workspace_bytes,
                         static_cast<cudaStream_t>(stream), false);
}

extern "C" int bitsknn_sharded_search_fused(bitsknn_sharded* h, const float* d_points, const float* d_queries,
                                            int64_t n_local, int64_t q, int dim, int k, int mode, int32_t shard_begin,
                                            float* d_out_dist, int32_t* d_out_idx, void* d_fused_workspace,
                                            size_t fused_workspace_bytes, void* d_workspace, size_t workspace_bytes,
                                            bitsknn_stream_t stream)
{
    return search_fused(h, d_points, d_queries, n_local, q, dim, k, mode, shard_begin, d_out_dist, d_out_idx,
                        d_fused_workspace, fused_workspace_bytes, d_workspace, workspace_bytes,
                        static_cast<cudaStream_t>(stream), true);
}

extern "C" int bitsknn_sharded_drain(bitsknn_sharded* h, bitsknn_stream_t stream)
{
    if (h == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    for (int s = 0; s < SLOTS; ++s)
    {
        if (h->slot_used[s])
        {
            BITSKNN_CUDA_TRY(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), h->search_done[s], 0));
        }
    }
    return BITSKNN_OK;
}
