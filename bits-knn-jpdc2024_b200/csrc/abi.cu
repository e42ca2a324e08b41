// Error reporting, tuning registry and the device status word shared by every entry point.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>

#include "common.cuh"
#include "ptx.cuh"

namespace bitsknn
{

namespace
{

thread_local std::string g_last_error;

__device__ int g_device_status = 0;

struct tuning_entry
{
    const char* key;
    int value;
    int min;
    int max;
};

std::mutex g_tuning_mutex;
tuning_entry g_tuning[] = {
    {"select.stage_bytes", 0, 0, 65536},
    {"select.stages", 0, 0, 8},
    {"select.merge_at", 0, 0, 190},
    {"select.unroll", 0, 0, 4},
    {"select.threads", 0, 0, 1024},
    {"select.ipt", 0, 0, 4},
    {"fused.variant", 2, 0, 2},
    {"fused.tc_mma_n", 0, 0, 256},
    {"fused.parts", 0, 0, 64},
    {"fused.tc_cap", 0, 0, 32},
    {"fused.tc_fold_above", 0, 0, 31},
    {"fused.tc_tf32_plain", 0, 0, 2},
    {"profile.kernel_events", 0, 0, 1},
};

// kernel timing slots: one pair of events per kernel name (names are string literals)
struct timing_slot
{
    const char* name;
    cudaEvent_t begin;
    cudaEvent_t end;
    bool recorded;
};
constexpr int MAX_TIMING_SLOTS = 16;
std::mutex g_timing_mutex;
timing_slot g_timing[MAX_TIMING_SLOTS] = {};
int g_timing_count = 0;

timing_slot* timing_slot_of(const char* name, bool create)
{
    std::lock_guard<std::mutex> lock{g_timing_mutex};
    for (int i = 0; i < g_timing_count; ++i)
    {
        if (std::strcmp(g_timing[i].name, name) == 0)
        {
            return &g_timing[i];
        }
    }
    if (!create || g_timing_count == MAX_TIMING_SLOTS)
    {
        return nullptr;
    }
    timing_slot& slot = g_timing[g_timing_count];
    if (cudaEventCreate(&slot.begin) != cudaSuccess || cudaEventCreate(&slot.end) != cudaSuccess)
    {
        return nullptr;
    }
    slot.name = name;
    slot.recorded = false;
    ++g_timing_count;
    return &slot;
}

} // namespace

int fail(int code, const char* fmt, ...)
{
    char buffer[512];
    va_list args;
    va_start(args, fmt);
    vsnprintf(buffer, sizeof(buffer), fmt, args);
    va_end(args);
    g_last_error = buffer;
    return code;
}

int cuda_fail(cudaError_t err, const char* what, const char* file, int line)
{
    // same information the reference prints before throwing "CUDA error."
    // (include/bits/cuch.hpp:11-19): file:line, error name and message, the failing call
    return fail(BITSKNN_ERR_CUDA, "CUDA error. %s:%d %s: %s\n\t%s", file, line, cudaGetErrorName(err),
                cudaGetErrorString(err), what);
}

int* device_status_word()
{
    int* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_device_status) != cudaSuccess)
    {
        return nullptr;
    }
    return ptr;
}

kernel_scope::kernel_scope(const char* name, cudaStream_t stream) : slot_(nullptr), stream_(stream)
{
    if (tuning_value("profile.kernel_events", 0) != 0)
    {
        timing_slot* slot = timing_slot_of(name, true);
        if (slot != nullptr && cudaEventRecord(slot->begin, stream) == cudaSuccess)
        {
            slot_ = slot;
        }
    }
}

kernel_scope::~kernel_scope()
{
    if (slot_ != nullptr)
    {
        auto* slot = static_cast<timing_slot*>(slot_);
        slot->recorded = cudaEventRecord(slot->end, stream_) == cudaSuccess;
    }
}

int tuning_value(const char* key, int fallback)
{
    std::lock_guard<std::mutex> lock{g_tuning_mutex};
    for (const auto& entry : g_tuning)
    {
        if (std::strcmp(entry.key, key) == 0)
        {
            return entry.value;
        }
    }
    return fallback;
}

int balanced_parts(int64_t query_tiles, int slots, int64_t max_parts)
{
    int64_t best = 1;
    double best_eff = 0.0;
    for (int64_t parts = 1; parts <= std::max<int64_t>(max_parts, 1); ++parts)
    {
        const int64_t blocks = query_tiles * parts;
        const int64_t waves = (blocks + slots - 1) / slots;
        const double eff = static_cast<double>(blocks) / static_cast<double>(waves * slots);
        if (eff > best_eff + 0.02)
        {
            best_eff = eff;
            best = parts;
        }
    }
    return static_cast<int>(best);
}

int device_sm_count()
{
    int device = 0;
    int sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
    {
        return 148;
    }
    return sms;
}

} // namespace bitsknn

namespace bitsknn
{

namespace
{

// Waits, with a small poll limit, on a barrier phase that nothing will ever complete, and reports
// the expiry exactly like the production kernels do: status bit, normal return.
__global__ void selftest_wait_kernel(int* status, uint32_t limit)
{
    __shared__ uint64_t bar;
    if (threadIdx.x == 0)
    {
        ptx::mbar_init(&bar, 1);
        ptx::mbar_init_fence();
    }
    __syncthreads();
    if (!ptx::mbar_wait_bounded(&bar, 0, limit) && threadIdx.x == 0)
    {
        atomicOr(status, DEVICE_STATUS_TIMEOUT);
    }
}

} // namespace

} // namespace bitsknn

extern "C" int bitsknn_selftest_bounded_wait(bitsknn_stream_t stream)
{
    using namespace bitsknn;
    int* word = device_status_word();
    if (word == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cannot resolve the device status word");
    }
    selftest_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(word, 1024U);
    BITSKNN_CUDA_TRY(cudaGetLastError());
    return BITSKNN_OK;
}

extern "C" int bitsknn_version(void) { return 100; }

extern "C" const char* bitsknn_last_error_string(void) { return bitsknn::g_last_error.c_str(); }

extern "C" int bitsknn_device_status(bitsknn_stream_t stream)
{
    using namespace bitsknn;
    int* word = device_status_word();
    if (word == nullptr)
    {
        return fail(BITSKNN_ERR_CUDA, "CUDA error. cannot resolve the device status word");
    }
    int value = 0;
    auto s = static_cast<cudaStream_t>(stream);
    BITSKNN_CUDA_TRY(cudaMemcpyAsync(&value, word, sizeof(int), cudaMemcpyDeviceToHost, s));
    BITSKNN_CUDA_TRY(cudaStreamSynchronize(s));
    if (value != 0)
    {
        BITSKNN_CUDA_TRY(cudaMemsetAsync(word, 0, sizeof(int), s));
        BITSKNN_CUDA_TRY(cudaStreamSynchronize(s));
        return fail(BITSKNN_ERR_DEVICE_TIMEOUT, "a kernel gave up a bounded wait (status word 0x%x)", value);
    }
    return BITSKNN_OK;
}

extern "C" int bitsknn_set_tuning(const char* key, int value)
{
    using namespace bitsknn;
    if (key == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "tuning key is null");
    }
    std::lock_guard<std::mutex> lock{g_tuning_mutex};
    for (auto& entry : g_tuning)
    {
        if (std::strcmp(entry.key, key) == 0)
        {
            if (value < entry.min || value > entry.max)
            {
                return fail(BITSKNN_ERR_INVALID_ARGUMENT, "tuning value %d for '%s' outside [%d, %d]", value, key,
                            entry.min, entry.max);
            }
            if (std::strcmp(key, "select.unroll") == 0 && value != 0 && value != 2 && value != 4)
            {
                return fail(BITSKNN_ERR_INVALID_ARGUMENT, "tuning value %d for 'select.unroll': only 0, 2 and 4 exist",
                            value);
            }
            entry.value = value;
            return BITSKNN_OK;
        }
    }
    return fail(BITSKNN_ERR_INVALID_ARGUMENT, "unknown tuning key '%s'", key);
}

extern "C" int bitsknn_kernel_ms(const char* kernel, float* ms)
{
    using namespace bitsknn;
    if (kernel == nullptr || ms == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "null pointer argument");
    }
    timing_slot* slot = timing_slot_of(kernel, false);
    if (slot == nullptr || !slot->recorded)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "no timed launch of '%s' (set \"profile.kernel_events\" to 1 first)",
                    kernel);
    }
    BITSKNN_CUDA_TRY(cudaEventSynchronize(slot->end));
    BITSKNN_CUDA_TRY(cudaEventElapsedTime(ms, slot->begin, slot->end));
    return BITSKNN_OK;
}

extern "C" const char* bitsknn_tuning_key(int index)
{
    using namespace bitsknn;
    constexpr int count = static_cast<int>(sizeof(g_tuning) / sizeof(g_tuning[0]));
    return index >= 0 && index < count ? g_tuning[index].key : nullptr;
}

extern "C" int bitsknn_get_tuning(const char* key, int* value)
{
    using namespace bitsknn;
    if (key == nullptr || value == nullptr)
    {
        return fail(BITSKNN_ERR_INVALID_ARGUMENT, "tuning key or output is null");
    }
    std::lock_guard<std::mutex> lock{g_tuning_mutex};
    for (const auto& entry : g_tuning)
    {
        if (std::strcmp(entry.key, key) == 0)
        {
            *value = entry.value;
            return BITSKNN_OK;
        }
    }
    return fail(BITSKNN_ERR_INVALID_ARGUMENT, "unknown tuning key '%s'", key);
}
