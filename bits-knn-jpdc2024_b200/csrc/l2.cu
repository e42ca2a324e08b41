#include "common.cuh"
using namespace bitsknn;
extern "C" size_t bitsknn_l2_workspace_bytes(int64_t, int64_t, int, int) { return 0; }
extern "C" int bitsknn_l2(const float*, const float*, int64_t, int64_t, int, int, float*, int64_t, void*, size_t,
                          bitsknn_stream_t)
{
    return fail(BITSKNN_ERR_UNSUPPORTED_MODE, "distance kernel not built yet");
}
