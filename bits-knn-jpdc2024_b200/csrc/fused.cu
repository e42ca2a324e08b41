#include "common.cuh"
using namespace bitsknn;
extern "C" int bitsknn_fused(const float*, const float*, int64_t, int64_t, int, int, int, int32_t, float*, int32_t*,
                             bitsknn_stream_t)
{
    return fail(BITSKNN_ERR_UNSUPPORTED_MODE, "fused kernel not built yet");
}
