#include "common.cuh"
namespace bitsknn
{
size_t l2_tc_workspace_bytes(int64_t, int64_t, int, int) { return 0; }
int l2_tc_launch(const float*, const float*, int64_t, int64_t, int, int, float*, int64_t, void*, size_t, cudaStream_t)
{
    return fail(BITSKNN_ERR_UNSUPPORTED_MODE, "tensor-core distance modes are not built yet");
}
} // namespace bitsknn
