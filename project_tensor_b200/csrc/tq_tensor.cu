// placeholder while the exact path is brought up
#include "tq_common.cuh"
bool tq_tensor_supported(int, int) { return false; }
int tq_tensor_plan_init(tq_plan*, const float*, const float*, const float*) { return TQ_OK; }
void tq_tensor_plan_free(tq_plan*) {}
int tq_launch_tensor_quantize(const tq_plan*, bool, const float*, int64_t, uint32_t*, uint32_t*, float*, float*, uint32_t*, cudaStream_t) {
    return tq_fail(TQ_ERR_UNSUPPORTED, "tensor path not built");
}
