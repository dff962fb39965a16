// FastExperts placeholder (replaced by the tcgen05 grouped GEMM).
#include "common.cuh"
struct glmflash_fast_experts { int unused; };
extern "C" int glmflash_fast_experts_new(const glmflash_config *, size_t, glmflash_fast_experts **out) {
    if (out) *out = nullptr;
    return gf::fail("fast experts: not built yet");
}
extern "C" void glmflash_fast_experts_free(glmflash_fast_experts *) {}
extern "C" int glmflash_fast_experts_run(glmflash_fast_experts *, void *, const glmflash_weights *, const void *, int,
                                         const int32_t *, const int32_t *, const int32_t *, const int32_t *, int, int, int) {
    return gf::fail("fast experts: not built yet");
}
extern "C" float *glmflash_fast_experts_output(const glmflash_fast_experts *) { return nullptr; }
extern "C" const uint16_t *glmflash_fast_experts_xd(const glmflash_fast_experts *) { return nullptr; }
