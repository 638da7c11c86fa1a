// Prefill GEMM (placeholder while the tcgen05 kernel is brought up).
#include "fk_common.cuh"

FK_EXPORT int fk_gemm(fk_ctx* ctx, void* stream, fk_weight w, int mat, const float* x_dev, int m, float* out_dev) {
    (void)ctx; (void)stream; (void)w; (void)mat; (void)x_dev; (void)m; (void)out_dev;
    return fk_fail(FK_UNSUPPORTED, "gemm: not built yet");
}
FK_EXPORT int fk_gemm_grouped(fk_ctx* ctx, void* stream, fk_weight w, const int* group_off_dev, const int* gather_dev,
                              const float* x_dev, int pairs, float* out_dev) {
    (void)ctx; (void)stream; (void)w; (void)group_off_dev; (void)gather_dev; (void)x_dev; (void)pairs; (void)out_dev;
    return fk_fail(FK_UNSUPPORTED, "gemm_grouped: not built yet");
}
