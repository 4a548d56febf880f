/* ref_shim_quant.c -- exports the reference's int4 row quantiser
 * (c/tools/kernel_check.c:27-35) and group-scaled int4 GEMM (c/quant.h:167-202)
 * by #including the unmodified reference sources in place.  TEST
 * INFRASTRUCTURE ONLY; see ref_shim.c. */
#define main kernel_check_main_unused
#include "tools/kernel_check.c"
#undef main
#include "quant.h"

#define REF_API __attribute__((visibility("default")))

REF_API void ref_quant_rows_i4(const float *w, int rows, int I, uint8_t *packed, float *scale) {
    for (int r = 0; r < rows; r++)
        quant_row_i4(w + (int64_t)r * I, I, packed + (int64_t)r * (I / 2), scale + r);
}
REF_API void ref_matmul_i4_grouped(float *y, const float *x, const uint8_t *q4, const float *scale,
                                   int S, int I, int O, int gs) {
    matmul_i4_grouped(y, x, q4, scale, S, I, O, gs);
}
