/* Elementwise test entry points next to the fused CE (names and signatures of the reference's
 * src/kernels/elementwise/capi_ew.h:22,29-30,36). Conventions as in capi.h. */
#ifndef MARINCPP_CAPI_EW_H
#define MARINCPP_CAPI_EW_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

int64_t nm_norm_partial_rows(int64_t T);
/* out[col] (+)= fixed-order sum over n_blocks partial rows [n_blocks, width]; round_bf16 rounds the reduced value */
int nm_reduce_partials_rows(const float* partial, int n_blocks, int width, float* out, int accumulate, int round_bf16,
                            void* stream);
/* out[0] = sum(x[0..n)) in a fixed order (the trainer sums the CE's loss_partial slots with it) */
int nm_sum_fixed(const float* x, int64_t n, float* out, void* stream);
/* raw partials of the RMSNorm backward ([nm_norm_partial_rows(T), D] f32) */
int nm_rmsnorm_bwd_add_partial(int dtype, int rounding, const void* dy, const void* x, const void* gain,
                               const float* rstd, const void* dres, void* dx, float* dgain_partial, int64_t T, int D,
                               float eps, void* stream);

#ifdef __cplusplus
}
#endif
#endif
