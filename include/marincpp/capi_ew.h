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

/* The sandwich tail backward with raw gain-gradient partials ([nm_norm_partial_rows(T), D] f32 each, nullptr: skipped),
 * as the trainer calls it with buffers of its memory plan; nm_sandwich_tail_bwd (capi.h) is the same kernel followed by
 * the fixed-order reduction of the partials. */
int nm_sandwich_tail_bwd_partial(int dtype, int rounding, const void* dx_out, const void* da_next, const void* x_out,
                                 const void* g_next, const float* rstd_next, const void* branch, const void* g_post,
                                 const float* rstd_post, void* dx_in, void* dbranch, float* pg_next, float* pg_post,
                                 int64_t T, int D, float eps, void* stream);
/* The norm backward kernels (nm_rmsnorm_bwd_add, nm_rmsnorm_bwd_add_partial, nm_sandwich_tail_bwd) stage their operands
 * through a ring in shared memory whose waits are bounded; one that ran out leaves a bit in a per-GPU word built into the
 * library. This reads the word after the stream's work (it synchronises the stream), clears it when set, and returns
 * NM_ERR_DEVICE with the bits in *status_host when it was not 0. */
int nm_norm_bwd_device_status(void* stream, uint32_t* status_host);
/* Test hook: a millisecond-bounded wait on a barrier that nothing completes (limit_cycles <= 2e6), pointed at that word:
 * afterwards nm_norm_bwd_device_status reports what a kernel whose wait ran out would have left. */
int nm_norm_bwd_test_timeout(int64_t limit_cycles, void* stream);

#ifdef __cplusplus
}
#endif
#endif
