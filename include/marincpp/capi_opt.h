/* C ABI of the LM head's AdamH update (the optimizer step that consumes the fused cross-entropy's dW). Conventions as
 * in capi.h: device pointers, `stream` is a cudaStream_t passed as void* (NULL = legacy default stream), int status
 * returns (NM_OK / NM_ERR_*), message in nm_last_error(). */
#pragma once

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference include/marincpp/capi.h:107-110 (src/optim/capi_optim.cpp:202-219): one AdamH update of one 2-D tensor
 * p[rows, cols] f32 (p16: optional bf16 copy of the new p) from gradient g and moments mu, nu, at update count t >= 1
 * with learning rate eta; when `clip` is non-zero the gradient is first scaled as (g / clip_gn) * max_norm.
 * Row blocks (optional; NULL, NULL, NULL, 0 = none; device arrays): block_of_row[rows] in [0, n_blocks),
 * block_lr_mult[n_blocks] (NULL: 1), block_frozen[n_blocks] (NULL: none). A block uses eta * its multiplier and takes
 * its AdamH norms over its own rows; the rows of a frozen block keep p, mu, nu and p16. With row blocks the call copies
 * block_of_row to the host to validate it and synchronises the stream (as the reference's does); without, it does not
 * synchronise. */
int nm_adamh_update(float* p, void* p16, const float* g, float* mu, float* nu, int64_t rows, int64_t cols, int64_t t,
                    float eta, float b1, float b2, float eps, float clip_gn, int clip, float max_norm,
                    const int32_t* block_of_row, const float* block_lr_mult, const uint8_t* block_frozen,
                    int n_blocks, void* stream);

/* reference include/marincpp/capi.h:111-114: one plain Adam update of one tensor, p += (-adam_lr) a with the same
 * moments, bias corrections and clip as above and no projection (the rule of the final norm's gain, whose gradient the
 * readout entry point produces). Row blocks as above (multiplier on adam_lr, frozen blocks). */
int nm_adam_update(float* p, void* p16, const float* g, float* mu, float* nu, int64_t rows, int64_t cols, int64_t t,
                   float adam_lr, float b1, float b2, float eps, float clip_gn, int clip, float max_norm,
                   const int32_t* block_of_row, const float* block_lr_mult, const uint8_t* block_frozen,
                   int n_blocks, void* stream);

/* ---- ZeRO-1 form (the design of the reference's include/marincpp/comm.hpp:22-71; no C entry points there) -------- */

/* nm_grad_reducer_create (capi_ce.h) with a reduction to owners: every bucket is reduce-scattered (f32), rank r keeps
 * the summed gradient on its element range of each bucket only. */
int nm_grad_reducer_create_owners(void* comm, float* grad, int V, int D, int n_buckets, void** reducer_out);
/* ZeRO-2 for the vocabulary-sized gradient (declared, not implemented, by the reference: GradReducer::microbatch_done,
 * include/marincpp/comm.hpp:52-53). Attach an owners reducer to the backward of every microbatch and call
 * nm_grad_reducer_microbatch_done after each: this rank's owned elements of every bucket are added into owned_acc
 * (packed, nm_grad_reducer_owned_elems f32) and the whole [V, D] gradient buffer is zeroed for the next microbatch.
 * nm_grad_reducer_owned_to_grad copies the packed sums back into the owned ranges before the optimizer step. */
int64_t nm_grad_reducer_owned_elems(void* reducer);
int nm_grad_reducer_microbatch_done(void* reducer, float* owned_acc, void* stream);
int nm_grad_reducer_owned_to_grad(void* reducer, const float* owned_acc, void* stream);

/* An updater for the head [V, D]. reducer: NULL (one rank owns everything) or a handle from
 * nm_grad_reducer_create_owners over the same gradient. */
int nm_head_adamh_create(int V, int D, void* reducer, void** out);
int nm_head_adamh_destroy(void* h);
/* number of f32 elements of the caller's p / mu / nu arrays (owned elements only) */
int64_t nm_head_adamh_owned_elems(void* h);
/* the owned ranges: up to `cap` entries of (offset into the flat tensor, offset into the compact arrays, length) */
int nm_head_adamh_ranges(void* h, int cap, int64_t* global_off_host, int64_t* compact_off_host, int64_t* len_host,
                         int* n_out);
/* p_owned = f32(w16) on the owned ranges */
int nm_head_adamh_init_master(void* h, const void* w16, float* p_owned, void* stream);
/* One update: clip by the head's own gradient norm (max_grad_norm <= 0: none), AdamH on owned elements, bf16 copy
 * into w16 and (with a reducer) all-gather of w16. Waits for the reducer's buckets on `stream` first. */
int nm_head_adamh_step(void* h, int64_t t, float eta, float b1, float b2, float eps, float max_grad_norm,
                       float grad_scale, const float* grad, float* p_owned, float* mu_owned, float* nu_owned,
                       void* w16, void* stream);
/* The same update with the all-gather of w16 issued on the reducer's communication stream (it then overlaps whatever
 * `stream` does next); nm_head_adamh_wait_params makes `stream` wait for it before w16 is read again. */
int nm_head_adamh_step_async(void* h, int64_t t, float eta, float b1, float b2, float eps, float max_grad_norm,
                             float grad_scale, const float* grad, float* p_owned, float* mu_owned, float* nu_owned,
                             void* w16, void* stream);
int nm_head_adamh_wait_params(void* h, void* stream);
/* the last step's scalars (4 doubles: sum g^2, sum p^2, sum a^2, sum p a over the whole tensor) copied to the host
 * after the work on `stream` (synchronises that stream) */
int nm_head_adamh_scalars(void* h, double* out4_host, void* stream);

#ifdef __cplusplus
}
#endif
