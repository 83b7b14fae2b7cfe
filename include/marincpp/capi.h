/* C ABI of libmarincpp_kernels.so, the fused LM-head cross-entropy part. Same names, argument order and status
 * convention as the reference's include/marincpp/capi.h (:14-17 status codes, :23-26 basics, :91-98 the CE block), so a
 * program or a ctypes harness (reference tests/s5/nmce.py:22-23) bound to the reference library binds to this one.
 * All pointers are device pointers unless named *_host. `stream` is a cudaStream_t (NULL = legacy default stream).
 * Every int function returns NM_OK (0) on success, else NM_ERR_INVALID (1: bad argument or unmet requirement),
 * NM_ERR_DEVICE (2: a CUDA or NCCL call failed, or a kernel reported a timed-out wait) or NM_ERR_INTERNAL (3);
 * nm_last_error() returns the message (thread-local). Only nm_* symbols are exported (csrc/capi.map).
 * The calls allocate nothing and never synchronise; the caller owns every buffer, the workspace included.
 * There is no CPU path: without a CUDA device every compute entry point returns NM_ERR_DEVICE. */
#ifndef MARINCPP_CAPI_H
#define MARINCPP_CAPI_H

#include <stdint.h>

#define NM_OK 0
#define NM_ERR_INVALID 1
#define NM_ERR_DEVICE 2
#define NM_ERR_INTERNAL 3

#ifdef __cplusplus
extern "C" {
#endif

/* reference include/marincpp/capi.h:23-26, src/core/capi_core.cpp:20-36 */
const char* nm_version(void);        /* build identifier of this library */
const char* nm_last_error(void);
int nm_device_arch(void);            /* 100 on a B200; 0 on a CUDA error (nm_last_error says which) */

/* ---- fused linear cross-entropy; impl 0 A, 1 B1, 2 B1.5, 3 B2 (all run the one sm_100a pipeline); rounding
 *      0 levanter, 1 accurate; io and logits_store: 0 f32, 1 bf16; dw_round 0 none, 1 per-chunk bf16 (strict).
 *      reference include/marincpp/capi.h:93-98, src/kernels/cross_entropy/capi_ce.cpp:37-56 ------------------------ */
uint64_t nm_ce_workspace_bytes(int impl, int64_t T, int D, int V, int chunk_rows, int logits_store);  /* 0 on error */
int nm_fused_linear_ce(int impl, int rounding, int io, int logits_store, const void* x, const void* w,
                       const int32_t* targets, const float* weight, const float* grad_scale, const float* logit_bias,
                       float* loss_tok, float* lse, float* loss_partial, void* dx /*nullable*/, int accumulate_dx,
                       float* dw /*nullable*/, float* dw_microbatch /*nullable*/, int dw_round, int forward_only,
                       int64_t T, int D, int V, int chunk_rows, void* workspace, void* stream);

/* ---- the step on either side of the fused CE (reference include/marincpp/capi.h:29-31, 36-48): the metadata kernel
 *      that produces targets and weights, the RMSNorm pair of the readout head, and the sandwich tail whose forward
 *      produces the CE input (final norm) and whose backward consumes the CE's dX. dtype: storage of the row tensors
 *      and gains, 1 = bf16 (the model's; the tuned kernels), 0 = f32 (f32 throughout, both rounding modes alike: the
 *      reference's own tests use it to tell math errors from rounding).
 *      dgain / dg_next / dg_post: f32 [D], overwritten with the fixed-order reduction of the per-part partials,
 *      rounded to bf16 under levanter rounding with bf16 storage; NULL skips it (these entry points make a stream-ordered allocation
 *      for the partials, as the reference's test entry points do) ------------------------------------------------ */
int nm_doc_meta(const int32_t* tokens, const uint8_t* row_valid, int rows, int S, int32_t eos, int max_segs,
                int32_t* targets, float* weight, int32_t* pos, int32_t* cu_seqlens, int32_t* n_segs,
                int32_t* row_seg_start, uint32_t* overflow, void* stream);
int nm_rmsnorm_fwd(int dtype, int rounding, const void* x, const void* gain, void* y, float* rstd, int64_t T, int D,
                   float eps, void* stream);
int nm_rmsnorm_bwd_add(int dtype, int rounding, const void* dy, const void* x, const void* gain, const float* rstd,
                       const void* dres, void* dx, float* dgain, int64_t T, int D, float eps, void* stream);
int nm_sandwich_tail_fwd(int dtype, int rounding, const void* branch, const void* x_in, const void* g_post,
                         const void* g_next, void* x_out, void* a_next, float* rstd_post, float* rstd_next, int64_t T,
                         int D, float eps, void* stream);
int nm_sandwich_tail_bwd(int dtype, int rounding, const void* dx_out, const void* da_next, const void* x_out,
                         const void* g_next, const float* rstd_next, const void* branch, const void* g_post,
                         const float* rstd_post, void* dx_in, void* dbranch, float* dg_next, float* dg_post,
                         int64_t T, int D, float eps, void* stream);

#ifdef __cplusplus
}
#endif

#endif
