/* Further C entry points of the fused CE in libmarincpp_kernels.so. The first block has the names and signatures of
 * the reference's src/kernels/cross_entropy/capi_ce.h:17-35 (test and bench entry points); the second block holds the
 * extensions of this library: z-loss / ignore-index, and the data-parallel dW reduction. Conventions as in capi.h. */
#ifndef MARINCPP_CAPI_CE_H
#define MARINCPP_CAPI_CE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* reference capi_ce.h:17-19. This library has one kernel set, so the arguments only update the recorded setting;
 * returns the previous setting packed as dgrad | wgrad << 1 | sm90 << 2 (sm90 < 0: unchanged). */
int nm_ce_set_backends(int dgrad_own, int wgrad_own, int sm90);
/* reference capi_ce.h:20-21. The statistics exponential here is always ex2.approx on a pre-scaled argument; the
 * switch is recorded and returned for callers that toggle it. */
int nm_ce_set_fast_stats_exp(int on);
/* reference capi_ce.h:22-23: dw += f32(bf16(dw_microbatch)); dw_microbatch = 0 (n = V * D) */
int nm_ce_finish_microbatch(float* dw, float* dw_microbatch, int64_t n, void* stream);
/* reference capi_ce.h:24-25: *out = mult / sum(w[0..n)) in f32, fixed summation order */
int nm_ce_grad_scale(const float* w, int64_t n, float mult, float* out, void* stream);
/* reference capi_ce.h:26-31: one readout head (norm of `state`, CE against w, dW into dw, d(state) added into d_state,
 * gain partials [nm_norm_partial_rows(T), D] into dgain_partial) */
int nm_ce_readout(int impl, int rounding, int logits_store, const void* state, const void* norm_gain,
                  float* norm_rstd_ws, void* norm_out_ws, const void* w, float* dw, float* dgain_partial,
                  const float* grad_scale, void* d_state, int visible_dims, const int32_t* targets,
                  const float* weight, float* loss_tok, float* lse, float* loss_partial, int forward_only, int64_t T,
                  int D, int V, int chunk_rows, float eps, void* workspace, void* stream);
/* reference capi_ce.h:32-34: the in-place dlogits pass alone over a logits store [rows, ldS]. `gscale` holds the
 * per-row factor g; the store is rewritten as bf16 g (p - onehot). logits_store 0 f32, 1 bf16. */
int nm_ce_dlogits(int logits_store, void* store, int64_t ldS, const float* lse, const float* gscale,
                  const int32_t* targets, int rows, int V, void* stream);
/* reference capi_ce.h:35: compute capability as the CE dispatch sees it (100 on a B200) */
int nm_ce_device_arch(void);

/* ---------------------------------------------------------------------------------------------- extensions
 * (no counterpart in the reference, whose CE has neither a z-loss nor an ignore index: docs/spec/model.md:277) */

/* nm_fused_linear_ce plus: z_loss_weight L (loss += L lse^2, dz = g (p (1 + 2 L lse) - onehot)), ignore_index (a
 * target equal to it is ignored like a target outside [0, V)), and dw_reducer (NULL, or a handle from
 * nm_grad_reducer_create: the dW kernel of the last chunk is issued per vocabulary bucket and each bucket's all-reduce
 * is enqueued on the reducer's stream as soon as that bucket is final, overlapping the last chunk's dX kernel). */
int nm_fused_linear_ce_ex(int impl, int rounding, int io, int logits_store, const void* x, const void* w,
                          const int32_t* targets, const float* weight, const float* grad_scale,
                          const float* logit_bias, float* loss_tok, float* lse, float* loss_partial, void* dx,
                          int accumulate_dx, float* dw, float* dw_microbatch, int dw_round, int forward_only,
                          int64_t T, int D, int V, int chunk_rows, void* workspace, void* stream,
                          float z_loss_weight, int32_t ignore_index, void* dw_reducer);

/* Status word of the device-side waits: every mbarrier wait in the tcgen05 kernels is bounded; a wait that runs out
 * sets a bit in a per-workspace word and the kernel returns. Reads the word of `workspace` (synchronises `stream`). */
int nm_ce_device_status(void* workspace, void* stream, uint32_t* status_host);

/* Per-kernel-class device timing for benches (the role of the reference's tests/s5/bench_ce.py event timing, moved
 * inside the call so that each kernel class is timed on the stream it is launched on). enable(n > 0) creates 2 n CUDA
 * events and makes every later call bracket each launch with a pair (up to n launches between two reads);
 * enable(0) frees them. read() waits for the recorded events and returns, per class (0 logits, 1 finalize, 2 dlogits
 * pass, 3 dW, 4 dX, 5 chunk loss), the summed milliseconds and the number of launches since the previous read. */
int nm_ce_profile_enable(int max_launches);
int nm_ce_profile_read(double* ms_host /*[6]*/, int* launches_host /*[6]*/);

/* Exercises the time-out path of the bounded device waits without hanging anything: one small CTA waits on an mbarrier
 * that nobody completes, with a limit of `limit_cycles` SM clocks (at most 2e6, about a millisecond). The waiting
 * thread must OR the epilogue-wait bit (4) into *status and raise the CTA's abort flag; a second thread waiting on the
 * same barrier with a long limit must leave through that flag (*saw_abort = 1). The kernel then returns normally. */
int nm_ce_test_wait_timeout(uint32_t* status, int64_t limit_cycles, int* saw_abort, void* stream);

/* A chunk size for a call of T rows on the current device: min(T, 128 x SM count) rows (18944 on a B200). With it the
 * tile counts of the logits and dX kernels of every full chunk are whole multiples of the SM count (one persistent CTA
 * per SM, 128-row tiles), so no wave of tiles runs part-filled; 16384 leaves the dX kernel at 86 % of its last wave
 * for hidden sizes up to 1024. Returns 0 without a device. No counterpart in the reference (its callers pass 16384). */
int nm_ce_suggest_chunk_rows(int64_t T);

/* How many CTAs work on one accumulator tile in the logits, dX and dW contractions: 0 = one CTA per 128 x 256 tile,
 * non-zero = a pair of CTAs on one TPC per 256 x 256 tile (tcgen05 cta_group::2; the B operand is staged once per
 * pair), negative = chosen per launch (the default: pairs where they were measured to pay: the dX and dW contractions
 * of calls with hidden size up to 512 and at most 16384 rows per chunk, the logits contraction of calls with hidden
 * size 1024 .. 2048 and at least 4096 rows per chunk; one CTA per tile otherwise). Results are
 * bit-identical between the two forms. Process-wide; call it while no CE call is in flight. No
 * counterpart in the reference (its nm_ce_set_backends chooses between its own kernels and cuBLASLt). */
int nm_ce_set_cta_pair(int logits, int dgrad, int wgrad);

/* How the two gradient contractions of a chunk get the normalised gradient n and which tile form they use:
 * 0 = an in-place pass over the logits store writes n, dX / dW run on 128 x 256 tiles; 1 = the same pass, dX / dW on
 * CTA pairs with 256 x 512 tiles (one 512-column TMEM accumulator); 2 = no pass: dX / dW read the raw logits and form
 * n in shared memory ahead of the tensor-core instructions (256 x 512 tiles); -1 = chosen per call (the default: 2 for
 * hidden sizes up to 1024, else 0). Loss, lse and dX are bit-identical across the three; dW differs only by summation
 * order between tile forms. Calls with an f32 logits store or f32 io always take form 0. Process-wide. No counterpart
 * in the reference (its nm_ce_set_backends chooses between its own kernels and cuBLASLt). */
int nm_ce_set_grad_path(int path);

/* Order of the last chunk of a call whose dW goes through a bucketed reducer: 0 (default) = the dW buckets first and dX
 * beside their reductions (always the order when dx aliases x); 1 = when dx does not alias x, dX runs first on every SM
 * and only the dW buckets share the GPU with the reductions. Results do not depend on it. Process-wide. No counterpart
 * in the reference. */
int nm_ce_set_tail_order(int order);

/* One of the tcgen05 contractions alone, for unit tests and ncu (kind 0: C[M,N] f32 = A[M,K] B[N,K]^T, both
 * K-major; 1: C[M,N] f32 = A[M,K] B[K,N], B N-major; 2: C[M,N] f32 = A[K,M]^T B[K,N], both MN-major; kind + 4: the same
 * with CTA pairs; kind + 8 (kinds 1 and 2): the 256 x 512-tile pair kernel; kind + 8 + 16: that kernel with A holding
 * raw logits that it turns into a p - b onehot(target) on the fly, `row_factors` being a device array of
 * {float e, a, b; int32 target} per row of the logits (rows = M for kind 1, K for kind 2), NULL otherwise). bf16
 * operands, row-major with leading dimensions in elements; `status` is a device uint32 the kernel ORs its wait errors
 * into. */
int nm_ce_test_gemm(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc, int M,
                    int N, int K, uint32_t* status, const void* row_factors, void* stream);

/* Forward only (per-token loss, lse, per-chunk loss sums; bf16 x and W) WITHOUT a caller workspace and without any
 * allocation: the scratch of one chunk lives in a 16 MiB device array built into the library (held by every GPU that
 * loads it). This entry point has no counterpart in the reference. It is for callers that cannot allocate: a trainer
 * whose single up-front arena has no region planned for an extra evaluation or probe call, or a thread that runs while
 * a stream capture is open, when cudaMalloc is not permitted. Same results as nm_fused_linear_ce_ex with
 * forward_only = 1 and the same chunk_rows. With r = min(chunk_rows, T) it needs 256 + 8 ceil(V / 256) r + 4 r bytes
 * of scratch (r <= 4096 at V = 128256); a larger request returns NM_ERR_INVALID. The first call on a device resolves
 * the array's device address: make it before any stream capture. All calls on a GPU share the array: calls whose
 * kernels may overlap on the device race and must be serialised by the caller. lse and loss_partial may be NULL. */
int nm_ce_forward_noalloc(const void* x, const void* w, const int32_t* targets, const float* weight, float* loss_tok,
                          float* lse, float* loss_partial, int64_t T, int D, int V, int chunk_rows,
                          float z_loss_weight, int32_t ignore_index, void* stream);
/* The wait-status word of the calls above on the current device (nm_ce_device_status needs a workspace pointer, which
 * a caller of nm_ce_forward_noalloc never holds): copies word 0 of the built-in array to *status_host, synchronises
 * `stream`, and returns NM_ERR_DEVICE when a bit is set (a bounded wait inside a kernel ran out: discard that call's
 * losses). Allocates nothing. Each nm_ce_forward_noalloc clears the word when it starts, so read it after the call
 * you care about and before the next one. No counterpart in the reference. */
int nm_ce_forward_noalloc_status(void* stream, uint32_t* status_host);
/* Test hook for the line above: points the short wait probe of nm_ce_test_wait_timeout at that status word. */
int nm_ce_forward_noalloc_test_timeout(int64_t limit_cycles, void* stream);

/* ---- sampled-softmax head (C++: include/marincpp/kernels/sampled_head.hpp). The reference names this head in its
 *      output-head design (include/marincpp/model.hpp:236-239, docs/DESIGN.md:958) and ships no code for it. The
 *      candidate set is the sorted unique set of the call's counted targets plus n_negatives ids
 *      (neg_offset + j * nm_ce_sampled_stride(V)) mod V; W is gathered to W_P [p_max, D], the fused CE runs over the
 *      candidate columns (unused ones masked out of the softmax), and dW_P is added into dw at the candidate rows.
 *      p_max (a multiple of 8) must be at least min(V, T + n_negatives). x, w, dx bf16; dw [V, D] f32 (+=).
 *      candidates_out [p_max] (sorted ids, -1 beyond the count) and n_candidates_out (device int) are optional. ------ */
int64_t nm_ce_sampled_stride(int64_t V);
uint64_t nm_ce_sampled_workspace_bytes(int64_t T, int D, int V, int p_max, int chunk_rows, int logits_store);
int nm_ce_sampled_head(int rounding, int logits_store, const void* x, const void* w, const int32_t* targets,
                       const float* weight, const float* grad_scale, float* loss_tok, float* lse, float* loss_partial,
                       void* dx, int accumulate_dx, float* dw, int forward_only, int64_t T, int D, int V,
                       int n_negatives, int64_t neg_offset, int p_max, int chunk_rows, int32_t* candidates_out,
                       int32_t* n_candidates_out, void* workspace, void* stream, float z_loss_weight,
                       int32_t ignore_index);

/* ---- data-parallel dW reduction over NCCL (the role of the reference's include/marincpp/comm.hpp:22-58 GradReducer
 *      and of src/train/trainer.cpp:50,139): one communicator per process (one process per GPU) ------------------- */
int nm_comm_unique_id(void* id128_host);                       /* rank 0: 128 bytes to broadcast to the other ranks */
int nm_comm_create(const void* id128_host, int nranks, int rank, void** comm_out);   /* current device */
int nm_comm_destroy(void* comm);
int nm_comm_allreduce_f32(void* comm, float* buf, int64_t n, void* stream);           /* in place, sum */
/* A reducer over one gradient buffer grad[V, D] f32 split into n_buckets contiguous vocabulary ranges (multiples of
 * 128 rows). reduce_dtype 0: f32 in place; 1: each bucket is cast to bf16 into `staging` (V * D * 2 bytes, caller
 * owned), all-reduced in bf16 and cast back. */
int nm_grad_reducer_create(void* comm, float* grad, int V, int D, int n_buckets, int reduce_dtype, void* staging,
                           void** reducer_out);
/* the vocabulary ranges such a reducer uses (host arithmetic only): v0/v1 hold up to n_buckets entries, *n_out the
 * number of buckets actually made (whole 128-row tiles; fewer buckets than asked when V has fewer tiles) */
int nm_grad_bucket_ranges(int V, int n_buckets, int* v0_host, int* v1_host, int* n_out);
int nm_grad_reducer_destroy(void* reducer);
/* all buckets, in order, after the work already on `stream` (no overlap: what trainer.cpp:139 does) */
int nm_grad_reducer_reduce_all(void* reducer, void* stream);
/* make `stream` wait for every bucket reduction enqueued so far */
int nm_grad_reducer_wait(void* reducer, void* stream);

#ifdef __cplusplus
}
#endif

#endif
