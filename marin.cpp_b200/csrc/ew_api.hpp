// The RMSNorm pair the readout head calls around the fused CE (bf16 storage). Semantics follow the reference's
// src/kernels/elementwise/rmsnorm_kernels.cuh:3-9:
//   levanter  forward   ms = sum(x^2) / D; r = rsqrt(ms + eps); y = bf16(x r); out = bf16(g y)
//             backward  a = bf16(g dy); dg += f32(bf16(dy y)); s = sum(x a); c = (s (-0.5 (r / (ms + eps)))) / D;
//                       dx = bf16(a r + c (2 x)); with a residual gradient: bf16(dres + bf16(dx))
//   accurate  f32 throughout, one rounding per stored output (dg accumulates dy x r in f32)
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "marincpp/core.hpp"

namespace nm::ew {

// the row kernels read and write 16-byte pieces: every (non-null) pointer given to them must be 16-byte aligned
template <class... P>
inline bool aligned16(P... p) {
  return ((reinterpret_cast<uintptr_t>(p) % 16 == 0) && ...);
}

// Number of gain-gradient partial rows the backward writes for T rows on the current device:
// min(1024, ceil(T / 16), 4 x SMs) parts of consecutive rows (reference ew_api.hpp:18-21).
int64_t norm_partial_rows(int64_t T);

void rmsnorm_fwd(const bf16_t* x, const bf16_t* gain, bf16_t* y, float* rstd, int64_t T, int D, float eps,
                 cudaStream_t st, Rounding r = Rounding::Levanter);
// dx = norm backward of dy (+ dres when given; dres may equal dx); dgain_partial [norm_partial_rows(T), D] or nullptr
void rmsnorm_bwd_add(const bf16_t* dy, const bf16_t* x, const bf16_t* gain, const float* rstd, const bf16_t* dres,
                     bf16_t* dx, float* dgain_partial, int64_t T, int D, float eps, cudaStream_t st,
                     Rounding r = Rounding::Levanter);


// Sandwich tail (ew_sandwich.cu): y = g_post ? norm(branch; g_post) : branch; x_out = bf16(x_in + y);
// a_next = norm(x_out; g_next) (a_next may be nullptr). Reference elementwise.hpp:101-122.
void sandwich_tail_fwd(const bf16_t* branch, const bf16_t* x_in, const bf16_t* g_post, const bf16_t* g_next,
                       bf16_t* x_out, bf16_t* a_next, float* rstd_post, float* rstd_next, int64_t T, int D, float eps,
                       cudaStream_t st, Rounding r = Rounding::Levanter);
// dx_mid = dx_out + norm_next_bwd(da_next); dx_in = dx_mid (may alias dx_out); dbranch = norm_post_bwd(dx_mid) or
// dx_mid; gain partials [norm_partial_rows(T), D] (nullptr: skipped)
void sandwich_tail_bwd(const bf16_t* dx_out, const bf16_t* da_next, const bf16_t* x_out, const bf16_t* g_next,
                       const float* rstd_next, const bf16_t* branch, const bf16_t* g_post, const float* rstd_post,
                       bf16_t* dx_in, bf16_t* dbranch, float* pg_next, float* pg_post, int64_t T, int D, float eps,
                       cudaStream_t st, Rounding r = Rounding::Levanter);

// f32-storage forms (ew_norm_f32.cu): the same entry points for float tensors and gains, f32 throughout (both rounding
// modes coincide); the reference's tests use them to tell math errors from rounding. Not a hot path.
void rmsnorm_fwd_f32(const float* x, const float* gain, float* y, float* rstd, int64_t T, int D, float eps, cudaStream_t st);
void rmsnorm_bwd_add_f32(const float* dy, const float* x, const float* gain, const float* rstd, const float* dres, float* dx,
                         float* dgain_partial, int64_t T, int D, float eps, cudaStream_t st);
void sandwich_tail_fwd_f32(const float* branch, const float* x_in, const float* g_post, const float* g_next, float* x_out,
                           float* a_next, float* rstd_post, float* rstd_next, int64_t T, int D, float eps, cudaStream_t st);
void sandwich_tail_bwd_f32(const float* dx_out, const float* da_next, const float* x_out, const float* g_next,
                           const float* rstd_next, const float* branch, const float* g_post, const float* rstd_post,
                           float* dx_in, float* dbranch, float* pg_next, float* pg_post, int64_t T, int D, float eps,
                           cudaStream_t st);

// The word the norm backward kernels OR their error bits into when one of their bounded waits runs out (one per GPU,
// zero-initialised, address looked up on first use: make the first backward call on a device outside a stream capture).
// read_row_status copies it to the host after the stream's work, clears it when set, and returns it.
uint32_t* row_status_word();
uint32_t read_row_status(cudaStream_t st);

// Microbatch metadata from token rows [rows, S] (ew_misc.cu): targets (next token; the last position wraps and has
// weight 0), weight (0 for an invalid row), pos, per-row segment starts [rows, max_segs + 1] (padded with S), packed
// cu_seqlens [rows * max_segs + 1] (padded with rows * S), the segment count, and an overflow flag set when a row
// holds more than max_segs segments. Reference elementwise.hpp DocMetaArgs, doc_meta.cu.
void doc_meta(const int32_t* tokens, const uint8_t* row_valid, int rows, int S, int32_t eos, int max_segs,
              int32_t* targets, float* weight, int32_t* pos, int32_t* cu_seqlens, int32_t* n_segs,
              int32_t* row_seg_start, uint32_t* overflow, cudaStream_t st);
void sum_fixed(const float* x, int64_t n, float* out, cudaStream_t st);     // fixed-order sum (loss slots)
void reduce_partials_rows(const float* partial, int n_blocks, int width, float* out, bool accumulate, bool round_bf16,
                          cudaStream_t st);

}  // namespace nm::ew
