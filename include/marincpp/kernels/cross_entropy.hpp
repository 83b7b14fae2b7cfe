// Fused linear (LM-head) cross-entropy for sm_100a: x [T, D] x W [V, D] -> per-token CE, dX, dW (+= f32).
//
// The public C++ surface of the reference's include/marincpp/kernels/cross_entropy.hpp:41-98 (CeImpl, CeShape, CeArgs,
// ce_workspace_bytes, fused_linear_ce, ce_finish_microbatch, ReadoutCall, run_readout), field for field, so the
// reference's call site (src/model/baseline.cpp:366-373) links against this library unchanged. Two trailing, defaulted
// CeArgs fields add what the reference does not have: a z-loss weight and an explicit ignore index.
//
// Math per row t (natural log), g_t = weight[t] * (*grad_scale), z-loss weight L (0 reproduces the reference):
//   z      = x_t W^T                       bf16 operands, f32 accumulate on the tensor cores
//   lse_t  = m + log(sum exp(z - m))       from the f32 accumulators
//   loss_t = lse_t - z[target_t] + L lse_t^2          (0 for an ignored row)
//   p      = exp(z_s - lse_t)              z_s = the stored logit of the chunk: f32(bf16(z)) (bf16 store) or z (f32)
//   dz     = g_t (p (1 + 2 L lse_t) - onehot(target_t))
//   dx_t   = bf16(dz W)                    dW += dz^T x   (f32)
// A row is ignored (no loss, no gradient) when weight[t] == 0, target_t is outside [0, V), or target_t == ignore_index.
//
// How this library computes it: rows are processed in chunks of chunk_rows. Per chunk: one tcgen05 kernel forms the
// logits tile by tile in TMEM, keeps per-(row, 256-column tile) partial (max, sum exp) and writes the bf16 (or f32)
// logits of the chunk to the workspace store; a row kernel merges the partials in ascending tile order; a streaming
// pass rewrites the store in place as the bf16 matrix n = w_t (p (1 + 2 L lse) - onehot), i.e. dz without the common
// factor *grad_scale (so the dominant -1 at the target is exact in bf16 whatever the value of grad_scale); two tcgen05
// kernels contract n with W (dX) and with x (dW) and apply *grad_scale in f32 in their epilogues. The full [T, V]
// logits are never materialised; only the store of one chunk exists. Every implementation value (A, B1, B1.5, B2) of
// the reference maps to this one pipeline.
#pragma once

#include <cstdint>

#include "marincpp/core.hpp"

namespace nm {

class GemmCache;   // trunk GEMM planner of the reference trainer; the CE path ignores it (reference ce_api.cpp:284)

enum class CeImpl : uint8_t { A = 0, B1 = 1, B1_5 = 2, B2 = 3 };

struct CeShape {
  int64_t T;          // rows (tokens) in the call
  int D, V;
  int chunk_rows;     // rows per chunk (bounds the logits store: chunk_rows * round_up(V, 8) elements)
  DType logits_store; // bf16 or f32
  DType io = DType::bf16;   // bf16, or f32 (implementation A only, as in the reference)
};

struct CeArgs {
  const void* x;             // [T, D]
  const void* w;             // [V, D]
  const int32_t* targets;    // [T]
  const float* weight;       // [T]
  const float* grad_scale;   // device scalar
  const float* logit_bias;   // [V] or nullptr (implementation A only)
  float* loss_tok;           // [T] per-token loss (0 where ignored)
  float* lse;                // [T] or nullptr
  float* loss_partial;       // [ceil(T / chunk_rows)] f32 sum of weight * loss per chunk, or nullptr
  void* dx;                  // [T, D] or nullptr; may alias x (not together with accumulate_dx)
  bool accumulate_dx;        // dx +=
  float* dw;                 // [V, D] f32 accumulator (+=) or nullptr
  float* dw_microbatch;      // CeDwRound::PerChunkBf16: per-microbatch f32 accumulator [V, D]
  CeDwRound dw_round;
  bool forward_only;         // statistics and loss only (no store, no gradients)
  // ---- extensions (not in the reference; defaults reproduce it) ----
  float z_loss_weight = 0.f;            // L above
  int32_t ignore_index = INT32_MIN;     // a target equal to this is ignored even when it lies inside [0, V)
  void* dw_reducer = nullptr;           // nm::GradReducer* (comm.hpp): the last chunk's dW is issued per bucket and
                                        // each bucket's all-reduce starts as its vocabulary range retires
};

uint64_t ce_workspace_bytes(CeImpl impl, const CeShape& s);
void fused_linear_ce(CeImpl impl, Rounding r, const CeShape& s, const CeArgs& a, void* ws, GemmCache& gemm,
                     cudaStream_t st);
// Strict mode only: dw += f32(bf16(dw_microbatch)); dw_microbatch = 0.
void ce_finish_microbatch(const CeShape& s, const CeArgs& a, cudaStream_t st);

// One readout head (pls): RMSNorm of `state`, CE against w with dX written over the norm output, RMSNorm backward
// added into d_state, gain partials. Field order as the reference's ReadoutCall (cross_entropy.hpp:84-96).
struct ReadoutCall {
  int layer;
  const bf16_t* state;           // [T, D]
  const bf16_t* norm_gain;       // [D]
  float* norm_rstd_ws;           // [T]
  bf16_t* norm_out_ws;           // [T, D]
  const bf16_t* w;               // [V, D]
  float* dw;                     // [V, D] f32 (nullptr: detached head)
  float* dgain_partial;          // [norm_partial_rows(T), D] or nullptr
  const float* grad_scale;       // device scalar
  bf16_t* d_state;               // [T, D] gradient w.r.t. the readout state, added into (nullptr: none)
  int visible_dims;              // coordinates >= visible_dims of the normed input are zeroed
};
void run_readout(CeImpl impl, Rounding r, const CeShape& s, const ReadoutCall& c, const CeArgs& base, void* ws,
                 GemmCache& gemm, cudaStream_t st);

}  // namespace nm
