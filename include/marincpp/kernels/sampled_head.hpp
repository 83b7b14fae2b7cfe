// Sampled-softmax output head on top of the fused linear cross-entropy.
//
// The reference names this head in its output-head design (include/marincpp/model.hpp:236-239: "candidates =
// sort-unique targets of the device microbatch + golden-ratio stride negatives, remapped targets, gathered W_P, fused CE,
// unique-row scatter of dW_P", docs/DESIGN.md:958) and gates it against a float64 full-vocabulary CE whose logits are
// masked to the candidate set (docs/DESIGN.md:1283); it ships no source for it. This is that head, built from the
// description, everything on the device and stream-ordered (no host synchronisation, nothing allocated):
//
//   1. candidates  C = sorted unique { target_t : row t counts } u { (neg_offset + j * stride(V)) mod V : j < n_negatives },
//                  stride(V) = the integer nearest V (sqrt(5) - 1) / 2 made coprime with V (sampled_stride below), so
//                  consecutive negatives spread over the vocabulary and never repeat within V draws.
//   2. remap       target_t -> position of target_t in C (ignored rows stay ignored)
//   3. gather      W_P[i, :] = W[C[i], :] for i < |C|; rows |C| .. p_max - 1 are zero
//   4. fused CE    on x [T, D] and W_P [p_max, D] with the columns |C| .. p_max - 1 masked out of the softmax (a logit
//                  bias of -1e30 on them): loss, lse, dX as for a vocabulary of exactly C; dW_P [p_max, D] f32
//   5. scatter     dW[C[i], :] += dW_P[i, :] for i < |C| (the rows are unique: plain adds, no atomics)
//
// p_max bounds |C| and sizes the workspace; it must be at least min(V, T + n_negatives) so that no microbatch can
// overflow it (the reference plans a data-dependent fallback to the full head instead; with this bound none is needed).
#pragma once

#include <cstdint>

#include "marincpp/core.hpp"
#include "marincpp/kernels/cross_entropy.hpp"

namespace nm {

// The stride of the negatives: round(V * 0.6180339887...) moved up to the next value coprime with V (1 for V <= 2).
int64_t sampled_stride(int64_t V);

struct SampledHeadShape {
  int64_t T;           // rows in the call
  int D, V;
  int p_max;           // capacity of the candidate set (multiple of 8); >= min(V, T + n_negatives)
  int chunk_rows;
  DType logits_store;  // bf16 or f32, as CeShape
};

struct SampledHeadArgs {
  const void* x;             // [T, D] bf16
  const void* w;             // [V, D] bf16, the full head
  const int32_t* targets;    // [T] ids in the full vocabulary
  const float* weight;       // [T]
  const float* grad_scale;   // device scalar
  float* loss_tok;           // [T]
  float* lse;                // [T] or nullptr: log-sum-exp over the candidate set
  float* loss_partial;       // [ceil(T / chunk_rows)] or nullptr
  void* dx;                  // [T, D] or nullptr; may alias x
  bool accumulate_dx;
  float* dw;                 // [V, D] f32 (+= on the candidate rows) or nullptr
  bool forward_only;
  int n_negatives;           // strided negatives added to the targets
  int64_t neg_offset;        // first negative id (any value; taken mod V): vary it per step
  float z_loss_weight = 0.f;
  int32_t ignore_index = INT32_MIN;
  int32_t* candidates_out = nullptr;     // [p_max] the sorted candidate ids (entries >= the count are -1), optional
  int32_t* n_candidates_out = nullptr;   // device int: |C|, optional
};

uint64_t sampled_head_workspace_bytes(const SampledHeadShape& s);
void sampled_head(Rounding r, const SampledHeadShape& s, const SampledHeadArgs& a, void* ws, cudaStream_t st);

}  // namespace nm
