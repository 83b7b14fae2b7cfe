// AdamH update of the LM head on the elements a rank owns (ZeRO-1), next to the fused cross-entropy that produces the
// head's gradient. Algorithm and operation order: the reference's docs/spec/optim.md:264-286 (AdamH = Adam direction,
// then the norm-preserving projection of a 2-D parameter with one Frobenius norm over the whole [V, D] matrix),
// :123-171 (the group's own clip by its gradient norm), src/kernels/optim/optk_adam.cu:1-26,84-221. The reference runs
// it inside its multi-tensor optimizer engine (src/optim/engine.cpp) over "owned slices" planned by
// include/marincpp/comm.hpp:22-71 (GradReducer reduces buckets to their owners, ParamGather all-gathers the updated
// bf16 parameters); this header is that design for the one tensor on this path.
//
//   per step, on each rank:   dW buckets --reduce-scatter--> owned gradient ranges        (GradReducer, to_owners)
//                             sum g^2 over owned ranges --all-reduce (1 f64)--> clip norm
//                             pass 1: mu, nu, sums of p^2, a^2, p a --all-reduce (3 f64)--> n, m, ||w||
//                             pass 2: p <- p + ((w / ||w||) n - p);  W16[owned] <- bf16(p)
//                             W16 --all-gather per bucket--> full bf16 replica for the next forward
#pragma once

#include <cstdint>

#include "marincpp/comm.hpp"
#include "marincpp/core.hpp"

namespace nm {

struct AdamHStep {
  int64_t t = 1;                 // update count, first update 1 (bias corrections 1 - b^t)
  float eta = 0.02f;             // the main learning rate of this update
  float b1 = 0.9f, b2 = 0.98f, eps = 1e-20f;
  float max_grad_norm = 1.0f;    // <= 0: no clip
  float grad_scale = 1.0f;       // the gradient is multiplied by this first (1 / microbatches)
  // bias corrections 1 - b^t from the trainer's schedule tables (the reference computes them with XLA's f32 pow,
  // docs/spec/optim.md:322-335); 0 = computed here as f32(1 - pow(f32(b), t)) with the power taken in f64, which can
  // differ from that table by one ulp of b^t (AdamH divides the factor out again, plain Adam does not)
  float bc1 = 0.f, bc2 = 0.f;
  // With a reducer: run the all-gather of the bf16 replica on the reducer's communication stream instead of `st` (the
  // reference's ParamGather design, include/marincpp/comm.hpp:60-71: the gather of step k travels while the trunk of
  // step k + 1 runs); whatever reads the replica next must call wait_params first.
  bool gather_on_comm_stream = false;
};

class HeadAdamH {
 public:
  // reducer == nullptr: one rank owns the whole tensor. Otherwise a GradReducer made with to_owners = true over the
  // same [V, D] gradient: its buckets' owned ranges are this rank's elements.
  HeadAdamH(int V, int D, GradReducer* reducer);
  ~HeadAdamH();
  HeadAdamH(const HeadAdamH&) = delete;
  HeadAdamH& operator=(const HeadAdamH&) = delete;

  int64_t owned_elems() const { return owned_; }   // length of the caller's p, mu, nu arrays (f32 each)
  int n_ranges() const;
  void range(int i, int64_t& global_off, int64_t& compact_off, int64_t& len) const;

  // p_owned[compact] = f32(w16[global]) over the owned ranges (start of training: master copy from the replica)
  void init_master(const bf16_t* w16, float* p_owned, cudaStream_t st) const;

  // One update. grad: the [V, D] f32 gradient (with a reducer: after its buckets were reduced to their owners; the call
  // waits for the reducer on `st`). p_owned, mu_owned, nu_owned: this rank's master parameters and moments, compact.
  // w16: the [V, D] bf16 replica, rewritten on owned ranges and, with a reducer, all-gathered. Everything runs on `st`;
  // nothing is allocated and the host is not synchronised. One step at a time per object (its scalars and block
  // partials live in device memory the object owns); the object belongs to the device that was current when it was made.
  void step(const AdamHStep& s, const float* grad, float* p_owned, float* mu_owned, float* nu_owned, bf16_t* w16,
            cudaStream_t st);

  // `st` waits for the last all-gather issued with gather_on_comm_stream (no-op otherwise)
  void wait_params(cudaStream_t st);

  // the step's scalars on the device (f64: sum g^2, sum p^2, sum a^2, sum p a over the whole tensor), for tests
  const double* scalars() const { return scal_; }

 private:
  struct Impl;
  Impl* impl_;
  GradReducer* reducer_;
  int V_, D_;
  int64_t owned_ = 0;
  double* scal_ = nullptr;
  double* partial_ = nullptr;
  cudaEvent_t applied_ = nullptr, gathered_ = nullptr;
  bool gather_pending_ = false;
};

// The reference's one-tensor entry point (include/marincpp/capi.h:107-110, src/optim/capi_optim.cpp:202-219): the
// whole [rows, cols] tensor on one GPU, clip state given by the caller. Optional row blocks (device arrays; nullptr /
// 0 = none): block_of_row[rows] in [0, n_blocks), block_lr_mult[n_blocks] (nullable: 1), block_frozen[n_blocks]
// (nullable: none); a block has its own learning-rate multiplier and its own AdamH norms, a frozen block's rows keep
// p, mu, nu and enter no norm (reference src/optim/capi_optim.cpp:103-128). With row blocks the call copies
// block_of_row to the host to validate it and synchronises the stream, as the reference's does.
struct RowBlocks {
  const int32_t* block_of_row = nullptr;
  const float* block_lr_mult = nullptr;
  const uint8_t* block_frozen = nullptr;
  int n_blocks = 0;
};
void adamh_update(float* p, bf16_t* p16, const float* g, float* mu, float* nu, int64_t rows, int64_t cols, int64_t t,
                  float eta, float b1, float b2, float eps, float clip_gn, bool clip, float max_norm, cudaStream_t st,
                  const RowBlocks& blocks = RowBlocks{});

// The reference's one-tensor Adam entry point (include/marincpp/capi.h:111-114): p += (-adam_lr) a, no projection; for
// the tensors beside the head on this path (the final norm's gain). Row blocks as above.
void adam_update(float* p, bf16_t* p16, const float* g, float* mu, float* nu, int64_t rows, int64_t cols, int64_t t,
                 float adam_lr, float b1, float b2, float eps, float clip_gn, bool clip, float max_norm, cudaStream_t st,
                 const RowBlocks& blocks = RowBlocks{});

}  // namespace nm
