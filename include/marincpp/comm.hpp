// Data-parallel reduction of the LM-head gradient over NCCL: the part of the reference's communication design that
// the fused CE path touches. The reference declares a bucketed GradReducer (include/marincpp/comm.hpp:22-58) but ships
// no implementation; its trainer all-reduces the whole f32 gradient once per step on the compute stream
// (src/train/trainer.cpp:50,139). Here: one communicator per process (one process per GPU), a dedicated communication
// stream, and a reducer over dW [V, D] split into vocabulary-range buckets. The fused CE issues the dW kernel of its
// last chunk bucket by bucket and calls bucket_ready() after each, so the all-reduce of bucket i runs on the
// communication stream while the dW kernel of bucket i + 1 and then the dX kernel run on the compute stream.
#pragma once

#include <cstdint>
#include <vector>

#include "marincpp/core.hpp"

typedef struct CUevent_st* cudaEvent_t;

namespace nm {

// SMs the compute kernels leave to NCCL while a bucket reduction may be in flight (and the CTA cap given to NCCL).
// The tcgen05 kernels are persistent with one CTA per SM and nearly all of its shared memory, so a collective's CTAs
// cannot share an SM with them: without free SMs the all-reduce would only start when the compute kernel ends.
inline constexpr int kCommSms = 16;
// The value in effect: kCommSms, or the environment variable NM_COMM_SMS (4 .. 64) read once per process.
int comm_sms();

class Comm {
 public:
  static void unique_id(void* id128_host);                     // rank 0; 128 bytes
  Comm(const void* id128_host, int nranks, int rank);          // binds the current device
  ~Comm();
  Comm(const Comm&) = delete;
  Comm& operator=(const Comm&) = delete;
  int nranks() const { return nranks_; }
  int rank() const { return rank_; }
  cudaStream_t stream() const { return stream_; }              // the communication stream
  void allreduce_sum(void* buf, int64_t n, DType dt, cudaStream_t st);   // in place; dt f32, bf16 or f64
  // buf holds nranks * count f32 elements; afterwards elements [rank * count, (rank + 1) * count) hold the sum over
  // ranks (in place); the other parts are unspecified
  void reduce_scatter_sum_f32(float* buf, int64_t count, cudaStream_t st);
  // every rank's part [rank * count, (rank + 1) * count) of buf is gathered into buf on every rank (in place)
  void allgather(void* buf, int64_t count, DType dt, cudaStream_t st);
  void group_start();
  void group_end();
 private:
  void* comm_ = nullptr;
  cudaStream_t stream_ = nullptr;
  int nranks_ = 1, rank_ = 0, device_ = 0;
};

// Splits [0, V) into at most n_buckets contiguous ranges of whole 128-row tiles (the last ends at V), sizes as even as
// the tile count allows. Returns the number of buckets (pure host arithmetic).
int grad_bucket_ranges(int V, int n_buckets, std::vector<int>& v0, std::vector<int>& v1);

class GradReducer {
 public:
  // grad [V, D] f32; n_buckets contiguous vocabulary ranges whose sizes are multiples of 128 rows (the last takes the
  // remainder). reduce_dtype f32: in place. bf16: each bucket is cast into `staging` (V * D bf16, caller owned),
  // all-reduced there and cast back (wire bytes halved; the sum is then a bf16 sum).
  // to_owners (ZeRO-1, the reference's include/marincpp/comm.hpp:36-44 design): each bucket is reduce-scattered
  // instead of all-reduced: rank r ends up with the sum on elements [r, r + 1) * n / nranks of the bucket's n = rows * D
  // elements only (its owned range; f32 only, n must divide by nranks), for an optimizer that updates owned elements
  // and all-gathers the updated bf16 parameters (HeadAdamH). Wire bytes per parameter 4 + 2 instead of 8.
  GradReducer(Comm& comm, float* grad, int V, int D, int n_buckets, DType reduce_dtype, void* staging,
              bool to_owners = false);
  ~GradReducer();
  GradReducer(const GradReducer&) = delete;
  GradReducer& operator=(const GradReducer&) = delete;
  int n_buckets() const { return int(v0_.size()); }
  void range(int b, int& v0, int& v1) const { v0 = v0_[b]; v1 = v1_[b]; }
  bool to_owners() const { return to_owners_; }
  Comm& comm() const { return comm_; }
  int V() const { return V_; }
  int D() const { return D_; }
  // to_owners: this rank's element range of bucket b (offset into grad, length)
  void owned_range(int b, int64_t& offset, int64_t& len) const;
  // Bucket b of grad is final on `compute`: its all-reduce is enqueued on the communication stream behind an event.
  void bucket_ready(int b, cudaStream_t compute);
  void reduce_all(cudaStream_t compute);       // every bucket, after the work already on `compute`
  void wait(cudaStream_t st);                  // st waits for every bucket reduction enqueued so far
  // ZeRO-2 for this vocabulary-sized gradient (the reference declares it as GradReducer::microbatch_done,
  // include/marincpp/comm.hpp:52-53, "reduce-scatter those gradients after every microbatch", and does not implement it).
  // With a reduction to owners, attach the reducer to the backward of EVERY microbatch and call microbatch_done after
  // each: on `st`, once the bucket reductions enqueued so far are complete, this rank's owned elements of every bucket
  // are added into `owned_acc` (packed, bucket after bucket, owned_elems() f32) and the whole [V, D] buffer is set to
  // zero for the next microbatch. A rank's persistent gradient state is then owned_acc alone, 1 / nranks of V * D; the
  // [V, D] buffer is scratch between microbatches (it can be shared with anything else that is dead by then).
  int64_t owned_elems() const;
  void microbatch_done(float* owned_acc, cudaStream_t st);
  // Before the optimizer step: the packed sums go back into this rank's owned ranges of the gradient buffer, where an
  // optimizer on owned elements (HeadAdamH) reads them.
  void owned_to_grad(const float* owned_acc, cudaStream_t st);
 private:
  Comm& comm_;
  float* grad_;
  int V_, D_;
  DType dtype_;
  void* staging_;
  bool to_owners_ = false;
  std::vector<int> v0_, v1_;
  std::vector<cudaEvent_t> ready_;
  cudaEvent_t done_ = nullptr;
};

}  // namespace nm
