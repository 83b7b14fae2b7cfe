// Host side of the LM head's AdamH update (include/marincpp/kernels/head_optim.hpp) and its C ABI (capi_opt.h).
#include <cuda_runtime.h>

#include <charconv>
#include <cmath>
#include <cstdlib>
#include <string>
#include <vector>

#include "abi_guard.hpp"
#include "marincpp/capi_opt.h"
#include "marincpp/kernels/head_optim.hpp"
#include "opt_internal.hpp"

namespace nm {
namespace {

// The shortest decimal that reads back as the f32 value, as a double: 0.9f -> 0.9, so that 1 - b is formed in f64 from
// the decimal constant and rounded to f32 once, as the reference's source program does (docs/spec/optim.md:296-303;
// src/optim/capi_optim.cpp:61-67).
double decimal_of(float x) {
  char buf[48];
  const auto r = std::to_chars(buf, buf + sizeof(buf) - 1, x);
  NM_REQUIRE(r.ec == std::errc(), "adamh: decimal conversion failed");
  *r.ptr = '\0';
  return std::strtod(buf, nullptr);
}

opt::Hyper make_hyper(int64_t t, float eta, float b1, float b2, float eps, float grad_scale) {
  NM_REQUIRE(t >= 1 && t < (int64_t(1) << 24), "adamh: update count t must be in [1, 2^24)");
  NM_REQUIRE(b1 >= 0.f && b1 < 1.f && b2 >= 0.f && b2 < 1.f, "adamh: betas in [0, 1)");
  opt::Hyper h{};
  h.eta = eta;
  h.b1 = b1;
  h.b2 = b2;
  h.one_minus_b1 = static_cast<float>(1.0 - decimal_of(b1));
  h.one_minus_b2 = static_cast<float>(1.0 - decimal_of(b2));
  h.eps = static_cast<float>(decimal_of(eps));
  // 1 - b^t in f32 (src/optim/capi_optim.cpp:69-72); AdamH divides the factors out again in its projection
  h.bc1 = 1.0f - static_cast<float>(std::pow(static_cast<double>(b1), static_cast<double>(t)));
  h.bc2 = 1.0f - static_cast<float>(std::pow(static_cast<double>(b2), static_cast<double>(t)));
  h.grad_scale = grad_scale;
  h.max_norm = 1.f;
  h.clip_gn = 1.f;
  return h;
}

// Row blocks of a one-tensor call: validated on the host (block ids in range), as the reference does.
bool make_block_tab(const RowBlocks& rb, int64_t rows, cudaStream_t st, opt::BlockTab& bt) {
  if (!rb.block_of_row) {
    NM_REQUIRE(!rb.block_lr_mult && !rb.block_frozen && rb.n_blocks == 0,
               "optimizer update: block_lr_mult / block_frozen / n_blocks need block_of_row");
    return false;
  }
  NM_REQUIRE(rb.n_blocks > 0 && rb.n_blocks <= 65535, "optimizer update: n_blocks must be in [1, 65535] with block_of_row");
  std::vector<int32_t> host(static_cast<size_t>(rows));
  NM_CUDA(cudaMemcpyAsync(host.data(), rb.block_of_row, size_t(rows) * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
  NM_CUDA(cudaStreamSynchronize(st));
  for (int32_t b : host) NM_REQUIRE(b >= 0 && b < rb.n_blocks, "optimizer update: block_of_row out of range");
  bt = opt::BlockTab{rb.block_of_row, rb.block_lr_mult, rb.block_frozen, rb.n_blocks};
  return true;
}

}  // namespace

struct HeadAdamH::Impl {
  opt::Ranges r;
};

HeadAdamH::HeadAdamH(int V, int D, GradReducer* reducer) : impl_(new Impl), reducer_(reducer), V_(V), D_(D) {
  try {
    NM_REQUIRE(V > 0 && D > 0, "head adamh: V, D > 0");
    opt::Ranges& r = impl_->r;
    if (reducer) {
      NM_REQUIRE(reducer->to_owners(), "head adamh: the reducer must reduce to owners");
      NM_REQUIRE(reducer->V() == V && reducer->D() == D, "head adamh: the reducer covers another shape");
      NM_REQUIRE(reducer->n_buckets() <= opt::kMaxRanges, "head adamh: at most 64 buckets");
      r.n = reducer->n_buckets();
      int64_t c = 0;
      for (int b = 0; b < r.n; ++b) {
        reducer->owned_range(b, r.goff[b], r.len[b]);
        r.coff[b] = c;
        c += r.len[b];
      }
      owned_ = c;
    } else {
      r.n = 1;
      r.goff[0] = 0, r.coff[0] = 0, r.len[0] = int64_t(V) * D;
      owned_ = r.len[0];
    }
    NM_CUDA(cudaMalloc(&scal_, opt::kNumScalars * sizeof(double)));
    NM_CUDA(cudaMalloc(&partial_, size_t(opt::kMaxBlocksTotal) * 3 * sizeof(double)));
    NM_CUDA(cudaMemset(scal_, 0, opt::kNumScalars * sizeof(double)));
    NM_CUDA(cudaEventCreateWithFlags(&applied_, cudaEventDisableTiming));
    NM_CUDA(cudaEventCreateWithFlags(&gathered_, cudaEventDisableTiming));
  } catch (...) {
    if (applied_) cudaEventDestroy(applied_);
    if (gathered_) cudaEventDestroy(gathered_);
    if (scal_) cudaFree(scal_);
    if (partial_) cudaFree(partial_);
    delete impl_;
    throw;
  }
}

HeadAdamH::~HeadAdamH() {
  if (applied_) cudaEventDestroy(applied_);
  if (gathered_) cudaEventDestroy(gathered_);
  if (scal_) cudaFree(scal_);
  if (partial_) cudaFree(partial_);
  delete impl_;
}

int HeadAdamH::n_ranges() const { return impl_->r.n; }
void HeadAdamH::range(int i, int64_t& global_off, int64_t& compact_off, int64_t& len) const {
  NM_REQUIRE(i >= 0 && i < impl_->r.n, "head adamh: range index");
  global_off = impl_->r.goff[i], compact_off = impl_->r.coff[i], len = impl_->r.len[i];
}

void HeadAdamH::init_master(const bf16_t* w16, float* p_owned, cudaStream_t st) const {
  NM_REQUIRE(w16 && p_owned, "head adamh: w16 and p_owned required");
  opt::launch_master_from_bf16(impl_->r, w16, p_owned, st);
}

void HeadAdamH::step(const AdamHStep& s, const float* grad, float* p_owned, float* mu_owned, float* nu_owned,
                     bf16_t* w16, cudaStream_t st) {
  NM_REQUIRE(grad && p_owned && mu_owned && nu_owned, "head adamh: grad, p, mu, nu required");
  opt::Hyper h = make_hyper(s.t, s.eta, s.b1, s.b2, s.eps, s.grad_scale);
  if (s.bc1 > 0.f) h.bc1 = s.bc1;
  if (s.bc2 > 0.f) h.bc2 = s.bc2;
  const opt::Ranges& r = impl_->r;
  Comm* comm = reducer_ && reducer_->comm().nranks() > 1 ? &reducer_->comm() : nullptr;
  if (reducer_) reducer_->wait(st);
  if (s.max_grad_norm > 0.f) {
    // the head is its own clip group (docs/spec/optim.md:151-165): gn = ||g * grad_scale|| over the whole tensor
    opt::launch_sumsq(grad, r, h.grad_scale, partial_, scal_ + opt::kSumG, false, st);
    if (comm) comm->allreduce_sum(scal_ + opt::kSumG, 1, DType::f64, st);
    h.clip_mode = 2;
    h.max_norm = s.max_grad_norm;
  }
  opt::launch_moments(r, grad, p_owned, mu_owned, nu_owned, h, scal_, partial_, st);
  if (comm) comm->allreduce_sum(scal_ + opt::kSumPP, 3, DType::f64, st);
  opt::launch_apply(r, p_owned, mu_owned, nu_owned, w16, h, scal_, st);
  if (comm && w16) {
    // every bucket of the bf16 replica is completed from its owners' parts
    cudaStream_t gs = st;
    if (s.gather_on_comm_stream) {
      gs = comm->stream();
      NM_CUDA(cudaEventRecord(applied_, st));
      NM_CUDA(cudaStreamWaitEvent(gs, applied_, 0));
    }
    comm->group_start();
    for (int b = 0; b < r.n; ++b) {
      int v0, v1;
      reducer_->range(b, v0, v1);
      comm->allgather(w16 + int64_t(v0) * D_, r.len[b], DType::bf16, gs);
    }
    comm->group_end();
    if (s.gather_on_comm_stream) {
      NM_CUDA(cudaEventRecord(gathered_, gs));
      gather_pending_ = true;
    }
  }
}

void HeadAdamH::wait_params(cudaStream_t st) {
  if (!gather_pending_) return;
  NM_CUDA(cudaStreamWaitEvent(st, gathered_, 0));
  gather_pending_ = false;
}

void adamh_update(float* p, bf16_t* p16, const float* g, float* mu, float* nu, int64_t rows, int64_t cols, int64_t t,
                  float eta, float b1, float b2, float eps, float clip_gn, bool clip, float max_norm, cudaStream_t st,
                  const RowBlocks& blocks) {
  NM_REQUIRE(p && g && mu && nu, "adamh_update: p, g, mu, nu required");
  NM_REQUIRE(rows > 0 && cols > 0, "adamh_update: rows, cols > 0");
  opt::Hyper h = make_hyper(t, eta, b1, b2, eps, 1.0f);
  h.clip_mode = 1;
  h.clip = clip ? 1 : 0;
  h.clip_gn = clip_gn;
  h.max_norm = max_norm;
  opt::BlockTab bt{};
  if (make_block_tab(blocks, rows, st, bt)) {
    double* scratch = nullptr;
    const size_t n_doubles = size_t(rows) * 3 + size_t(bt.n_blocks) * 3;
    NM_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&scratch), n_doubles * sizeof(double), st));
    try {
      opt::launch_blk_adamh(g, p, mu, nu, p16, rows, cols, h, bt, scratch, scratch + size_t(rows) * 3, st);
    } catch (...) {
      cudaFreeAsync(scratch, st);
      throw;
    }
    NM_CUDA(cudaFreeAsync(scratch, st));
    return;
  }
  opt::Ranges r;
  r.n = 1;
  r.goff[0] = 0, r.coff[0] = 0, r.len[0] = rows * cols;
  // scratch for the block partials and the scalars, stream-ordered (no host synchronisation)
  double* scratch = nullptr;
  const size_t bytes = (size_t(opt::kMaxBlocksTotal) * 3 + opt::kNumScalars) * sizeof(double);
  NM_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&scratch), bytes, st));
  double* scal = scratch + size_t(opt::kMaxBlocksTotal) * 3;
  try {
    opt::launch_moments(r, g, p, mu, nu, h, scal, scratch, st);
    opt::launch_apply(r, p, mu, nu, p16, h, scal, st);
  } catch (...) {
    cudaFreeAsync(scratch, st);
    throw;
  }
  NM_CUDA(cudaFreeAsync(scratch, st));
}

void adam_update(float* p, bf16_t* p16, const float* g, float* mu, float* nu, int64_t rows, int64_t cols, int64_t t,
                 float adam_lr, float b1, float b2, float eps, float clip_gn, bool clip, float max_norm, cudaStream_t st,
                 const RowBlocks& blocks) {
  NM_REQUIRE(p && g && mu && nu, "adam_update: p, g, mu, nu required");
  NM_REQUIRE(rows > 0 && cols > 0, "adam_update: rows, cols > 0");
  opt::Hyper h = make_hyper(t, adam_lr, b1, b2, eps, 1.0f);
  h.clip_mode = 1;
  h.clip = clip ? 1 : 0;
  h.clip_gn = clip_gn;
  h.max_norm = max_norm;
  opt::BlockTab bt{};
  if (make_block_tab(blocks, rows, st, bt)) {
    opt::launch_blk_adam(g, p, mu, nu, p16, rows, cols, h, bt, st);
    return;
  }
  opt::Ranges r;
  r.n = 1;
  r.goff[0] = 0, r.coff[0] = 0, r.len[0] = rows * cols;
  opt::launch_adam(r, g, p, mu, nu, p16, h, nullptr, st);
}

}  // namespace nm

// ------------------------------------------------------------------------------------------------ C ABI
namespace {
cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }
nm::HeadAdamH* H(void* h) {
  NM_REQUIRE(h, "head adamh: null handle");
  return static_cast<nm::HeadAdamH*>(h);
}
}  // namespace

extern "C" {

int nm_adamh_update(float* p, void* p16, const float* g, float* mu, float* nu, int64_t rows, int64_t cols, int64_t t,
                    float eta, float b1, float b2, float eps, float clip_gn, int clip, float max_norm,
                    const int32_t* block_of_row, const float* block_lr_mult, const uint8_t* block_frozen, int n_blocks,
                    void* stream) {
  return nm::abi::guarded([&] {
    nm::adamh_update(p, static_cast<nm::bf16_t*>(p16), g, mu, nu, rows, cols, t, eta, b1, b2, eps, clip_gn, clip != 0,
                     max_norm, S(stream), nm::RowBlocks{block_of_row, block_lr_mult, block_frozen, n_blocks});
  });
}

int nm_adam_update(float* p, void* p16, const float* g, float* mu, float* nu, int64_t rows, int64_t cols, int64_t t,
                   float adam_lr, float b1, float b2, float eps, float clip_gn, int clip, float max_norm,
                   const int32_t* block_of_row, const float* block_lr_mult, const uint8_t* block_frozen, int n_blocks,
                   void* stream) {
  return nm::abi::guarded([&] {
    nm::adam_update(p, static_cast<nm::bf16_t*>(p16), g, mu, nu, rows, cols, t, adam_lr, b1, b2, eps, clip_gn,
                    clip != 0, max_norm, S(stream), nm::RowBlocks{block_of_row, block_lr_mult, block_frozen, n_blocks});
  });
}

int nm_grad_reducer_create_owners(void* comm, float* grad, int V, int D, int n_buckets, void** reducer_out) {
  return nm::abi::guarded([&] {
    NM_REQUIRE(comm && reducer_out, "nm_grad_reducer_create_owners: comm and reducer_out required");
    *reducer_out =
        new nm::GradReducer(*static_cast<nm::Comm*>(comm), grad, V, D, n_buckets, nm::DType::f32, nullptr, true);
  });
}

int64_t nm_grad_reducer_owned_elems(void* reducer) {
  int64_t n = 0;
  const int rc = nm::abi::guarded([&] {
    NM_REQUIRE(reducer, "nm_grad_reducer_owned_elems: reducer required");
    n = static_cast<nm::GradReducer*>(reducer)->owned_elems();
  });
  return rc == NM_OK ? n : 0;
}
int nm_grad_reducer_microbatch_done(void* reducer, float* owned_acc, void* stream) {
  return nm::abi::guarded([&] {
    NM_REQUIRE(reducer, "nm_grad_reducer_microbatch_done: reducer required");
    static_cast<nm::GradReducer*>(reducer)->microbatch_done(owned_acc, static_cast<cudaStream_t>(stream));
  });
}
int nm_grad_reducer_owned_to_grad(void* reducer, const float* owned_acc, void* stream) {
  return nm::abi::guarded([&] {
    NM_REQUIRE(reducer, "nm_grad_reducer_owned_to_grad: reducer required");
    static_cast<nm::GradReducer*>(reducer)->owned_to_grad(owned_acc, static_cast<cudaStream_t>(stream));
  });
}

int nm_head_adamh_create(int V, int D, void* reducer, void** out) {
  return nm::abi::guarded([&] {
    NM_REQUIRE(out, "nm_head_adamh_create: out required");
    *out = new nm::HeadAdamH(V, D, static_cast<nm::GradReducer*>(reducer));
  });
}
int nm_head_adamh_destroy(void* h) {
  return nm::abi::guarded([&] { delete static_cast<nm::HeadAdamH*>(h); });
}
int64_t nm_head_adamh_owned_elems(void* h) {
  int64_t n = 0;
  return nm::abi::guarded([&] { n = H(h)->owned_elems(); }) == NM_OK ? n : 0;
}
int nm_head_adamh_ranges(void* h, int cap, int64_t* global_off_host, int64_t* compact_off_host, int64_t* len_host,
                         int* n_out) {
  return nm::abi::guarded([&] {
    NM_REQUIRE(global_off_host && compact_off_host && len_host && n_out, "nm_head_adamh_ranges: outputs required");
    const int n = H(h)->n_ranges();
    *n_out = n;
    for (int i = 0; i < n && i < cap; ++i) H(h)->range(i, global_off_host[i], compact_off_host[i], len_host[i]);
  });
}
int nm_head_adamh_init_master(void* h, const void* w16, float* p_owned, void* stream) {
  return nm::abi::guarded([&] { H(h)->init_master(static_cast<const nm::bf16_t*>(w16), p_owned, S(stream)); });
}
int nm_head_adamh_step(void* h, int64_t t, float eta, float b1, float b2, float eps, float max_grad_norm,
                       float grad_scale, const float* grad, float* p_owned, float* mu_owned, float* nu_owned, void* w16,
                       void* stream) {
  return nm::abi::guarded([&] {
    nm::AdamHStep s;
    s.t = t, s.eta = eta, s.b1 = b1, s.b2 = b2, s.eps = eps, s.max_grad_norm = max_grad_norm, s.grad_scale = grad_scale;
    H(h)->step(s, grad, p_owned, mu_owned, nu_owned, static_cast<nm::bf16_t*>(w16), S(stream));
  });
}
int nm_head_adamh_step_async(void* h, int64_t t, float eta, float b1, float b2, float eps, float max_grad_norm,
                             float grad_scale, const float* grad, float* p_owned, float* mu_owned, float* nu_owned,
                             void* w16, void* stream) {
  return nm::abi::guarded([&] {
    nm::AdamHStep s;
    s.t = t, s.eta = eta, s.b1 = b1, s.b2 = b2, s.eps = eps, s.max_grad_norm = max_grad_norm, s.grad_scale = grad_scale;
    s.gather_on_comm_stream = true;
    H(h)->step(s, grad, p_owned, mu_owned, nu_owned, static_cast<nm::bf16_t*>(w16), S(stream));
  });
}
int nm_head_adamh_wait_params(void* h, void* stream) {
  return nm::abi::guarded([&] { H(h)->wait_params(S(stream)); });
}
int nm_head_adamh_scalars(void* h, double* out4_host, void* stream) {
  return nm::abi::guarded([&] {
    NM_REQUIRE(out4_host, "nm_head_adamh_scalars: output required");
    NM_CUDA(cudaMemcpyAsync(out4_host, H(h)->scalars(), 4 * sizeof(double), cudaMemcpyDeviceToHost, S(stream)));
    NM_CUDA(cudaStreamSynchronize(S(stream)));
  });
}

}  // extern "C"
