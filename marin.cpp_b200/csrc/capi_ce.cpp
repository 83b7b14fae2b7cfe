// C ABI of the fused linear cross-entropy (include/marincpp/capi.h, capi_ce.h). Argument validation mirrors the
// reference's src/kernels/cross_entropy/capi_ce.cpp:15-31.
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "capi_util.hpp"
#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "marincpp/capi.h"
#include "marincpp/capi_ce.h"
#include "marincpp/capi_ew.h"
#include "marincpp/comm.hpp"

namespace {

cudaStream_t S(void* p) { return static_cast<cudaStream_t>(p); }

nm::CeImpl impl_of(int i) {
  if (i < 0 || i > 3) nm::fatal(NM_WHERE, "impl must be 0 (A), 1 (B1), 2 (B1.5) or 3 (B2), got " + std::to_string(i));
  return static_cast<nm::CeImpl>(i);
}
nm::Rounding rounding_of(int r) {
  if (r != 0 && r != 1) nm::fatal(NM_WHERE, "rounding must be 0 (levanter) or 1 (accurate), got " + std::to_string(r));
  return r == 0 ? nm::Rounding::Levanter : nm::Rounding::Accurate;
}
nm::DType dtype_of(int d, const char* what) {
  if (d != 0 && d != 1) nm::fatal(NM_WHERE, std::string(what) + " must be 0 (f32) or 1 (bf16), got " + std::to_string(d));
  return d == 0 ? nm::DType::f32 : nm::DType::bf16;
}
nm::CeShape shape(int io, int logits_store, int64_t T, int D, int V, int chunk_rows) {
  return nm::CeShape{T, D, V, chunk_rows, dtype_of(logits_store, "logits_store"), dtype_of(io, "io")};
}

int ce_call(int impl, int rounding, int io, int logits_store, const void* x, const void* w, const int32_t* targets,
            const float* weight, const float* grad_scale, const float* logit_bias, float* loss_tok, float* lse,
            float* loss_partial, void* dx, int accumulate_dx, float* dw, float* dw_microbatch, int dw_round,
            int forward_only, int64_t T, int D, int V, int chunk_rows, void* workspace, void* stream,
            float z_loss_weight, int32_t ignore_index, void* dw_reducer) {
  return nm::capi_call([&] {
    if (dw_round != 0 && dw_round != 1) nm::fatal(NM_WHERE, "dw_round must be 0 or 1");
    nm::CeArgs a{x, w, targets, weight, grad_scale, logit_bias, loss_tok, lse, loss_partial, dx, accumulate_dx != 0,
                 dw, dw_microbatch, dw_round ? nm::CeDwRound::PerChunkBf16 : nm::CeDwRound::None, forward_only != 0,
                 z_loss_weight, ignore_index, dw_reducer};
    nm::ce::run(impl_of(impl), rounding_of(rounding), shape(io, logits_store, T, D, V, chunk_rows), a, workspace,
                S(stream));
  });
}

}  // namespace

extern "C" {

uint64_t nm_ce_workspace_bytes(int impl, int64_t T, int D, int V, int chunk_rows, int logits_store) {
  uint64_t r = 0;
  const int st = nm::capi_call(
      [&] { r = nm::ce_workspace_bytes(impl_of(impl), shape(1, logits_store, T, D, V, chunk_rows)); });
  return st == NM_OK ? r : 0;
}

int nm_fused_linear_ce(int impl, int rounding, int io, int logits_store, const void* x, const void* w,
                       const int32_t* targets, const float* weight, const float* grad_scale, const float* logit_bias,
                       float* loss_tok, float* lse, float* loss_partial, void* dx, int accumulate_dx, float* dw,
                       float* dw_microbatch, int dw_round, int forward_only, int64_t T, int D, int V, int chunk_rows,
                       void* workspace, void* stream) {
  return ce_call(impl, rounding, io, logits_store, x, w, targets, weight, grad_scale, logit_bias, loss_tok, lse,
                 loss_partial, dx, accumulate_dx, dw, dw_microbatch, dw_round, forward_only, T, D, V, chunk_rows,
                 workspace, stream, 0.f, INT32_MIN, nullptr);
}

int nm_fused_linear_ce_ex(int impl, int rounding, int io, int logits_store, const void* x, const void* w,
                          const int32_t* targets, const float* weight, const float* grad_scale,
                          const float* logit_bias, float* loss_tok, float* lse, float* loss_partial, void* dx,
                          int accumulate_dx, float* dw, float* dw_microbatch, int dw_round, int forward_only,
                          int64_t T, int D, int V, int chunk_rows, void* workspace, void* stream,
                          float z_loss_weight, int32_t ignore_index, void* dw_reducer) {
  return ce_call(impl, rounding, io, logits_store, x, w, targets, weight, grad_scale, logit_bias, loss_tok, lse,
                 loss_partial, dx, accumulate_dx, dw, dw_microbatch, dw_round, forward_only, T, D, V, chunk_rows,
                 workspace, stream, z_loss_weight, ignore_index, dw_reducer);
}

int nm_ce_set_backends(int dgrad_own, int wgrad_own, int sm90) {
  auto& s = nm::ce::settings();
  const int prev = (s.dgrad_own ? 1 : 0) | (s.wgrad_own ? 1 : 0) << 1 | s.sm90 << 2;
  s.dgrad_own = dgrad_own != 0;
  s.wgrad_own = wgrad_own != 0;
  if (sm90 >= 0) s.sm90 = sm90 & 3;
  return prev;
}

int nm_ce_set_fast_stats_exp(int on) {
  const int prev = nm::ce::settings().fast_stats_exp;
  nm::ce::settings().fast_stats_exp = on != 0;
  return prev;
}

int nm_ce_finish_microbatch(float* dw, float* dw_microbatch, int64_t n, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(dw && dw_microbatch && n >= 0, "nm_ce_finish_microbatch: dw, dw_microbatch, n >= 0");
    nm::ce::launch_finish_microbatch(dw, dw_microbatch, n, S(stream));
  });
}

int nm_ce_grad_scale(const float* w, int64_t n, float mult, float* out, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(w && out && n >= 0, "nm_ce_grad_scale: w, out, n >= 0");
    nm::ce::launch_sum_scale(w, n, mult, out, S(stream));
  });
}

int nm_ce_readout(int impl, int rounding, int logits_store, const void* state, const void* norm_gain,
                  float* norm_rstd_ws, void* norm_out_ws, const void* w, float* dw, float* dgain_partial,
                  const float* grad_scale, void* d_state, int visible_dims, const int32_t* targets,
                  const float* weight, float* loss_tok, float* lse, float* loss_partial, int forward_only, int64_t T,
                  int D, int V, int chunk_rows, float eps, void* workspace, void* stream) {
  return nm::capi_call([&] {
    nm::ReadoutCall c{0, static_cast<const nm::bf16_t*>(state), static_cast<const nm::bf16_t*>(norm_gain), norm_rstd_ws,
                      static_cast<nm::bf16_t*>(norm_out_ws), static_cast<const nm::bf16_t*>(w), dw, dgain_partial,
                      grad_scale, static_cast<nm::bf16_t*>(d_state), visible_dims};
    nm::CeArgs base{};
    base.targets = targets;
    base.weight = weight;
    base.loss_tok = loss_tok;
    base.lse = lse;
    base.loss_partial = loss_partial;
    base.dw_round = nm::CeDwRound::None;
    base.forward_only = forward_only != 0;
    nm::ce::readout(impl_of(impl), rounding_of(rounding), shape(1, logits_store, T, D, V, chunk_rows), c, base, eps,
                    workspace, S(stream));
  });
}

int nm_ce_dlogits(int logits_store, void* store, int64_t ldS, const float* lse, const float* gscale,
                  const int32_t* targets, int rows, int V, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(store && lse && gscale && targets && rows >= 0 && V > 0 && ldS >= V && ldS % 8 == 0,
               "nm_ce_dlogits: store, lse, gscale, targets, ldS >= V, ldS % 8 == 0");
    nm::ce::DzArgs a{store, ldS, dtype_of(logits_store, "logits_store") == nm::DType::f32, lse, gscale, gscale,
                     targets, rows, V};
    nm::ce::launch_dlogits_inplace(a, S(stream));
  });
}

int nm_ce_device_arch(void) {
  int a = 0;
  return nm::capi_call([&] { a = nm::ce::device_arch(); }) == NM_OK ? a : 0;
}

int nm_ce_device_status(void* workspace, void* stream, uint32_t* status_host) {
  return nm::capi_call([&] {
    NM_REQUIRE(workspace && status_host, "nm_ce_device_status: workspace and status_host required");
    NM_CUDA(cudaMemcpyAsync(status_host, workspace, 4, cudaMemcpyDeviceToHost, S(stream)));
    NM_CUDA(cudaStreamSynchronize(S(stream)));
    if (*status_host)
      throw nm::DeviceError("fused CE: a bounded device-side wait ran out (status bits " + std::to_string(*status_host) +
                            ": 1 TMA producer, 2 UMMA issuer, 4 epilogue, 8 accumulator hand-back)");
  });
}

int nm_ce_profile_enable(int max_launches) {
  return nm::capi_call([&] { nm::ce::profile_enable(max_launches); });
}
int nm_ce_profile_read(double* ms_host, int* launches_host) {
  return nm::capi_call([&] {
    NM_REQUIRE(ms_host && launches_host, "nm_ce_profile_read: two host arrays of 6 entries required");
    nm::ce::profile_read(ms_host, launches_host);
  });
}

int nm_ce_test_wait_timeout(uint32_t* status, int64_t limit_cycles, int* saw_abort, void* stream) {
  return nm::capi_call(
      [&] { nm::ce::launch_wait_timeout_probe(status, static_cast<long long>(limit_cycles), saw_abort, S(stream)); });
}

int nm_ce_suggest_chunk_rows(int64_t T) {
  int rows = 0;
  const int rc = nm::capi_call([&] {
    const int64_t full = int64_t(128) * nm::ce::sm_count();
    rows = int(T < full ? (T > 0 ? T : 1) : full);
  });
  return rc == NM_OK ? rows : 0;
}

int nm_ce_set_cta_pair(int logits, int dgrad, int wgrad) {
  return nm::capi_call([&] { nm::ce::set_cta_pair(logits, dgrad, wgrad); });
}

int nm_ce_test_gemm(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc, int M,
                    int N, int K, uint32_t* status, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(a && b && c, "nm_ce_test_gemm: a, b, c required");
    nm::ce::launch_test_gemm(kind, a, lda, b, ldb, c, ldc, M, N, K, status, S(stream));
  });
}

// ---- RMSNorm pair of the readout head
int nm_rmsnorm_fwd(int dtype, int rounding, const void* x, const void* gain, void* y, float* rstd, int64_t T, int D,
                   float eps, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(dtype == 1, "nm_rmsnorm_fwd: bf16 storage (dtype 1) only");
    nm::ew::rmsnorm_fwd(static_cast<const nm::bf16_t*>(x), static_cast<const nm::bf16_t*>(gain),
                        static_cast<nm::bf16_t*>(y), rstd, T, D, eps, S(stream), rounding_of(rounding));
  });
}
int64_t nm_norm_partial_rows(int64_t T) {
  int64_t r = 0;
  return nm::capi_call([&] { r = nm::ew::norm_partial_rows(T); }) == NM_OK ? r : 0;
}
int nm_rmsnorm_bwd_add_partial(int dtype, int rounding, const void* dy, const void* x, const void* gain,
                               const float* rstd, const void* dres, void* dx, float* dgain_partial, int64_t T, int D,
                               float eps, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(dtype == 1, "nm_rmsnorm_bwd_add_partial: bf16 storage (dtype 1) only");
    nm::ew::rmsnorm_bwd_add(static_cast<const nm::bf16_t*>(dy), static_cast<const nm::bf16_t*>(x),
                            static_cast<const nm::bf16_t*>(gain), rstd, static_cast<const nm::bf16_t*>(dres),
                            static_cast<nm::bf16_t*>(dx), dgain_partial, T, D, eps, S(stream), rounding_of(rounding));
  });
}

int nm_rmsnorm_bwd_add(int dtype, int rounding, const void* dy, const void* x, const void* gain, const float* rstd,
                       const void* dres, void* dx, float* dgain, int64_t T, int D, float eps, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(dtype == 1, "nm_rmsnorm_bwd_add: bf16 storage (dtype 1) only");
    const nm::Rounding r = rounding_of(rounding);
    const int64_t rows = nm::ew::norm_partial_rows(T);
    float* part = nullptr;   // test path, as in the reference: the partial buffer is a stream-ordered allocation
    if (dgain) NM_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&part), size_t(rows) * D * 4, S(stream)));
    nm::ew::rmsnorm_bwd_add(static_cast<const nm::bf16_t*>(dy), static_cast<const nm::bf16_t*>(x),
                            static_cast<const nm::bf16_t*>(gain), rstd, static_cast<const nm::bf16_t*>(dres),
                            static_cast<nm::bf16_t*>(dx), part, T, D, eps, S(stream), r);
    if (dgain) {
      nm::ew::reduce_partials_rows(part, int(rows), D, dgain, false, r == nm::Rounding::Levanter, S(stream));
      NM_CUDA(cudaFreeAsync(part, S(stream)));
    }
  });
}
int nm_sandwich_tail_fwd(int dtype, int rounding, const void* branch, const void* x_in, const void* g_post,
                         const void* g_next, void* x_out, void* a_next, float* rstd_post, float* rstd_next, int64_t T,
                         int D, float eps, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(dtype == 1, "nm_sandwich_tail_fwd: bf16 storage (dtype 1) only");
    auto B = [](const void* p) { return static_cast<const nm::bf16_t*>(p); };
    nm::ew::sandwich_tail_fwd(B(branch), B(x_in), B(g_post), B(g_next), static_cast<nm::bf16_t*>(x_out),
                              static_cast<nm::bf16_t*>(a_next), rstd_post, rstd_next, T, D, eps, S(stream),
                              rounding_of(rounding));
  });
}
int nm_sandwich_tail_bwd(int dtype, int rounding, const void* dx_out, const void* da_next, const void* x_out,
                         const void* g_next, const float* rstd_next, const void* branch, const void* g_post,
                         const float* rstd_post, void* dx_in, void* dbranch, float* dg_next, float* dg_post,
                         int64_t T, int D, float eps, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(dtype == 1, "nm_sandwich_tail_bwd: bf16 storage (dtype 1) only");
    const nm::Rounding r = rounding_of(rounding);
    const int64_t rows = nm::ew::norm_partial_rows(T);
    float* part = nullptr;   // test path: two partial buffers in one stream-ordered allocation
    NM_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&part), size_t(rows) * D * 4 * 2, S(stream)));
    float* pn = part;
    float* pp = part + size_t(rows) * D;
    auto B = [](const void* p) { return static_cast<const nm::bf16_t*>(p); };
    nm::ew::sandwich_tail_bwd(B(dx_out), B(da_next), B(x_out), B(g_next), rstd_next, B(branch), B(g_post), rstd_post,
                              static_cast<nm::bf16_t*>(dx_in), static_cast<nm::bf16_t*>(dbranch), dg_next ? pn : nullptr,
                              (dg_post && g_post) ? pp : nullptr, T, D, eps, S(stream), r);
    const bool rbf = r == nm::Rounding::Levanter;
    if (dg_next) nm::ew::reduce_partials_rows(pn, int(rows), D, dg_next, false, rbf, S(stream));
    if (dg_post && g_post) nm::ew::reduce_partials_rows(pp, int(rows), D, dg_post, false, rbf, S(stream));
    NM_CUDA(cudaFreeAsync(part, S(stream)));
  });
}
int nm_doc_meta(const int32_t* tokens, const uint8_t* row_valid, int rows, int S_, int32_t eos, int max_segs,
                int32_t* targets, float* weight, int32_t* pos, int32_t* cu_seqlens, int32_t* n_segs,
                int32_t* row_seg_start, uint32_t* overflow, void* stream) {
  return nm::capi_call([&] {
    nm::ew::doc_meta(tokens, row_valid, rows, S_, eos, max_segs, targets, weight, pos, cu_seqlens, n_segs,
                     row_seg_start, overflow, S(stream));
  });
}
int nm_sum_fixed(const float* x, int64_t n, float* out, void* stream) {
  return nm::capi_call([&] { nm::ew::sum_fixed(x, n, out, S(stream)); });
}
int nm_reduce_partials_rows(const float* partial, int n_blocks, int width, float* out, int accumulate, int round_bf16,
                            void* stream) {
  return nm::capi_call([&] {
    nm::ew::reduce_partials_rows(partial, n_blocks, width, out, accumulate != 0, round_bf16 != 0, S(stream));
  });
}

// ---- data-parallel dW reduction
int nm_comm_unique_id(void* id128_host) {
  return nm::capi_call([&] { nm::Comm::unique_id(id128_host); });
}
int nm_comm_create(const void* id128_host, int nranks, int rank, void** comm_out) {
  return nm::capi_call([&] {
    NM_REQUIRE(comm_out, "nm_comm_create: comm_out required");
    *comm_out = new nm::Comm(id128_host, nranks, rank);
  });
}
int nm_comm_destroy(void* comm) {
  return nm::capi_call([&] { delete static_cast<nm::Comm*>(comm); });
}
int nm_comm_allreduce_f32(void* comm, float* buf, int64_t n, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(comm && buf, "nm_comm_allreduce_f32: comm and buf required");
    static_cast<nm::Comm*>(comm)->allreduce_sum(buf, n, nm::DType::f32, S(stream));
  });
}
int nm_grad_reducer_create(void* comm, float* grad, int V, int D, int n_buckets, int reduce_dtype, void* staging,
                           void** reducer_out) {
  return nm::capi_call([&] {
    NM_REQUIRE(comm && reducer_out, "nm_grad_reducer_create: comm and reducer_out required");
    *reducer_out = new nm::GradReducer(*static_cast<nm::Comm*>(comm), grad, V, D, n_buckets,
                                       dtype_of(reduce_dtype, "reduce_dtype"), staging);
  });
}
int nm_grad_bucket_ranges(int V, int n_buckets, int* v0_host, int* v1_host, int* n_out) {
  return nm::capi_call([&] {
    NM_REQUIRE(v0_host && v1_host && n_out, "nm_grad_bucket_ranges: output arrays required");
    std::vector<int> a, b;
    *n_out = nm::grad_bucket_ranges(V, n_buckets, a, b);
    for (int i = 0; i < *n_out; ++i) { v0_host[i] = a[size_t(i)]; v1_host[i] = b[size_t(i)]; }
  });
}
int nm_grad_reducer_destroy(void* reducer) {
  return nm::capi_call([&] { delete static_cast<nm::GradReducer*>(reducer); });
}
int nm_grad_reducer_reduce_all(void* reducer, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(reducer, "nm_grad_reducer_reduce_all: reducer required");
    static_cast<nm::GradReducer*>(reducer)->reduce_all(S(stream));
  });
}
int nm_grad_reducer_wait(void* reducer, void* stream) {
  return nm::capi_call([&] {
    NM_REQUIRE(reducer, "nm_grad_reducer_wait: reducer required");
    static_cast<nm::GradReducer*>(reducer)->wait(S(stream));
  });
}

}  // extern "C"
