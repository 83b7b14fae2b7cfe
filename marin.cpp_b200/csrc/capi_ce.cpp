// The extern "C" surface of the fused linear cross-entropy (include/marincpp/capi.h, capi_ce.h, capi_ew.h): integer
// codes are decoded into the C++ enums, the C++ layer (ce_api.cpp, ew_*.cu, comm.cpp) does the work, and
// abi::guarded turns whatever it throws into a status. The names, argument orders and code values are the reference's
// (include/marincpp/capi.h:93-98, src/kernels/cross_entropy/capi_ce.h:17-35).
#include <cuda_runtime.h>

#include <string>
#include <vector>

#include "abi_guard.hpp"
#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "marincpp/capi.h"
#include "marincpp/capi_ce.h"
#include "marincpp/capi_ew.h"
#include "marincpp/comm.hpp"

namespace {

using nm::abi::guarded;
using nm::abi::guarded_value;

cudaStream_t S(void* p) { return static_cast<cudaStream_t>(p); }

// An integer code of the C ABI with its legal range; `legend` lists what the values mean for the error message.
int code_in_range(const char* name, int value, int lo, int hi, const char* legend) {
  if (value < lo || value > hi)
    nm::fatal(NM_WHERE, std::string(name) + " = " + std::to_string(value) + " is not one of " + legend);
  return value;
}
nm::CeImpl impl_of(int code) {
  return static_cast<nm::CeImpl>(code_in_range("impl", code, 0, 3, "0 (A), 1 (B1), 2 (B1.5), 3 (B2)"));
}
nm::Rounding rounding_of(int code) {
  return code_in_range("rounding", code, 0, 1, "0 (levanter), 1 (accurate)") == 0 ? nm::Rounding::Levanter
                                                                                   : nm::Rounding::Accurate;
}
nm::DType dtype_of(int code, const char* name) {
  return code_in_range(name, code, 0, 1, "0 (f32), 1 (bf16)") == 0 ? nm::DType::f32 : nm::DType::bf16;
}
nm::CeShape shape_of(int io, int logits_store, int64_t T, int D, int V, int chunk_rows) {
  nm::CeShape s{};
  s.T = T;
  s.D = D;
  s.V = V;
  s.chunk_rows = chunk_rows;
  s.logits_store = dtype_of(logits_store, "logits_store");
  s.io = dtype_of(io, "io");
  return s;
}

// Both fused-CE entry points funnel into this: the plain one passes the neutral values of the three extensions.
struct CeExtras {
  float z_loss_weight = 0.f;
  int32_t ignore_index = INT32_MIN;
  void* dw_reducer = nullptr;
};

int fused_ce(int impl, int rounding, int io, int logits_store, const void* x, const void* w, const int32_t* targets,
             const float* weight, const float* grad_scale, const float* logit_bias, float* loss_tok, float* lse,
             float* loss_partial, void* dx, int accumulate_dx, float* dw, float* dw_microbatch, int dw_round,
             int forward_only, int64_t T, int D, int V, int chunk_rows, void* workspace, void* stream,
             const CeExtras& extra) {
  return guarded([&] {
    nm::CeArgs a{};
    a.x = x;
    a.w = w;
    a.targets = targets;
    a.weight = weight;
    a.grad_scale = grad_scale;
    a.logit_bias = logit_bias;
    a.loss_tok = loss_tok;
    a.lse = lse;
    a.loss_partial = loss_partial;
    a.dx = dx;
    a.accumulate_dx = accumulate_dx != 0;
    a.dw = dw;
    a.dw_microbatch = dw_microbatch;
    a.dw_round = code_in_range("dw_round", dw_round, 0, 1, "0 (none), 1 (per-chunk bf16)") ? nm::CeDwRound::PerChunkBf16
                                                                                           : nm::CeDwRound::None;
    a.forward_only = forward_only != 0;
    a.z_loss_weight = extra.z_loss_weight;
    a.ignore_index = extra.ignore_index;
    a.dw_reducer = extra.dw_reducer;
    nm::ce::run(impl_of(impl), rounding_of(rounding), shape_of(io, logits_store, T, D, V, chunk_rows), a, workspace,
                S(stream));
  });
}

}  // namespace

extern "C" {

uint64_t nm_ce_workspace_bytes(int impl, int64_t T, int D, int V, int chunk_rows, int logits_store) {
  return guarded_value<uint64_t>(0, [&] {
    // sized for bf16 io; implementation A's layout always includes what its f32-io form adds
    return nm::ce_workspace_bytes(impl_of(impl), shape_of(1, logits_store, T, D, V, chunk_rows));
  });
}

int nm_fused_linear_ce(int impl, int rounding, int io, int logits_store, const void* x, const void* w,
                       const int32_t* targets, const float* weight, const float* grad_scale, const float* logit_bias,
                       float* loss_tok, float* lse, float* loss_partial, void* dx, int accumulate_dx, float* dw,
                       float* dw_microbatch, int dw_round, int forward_only, int64_t T, int D, int V, int chunk_rows,
                       void* workspace, void* stream) {
  return fused_ce(impl, rounding, io, logits_store, x, w, targets, weight, grad_scale, logit_bias, loss_tok, lse,
                  loss_partial, dx, accumulate_dx, dw, dw_microbatch, dw_round, forward_only, T, D, V, chunk_rows,
                  workspace, stream, CeExtras{});
}

int nm_fused_linear_ce_ex(int impl, int rounding, int io, int logits_store, const void* x, const void* w,
                          const int32_t* targets, const float* weight, const float* grad_scale,
                          const float* logit_bias, float* loss_tok, float* lse, float* loss_partial, void* dx,
                          int accumulate_dx, float* dw, float* dw_microbatch, int dw_round, int forward_only,
                          int64_t T, int D, int V, int chunk_rows, void* workspace, void* stream,
                          float z_loss_weight, int32_t ignore_index, void* dw_reducer) {
  return fused_ce(impl, rounding, io, logits_store, x, w, targets, weight, grad_scale, logit_bias, loss_tok, lse,
                  loss_partial, dx, accumulate_dx, dw, dw_microbatch, dw_round, forward_only, T, D, V, chunk_rows,
                  workspace, stream, CeExtras{z_loss_weight, ignore_index, dw_reducer});
}

// One kernel set exists, so the reference's backend switches are bookkeeping: stored, and handed back on the next call.
int nm_ce_set_backends(int dgrad_own, int wgrad_own, int sm90) {
  return nm::ce::exchange_backends(dgrad_own, wgrad_own, sm90);
}
int nm_ce_set_fast_stats_exp(int on) { return nm::ce::exchange_fast_stats_exp(on); }

int nm_ce_finish_microbatch(float* dw, float* dw_microbatch, int64_t n, void* stream) {
  return guarded([&] {
    NM_REQUIRE(dw != nullptr && dw_microbatch != nullptr, "nm_ce_finish_microbatch: both accumulators are required");
    NM_REQUIRE(n >= 0, "nm_ce_finish_microbatch: negative element count");
    nm::ce::launch_finish_microbatch(dw, dw_microbatch, n, S(stream));
  });
}

int nm_ce_grad_scale(const float* w, int64_t n, float mult, float* out, void* stream) {
  return guarded([&] {
    NM_REQUIRE(w != nullptr && out != nullptr, "nm_ce_grad_scale: the weights and the output scalar are required");
    NM_REQUIRE(n >= 0, "nm_ce_grad_scale: negative element count");
    nm::ce::launch_sum_scale(w, n, mult, out, S(stream));
  });
}

int nm_ce_readout(int impl, int rounding, int logits_store, const void* state, const void* norm_gain,
                  float* norm_rstd_ws, void* norm_out_ws, const void* w, float* dw, float* dgain_partial,
                  const float* grad_scale, void* d_state, int visible_dims, const int32_t* targets,
                  const float* weight, float* loss_tok, float* lse, float* loss_partial, int forward_only, int64_t T,
                  int D, int V, int chunk_rows, float eps, void* workspace, void* stream) {
  return guarded([&] {
    using B = nm::bf16_t;
    nm::ReadoutCall head{};
    head.layer = 0;
    head.state = static_cast<const B*>(state);
    head.norm_gain = static_cast<const B*>(norm_gain);
    head.norm_rstd_ws = norm_rstd_ws;
    head.norm_out_ws = static_cast<B*>(norm_out_ws);
    head.w = static_cast<const B*>(w);
    head.dw = dw;
    head.dgain_partial = dgain_partial;
    head.grad_scale = grad_scale;
    head.d_state = static_cast<B*>(d_state);
    head.visible_dims = visible_dims;
    nm::CeArgs shared{};   // what every head of a step has in common: the labels and where the losses go
    shared.targets = targets;
    shared.weight = weight;
    shared.loss_tok = loss_tok;
    shared.lse = lse;
    shared.loss_partial = loss_partial;
    shared.dw_round = nm::CeDwRound::None;
    shared.forward_only = forward_only != 0;
    nm::ce::readout(impl_of(impl), rounding_of(rounding), shape_of(1, logits_store, T, D, V, chunk_rows), head, shared,
                    eps, workspace, S(stream));
  });
}

int nm_ce_dlogits(int logits_store, void* store, int64_t ldS, const float* lse, const float* gscale,
                  const int32_t* targets, int rows, int V, void* stream) {
  return guarded([&] {
    NM_REQUIRE(store != nullptr && lse != nullptr && gscale != nullptr && targets != nullptr,
               "nm_ce_dlogits: store, lse, gscale and targets are required");
    NM_REQUIRE(rows >= 0 && V > 0 && ldS >= V && ldS % 8 == 0,
               "nm_ce_dlogits: rows >= 0, V > 0 and a row pitch ldS >= V that is a multiple of 8");
    nm::ce::DzArgs a{};
    a.store = store;
    a.ldS = ldS;
    a.store_f32 = dtype_of(logits_store, "logits_store") == nm::DType::f32;
    a.lse = lse;
    a.ga = gscale;   // dz = g (p - onehot): the same factor on both terms
    a.gb = gscale;
    a.targets = targets;
    a.rows = rows;
    a.V = V;
    nm::ce::launch_dlogits_inplace(a, S(stream));
  });
}

int nm_ce_device_arch(void) {
  return guarded_value<int>(0, [] { return nm::ce::device_arch(); });
}

int nm_ce_device_status(void* workspace, void* stream, uint32_t* status_host) {
  return guarded([&] {
    NM_REQUIRE(workspace && status_host, "nm_ce_device_status: workspace and status_host required");
    NM_CUDA(cudaMemcpyAsync(status_host, workspace, 4, cudaMemcpyDeviceToHost, S(stream)));
    NM_CUDA(cudaStreamSynchronize(S(stream)));
    if (*status_host)
      throw nm::DeviceError("fused CE: a bounded device-side wait ran out (status bits " + std::to_string(*status_host) +
                            ": 1 TMA producer, 2 UMMA issuer, 4 epilogue, 8 accumulator hand-back, 16 transform)");
  });
}

int nm_ce_profile_enable(int max_launches) {
  return guarded([&] { nm::ce::profile_enable(max_launches); });
}
int nm_ce_profile_read(double* ms_host, int* launches_host) {
  return guarded([&] {
    NM_REQUIRE(ms_host && launches_host, "nm_ce_profile_read: two host arrays of 6 entries required");
    nm::ce::profile_read(ms_host, launches_host);
  });
}

int nm_ce_test_wait_timeout(uint32_t* status, int64_t limit_cycles, int* saw_abort, void* stream) {
  return guarded(
      [&] { nm::ce::launch_wait_timeout_probe(status, static_cast<long long>(limit_cycles), saw_abort, S(stream)); });
}

int nm_ce_suggest_chunk_rows(int64_t T) {
  int rows = 0;
  const int rc = guarded([&] {
    const int64_t full = int64_t(128) * nm::ce::sm_count();
    rows = int(T < full ? (T > 0 ? T : 1) : full);
  });
  return rc == NM_OK ? rows : 0;
}

int nm_ce_set_cta_pair(int logits, int dgrad, int wgrad) {
  return guarded([&] { nm::ce::set_cta_pair(logits, dgrad, wgrad); });
}

int nm_ce_set_tail_order(int order) {
  return guarded([&] { nm::ce::set_tail_order(order); });
}

int nm_ce_set_grad_path(int path) {
  return guarded([&] { nm::ce::set_grad_path(path); });
}

int nm_ce_test_gemm(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc, int M,
                    int N, int K, uint32_t* status, const void* row_factors, void* stream) {
  return guarded([&] {
    NM_REQUIRE(a && b && c, "nm_ce_test_gemm: a, b, c required");
    NM_REQUIRE(reinterpret_cast<uintptr_t>(row_factors) % 16 == 0, "nm_ce_test_gemm: row_factors must be 16-byte aligned");
    nm::ce::launch_test_gemm(kind, a, lda, b, ldb, c, ldc, M, N, K, status,
                             static_cast<const nm::ce::RowFactors*>(row_factors), S(stream));
  });
}

// ---- RMSNorm pair of the readout head
int nm_rmsnorm_fwd(int dtype, int rounding, const void* x, const void* gain, void* y, float* rstd, int64_t T, int D,
                   float eps, void* stream) {
  return guarded([&] {
    if (dtype == 0)
      return nm::ew::rmsnorm_fwd_f32(static_cast<const float*>(x), static_cast<const float*>(gain), static_cast<float*>(y),
                                     rstd, T, D, eps, S(stream));
    NM_REQUIRE(dtype == 1, "nm_rmsnorm_fwd: storage 0 (f32) or 1 (bf16)");
    nm::ew::rmsnorm_fwd(static_cast<const nm::bf16_t*>(x), static_cast<const nm::bf16_t*>(gain),
                        static_cast<nm::bf16_t*>(y), rstd, T, D, eps, S(stream), rounding_of(rounding));
  });
}
int64_t nm_norm_partial_rows(int64_t T) {
  int64_t r = 0;
  return guarded([&] { r = nm::ew::norm_partial_rows(T); }) == NM_OK ? r : 0;
}
int nm_rmsnorm_bwd_add_partial(int dtype, int rounding, const void* dy, const void* x, const void* gain,
                               const float* rstd, const void* dres, void* dx, float* dgain_partial, int64_t T, int D,
                               float eps, void* stream) {
  return guarded([&] {
    if (dtype == 0)
      return nm::ew::rmsnorm_bwd_add_f32(static_cast<const float*>(dy), static_cast<const float*>(x),
                                         static_cast<const float*>(gain), rstd, static_cast<const float*>(dres),
                                         static_cast<float*>(dx), dgain_partial, T, D, eps, S(stream));
    NM_REQUIRE(dtype == 1, "nm_rmsnorm_bwd_add_partial: storage 0 (f32) or 1 (bf16)");
    nm::ew::rmsnorm_bwd_add(static_cast<const nm::bf16_t*>(dy), static_cast<const nm::bf16_t*>(x),
                            static_cast<const nm::bf16_t*>(gain), rstd, static_cast<const nm::bf16_t*>(dres),
                            static_cast<nm::bf16_t*>(dx), dgain_partial, T, D, eps, S(stream), rounding_of(rounding));
  });
}

int nm_rmsnorm_bwd_add(int dtype, int rounding, const void* dy, const void* x, const void* gain, const float* rstd,
                       const void* dres, void* dx, float* dgain, int64_t T, int D, float eps, void* stream) {
  return guarded([&] {
    NM_REQUIRE(dtype == 0 || dtype == 1, "nm_rmsnorm_bwd_add: storage 0 (f32) or 1 (bf16)");
    const nm::Rounding r = rounding_of(rounding);
    const int64_t rows = nm::ew::norm_partial_rows(T);
    float* part = nullptr;   // test path, as in the reference: the partial buffer is a stream-ordered allocation
    if (dgain) NM_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&part), size_t(rows) * D * 4, S(stream)));
    if (dtype == 0)
      nm::ew::rmsnorm_bwd_add_f32(static_cast<const float*>(dy), static_cast<const float*>(x),
                                  static_cast<const float*>(gain), rstd, static_cast<const float*>(dres),
                                  static_cast<float*>(dx), part, T, D, eps, S(stream));
    else
      nm::ew::rmsnorm_bwd_add(static_cast<const nm::bf16_t*>(dy), static_cast<const nm::bf16_t*>(x),
                              static_cast<const nm::bf16_t*>(gain), rstd, static_cast<const nm::bf16_t*>(dres),
                              static_cast<nm::bf16_t*>(dx), part, T, D, eps, S(stream), r);
    if (dgain) {
      // the reduced gain gradient is a bf16 value only where the gains are stored in bf16 under levanter rounding
      nm::ew::reduce_partials_rows(part, int(rows), D, dgain, false, dtype == 1 && r == nm::Rounding::Levanter, S(stream));
      NM_CUDA(cudaFreeAsync(part, S(stream)));
    }
  });
}
int nm_sandwich_tail_fwd(int dtype, int rounding, const void* branch, const void* x_in, const void* g_post,
                         const void* g_next, void* x_out, void* a_next, float* rstd_post, float* rstd_next, int64_t T,
                         int D, float eps, void* stream) {
  return guarded([&] {
    auto F = [](const void* p) { return static_cast<const float*>(p); };
    if (dtype == 0)
      return nm::ew::sandwich_tail_fwd_f32(F(branch), F(x_in), F(g_post), F(g_next), static_cast<float*>(x_out),
                                           static_cast<float*>(a_next), rstd_post, rstd_next, T, D, eps, S(stream));
    NM_REQUIRE(dtype == 1, "nm_sandwich_tail_fwd: storage 0 (f32) or 1 (bf16)");
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
  return guarded([&] {
    NM_REQUIRE(dtype == 0 || dtype == 1, "nm_sandwich_tail_bwd: storage 0 (f32) or 1 (bf16)");
    const nm::Rounding r = rounding_of(rounding);
    const int64_t rows = nm::ew::norm_partial_rows(T);
    float* part = nullptr;   // test path: two partial buffers in one stream-ordered allocation
    const bool want_partials = dg_next || (dg_post && g_post);
    if (want_partials) NM_CUDA(cudaMallocAsync(reinterpret_cast<void**>(&part), size_t(rows) * D * 4 * 2, S(stream)));
    float* pn = part;
    float* pp = part + size_t(rows) * D;
    auto B = [](const void* p) { return static_cast<const nm::bf16_t*>(p); };
    auto F = [](const void* p) { return static_cast<const float*>(p); };
    if (dtype == 0)
      nm::ew::sandwich_tail_bwd_f32(F(dx_out), F(da_next), F(x_out), F(g_next), rstd_next, F(branch), F(g_post), rstd_post,
                                    static_cast<float*>(dx_in), static_cast<float*>(dbranch), dg_next ? pn : nullptr,
                                    (dg_post && g_post) ? pp : nullptr, T, D, eps, S(stream));
    else
      nm::ew::sandwich_tail_bwd(B(dx_out), B(da_next), B(x_out), B(g_next), rstd_next, B(branch), B(g_post), rstd_post,
                                static_cast<nm::bf16_t*>(dx_in), static_cast<nm::bf16_t*>(dbranch), dg_next ? pn : nullptr,
                                (dg_post && g_post) ? pp : nullptr, T, D, eps, S(stream), r);
    const bool rbf = dtype == 1 && r == nm::Rounding::Levanter;
    if (dg_next) nm::ew::reduce_partials_rows(pn, int(rows), D, dg_next, false, rbf, S(stream));
    if (dg_post && g_post) nm::ew::reduce_partials_rows(pp, int(rows), D, dg_post, false, rbf, S(stream));
    if (want_partials) NM_CUDA(cudaFreeAsync(part, S(stream)));
  });
}
int nm_sandwich_tail_bwd_partial(int dtype, int rounding, const void* dx_out, const void* da_next, const void* x_out,
                                 const void* g_next, const float* rstd_next, const void* branch, const void* g_post,
                                 const float* rstd_post, void* dx_in, void* dbranch, float* pg_next, float* pg_post,
                                 int64_t T, int D, float eps, void* stream) {
  return guarded([&] {
    auto F = [](const void* p) { return static_cast<const float*>(p); };
    if (dtype == 0)
      return nm::ew::sandwich_tail_bwd_f32(F(dx_out), F(da_next), F(x_out), F(g_next), rstd_next, F(branch), F(g_post),
                                           rstd_post, static_cast<float*>(dx_in), static_cast<float*>(dbranch), pg_next,
                                           pg_post, T, D, eps, S(stream));
    NM_REQUIRE(dtype == 1, "nm_sandwich_tail_bwd_partial: storage 0 (f32) or 1 (bf16)");
    auto B = [](const void* p) { return static_cast<const nm::bf16_t*>(p); };
    nm::ew::sandwich_tail_bwd(B(dx_out), B(da_next), B(x_out), B(g_next), rstd_next, B(branch), B(g_post), rstd_post,
                              static_cast<nm::bf16_t*>(dx_in), static_cast<nm::bf16_t*>(dbranch), pg_next, pg_post, T, D,
                              eps, S(stream), rounding_of(rounding));
  });
}
int nm_doc_meta(const int32_t* tokens, const uint8_t* row_valid, int rows, int S_, int32_t eos, int max_segs,
                int32_t* targets, float* weight, int32_t* pos, int32_t* cu_seqlens, int32_t* n_segs,
                int32_t* row_seg_start, uint32_t* overflow, void* stream) {
  return guarded([&] {
    nm::ew::doc_meta(tokens, row_valid, rows, S_, eos, max_segs, targets, weight, pos, cu_seqlens, n_segs,
                     row_seg_start, overflow, S(stream));
  });
}
int nm_norm_bwd_device_status(void* stream, uint32_t* status_host) {
  return guarded([&] {
    NM_REQUIRE(status_host != nullptr, "nm_norm_bwd_device_status: status_host is required");
    *status_host = nm::ew::read_row_status(S(stream));
    if (*status_host != 0)
      throw nm::DeviceError("norm backward: a bounded device-side wait ran out (status bits " +
                            std::to_string(*status_host) + "); the gradients of that call are invalid");
  });
}
// Test hook: runs the short bounded-wait probe of nm_ce_test_wait_timeout against the norm kernels' status word, so that
// the word afterwards holds what a norm backward kernel whose wait ran out would have left.
int nm_norm_bwd_test_timeout(int64_t limit_cycles, void* stream) {
  return guarded([&] {
    uint32_t* word = nm::ew::row_status_word();
    nm::ce::launch_wait_timeout_probe(word, static_cast<long long>(limit_cycles), reinterpret_cast<int*>(word + 1),
                                      S(stream));
  });
}
int nm_sum_fixed(const float* x, int64_t n, float* out, void* stream) {
  return guarded([&] { nm::ew::sum_fixed(x, n, out, S(stream)); });
}
int nm_reduce_partials_rows(const float* partial, int n_blocks, int width, float* out, int accumulate, int round_bf16,
                            void* stream) {
  return guarded([&] {
    nm::ew::reduce_partials_rows(partial, n_blocks, width, out, accumulate != 0, round_bf16 != 0, S(stream));
  });
}

// ---- data-parallel dW reduction
int nm_comm_unique_id(void* id128_host) {
  return guarded([&] { nm::Comm::unique_id(id128_host); });
}
int nm_comm_create(const void* id128_host, int nranks, int rank, void** comm_out) {
  return guarded([&] {
    NM_REQUIRE(comm_out, "nm_comm_create: comm_out required");
    *comm_out = new nm::Comm(id128_host, nranks, rank);
  });
}
int nm_comm_destroy(void* comm) {
  return guarded([&] { delete static_cast<nm::Comm*>(comm); });
}
int nm_comm_allreduce_f32(void* comm, float* buf, int64_t n, void* stream) {
  return guarded([&] {
    NM_REQUIRE(comm && buf, "nm_comm_allreduce_f32: comm and buf required");
    static_cast<nm::Comm*>(comm)->allreduce_sum(buf, n, nm::DType::f32, S(stream));
  });
}
int nm_grad_reducer_create(void* comm, float* grad, int V, int D, int n_buckets, int reduce_dtype, void* staging,
                           void** reducer_out) {
  return guarded([&] {
    NM_REQUIRE(comm && reducer_out, "nm_grad_reducer_create: comm and reducer_out required");
    *reducer_out = new nm::GradReducer(*static_cast<nm::Comm*>(comm), grad, V, D, n_buckets,
                                       dtype_of(reduce_dtype, "reduce_dtype"), staging);
  });
}
int nm_grad_bucket_ranges(int V, int n_buckets, int* v0_host, int* v1_host, int* n_out) {
  return guarded([&] {
    NM_REQUIRE(v0_host && v1_host && n_out, "nm_grad_bucket_ranges: output arrays required");
    std::vector<int> a, b;
    *n_out = nm::grad_bucket_ranges(V, n_buckets, a, b);
    for (int i = 0; i < *n_out; ++i) { v0_host[i] = a[size_t(i)]; v1_host[i] = b[size_t(i)]; }
  });
}
int nm_grad_reducer_destroy(void* reducer) {
  return guarded([&] { delete static_cast<nm::GradReducer*>(reducer); });
}
int nm_grad_reducer_reduce_all(void* reducer, void* stream) {
  return guarded([&] {
    NM_REQUIRE(reducer, "nm_grad_reducer_reduce_all: reducer required");
    static_cast<nm::GradReducer*>(reducer)->reduce_all(S(stream));
  });
}
int nm_grad_reducer_wait(void* reducer, void* stream) {
  return guarded([&] {
    NM_REQUIRE(reducer, "nm_grad_reducer_wait: reducer required");
    static_cast<nm::GradReducer*>(reducer)->wait(S(stream));
  });
}

}  // extern "C"
