// Host side of the fused linear cross-entropy: workspace layout, argument checks, the per-chunk schedule, the readout
// head and the public C++ entry points of include/marincpp/kernels/cross_entropy.hpp. Behaviour follows the
// reference's src/kernels/cross_entropy/ce_api.cpp: check_shape :52-57, the requirements of run :133-145, the chunk
// loop :153-239 (dW before dX so dX may overwrite x), readout :243-275.
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <map>
#include <mutex>
#include <string>
#include <vector>

#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "marincpp/comm.hpp"

namespace nm {
namespace ce {
namespace {

int dev_attr(cudaDeviceAttr at) {
  static std::mutex mu;
  static std::map<std::pair<int, int>, int> cache;
  int dev = 0;
  NM_CUDA(cudaGetDevice(&dev));
  std::lock_guard<std::mutex> lk(mu);
  const auto key = std::make_pair(dev, int(at));
  auto it = cache.find(key);
  if (it != cache.end()) return it->second;
  int v = 0;
  NM_CUDA(cudaDeviceGetAttribute(&v, at, dev));
  cache[key] = v;
  return v;
}

const char* impl_name(CeImpl i) {
  switch (i) {
    case CeImpl::A: return "A";
    case CeImpl::B1: return "B1";
    case CeImpl::B1_5: return "B1.5";
    case CeImpl::B2: return "B2";
  }
  return "?";
}

void check_shape(CeImpl impl, const CeShape& s) {
  NM_REQUIRE(s.T >= 0 && s.D > 0 && s.V > 0, "fused CE: T >= 0, D > 0, V > 0");
  NM_REQUIRE(s.D % 8 == 0, "fused CE: D must be a multiple of 8");
  NM_REQUIRE(s.chunk_rows > 0, "fused CE: chunk_rows must be positive");
  NM_REQUIRE(s.logits_store == DType::bf16 || s.logits_store == DType::f32, "fused CE: logits store bf16 or f32");
  NM_REQUIRE(s.io == DType::bf16 || (s.io == DType::f32 && impl == CeImpl::A),
             std::string("fused CE: io f32 (the f32 policy) runs only implementation A, not ") + impl_name(impl));
}

template <class T>
T* byte_offset(T* p, int64_t bytes) {
  using B = std::conditional_t<std::is_const_v<T>, const uint8_t, uint8_t>;
  return p ? reinterpret_cast<T*>(reinterpret_cast<B*>(p) + bytes) : nullptr;
}

// extra regions of the f32-io path (implementation A only): split copies of the x chunk and of W
struct WsF32 {
  void* xs = nullptr;       // [chunk_rows, 3 D] bf16: (hi | hi | lo)
  void* wsplit = nullptr;   // [V, 3 D] bf16: (hi | lo | hi)
};

Ws carve_all(CeImpl impl, const CeShape& s, void* base, WsF32* f32) {
  Ws w;
  const int64_t rows = s.chunk_rows;
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) -> void* {
    off = uint64_t(round_up(int64_t(off), 256));
    void* p = base ? static_cast<uint8_t*>(base) + off : nullptr;
    off += bytes;
    return p;
  };
  w.status = static_cast<uint32_t*>(take(256));
  w.ldS = store_ld(s.V);
  w.store = take(uint64_t(rows) * w.ldS * dtype_size(s.logits_store));
  w.NT = stats_tiles(s.V);
  w.ldT = rows;
  w.tmax = static_cast<float*>(take(uint64_t(w.NT) * rows * 4));
  w.tsum = static_cast<float*>(take(uint64_t(w.NT) * rows * 4));
  w.lse = static_cast<float*>(take(uint64_t(rows) * 4));
  w.rowa = static_cast<float*>(take(uint64_t(rows) * 4));
  w.rowb = static_cast<float*>(take(uint64_t(rows) * 4));
  if (impl == CeImpl::A) {   // the C ABI sizes the workspace without knowing io, so A always carries the f32-io regions
    void* xs = take(uint64_t(rows) * 3 * s.D * 2);
    void* wsp = take(uint64_t(s.V) * 3 * s.D * 2);
    if (f32) { f32->xs = xs; f32->wsplit = wsp; }
  }
  off = uint64_t(round_up(int64_t(off), 256));
  w.bytes = off;
  return w;
}

}  // namespace

Ws carve(CeImpl impl, const CeShape& s, void* base) { return carve_all(impl, s, base, nullptr); }

int device_arch() {
  return dev_attr(cudaDevAttrComputeCapabilityMajor) * 10 + dev_attr(cudaDevAttrComputeCapabilityMinor);
}
int sm_count() { return dev_attr(cudaDevAttrMultiProcessorCount); }

Settings& settings() {
  static Settings s;
  return s;
}

// ------------------------------------------------------------------------------------------------ profiling
namespace {
struct Prof {
  std::mutex mu;
  std::vector<cudaEvent_t> ev;   // 2 per slot
  std::vector<int> cls;
  int used = 0;
  bool on = false;
} g_prof;
}  // namespace

void profile_enable(int max_launches) {
  std::lock_guard<std::mutex> lk(g_prof.mu);
  for (auto e : g_prof.ev) cudaEventDestroy(e);
  g_prof.ev.clear();
  g_prof.cls.assign(size_t(max_launches > 0 ? max_launches : 0), 0);
  g_prof.used = 0;
  g_prof.on = max_launches > 0;
  for (int i = 0; i < 2 * max_launches; ++i) {
    cudaEvent_t e;
    NM_CUDA(cudaEventCreate(&e));
    g_prof.ev.push_back(e);
  }
}

void profile_read(double* ms, int* launches) {
  std::lock_guard<std::mutex> lk(g_prof.mu);
  for (int c = 0; c < kProfClasses; ++c) { ms[c] = 0; launches[c] = 0; }
  for (int i = 0; i < g_prof.used; ++i) {
    NM_CUDA(cudaEventSynchronize(g_prof.ev[2 * i + 1]));
    float t = 0.f;
    NM_CUDA(cudaEventElapsedTime(&t, g_prof.ev[2 * i], g_prof.ev[2 * i + 1]));
    ms[g_prof.cls[i]] += t;
    launches[g_prof.cls[i]] += 1;
  }
  g_prof.used = 0;
}

// Every launch of the path also sits in an NVTX range named after its kernel class (header-only NVTX 3: a no-op
// unless a profiler is attached), so that ncu / nsys can select e.g. `--nvtx --nvtx-include "ce.logits/"`.
static const char* const kProfNames[kProfClasses] = {"ce.logits", "ce.finalize", "ce.dlogits", "ce.dw", "ce.dx",
                                                     "ce.chunk_loss"};

ProfScope::ProfScope(int cls, cudaStream_t st) : slot_(-1), st_(st) {
  nvtxRangePushA(kProfNames[cls]);
  if (!g_prof.on) return;
  std::lock_guard<std::mutex> lk(g_prof.mu);
  if (g_prof.used >= int(g_prof.cls.size())) return;
  slot_ = g_prof.used++;
  g_prof.cls[slot_] = cls;
  cudaEventRecord(g_prof.ev[2 * slot_], st_);
}
ProfScope::~ProfScope() {
  if (slot_ >= 0) cudaEventRecord(g_prof.ev[2 * slot_ + 1], st_);
  nvtxRangePop();
}

// ------------------------------------------------------------------------------------------------ one call
void run(CeImpl impl, Rounding r, const CeShape& s, const CeArgs& a, void* ws, cudaStream_t st) {
  check_shape(impl, s);
  if (s.T == 0) return;
  NM_REQUIRE(a.x && a.w && a.targets && a.weight && a.loss_tok && ws, "fused CE: x, w, targets, weight, loss_tok and "
                                                                       "the workspace are required");
  const bool grads = !a.forward_only && (a.dx || a.dw);
  const bool strict_dw = a.dw && a.dw_round == CeDwRound::PerChunkBf16;
  if (grads) NM_REQUIRE(a.grad_scale, "fused CE: gradients need grad_scale");
  if (strict_dw) NM_REQUIRE(a.dw_microbatch && s.io == DType::bf16,
                            "fused CE: CeDwRound::PerChunkBf16 needs dw_microbatch (and bf16 io)");
  NM_REQUIRE(!(a.dx && a.dx == a.x && a.accumulate_dx), "fused CE: dx == x cannot accumulate");
  if (impl != CeImpl::A) NM_REQUIRE(!a.logit_bias, "fused CE: logit_bias is implemented only by implementation A");
  NM_REQUIRE(reinterpret_cast<uintptr_t>(ws) % 256 == 0, "fused CE: the workspace must be 256-byte aligned");
  // x, w and dw are checked where their tensor maps are made; dx is written with 16-byte vector stores
  NM_REQUIRE(reinterpret_cast<uintptr_t>(a.dx) % 16 == 0, "fused CE: dx must be 16-byte aligned");
  NM_REQUIRE(reinterpret_cast<uintptr_t>(a.dw_microbatch) % 16 == 0, "fused CE: dw_microbatch must be 16-byte aligned");
  NM_REQUIRE(device_arch() >= 100, "fused CE: this library holds only sm_100a kernels (tcgen05 / TMEM); the current "
                                   "device is sm_" + std::to_string(device_arch()));

  WsF32 wf;
  const Ws w = carve_all(impl, s, ws, &wf);
  const bool f32io = s.io == DType::f32;
  const bool store_f32 = s.logits_store == DType::f32;
  const int D = s.D, V = s.V;
  const int Dk = f32io ? 3 * D : D;            // contraction length of the logits GEMM
  const int64_t io_bytes = int64_t(dtype_size(s.io));
  const int64_t n_chunks = (s.T + s.chunk_rows - 1) / s.chunk_rows;
  float* dw_target = strict_dw ? a.dw_microbatch : a.dw;
  GradReducer* reducer = static_cast<GradReducer*>(a.dw_reducer);
  if (reducer) NM_REQUIRE(a.dw && !strict_dw && grads, "fused CE: a dW reducer needs dw, gradients and dw_round none");

  NM_CUDA(cudaMemsetAsync(w.status, 0, 4, st));
  const void* w_logits = a.w;
  if (f32io) {
    launch_split3(static_cast<const float*>(a.w), wf.wsplit, V, D, 1, st);
    w_logits = wf.wsplit;
  }

  for (int64_t c = 0; c < n_chunks; ++c) {
    const int64_t r0 = c * s.chunk_rows;
    const int n = int(std::min<int64_t>(s.chunk_rows, s.T - r0));
    const void* x_c = byte_offset(a.x, r0 * D * io_bytes);
    const int32_t* tg_c = a.targets + r0;
    const float* wt_c = a.weight + r0;
    float* loss_c = a.loss_tok + r0;
    float* lse_c = a.lse ? a.lse + r0 : w.lse;
    void* dx_c = grads ? byte_offset(a.dx, r0 * D * io_bytes) : nullptr;

    const void* x_logits = x_c;
    if (f32io) {
      launch_split3(static_cast<const float*>(x_c), wf.xs, n, D, 0, st);
      x_logits = wf.xs;
    }
    // loss_tok doubles as the z[target] scratch between the logits kernel and the finalize
    LogitsArgs la{x_logits, w_logits, a.logit_bias, tg_c, n, Dk, V, grads ? w.store : nullptr, w.ldS, store_f32,
                  w.tmax, w.tsum, w.ldT, loss_c, w.status};
    { ProfScope ps(0, st); launch_logits(la, st); }
    FinalizeArgs fa{w.tmax, w.tsum, w.ldT, w.NT, loss_c, tg_c, wt_c, n, V, a.z_loss_weight, a.ignore_index, grads,
                    lse_c, loss_c, w.rowa, w.rowb};
    { ProfScope ps(1, st); launch_finalize(fa, st); }
    if (grads) {
      DzArgs za{w.store, w.ldS, store_f32, lse_c, w.rowa, w.rowb, tg_c, n, V};
      { ProfScope ps(2, st); launch_dlogits_inplace(za, st); }
      const int64_t ldn = store_f32 ? 2 * w.ldS : w.ldS;   // bf16 elements
      // dW first: every kernel that reads x runs before dX is written (dx may alias x)
      if (dw_target) {
        int reserve = 0;   // SMs left to the collective once a bucket reduction may be in flight
        auto wgrad = [&](int v0, int v1) {
          if (f32io) {   // x = hi + lo: two accumulating launches over the split copy (hi at column 0, lo at 2 D)
            WgradArgs g{w.store, ldn, wf.xs, int64_t(3) * D, n, D, V, v0, v1, a.grad_scale, dw_target, false, w.status};
            ProfScope ps(3, st);
            launch_wgrad(g, st);
            g.x = static_cast<const uint16_t*>(wf.xs) + 2 * D;
            launch_wgrad(g, st);
          } else {
            WgradArgs g{w.store, ldn, x_c, int64_t(D), n, D, V, v0, v1, a.grad_scale, dw_target, strict_dw, w.status};
            g.sm_reserve = reserve;
            ProfScope ps(3, st);
            launch_wgrad(g, st);
          }
        };
        if (reducer && c == n_chunks - 1) {
          for (int b = 0; b < reducer->n_buckets(); ++b) {
            int v0, v1;
            reducer->range(b, v0, v1);
            wgrad(v0, v1);
            reducer->bucket_ready(b, st);
            reserve = comm_sms();
          }
        } else {
          wgrad(0, V);
        }
      }
      if (dx_c) {
        ProfScope ps(4, st);
        if (f32io) {   // W = hi + lo (hi at column 0, lo at column D of the split copy)
          DgradArgs g{w.store, ldn, wf.wsplit, int64_t(3) * D, n, D, V, a.grad_scale, a.accumulate_dx ? dx_c : nullptr,
                      dx_c, 2, true, w.status};
          launch_dgrad(g, st);
          g.w = static_cast<const uint16_t*>(wf.wsplit) + D;
          g.dx_old = dx_c;
          launch_dgrad(g, st);
        } else {
          DgradArgs g{w.store, ldn, a.w, int64_t(D), n, D, V, a.grad_scale, a.accumulate_dx ? dx_c : nullptr, dx_c,
                      r == Rounding::Levanter ? 1 : 2, false, w.status};
          if (reducer && c == n_chunks - 1) g.sm_reserve = comm_sms();   // the bucket reductions run beside this kernel
          launch_dgrad(g, st);
        }
      }
    }
    if (a.loss_partial) { ProfScope ps(5, st); launch_chunk_loss(loss_c, wt_c, n, a.loss_partial + c, st); }
  }
}

// ------------------------------------------------------------------------------------------------ readout
void readout(CeImpl impl, Rounding r, const CeShape& s, const ReadoutCall& c, const CeArgs& base, float eps, void* ws,
             cudaStream_t st) {
  check_shape(impl, s);
  NM_REQUIRE(s.io == DType::bf16, "readout: bf16 io only");
  NM_REQUIRE(c.state && c.norm_gain && c.norm_rstd_ws && c.norm_out_ws && c.w, "readout: state, norm_gain, "
                                                                                "norm_rstd_ws, norm_out_ws, w required");
  NM_REQUIRE(c.visible_dims > 0 && c.visible_dims <= s.D, "readout: visible_dims in (0, D]");
  const int64_t T = s.T;
  const int D = s.D;
  if (T == 0) return;
  ew::rmsnorm_fwd(c.state, c.norm_gain, c.norm_out_ws, c.norm_rstd_ws, T, D, eps, st, r);
  if (c.visible_dims < D) launch_zero_cols(c.norm_out_ws, T, D, c.visible_dims, st);
  const bool need_dy = !base.forward_only && (c.d_state || c.dgain_partial);
  CeArgs a = base;
  a.x = c.norm_out_ws;
  a.w = c.w;
  a.dw = c.dw;
  a.grad_scale = c.grad_scale;
  a.dx = need_dy ? c.norm_out_ws : nullptr;   // dy over the normed input: every kernel that reads x runs before
  a.accumulate_dx = false;
  run(impl, r, s, a, ws, st);
  if (!need_dy) return;
  if (c.visible_dims < D) launch_zero_cols(c.norm_out_ws, T, D, c.visible_dims, st);
  bf16_t* dxo = c.d_state;
  if (!dxo) {   // gain gradient only: the norm's dX goes to the (now free) logits store
    const Ws w = carve(impl, s, ws);
    const uint64_t store_bytes = uint64_t(s.chunk_rows) * w.ldS * dtype_size(s.logits_store);
    NM_REQUIRE(uint64_t(T) * D * 2 <= store_bytes, "readout: the logits store is too small to hold the discarded norm dX");
    dxo = static_cast<bf16_t*>(w.store);
  }
  ew::rmsnorm_bwd_add(c.norm_out_ws, c.state, c.norm_gain, c.norm_rstd_ws, c.d_state, dxo, c.dgain_partial, T, D, eps,
                      st, r);
}

}  // namespace ce

// ------------------------------------------------------------------------------------------------ public API
uint64_t ce_workspace_bytes(CeImpl impl, const CeShape& s) {
  ce::check_shape(impl, s);
  return ce::carve(impl, s, nullptr).bytes;
}

void fused_linear_ce(CeImpl impl, Rounding r, const CeShape& s, const CeArgs& a, void* ws, GemmCache& gemm,
                     cudaStream_t st) {
  (void)gemm;   // the CE contractions are this library's own kernels
  ce::run(impl, r, s, a, ws, st);
}

void ce_finish_microbatch(const CeShape& s, const CeArgs& a, cudaStream_t st) {
  if (a.dw_round != CeDwRound::PerChunkBf16 || !a.dw) return;
  NM_REQUIRE(a.dw_microbatch, "ce_finish_microbatch: dw_microbatch required");
  ce::launch_finish_microbatch(a.dw, a.dw_microbatch, int64_t(s.V) * s.D, st);
}

void run_readout(CeImpl impl, Rounding r, const CeShape& s, const ReadoutCall& c, const CeArgs& base, void* ws,
                 GemmCache& gemm, cudaStream_t st) {
  (void)gemm;
  ce::readout(impl, r, s, c, base, 1e-5f, ws, st);   // ReadoutCall carries no eps; the reference passes 1e-5 too
}

}  // namespace nm
