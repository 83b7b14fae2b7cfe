// Host side of the fused linear cross-entropy: where the regions of a workspace lie, what makes a call valid, the
// order in which the kernels of one chunk are issued, the readout head, and the C++ entry points declared in
// include/marincpp/kernels/cross_entropy.hpp. What a caller may rely on is the reference's contract
// (src/kernels/cross_entropy/ce_api.cpp: the requirements of :52-57 and :133-145, dW issued before dX so that dX may
// overwrite x :199,226, one loss partial per chunk :238, the readout sequence :243-275); how it is met is this
// library's own.
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <string>
#include <vector>

#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "marincpp/comm.hpp"

namespace nm {
namespace ce {

// ------------------------------------------------------------------------------------------------ workspace layout
Regions layout_forward(Arena& arena, int V, int64_t rows) {
  Regions w;
  w.status = arena.take<uint32_t>(64);
  w.NT = stats_tiles(V);
  w.ldT = rows;
  w.tmax = arena.take<float>(uint64_t(w.NT) * rows);
  w.tsum = arena.take<float>(uint64_t(w.NT) * rows);
  w.lse = arena.take<float>(uint64_t(rows));
  w.bytes = arena.bytes();
  return w;
}

Regions layout_call(CeImpl impl, const CeShape& s, void* base) {
  Arena arena(base);
  const int64_t rows = s.chunk_rows;
  Regions w = layout_forward(arena, s.V, rows);
  w.rowf = arena.take<RowFactors>(uint64_t(rows));
  w.ldS = store_ld(s.V);
  w.store = arena.take<uint8_t>(uint64_t(rows) * w.ldS * dtype_size(s.logits_store));
  // The C ABI sizes a workspace from (impl, shape, store) without the io type, so implementation A always carries the
  // split copies its f32-io form needs.
  if (impl == CeImpl::A) {
    w.xs = arena.take<uint16_t>(uint64_t(rows) * 3 * s.D);
    w.wsplit = arena.take<uint16_t>(uint64_t(s.V) * 3 * s.D);
  }
  w.bytes = arena.bytes();
  return w;
}

// ------------------------------------------------------------------------------------------------ switches
namespace {
std::atomic<int> g_backends{3 << 2};        // dgrad | wgrad << 1 | sm90 << 2, as nm_ce_set_backends packs it
std::atomic<int> g_fast_stats_exp{0};
std::atomic<int> g_grad_path{kPathAuto};
std::atomic<int> g_tail_order{0};
}  // namespace

int exchange_backends(int dgrad_own, int wgrad_own, int sm90) {
  int old = g_backends.load(std::memory_order_relaxed), next;
  do {
    const int keep_sm90 = (old >> 2) & 3;
    next = (dgrad_own ? 1 : 0) | (wgrad_own ? 2 : 0) | ((sm90 >= 0 ? (sm90 & 3) : keep_sm90) << 2);
  } while (!g_backends.compare_exchange_weak(old, next, std::memory_order_relaxed));
  return old;
}
int exchange_fast_stats_exp(int on) { return g_fast_stats_exp.exchange(on ? 1 : 0, std::memory_order_relaxed); }

int tail_order() { return g_tail_order.load(std::memory_order_relaxed); }
void set_tail_order(int order) {
  NM_REQUIRE(order == 0 || order == 1, "tail order: 0 (dW buckets, then dX beside the reductions) or 1 (dX first)");
  g_tail_order.store(order, std::memory_order_relaxed);
}

void set_grad_path(int path) {
  NM_REQUIRE(path >= kPathAuto && path <= kFusedWide, "gradient path: -1 (per call), 0, 1 or 2");
  g_grad_path.store(path, std::memory_order_relaxed);
}

// Which form pays was measured per hidden size on a B200, all three forms in turn on the same box (131072 rows, vocabulary
// 128256; ms per step fused / pass + wide tiles / pass + 128 x 256 tiles): hidden 512: 48.6 / 55.5 / 56.3; 1024: 90.5 /
// 93.3 / 95.6; 2048: 177.2 / 177.8 / 174.4. Forming n inside the contractions removes the in-place pass (4 bytes per
// logit at the HBM rate: a fifth of the step at hidden 512) but every 512-column tile that reads a block of logits
// transforms it again, and the transform's shared-memory traffic slows the UMMAs it runs beside; at hidden 2048 (four
// tiles per block, a step that is bound by board power) that costs what the pass saved.
GradPath grad_path_for(int D, int rows, bool plain_bf16) {
  (void)rows;
  if (!plain_bf16) return kPassClassic;
  const int forced = g_grad_path.load(std::memory_order_relaxed);
  if (forced != kPathAuto) return GradPath(forced);
  return D <= 1024 ? kFusedWide : kPassClassic;
}

// ------------------------------------------------------------------------------------------------ profiling
namespace {
struct LaunchTimer {
  std::mutex mu;
  std::vector<cudaEvent_t> ev;   // begin / end per slot
  std::vector<int> cls;
  int used = 0;
  std::atomic<bool> on{false};
} g_timer;

// Every launch also sits in an NVTX range named after its kernel class (header-only NVTX 3: free unless a profiler is
// attached), so that a profiler can select one class, e.g. `--nvtx --nvtx-include "ce.dx/"`.
const char* const kClassName[kProfClasses] = {"ce.logits", "ce.finalize", "ce.dlogits", "ce.dw", "ce.dx",
                                              "ce.chunk_loss"};
}  // namespace

void profile_enable(int max_launches) {
  std::lock_guard<std::mutex> lock(g_timer.mu);
  g_timer.on.store(false, std::memory_order_release);
  for (cudaEvent_t e : g_timer.ev) cudaEventDestroy(e);
  g_timer.ev.clear();
  const int n = std::max(0, max_launches);
  g_timer.cls.assign(size_t(n), 0);
  g_timer.used = 0;
  for (int i = 0; i < 2 * n; ++i) {
    cudaEvent_t e;
    NM_CUDA(cudaEventCreate(&e));
    g_timer.ev.push_back(e);
  }
  g_timer.on.store(n > 0, std::memory_order_release);
}

void profile_read(double* ms, int* launches) {
  std::lock_guard<std::mutex> lock(g_timer.mu);
  std::fill(ms, ms + kProfClasses, 0.0);
  std::fill(launches, launches + kProfClasses, 0);
  for (int i = 0; i < g_timer.used; ++i) {
    float t = 0.f;
    NM_CUDA(cudaEventSynchronize(g_timer.ev[size_t(2 * i + 1)]));
    NM_CUDA(cudaEventElapsedTime(&t, g_timer.ev[size_t(2 * i)], g_timer.ev[size_t(2 * i + 1)]));
    ms[g_timer.cls[size_t(i)]] += t;
    launches[g_timer.cls[size_t(i)]] += 1;
  }
  g_timer.used = 0;
}

ProfScope::ProfScope(int cls, cudaStream_t st) : slot_(-1), st_(st) {
  nvtxRangePushA(kClassName[cls]);
  if (!g_timer.on.load(std::memory_order_acquire)) return;
  std::lock_guard<std::mutex> lock(g_timer.mu);
  if (!g_timer.on.load(std::memory_order_relaxed) || g_timer.used >= int(g_timer.cls.size())) return;
  slot_ = g_timer.used++;
  g_timer.cls[size_t(slot_)] = cls;
  cudaEventRecord(g_timer.ev[size_t(2 * slot_)], st_);
}
ProfScope::~ProfScope() {
  if (slot_ >= 0) {
    std::lock_guard<std::mutex> lock(g_timer.mu);
    if (size_t(2 * slot_ + 1) < g_timer.ev.size()) cudaEventRecord(g_timer.ev[size_t(2 * slot_ + 1)], st_);
  }
  nvtxRangePop();
}

// ------------------------------------------------------------------------------------------------ validation
namespace {

const char* spelled(CeImpl impl) {
  static const char* const names[] = {"A", "B1", "B1.5", "B2"};
  const unsigned i = unsigned(impl);
  return i < 4 ? names[i] : "(unknown)";
}

void require_shape(CeImpl impl, const CeShape& s) {
  NM_REQUIRE(s.T >= 0, "fused CE: the row count T cannot be negative");
  NM_REQUIRE(s.D > 0 && s.V > 0, "fused CE: hidden size D and vocabulary size V must be positive");
  NM_REQUIRE(s.D % 8 == 0, "fused CE: D must be a multiple of 8 (rows are moved in 16-byte pieces)");
  NM_REQUIRE(s.chunk_rows > 0, "fused CE: chunk_rows must be positive");
  const bool store_ok = s.logits_store == DType::bf16 || s.logits_store == DType::f32;
  NM_REQUIRE(store_ok, "fused CE: the logits store is bf16 or f32");
  const bool io_ok = s.io == DType::bf16 || (s.io == DType::f32 && impl == CeImpl::A);
  NM_REQUIRE(io_ok, std::string("fused CE: f32 x / W / dX is the f32 policy of implementation A; implementation ") +
                        spelled(impl) + " takes bf16");
}

// What a call asks for, derived once from its arguments after they have been found consistent.
struct CallKind {
  bool grads = false;       // any gradient wanted
  bool strict_dw = false;   // per-chunk bf16 rounding of dW into dw_microbatch
  bool f32io = false;
  bool store_f32 = false;
  GradReducer* reducer = nullptr;
};

bool aligned(const void* p, uintptr_t to) { return reinterpret_cast<uintptr_t>(p) % to == 0; }

CallKind require_call(CeImpl impl, const CeShape& s, const CeArgs& a, const void* ws, const RunOptions& opt) {
  CallKind k;
  NM_REQUIRE(a.x && a.w, "fused CE: x and w are required");
  NM_REQUIRE(a.targets && a.weight, "fused CE: targets and weight are required");
  NM_REQUIRE(a.loss_tok, "fused CE: loss_tok is required (it also carries z[target] between two kernels)");
  NM_REQUIRE(ws != nullptr, "fused CE: a workspace of nm_ce_workspace_bytes() bytes is required");
  NM_REQUIRE(aligned(ws, kArenaAlign), "fused CE: the workspace must be 256-byte aligned");
  k.grads = !a.forward_only && (a.dx != nullptr || a.dw != nullptr);
  k.strict_dw = a.dw != nullptr && a.dw_round == CeDwRound::PerChunkBf16;
  k.f32io = s.io == DType::f32;
  k.store_f32 = s.logits_store == DType::f32;
  k.reducer = static_cast<GradReducer*>(a.dw_reducer);
  if (k.grads) NM_REQUIRE(a.grad_scale != nullptr, "fused CE: a gradient call needs the device scalar grad_scale");
  if (k.strict_dw) {
    NM_REQUIRE(a.dw_microbatch != nullptr, "fused CE: CeDwRound::PerChunkBf16 accumulates into dw_microbatch");
    NM_REQUIRE(!k.f32io, "fused CE: CeDwRound::PerChunkBf16 is a bf16-io mode");
  }
  const bool inplace_accumulate = a.dx != nullptr && a.dx == a.x && a.accumulate_dx;
  NM_REQUIRE(!inplace_accumulate, "fused CE: dx may alias x or accumulate, not both");
  NM_REQUIRE(a.logit_bias == nullptr || impl == CeImpl::A || opt.allow_logit_bias,
             "fused CE: only implementation A takes a logit_bias");
  if (k.reducer) {
    NM_REQUIRE(a.dw != nullptr && k.grads && !k.strict_dw,
               "fused CE: a dW reducer goes with a dw gradient and CeDwRound::None");
  }
  // x, w and dw are checked where their tensor maps are built; these two are touched with 16-byte vector accesses
  NM_REQUIRE(aligned(a.dx, 16), "fused CE: dx must be 16-byte aligned");
  NM_REQUIRE(aligned(a.dw_microbatch, 16), "fused CE: dw_microbatch must be 16-byte aligned");
  const int arch = device_arch();
  NM_REQUIRE(arch >= 100, "fused CE: every kernel of this library is sm_100a code (tcgen05, TMEM, TMA); the current "
                          "device reports sm_" + std::to_string(arch) + " and there is no other path");
  return k;
}

const uint8_t* rows_from(const void* p, int64_t row, int64_t row_bytes) {
  return p ? static_cast<const uint8_t*>(p) + row * row_bytes : nullptr;
}
uint8_t* rows_from(void* p, int64_t row, int64_t row_bytes) {
  return p ? static_cast<uint8_t*>(p) + row * row_bytes : nullptr;
}

// The forward half of one chunk: logits tiles with their softmax partials, the merge into lse and loss, the chunk's
// loss sum. loss_tok doubles as the z[target] scratch between the first two kernels.
struct ChunkForward {
  const void* x; const void* w; int Dk;   // operands of the logits contraction and its length
  const float* bias;
  const int32_t* targets; const float* weight;
  float* loss_tok; float* lse; float* loss_partial;   // loss_partial: this chunk's slot, or nullptr
  int rows, V;
  float z_loss; int32_t ignore_index;
};

void forward_chunk(const Regions& w, const ChunkForward& c, bool keep_logits, bool store_f32, RowFactors* rowf,
                   cudaStream_t st) {
  LogitsArgs la{c.x, c.w, c.bias, c.targets, c.rows, c.Dk, c.V, keep_logits ? w.store : nullptr, w.ldS, store_f32,
                w.tmax, w.tsum, w.ldT, c.loss_tok, w.status};
  {
    ProfScope t(0, st);
    launch_logits(la, st);
  }
  FinalizeArgs fa{w.tmax, w.tsum, w.ldT, w.NT, c.loss_tok, c.targets, c.weight, c.rows, c.V, c.z_loss,
                  c.ignore_index, c.lse, c.loss_tok, rowf};
  {
    ProfScope t(1, st);
    launch_finalize(fa, st);
  }
  if (c.loss_partial) {
    ProfScope t(5, st);
    launch_chunk_loss(c.loss_tok, c.weight, c.rows, c.loss_partial, st);
  }
}

}  // namespace

void run_forward(const Regions& w, const void* x, const void* wmat, const int32_t* targets, const float* weight,
                 float* loss_tok, float* lse, float* loss_partial, int64_t T, int D, int V, int chunk_rows,
                 float z_loss, int32_t ignore_index, cudaStream_t st) {
  NM_CUDA(cudaMemsetAsync(w.status, 0, sizeof(uint32_t), st));
  int64_t slot = 0;
  for (int64_t r0 = 0; r0 < T; r0 += chunk_rows, ++slot) {
    const int n = int(std::min<int64_t>(chunk_rows, T - r0));
    ChunkForward c{rows_from(x, r0, int64_t(D) * 2), wmat, D, nullptr, targets + r0, weight + r0, loss_tok + r0,
                   lse ? lse + r0 : w.lse, loss_partial ? loss_partial + slot : nullptr, n, V, z_loss, ignore_index};
    forward_chunk(w, c, false, false, nullptr, st);
  }
}

// ------------------------------------------------------------------------------------------------ one call
void run(CeImpl impl, Rounding r, const CeShape& s, const CeArgs& a, void* ws, cudaStream_t st, const RunOptions& opt) {
  require_shape(impl, s);
  if (s.T == 0) return;
  const CallKind k = require_call(impl, s, a, ws, opt);
  const Regions w = layout_call(impl, s, ws);
  const int D = s.D, V = s.V;
  const int64_t io_row_bytes = int64_t(D) * int64_t(dtype_size(s.io));
  const int64_t last_r0 = (s.T - 1) / s.chunk_rows * int64_t(s.chunk_rows);
  float* dw_into = k.strict_dw ? a.dw_microbatch : a.dw;
  const GradPath path = grad_path_for(D, int(std::min<int64_t>(s.chunk_rows, s.T)), !k.store_f32 && !k.f32io);
  const bool wide = path != kPassClassic, fused = path == kFusedWide;

  NM_CUDA(cudaMemsetAsync(w.status, 0, sizeof(uint32_t), st));
  // f32 io: the contractions run on bf16 (hi, lo) splits; W is split once per call, x once per chunk
  const void* w_for_logits = a.w;
  if (k.f32io) {
    launch_split3(static_cast<const float*>(a.w), w.wsplit, V, D, 1, st);
    w_for_logits = w.wsplit;
  }

  int64_t slot = 0;
  for (int64_t r0 = 0; r0 < s.T; r0 += s.chunk_rows, ++slot) {
    const int n = int(std::min<int64_t>(s.chunk_rows, s.T - r0));
    const bool last_chunk = r0 == last_r0;
    const void* x_c = rows_from(a.x, r0, io_row_bytes);
    const void* x_for_logits = x_c;
    if (k.f32io) {
      launch_split3(static_cast<const float*>(x_c), w.xs, n, D, 0, st);
      x_for_logits = w.xs;
    }
    ChunkForward fwd{x_for_logits, w_for_logits, k.f32io ? 3 * D : D, a.logit_bias, a.targets + r0, a.weight + r0,
                     a.loss_tok + r0, a.lse ? a.lse + r0 : w.lse, a.loss_partial ? a.loss_partial + slot : nullptr,
                     n, V, a.z_loss_weight, a.ignore_index};
    forward_chunk(w, fwd, k.grads, k.store_f32, k.grads ? w.rowf : nullptr, st);
    if (!k.grads) continue;

    // ---- the gradient half. A operand of both contractions: the store, as n (after the pass) or as raw logits
    const RowFactors* on_the_fly = fused ? w.rowf : nullptr;
    if (!fused) {
      DzArgs za{w.store, w.ldS, k.store_f32, w.rowf, nullptr, nullptr, nullptr, nullptr, n, V, w.status};
      ProfScope t(2, st);
      launch_dlogits_inplace(za, st);
    }
    const int64_t ldn = k.store_f32 ? 2 * w.ldS : w.ldS;   // bf16 elements between rows of n

    const bool bucketed = k.reducer != nullptr && last_chunk;
    auto issue_dw = [&] {
      if (!dw_into) return;
      int reserve = 0;   // SMs left to the collective once a bucket reduction may be in flight
      auto wgrad_range = [&](int v0, int v1) {
        ProfScope t(3, st);
        if (k.f32io) {   // x = hi + lo: two accumulating launches over the split copy (hi at column 0, lo at 2 D)
          WgradArgs g{w.store, ldn, w.xs, int64_t(3) * D, n, D, V, v0, v1, a.grad_scale, dw_into, false, w.status};
          launch_wgrad(g, st);
          g.x = static_cast<const uint16_t*>(w.xs) + 2 * D;
          launch_wgrad(g, st);
        } else {
          WgradArgs g{w.store, ldn, x_c, int64_t(D), n, D, V, v0, v1, a.grad_scale, dw_into, k.strict_dw, w.status};
          g.sm_reserve = reserve;
          g.wide = wide;
          g.rowf = on_the_fly;
          launch_wgrad(g, st);
        }
      };
      if (bucketed) {
        // the last chunk completes dW range by range, and each range's reduction starts while the next is computed
        for (int b = 0; b < k.reducer->n_buckets(); ++b) {
          int v0 = 0, v1 = 0;
          k.reducer->range(b, v0, v1);
          wgrad_range(v0, v1);
          k.reducer->bucket_ready(b, st);
          reserve = comm_sms();
        }
      } else {
        wgrad_range(0, V);
      }
    };
    auto issue_dx = [&](bool beside_reductions) {
      if (!a.dx) return;
      void* dx_c = rows_from(a.dx, r0, io_row_bytes);
      ProfScope t(4, st);
      if (k.f32io) {   // W = hi + lo (hi at column 0, lo at column D of the split copy), f32 output accumulated
        DgradArgs g{w.store, ldn, w.wsplit, int64_t(3) * D, n, D, V, a.grad_scale, a.accumulate_dx ? dx_c : nullptr,
                    dx_c, 2, true, w.status};
        launch_dgrad(g, st);
        g.w = static_cast<const uint16_t*>(w.wsplit) + D;
        g.dx_old = dx_c;
        launch_dgrad(g, st);
      } else {
        DgradArgs g{w.store, ldn, a.w, int64_t(D), n, D, V, a.grad_scale, a.accumulate_dx ? dx_c : nullptr, dx_c,
                    r == Rounding::Levanter ? 1 : 2, false, w.status};
        if (beside_reductions) g.sm_reserve = comm_sms();
        g.wide = wide;
        g.rowf = on_the_fly;
        launch_dgrad(g, st);
      }
    };
    // The order of a chunk is dW, then dX: every kernel that reads x has been issued before dX (which may be x) is
    // written, and with a bucketed reducer the reductions of the dW buckets run beside the rest of dW and all of dX
    // (nothing exposed; the compute kernels leave the reducer its SMs). Optional (tail order 1) for the last chunk of
    // such a call when dX does not land on x: dX first, on every SM, and only the dW buckets share the GPU with the
    // reductions of their predecessors; the reduction of the last bucket is then exposed. Measured on 4 GPUs at
    // hidden 2048: 180.9 ms per step in the default order, 182.9 with dX first; on 2 GPUs the same.
    const bool dx_first = bucketed && a.dx != nullptr && a.dx != a.x && tail_order() == 1;
    if (dx_first) {
      issue_dx(false);
      issue_dw();
    } else {
      issue_dw();
      issue_dx(bucketed);
    }
  }
}

// ------------------------------------------------------------------------------------------------ readout
// One readout head: state -> RMSNorm -> fused CE whose dX lands on top of the normed activations -> RMSNorm backward
// into d_state (added) and the gain partials. Coordinates from visible_dims on are hidden from the head: zeroed in the
// normed input and again in the gradient that comes back.
void readout(CeImpl impl, Rounding r, const CeShape& s, const ReadoutCall& c, const CeArgs& base, float eps, void* ws,
             cudaStream_t st) {
  require_shape(impl, s);
  NM_REQUIRE(s.io == DType::bf16, "readout: the head runs on bf16 activations");
  NM_REQUIRE(c.state && c.norm_gain && c.w, "readout: state, norm_gain and w are required");
  NM_REQUIRE(c.norm_rstd_ws && c.norm_out_ws, "readout: the two norm work buffers are required");
  NM_REQUIRE(c.visible_dims >= 1 && c.visible_dims <= s.D, "readout: visible_dims must lie in [1, D]");
  if (s.T == 0) return;
  const bool hide = c.visible_dims < s.D;
  const bool wants_state_grad = !base.forward_only && (c.d_state != nullptr || c.dgain_partial != nullptr);

  ew::rmsnorm_fwd(c.state, c.norm_gain, c.norm_out_ws, c.norm_rstd_ws, s.T, s.D, eps, st, r);
  if (hide) launch_zero_cols(c.norm_out_ws, s.T, s.D, c.visible_dims, st);

  CeArgs call = base;
  call.x = c.norm_out_ws;
  call.w = c.w;
  call.grad_scale = c.grad_scale;
  call.dw = c.dw;
  call.dx = wants_state_grad ? static_cast<void*>(c.norm_out_ws) : nullptr;   // in place: legal, dW is issued first
  call.accumulate_dx = false;
  run(impl, r, s, call, ws, st);
  if (!wants_state_grad) return;

  if (hide) launch_zero_cols(c.norm_out_ws, s.T, s.D, c.visible_dims, st);
  bf16_t* norm_dx = c.d_state;
  if (norm_dx == nullptr) {
    // only the gain gradient is wanted: the norm's dX still has to be written somewhere, and the logits store is free
    const Regions w = layout_call(impl, s, ws);
    const uint64_t room = uint64_t(s.chunk_rows) * uint64_t(w.ldS) * dtype_size(s.logits_store);
    NM_REQUIRE(uint64_t(s.T) * uint64_t(s.D) * 2 <= room, "readout: no d_state given and the logits store cannot hold "
                                                          "the discarded norm gradient; use a larger chunk_rows");
    norm_dx = static_cast<bf16_t*>(w.store);
  }
  ew::rmsnorm_bwd_add(c.norm_out_ws, c.state, c.norm_gain, c.norm_rstd_ws, c.d_state, norm_dx, c.dgain_partial, s.T,
                      s.D, eps, st, r);
}

}  // namespace ce

// ------------------------------------------------------------------------------------------------ public C++ API
uint64_t ce_workspace_bytes(CeImpl impl, const CeShape& s) {
  ce::require_shape(impl, s);
  return ce::layout_call(impl, s, nullptr).bytes;
}

// The trunk's GEMM planner is accepted for signature compatibility and not used: the CE contractions are this
// library's own kernels.
void fused_linear_ce(CeImpl impl, Rounding r, const CeShape& s, const CeArgs& a, void* ws, GemmCache&, cudaStream_t st) {
  ce::run(impl, r, s, a, ws, st);
}

void ce_finish_microbatch(const CeShape& s, const CeArgs& a, cudaStream_t st) {
  const bool strict = a.dw != nullptr && a.dw_round == CeDwRound::PerChunkBf16;
  if (!strict) return;
  NM_REQUIRE(a.dw_microbatch != nullptr, "ce_finish_microbatch: the strict mode's dw_microbatch is missing");
  ce::launch_finish_microbatch(a.dw, a.dw_microbatch, int64_t(s.V) * int64_t(s.D), st);
}

void run_readout(CeImpl impl, Rounding r, const CeShape& s, const ReadoutCall& c, const CeArgs& base, void* ws,
                 GemmCache&, cudaStream_t st) {
  constexpr float kNormEps = 1e-5f;   // ReadoutCall has no eps field; this is the value the reference's trainer uses
  ce::readout(impl, r, s, c, base, kNormEps, ws, st);
}

}  // namespace nm
