// Internal API of the fused linear cross-entropy library: workspace regions, the plan of one call, kernel launchers,
// process-wide switches.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "device_info.hpp"
#include "marincpp/kernels/cross_entropy.hpp"

namespace nm::ce {

constexpr int kTileN = 256;   // vocabulary columns per (max, sumexp) partial = N of the logits UMMA tile
constexpr int kTileM = 128;   // rows per tile = M of every UMMA tile (one TMEM lane per row)

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline int64_t store_ld(int V) { return round_up(V, 8); }
inline int stats_tiles(int V) { return (V + kTileN - 1) / kTileN; }
inline int device_arch() { return current_device_info().arch; }   // 100 on a B200
inline int sm_count() { return current_device_info().sm_count; }

// ------------------------------------------------------------------------------------------------ workspace
// Hands out consecutive regions of one caller-owned block, each starting on a 256-byte boundary. With a null base it
// only measures. Every layout of the library (the full call, the forward-only call on the built-in scratch) is a
// sequence of take() calls on one of these, so sizing and placement cannot drift apart.
class Arena {
 public:
  explicit Arena(void* base) : base_(static_cast<uint8_t*>(base)) {}
  template <class T>
  T* take(uint64_t count) {
    cursor_ = uint64_t(round_up(int64_t(cursor_), int64_t(kArenaAlign)));
    T* p = base_ ? reinterpret_cast<T*>(base_ + cursor_) : nullptr;
    cursor_ += count * sizeof(T);
    return p;
  }
  uint64_t bytes() const { return uint64_t(round_up(int64_t(cursor_), int64_t(kArenaAlign))); }

 private:
  uint8_t* base_;
  uint64_t cursor_ = 0;
};

// Per-row factors of the normalised gradient n = a p - b onehot(target), p = 2^(z log2e + e), packed so that a kernel
// fetches them with one 16-byte load: e = -lse log2e, a = w_t (1 + 2 L lse), b = w_t (0 for an ignored row),
// target as int bits.
struct alignas(16) RowFactors {
  float e, a, b;
  int32_t target;
};

// Regions of one call, in workspace order:
//   status   256 B: word 0 = OR of the wait-error bits of every kernel launched on this workspace
//   tmax, tsum [NT, rows] f32 partial (max, sum exp) per 256-column tile, tile-major
//   lse      [rows] f32 (used when the caller passes no lse)
//   -- gradient calls only --
//   rowf     [rows] RowFactors
//   store    [rows, ldS] logits of the chunk (bf16 or f32; ldS = V rounded up to 8). Either read as they are by the
//            gradient contractions, which form n on the fly, or first rewritten in place as bf16 n (f32 store: over the
//            first half of each row)
//   f32 io only (implementation A): xs [rows, 3 D] and wsplit [V, 3 D] bf16 split copies of x and W
struct Regions {
  uint32_t* status = nullptr;
  float* tmax = nullptr; float* tsum = nullptr; int64_t ldT = 0; int NT = 0;
  float* lse = nullptr;
  RowFactors* rowf = nullptr;
  void* store = nullptr; int64_t ldS = 0;
  void* xs = nullptr; void* wsplit = nullptr;
  uint64_t bytes = 0;
};
Regions layout_forward(Arena& arena, int V, int64_t rows);                    // status .. lse
Regions layout_call(CeImpl impl, const CeShape& s, void* base);               // everything; base == nullptr: sizes only

// Process-wide switches. They are read by every call and may be written by any host thread: plain atomics, relaxed.
int exchange_backends(int dgrad_own, int wgrad_own, int sm90);   // recorded only (one kernel set); returns the old packing
int exchange_fast_stats_exp(int on);

// How the two gradient contractions of a chunk get their A operand and which tile geometry they use.
//   kPassClassic  the in-place pass rewrites the store as n; dX / dW run on 128 x 256 tiles (TMEM double-buffered)
//   kPassWide     the in-place pass; dX / dW run on CTA pairs with 256 x 512 tiles (one 512-column accumulator)
//   kFusedWide    no pass: dX / dW read the raw logits and form n in shared memory ahead of the UMMAs (wide tiles)
enum GradPath : int { kPathAuto = -1, kPassClassic = 0, kPassWide = 1, kFusedWide = 2 };
void set_grad_path(int path);                                    // kPathAuto (default): chosen per call
GradPath grad_path_for(int D, int rows, bool plain_bf16);        // plain_bf16: bf16 store and bf16 io
// Last chunk of a call with a bucketed dW reduction: 1 (default) = dX first on every SM when it does not overwrite x,
// then the dW buckets beside the reductions; 0 = dW buckets first, dX beside the reductions.
void set_tail_order(int order);
int tail_order();

// Optional per-kernel-class timing for benches: when enabled, run() brackets every launch with a pair of CUDA events on
// the call's stream (the events are created when profiling is enabled, never inside a call). Classes: 0 logits,
// 1 finalize, 2 dlogits pass, 3 dW, 4 dX, 5 chunk loss.
constexpr int kProfClasses = 6;
void profile_enable(int max_launches);                       // 0 disables and frees the events
void profile_read(double* ms, int* launches);                // sums per class since the last read; synchronises
struct ProfScope {                                           // records begin / end around one launch (no-op when off)
  ProfScope(int cls, cudaStream_t st);
  ~ProfScope();
  int slot_; cudaStream_t st_;
};

// One call (the C++ API and the C ABI both end here). Options that only callers inside the library may set:
struct RunOptions {
  bool allow_logit_bias = false;   // a logit bias with bf16 io and any implementation value (the sampled head's mask)
};
void run(CeImpl impl, Rounding r, const CeShape& s, const CeArgs& a, void* ws, cudaStream_t st,
         const RunOptions& opt = RunOptions{});
void readout(CeImpl impl, Rounding r, const CeShape& s, const ReadoutCall& c, const CeArgs& base, float eps, void* ws,
             cudaStream_t st);
// Forward only on caller-provided forward regions (layout_forward): what run() does for a call without gradients.
void run_forward(const Regions& w, const void* x, const void* wmat, const int32_t* targets, const float* weight,
                 float* loss_tok, float* lse, float* loss_partial, int64_t T, int D, int V, int chunk_rows,
                 float z_loss, int32_t ignore_index, cudaStream_t st);

// ------------------------------------------------------------------------------------------------ tcgen05 kernels
// z = x W^T tile by tile; per (row, 256-col tile) partial (max, sum exp(z - max)); z[target] -> zt; optional store.
struct LogitsArgs {
  const void* x; const void* w; const float* bias; const int32_t* targets;
  int rows, D, V;
  void* store; int64_t ldS; bool store_f32;   // store == nullptr: statistics only
  float* tmax; float* tsum; int64_t ldT;
  float* zt;                                   // [rows]; rows whose target is outside [0, V) are left untouched
  uint32_t* status;
};
void launch_logits(const LogitsArgs& a, cudaStream_t st);

// dx[rows, D] = scale * (n[rows, V] W[V, D]); n bf16 with leading dimension ldn (elements).
//   acc_mode 0: out = bf16(v); 1 (levanter): bf16(f32(old) + f32(bf16(v))); 2 (accurate): bf16(f32(old) + v)
// wide: CTA pairs on 256 x 512 tiles. rowf != nullptr (wide only): `n` holds the raw bf16 logits and the kernel forms
// the normalised gradient in shared memory from these per-row factors.
struct DgradArgs {
  const void* n; int64_t ldn; const void* w; int64_t ldw;   // ldw: row pitch of w in elements (D when contiguous)
  int rows, D, V;
  const float* scale;               // device scalar (*grad_scale)
  const void* dx_old; void* dx_out; int acc_mode; bool out_f32;
  uint32_t* status;
  int sm_reserve = 0;               // SMs left free (for a collective running beside this kernel)
  bool wide = false;
  const RowFactors* rowf = nullptr;
};
void launch_dgrad(const DgradArgs& a, cudaStream_t st);

// dw[v0 .. v1, D] += scale * (n[rows, v0 .. v1]^T x[rows, D]) in f32; round_bf16: += f32(bf16(.)) (strict mode).
struct WgradArgs {
  const void* n; int64_t ldn; const void* x; int64_t ldx;   // ldx: row pitch of x in elements (D when contiguous)
  int rows, D, V;
  int v0, v1;                       // vocabulary range of this launch (multiples of 128, or V)
  const float* scale; float* dw; bool round_bf16;
  uint32_t* status;
  int sm_reserve = 0;               // SMs left free (for a collective running beside this kernel)
  bool wide = false;
  const RowFactors* rowf = nullptr;
};
void launch_wgrad(const WgradArgs& a, cudaStream_t st);

// unit-test entry: one CTA whose bounded wait runs out after `limit_cycles` (<= 2e6) on a barrier nobody completes
void launch_wait_timeout_probe(uint32_t* status, long long limit_cycles, int* saw_abort, cudaStream_t st);

// CTAs per accumulator tile of the three classic contractions: 0 = one CTA per 128 x 256 tile, 1 = a pair of CTAs
// (cluster of two, one UMMA of M = 256 over both) per 256 x 256 tile, negative = chosen per launch (the default).
// Process-wide (atomic).
void set_cta_pair(int logits, int dgrad, int wgrad);

// unit-test entry: C f32 [M, N] = A B^T in the three operand layouts (kind 0 K/K, 1 K/MN, 2 MN/MN; + 4: CTA pairs;
// + 8: the wide pair kernel (kinds 1 and 2 only); + 16 with 8: A is transformed on the fly with `rowf`)
void launch_test_gemm(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc, int M,
                      int N, int K, uint32_t* status, const RowFactors* rowf, cudaStream_t st);

// ------------------------------------------------------------------------------------------------ row / streaming kernels
struct FinalizeArgs {
  const float* tmax; const float* tsum; int64_t ldT; int NT;
  const float* zt; const int32_t* targets; const float* weight;
  int rows, V; float z_loss; int32_t ignore_index;
  float* lse; float* loss_tok;        // loss_tok may equal zt
  RowFactors* rowf;                   // nullptr: a forward-only call
};
void launch_finalize(const FinalizeArgs& a, cudaStream_t st);
void launch_chunk_loss(const float* loss_tok, const float* weight, int rows, float* out, cudaStream_t st);

// store -> bf16 n in place (f32 store: over the first half of each row, ld 2 ldS). The per-row factors come packed
// (rowf) or, for the stand-alone entry point, as separate arrays: lse, the factor of p (ga) and of the onehot (gb).
struct DzArgs {
  void* store; int64_t ldS; bool store_f32;
  const RowFactors* rowf;
  const float* lse; const float* ga; const float* gb; const int32_t* targets;
  int rows, V;
  uint32_t* status = nullptr;           // where a timed-out wait of the kernel is recorded (may be null)
};
void launch_dlogits_inplace(const DzArgs& a, cudaStream_t st);

void launch_finish_microbatch(float* dw, float* dw_mb, int64_t n, cudaStream_t st);
void launch_zero_cols(void* x, int64_t rows, int D, int from, cudaStream_t st);   // bf16 x[:, from:] = 0
void launch_sum_scale(const float* w, int64_t n, float mult, float* out, cudaStream_t st);
void launch_add_f32(float* acc, const float* src, int64_t n, cudaStream_t st);   // acc += src
void launch_f32_to_bf16(const float* in, void* out, int64_t n, cudaStream_t st);
void launch_bf16_to_f32(const void* in, float* out, int64_t n, cudaStream_t st);
// f32 [rows, D] -> bf16 [rows, 3 D] holding (hi, hi, lo) (which == 0) or (hi, lo, hi) (which == 1) per row, so that
// the K = 3 D contraction of a (hi, hi, lo) matrix with a (hi, lo, hi) matrix is hi hi + hi lo + lo hi
void launch_split3(const float* in, void* out, int64_t rows, int D, int which, cudaStream_t st);

}  // namespace nm::ce
