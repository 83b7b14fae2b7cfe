// Internal API of the fused linear cross-entropy library: workspace layout, kernel launchers, process-wide switches.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

#include "marincpp/kernels/cross_entropy.hpp"

namespace nm::ce {

constexpr int kTileN = 256;   // vocabulary columns per (max, sumexp) partial = N of the logits UMMA tile
constexpr int kTileM = 128;   // rows per tile = M of every UMMA tile (one TMEM lane per row)

inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }
inline int64_t store_ld(int V) { return round_up(V, 8); }
inline int stats_tiles(int V) { return (V + kTileN - 1) / kTileN; }

// Workspace of one call; every region starts on a 256-byte boundary, in this order:
//   status   256 B: word 0 = OR of the wait-error bits of every kernel launched on this workspace
//   store    [chunk_rows, ldS] logits of the chunk (bf16 or f32; ldS = V rounded up to 8), rewritten in place as the
//            bf16 normalised gradient n = w_t (p (1 + 2 L lse) - onehot) (f32 store: over the first half of each row)
//   tmax, tsum [NT, chunk_rows] f32 partial (max, sum exp) per 256-column tile, tile-major
//   lse      [chunk_rows] f32 (used when the caller passes no lse)
//   rowa, rowb [chunk_rows] f32: per-row factors w_t (1 + 2 L lse_t) and w_t (0 for an ignored row)
//   f32 io only (implementation A): xs [chunk_rows, 3 D] and wsplit [V, 3 D] bf16 split copies of x and W
struct Ws {
  uint32_t* status = nullptr;
  void* store = nullptr; int64_t ldS = 0;
  float* tmax = nullptr; float* tsum = nullptr; int64_t ldT = 0; int NT = 0;
  float* lse = nullptr; float* rowa = nullptr; float* rowb = nullptr;
  uint64_t bytes = 0;
};
Ws carve(CeImpl impl, const CeShape& s, void* base);   // base == nullptr: sizes only

struct Settings {            // process-wide, recorded for callers that set them (one kernel set exists)
  int dgrad_own = 0, wgrad_own = 0, sm90 = 3;
  bool fast_stats_exp = false;
};
Settings& settings();

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

int device_arch();   // 100 on a B200 (cached per device)
int sm_count();

// One call (the C++ API and the C ABI both end here).
void run(CeImpl impl, Rounding r, const CeShape& s, const CeArgs& a, void* ws, cudaStream_t st);
void readout(CeImpl impl, Rounding r, const CeShape& s, const ReadoutCall& c, const CeArgs& base, float eps, void* ws,
             cudaStream_t st);

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
struct DgradArgs {
  const void* n; int64_t ldn; const void* w; int64_t ldw;   // ldw: row pitch of w in elements (D when contiguous)
  int rows, D, V;
  const float* scale;               // device scalar (*grad_scale)
  const void* dx_old; void* dx_out; int acc_mode; bool out_f32;
  uint32_t* status;
  int sm_reserve = 0;               // SMs left free (for a collective running beside this kernel)
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
};
void launch_wgrad(const WgradArgs& a, cudaStream_t st);

// unit-test entry: one CTA whose bounded wait runs out after `limit_cycles` (<= 2e6) on a barrier nobody completes
void launch_wait_timeout_probe(uint32_t* status, long long limit_cycles, int* saw_abort, cudaStream_t st);

// CTAs per accumulator tile of the three contractions: 0 = one CTA per 128 x 256 tile, 1 = a pair of CTAs (cluster of
// two, one UMMA of M = 256 over both) per 256 x 256 tile, negative = chosen per launch (the default). Process-wide;
// not to be changed while a call is in flight.
void set_cta_pair(int logits, int dgrad, int wgrad);

// unit-test entry: C f32 [M, N] = A B^T in the three operand layouts (kind 0 K/K, 1 K/MN, 2 MN/MN; + 4: CTA pairs)
void launch_test_gemm(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc, int M,
                      int N, int K, uint32_t* status, cudaStream_t st);

// ------------------------------------------------------------------------------------------------ row / streaming kernels
struct FinalizeArgs {
  const float* tmax; const float* tsum; int64_t ldT; int NT;
  const float* zt; const int32_t* targets; const float* weight;
  int rows, V; float z_loss; int32_t ignore_index; bool grads;
  float* lse; float* loss_tok; float* rowa; float* rowb;   // loss_tok may equal zt
};
void launch_finalize(const FinalizeArgs& a, cudaStream_t st);
void launch_chunk_loss(const float* loss_tok, const float* weight, int rows, float* out, cudaStream_t st);

// store -> bf16 n = rowa p - rowb onehot in place (f32 store: over the first half of each row, ld 2 ldS)
struct DzArgs {
  void* store; int64_t ldS; bool store_f32;
  const float* lse; const float* rowa; const float* rowb; const int32_t* targets;
  int rows, V;
};
void launch_dlogits_inplace(const DzArgs& a, cudaStream_t st);

void launch_finish_microbatch(float* dw, float* dw_mb, int64_t n, cudaStream_t st);
void launch_zero_cols(void* x, int64_t rows, int D, int from, cudaStream_t st);   // bf16 x[:, from:] = 0
void launch_sum_scale(const float* w, int64_t n, float mult, float* out, cudaStream_t st);
void launch_f32_to_bf16(const float* in, void* out, int64_t n, cudaStream_t st);
void launch_bf16_to_f32(const void* in, float* out, int64_t n, cudaStream_t st);
// f32 [rows, D] -> bf16 [rows, 3 D] holding (hi, hi, lo) (which == 0) or (hi, lo, hi) (which == 1) per row, so that
// the K = 3 D contraction of a (hi, hi, lo) matrix with a (hi, lo, hi) matrix is hi hi + hi lo + lo hi
void launch_split3(const float* in, void* out, int64_t rows, int D, int which, cudaStream_t st);

}  // namespace nm::ce
