// Sampled-softmax head (include/marincpp/kernels/sampled_head.hpp): the candidate set of a microbatch, the gathered
// head W_P, the fused CE over it, and the scatter of dW_P back into the full gradient. The reference describes this
// head (include/marincpp/model.hpp:236-239) without shipping it; the kernels here are small streaming kernels around the
// one fused-CE pipeline of this library.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <numeric>

#include "abi_guard.hpp"
#include "ce_internal.hpp"
#include "marincpp/capi_ce.h"
#include "marincpp/kernels/sampled_head.hpp"

namespace nm {
namespace {

// Bias of the unused candidate columns. Far below any real logit, so exp(z - lse) is exactly 0 in f32 for them, yet
// small enough that m * log2e stays accurate to ~1e-3 in the online softmax of a tile that holds only such columns
// (that tile's partial sum is then multiplied by exp(-30000 - max) = 0 when the tiles are merged).
constexpr float kMaskedLogit = -30000.f;

// mark[v] = 1 for every id that is a counted target or one of the strided negatives
__global__ void k_sampled_mark(const int32_t* __restrict__ targets, const float* __restrict__ weight, int64_t T, int V,
                               int32_t ignore_index, int n_neg, int64_t neg_first, int64_t stride, uint8_t* mark) {
  const int64_t n = T + n_neg;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    if (i < T) {
      const int32_t tg = targets[i];
      if (tg >= 0 && tg < V && tg != ignore_index && weight[i] != 0.f) mark[tg] = 1;
    } else {
      mark[(neg_first + (i - T) * stride) % V] = 1;
    }
  }
}

// One CTA walks the vocabulary in ascending order, 4096 ids per step (four per thread), and numbers the marked ones:
// remap[v] = position of v among the marked ids (or -1), cand[position] = v. Ascending ids give the sorted unique set
// directly. Then cand[count ..] = -1, bias[i] = 0 for i < count and the masked value beyond, and *count_out = count.
__global__ void __launch_bounds__(1024) k_sampled_compact(const uint8_t* __restrict__ mark, int V, int p_max,
                                                          int32_t* __restrict__ remap, int32_t* __restrict__ cand,
                                                          float* __restrict__ bias, int32_t* count_out,
                                                          int32_t* count_copy) {
  __shared__ int warp_total[32];
  __shared__ int running;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  for (int v0 = 0; v0 < V; v0 += 4096) {
    const int v = v0 + int(threadIdx.x) * 4;
    int m[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) m[q] = (v + q < V) ? int(mark[v + q]) : 0;
    const int mine = m[0] + m[1] + m[2] + m[3];
    int incl = mine;                                   // inclusive scan over the warp
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) warp_total[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int t = warp_total[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, t, o);
        if (lane >= o) t += up;
      }
      warp_total[lane] = t;                            // inclusive totals of the warps
    }
    __syncthreads();
    int pos = running + (warp ? warp_total[warp - 1] : 0) + incl - mine;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (v + q < V) {
        const bool in = m[q] != 0 && pos < p_max;      // p_max cannot be exceeded (checked on the host); belt and braces
        remap[v + q] = in ? pos : -1;
        if (in) cand[pos] = v + q;
        pos += m[q];
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) running += warp_total[31];
    __syncthreads();
  }
  const int count = min(running, p_max);
  for (int i = threadIdx.x; i < p_max; i += blockDim.x) {
    if (i >= count) cand[i] = -1;
    bias[i] = i < count ? 0.f : kMaskedLogit;
  }
  if (threadIdx.x == 0) {
    *count_out = count;
    if (count_copy) *count_copy = count;
  }
}

__global__ void k_sampled_remap_targets(const int32_t* __restrict__ targets, const float* __restrict__ weight, int64_t T,
                                        int V, int32_t ignore_index, const int32_t* __restrict__ remap,
                                        int32_t* __restrict__ out) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < T; i += int64_t(gridDim.x) * blockDim.x) {
    const int32_t tg = targets[i];
    const bool counts = tg >= 0 && tg < V && tg != ignore_index && weight[i] != 0.f;
    out[i] = counts ? remap[tg] : -1;
  }
}

// W_P[i, :] = W[cand[i], :] (16-byte pieces); rows at or beyond the count are zero
__global__ void k_sampled_gather(const uint4* __restrict__ w, const int32_t* __restrict__ cand, int p_max, int pieces,
                                 uint4* __restrict__ wp) {
  const int64_t n = int64_t(p_max) * pieces;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const int row = int(i / pieces), pc = int(i % pieces);
    const int32_t src = cand[row];
    wp[i] = src >= 0 ? w[int64_t(src) * pieces + pc] : make_uint4(0u, 0u, 0u, 0u);
  }
}

// dW[cand[i], :] += dW_P[i, :]; the candidate rows are distinct, so every element has one writer
__global__ void k_sampled_scatter_add(const float4* __restrict__ dwp, const int32_t* __restrict__ cand, int p_max,
                                      int quads, float4* __restrict__ dw) {
  const int64_t n = int64_t(p_max) * quads;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const int row = int(i / quads), q = int(i % quads);
    const int32_t dst = cand[row];
    if (dst < 0) continue;
    const float4 g = dwp[i];
    float4* o = dw + int64_t(dst) * quads + q;
    float4 cur = *o;
    cur.x = __fadd_rn(cur.x, g.x);
    cur.y = __fadd_rn(cur.y, g.y);
    cur.z = __fadd_rn(cur.z, g.z);
    cur.w = __fadd_rn(cur.w, g.w);
    *o = cur;
  }
}

int grid_for(int64_t n) {
  return int(std::max<int64_t>(1, std::min<int64_t>((n + 255) / 256, int64_t(ce::sm_count()) * 8)));
}

struct SampledRegions {
  uint8_t* mark; int32_t* remap; int32_t* cand; int32_t* count; int32_t* targets_p; float* bias;
  void* w_p; float* dw_p; void* ce_ws;
  uint64_t bytes;
};

CeShape ce_shape_of(const SampledHeadShape& s) {
  CeShape c{};
  c.T = s.T;
  c.D = s.D;
  c.V = s.p_max;
  c.chunk_rows = s.chunk_rows;
  c.logits_store = s.logits_store;
  c.io = DType::bf16;
  return c;
}

SampledRegions layout(const SampledHeadShape& s, void* base) {
  ce::Arena arena(base);
  SampledRegions r{};
  r.mark = arena.take<uint8_t>(uint64_t(s.V));
  r.remap = arena.take<int32_t>(uint64_t(s.V));
  r.cand = arena.take<int32_t>(uint64_t(s.p_max));
  r.count = arena.take<int32_t>(64);
  r.targets_p = arena.take<int32_t>(uint64_t(s.T));
  r.bias = arena.take<float>(uint64_t(s.p_max));
  r.w_p = arena.take<uint16_t>(uint64_t(s.p_max) * s.D);
  r.dw_p = arena.take<float>(uint64_t(s.p_max) * s.D);
  const uint64_t ce_bytes = ce_workspace_bytes(CeImpl::B1, ce_shape_of(s));
  r.ce_ws = arena.take<uint8_t>(ce_bytes);
  r.bytes = arena.bytes();
  return r;
}

void require_shape(const SampledHeadShape& s, int n_negatives) {
  NM_REQUIRE(s.T >= 0 && s.D > 0 && s.V > 0, "sampled head: T >= 0, D > 0, V > 0");
  NM_REQUIRE(s.D % 8 == 0, "sampled head: D must be a multiple of 8");
  NM_REQUIRE(s.p_max > 0 && s.p_max % 8 == 0, "sampled head: p_max must be a positive multiple of 8");
  NM_REQUIRE(n_negatives >= 0, "sampled head: n_negatives cannot be negative");
  const int64_t worst = std::min<int64_t>(s.V, s.T + n_negatives);
  NM_REQUIRE(s.p_max >= worst, "sampled head: p_max = " + std::to_string(s.p_max) + " could overflow; it must be at least "
                                   "min(V, T + n_negatives) = " + std::to_string(worst));
}

}  // namespace

int64_t sampled_stride(int64_t V) {
  if (V <= 2) return 1;
  int64_t s = int64_t(double(V) * 0.6180339887498949 + 0.5);
  s = std::max<int64_t>(1, std::min<int64_t>(s, V - 1));
  while (std::gcd(s, V) != 1) ++s;     // V - 1 is coprime with V, so this ends below V
  return s;
}

uint64_t sampled_head_workspace_bytes(const SampledHeadShape& s) {
  require_shape(s, 0);
  return layout(s, nullptr).bytes;
}

void sampled_head(Rounding r, const SampledHeadShape& s, const SampledHeadArgs& a, void* ws, cudaStream_t st) {
  require_shape(s, a.n_negatives);
  if (s.T == 0) return;
  NM_REQUIRE(a.x && a.w && a.targets && a.weight && a.loss_tok, "sampled head: x, w, targets, weight and loss_tok are "
                                                                "required");
  NM_REQUIRE(ws != nullptr && reinterpret_cast<uintptr_t>(ws) % kArenaAlign == 0,
             "sampled head: a 256-byte aligned workspace of sampled_head_workspace_bytes() bytes is required");
  NM_REQUIRE(reinterpret_cast<uintptr_t>(a.w) % 16 == 0 && reinterpret_cast<uintptr_t>(a.dw) % 16 == 0,
             "sampled head: w and dw must be 16-byte aligned");
  const SampledRegions g = layout(s, ws);
  const bool grads = !a.forward_only && (a.dx != nullptr || a.dw != nullptr);
  const int V = s.V, D = s.D;
  int64_t first = a.neg_offset % V;
  if (first < 0) first += V;

  // 1-2: candidates and remapped targets
  NM_CUDA(cudaMemsetAsync(g.mark, 0, size_t(V), st));
  k_sampled_mark<<<grid_for(s.T + a.n_negatives), 256, 0, st>>>(a.targets, a.weight, s.T, V, a.ignore_index,
                                                               a.n_negatives, first, sampled_stride(V), g.mark);
  k_sampled_compact<<<1, 1024, 0, st>>>(g.mark, V, s.p_max, g.remap, g.cand, g.bias, g.count, a.n_candidates_out);
  k_sampled_remap_targets<<<grid_for(s.T), 256, 0, st>>>(a.targets, a.weight, s.T, V, a.ignore_index, g.remap,
                                                         g.targets_p);
  if (a.candidates_out)
    NM_CUDA(cudaMemcpyAsync(a.candidates_out, g.cand, size_t(s.p_max) * 4, cudaMemcpyDeviceToDevice, st));
  // 3: gathered head
  k_sampled_gather<<<grid_for(int64_t(s.p_max) * (D / 8)), 256, 0, st>>>(static_cast<const uint4*>(a.w), g.cand,
                                                                       s.p_max, D / 8, static_cast<uint4*>(g.w_p));
  NM_CUDA(cudaGetLastError());
  // 4: the fused CE over the candidate columns; the unused ones are masked by the bias
  const bool want_dw = grads && a.dw != nullptr;
  if (want_dw) NM_CUDA(cudaMemsetAsync(g.dw_p, 0, size_t(s.p_max) * D * 4, st));
  CeArgs c{};
  c.x = a.x;
  c.w = g.w_p;
  c.targets = g.targets_p;
  c.weight = a.weight;
  c.grad_scale = a.grad_scale;
  c.logit_bias = g.bias;
  c.loss_tok = a.loss_tok;
  c.lse = a.lse;
  c.loss_partial = a.loss_partial;
  c.dx = grads ? a.dx : nullptr;
  c.accumulate_dx = a.accumulate_dx;
  c.dw = want_dw ? g.dw_p : nullptr;
  c.dw_microbatch = nullptr;
  c.dw_round = CeDwRound::None;
  c.forward_only = a.forward_only;
  c.z_loss_weight = a.z_loss_weight;
  c.ignore_index = INT32_MIN;            // ignored rows already carry target -1
  ce::RunOptions opt;
  opt.allow_logit_bias = true;
  ce::run(CeImpl::B1, r, ce_shape_of(s), c, g.ce_ws, st, opt);
  // 5: unique-row scatter
  if (want_dw) {
    k_sampled_scatter_add<<<grid_for(int64_t(s.p_max) * (D / 4)), 256, 0, st>>>(
        reinterpret_cast<const float4*>(g.dw_p), g.cand, s.p_max, D / 4, reinterpret_cast<float4*>(a.dw));
    NM_CUDA(cudaGetLastError());
  }
}

}  // namespace nm

extern "C" {

int64_t nm_ce_sampled_stride(int64_t V) {
  return nm::abi::guarded_value<int64_t>(0, [&] { return nm::sampled_stride(V); });
}

uint64_t nm_ce_sampled_workspace_bytes(int64_t T, int D, int V, int p_max, int chunk_rows, int logits_store) {
  return nm::abi::guarded_value<uint64_t>(0, [&] {
    NM_REQUIRE(logits_store == 0 || logits_store == 1, "logits_store must be 0 (f32) or 1 (bf16)");
    nm::SampledHeadShape s{T, D, V, p_max, chunk_rows, logits_store == 0 ? nm::DType::f32 : nm::DType::bf16};
    return nm::sampled_head_workspace_bytes(s);
  });
}

int nm_ce_sampled_head(int rounding, int logits_store, const void* x, const void* w, const int32_t* targets,
                       const float* weight, const float* grad_scale, float* loss_tok, float* lse, float* loss_partial,
                       void* dx, int accumulate_dx, float* dw, int forward_only, int64_t T, int D, int V,
                       int n_negatives, int64_t neg_offset, int p_max, int chunk_rows, int32_t* candidates_out,
                       int32_t* n_candidates_out, void* workspace, void* stream, float z_loss_weight,
                       int32_t ignore_index) {
  return nm::abi::guarded([&] {
    NM_REQUIRE(rounding == 0 || rounding == 1, "rounding must be 0 (levanter) or 1 (accurate)");
    NM_REQUIRE(logits_store == 0 || logits_store == 1, "logits_store must be 0 (f32) or 1 (bf16)");
    nm::SampledHeadShape s{T, D, V, p_max, chunk_rows, logits_store == 0 ? nm::DType::f32 : nm::DType::bf16};
    nm::SampledHeadArgs a{};
    a.x = x;
    a.w = w;
    a.targets = targets;
    a.weight = weight;
    a.grad_scale = grad_scale;
    a.loss_tok = loss_tok;
    a.lse = lse;
    a.loss_partial = loss_partial;
    a.dx = dx;
    a.accumulate_dx = accumulate_dx != 0;
    a.dw = dw;
    a.forward_only = forward_only != 0;
    a.n_negatives = n_negatives;
    a.neg_offset = neg_offset;
    a.z_loss_weight = z_loss_weight;
    a.ignore_index = ignore_index;
    a.candidates_out = candidates_out;
    a.n_candidates_out = n_candidates_out;
    nm::sampled_head(rounding == 0 ? nm::Rounding::Levanter : nm::Rounding::Accurate, s, a, workspace,
                     static_cast<cudaStream_t>(stream));
  });
}

}  // extern "C"
