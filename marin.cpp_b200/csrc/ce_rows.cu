// Row and streaming kernels of the fused linear cross-entropy (plain SIMT, HBM- or latency-bound): the merge of the
// per-tile softmax partials, the in-place rewrite of the logits store as the normalised gradient, the fixed-order loss
// and weight reductions, and the small helpers of the strict dW mode, the readout head and the f32-io path.
// Counterparts in the reference: k_ce_finalize_rows, k_ce_chunk_loss, k_ce_dlogits_bf16 / _f32
// (src/kernels/cross_entropy/ce_logits.cu:220-318) and ce_small.cu:22-61.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "ce_internal.hpp"
#include "ptx.cuh"

namespace nm::ce {
namespace {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// ------------------------------------------------------------------------------------------------ finalize
// 32 rows per CTA (lane = row), 8 warps: warp w merges the tile partials of segment w of the vocabulary in ascending
// order (m_w = max_i m_i, s_w = sum_i s_i exp(m_i - m_w)); warp 0 then merges the 8 segments in ascending order:
// M = max_w m_w (0 when not finite), S = sum_w s_w exp(m_w - M), lse = log S + M. The order depends only on the
// number of tiles, so lse and the loss do not depend on the chunk size or the launch geometry.
// loss = lse - z[target] + L lse^2 for a row that counts, else 0. rowb = weight (0 for an ignored target or a
// forward-only call), rowa = rowb (1 + 2 L lse): the two per-row factors of the normalised gradient.
constexpr int kFinWarps = 8;
__global__ void __launch_bounds__(32 * kFinWarps) k_ce_finalize_rows(FinalizeArgs p) {
  __shared__ float sm[kFinWarps][32], ss[kFinWarps][32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int r = blockIdx.x * 32 + lane;
  const bool on = r < p.rows;
  const int i0 = int(int64_t(p.NT) * w / kFinWarps), i1 = int(int64_t(p.NT) * (w + 1) / kFinWarps);
  float m = -INFINITY, s = 0.f;
  if (on) {
#pragma unroll 4
    for (int i = i0; i < i1; ++i) m = fmaxf(m, p.tmax[int64_t(i) * p.ldT + r]);
    const float mm = isfinite(m) ? m : 0.f;
#pragma unroll 4
    for (int i = i0; i < i1; ++i) {
      const int64_t o = int64_t(i) * p.ldT + r;
      s = __fadd_rn(s, __fmul_rn(p.tsum[o], expf(__fsub_rn(p.tmax[o], mm))));
    }
  }
  sm[w][lane] = m;
  ss[w][lane] = s;
  __syncthreads();
  if (w != 0 || !on) return;
  float M = -INFINITY;
#pragma unroll
  for (int k = 0; k < kFinWarps; ++k) M = fmaxf(M, sm[k][lane]);
  if (!isfinite(M)) M = 0.f;
  float S = 0.f;
#pragma unroll
  for (int k = 0; k < kFinWarps; ++k) {
    const float mk = isfinite(sm[k][lane]) ? sm[k][lane] : 0.f;
    S = __fadd_rn(S, __fmul_rn(ss[k][lane], expf(__fsub_rn(mk, M))));   // an empty segment has s = 0
  }
  const float lse = __fadd_rn(logf(S), M);
  const int tg = p.targets[r];
  const float wt = p.weight[r];
  const bool valid = tg >= 0 && tg < p.V && tg != p.ignore_index;
  float loss = 0.f;
  if (valid && wt != 0.f) {
    loss = __fsub_rn(lse, p.zt[r]);
    if (p.z_loss != 0.f) loss = __fadd_rn(loss, __fmul_rn(p.z_loss, __fmul_rn(lse, lse)));
  }
  p.lse[r] = lse;
  p.loss_tok[r] = loss;
  const float rb = (p.grads && valid) ? wt : 0.f;
  p.rowb[r] = rb;
  p.rowa[r] = (p.z_loss != 0.f) ? __fmul_rn(rb, __fmaf_rn(2.f * p.z_loss, lse, 1.f)) : rb;
}

// sum_t weight[t] * loss[t] by one CTA of 1024 threads: thread-strided sequential f32 sums, then a binary tree. The
// order is part of the contract (the per-chunk loss must not depend on the launch geometry).
__global__ void __launch_bounds__(1024) k_ce_chunk_loss(const float* loss, const float* w, int rows, float* out) {
  __shared__ float red[1024];
  float s = 0.f;
  for (int r = threadIdx.x; r < rows; r += 1024) s = __fadd_rn(s, __fmul_rn(w[r], loss[r]));
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if (int(threadIdx.x) < o) red[threadIdx.x] = __fadd_rn(red[threadIdx.x], red[threadIdx.x + o]);
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = red[0];
}

// out = mult / sum(w), same reduction order as above.
__global__ void __launch_bounds__(1024) k_sum_scale(const float* w, int64_t n, float mult, float* out) {
  __shared__ float red[1024];
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += 1024) s = __fadd_rn(s, w[i]);
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if (int(threadIdx.x) < o) red[threadIdx.x] = __fadd_rn(red[threadIdx.x], red[threadIdx.x + o]);
    __syncthreads();
  }
  if (threadIdx.x == 0) *out = __fdiv_rn(mult, red[0]);
}

// ------------------------------------------------------------------------------------------------ normalised gradient
// n = rowa p - rowb onehot, p = exp(z_s - lse) = 2^(z_s log2e - lse log2e); columns >= V are written as 0.
__device__ __forceinline__ float grad_n(float zs, float neg_lse2, float ra, float rb, bool is_target, bool ok) {
  const float p = nm::ptx::ex2_approx(fmaf(zs, kLog2e, neg_lse2));
  const float d = __fmul_rn(p, ra);
  const float r = is_target ? __fsub_rn(d, rb) : d;
  return ok ? r : 0.f;
}

// bf16 store, in place. Each thread owns one 16-byte piece (8 logits) of kDzRows consecutive rows; all loads of a
// thread are issued before its math, and the grid strides over row groups.
constexpr int kDzRows = 4;
__global__ void __launch_bounds__(256) k_ce_dlogits_bf16(DzArgs p) {
  const int npieces = int((p.V + 7) / 8);
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= npieces) return;
  const int v0 = c * 8;
  __nv_bfloat16* base = static_cast<__nv_bfloat16*>(p.store);
  for (int r0 = blockIdx.y * kDzRows; r0 < p.rows; r0 += gridDim.y * kDzRows) {
    uint4 raw[kDzRows];
#pragma unroll
    for (int q = 0; q < kDzRows; ++q)
      if (r0 + q < p.rows) raw[q] = *reinterpret_cast<const uint4*>(base + int64_t(r0 + q) * p.ldS + v0);
#pragma unroll
    for (int q = 0; q < kDzRows; ++q) {
      const int r = r0 + q;
      if (r < p.rows) {
        const float neg = -p.lse[r] * kLog2e, ra = p.rowa[r], rb = p.rowb[r];
        const int tg = p.targets[r];
        uint32_t u[4] = {raw[q].x, raw[q].y, raw[q].z, raw[q].w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int v = v0 + 2 * e;
          const float d0 = grad_n(bf_lo(u[e]), neg, ra, rb, v == tg, v < p.V);
          const float d1 = grad_n(bf_hi(u[e]), neg, ra, rb, v + 1 == tg, v + 1 < p.V);
          u[e] = pack2(d0, d1);
        }
        *reinterpret_cast<uint4*>(base + int64_t(r) * p.ldS + v0) = make_uint4(u[0], u[1], u[2], u[3]);
      }
    }
  }
}

// f32 store: the bf16 result of a row is packed over the first half of the same row (leading dimension 2 ldS in bf16
// elements). A CTA walks its row 1024 logits at a time in ascending order; the bytes a step writes, [2048 s, 2048 s +
// 2048), were read as f32 by this or an earlier step, and the barrier between a step's reads and writes orders them.
__global__ void __launch_bounds__(256) k_ce_dlogits_f32(DzArgs p) {
  for (int r = blockIdx.x; r < p.rows; r += gridDim.x) {
    const float* zr = static_cast<const float*>(p.store) + int64_t(r) * p.ldS;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(static_cast<float*>(p.store) + int64_t(r) * p.ldS);
    const float neg = -p.lse[r] * kLog2e, ra = p.rowa[r], rb = p.rowb[r];
    const int tg = p.targets[r];
    for (int s0 = 0; s0 < p.ldS; s0 += 1024) {
      const int v = s0 + int(threadIdx.x) * 4;
      float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
      if (v < p.ldS) z = *reinterpret_cast<const float4*>(zr + v);   // ldS % 8 == 0: whole float4s
      __syncthreads();
      if (v < p.ldS) {
        const float d0 = grad_n(z.x, neg, ra, rb, v == tg, v < p.V);
        const float d1 = grad_n(z.y, neg, ra, rb, v + 1 == tg, v + 1 < p.V);
        const float d2 = grad_n(z.z, neg, ra, rb, v + 2 == tg, v + 2 < p.V);
        const float d3 = grad_n(z.w, neg, ra, rb, v + 3 == tg, v + 3 < p.V);
        *reinterpret_cast<uint2*>(out + v) = make_uint2(pack2(d0, d1), pack2(d2, d3));
      }
    }
    __syncthreads();
  }
}

// ------------------------------------------------------------------------------------------------ small helpers
__global__ void k_finish_microbatch(float* dw, float* mb, int64_t n) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    dw[i] = __fadd_rn(dw[i], __bfloat162float(__float2bfloat16_rn(mb[i])));
    mb[i] = 0.f;
  }
}

__global__ void k_zero_cols_bf16(__nv_bfloat16* x, int64_t rows, int D, int from) {
  const int wdt = D - from;
  const int64_t n = rows * wdt;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    x[(i / wdt) * D + from + i % wdt] = __float2bfloat16_rn(0.f);
}

__global__ void k_f32_to_bf16(const float* in, __nv_bfloat16* out, int64_t n) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void k_bf16_to_f32(const __nv_bfloat16* in, float* out, int64_t n) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    out[i] = __bfloat162float(in[i]);
}

// f32 [rows, D] -> bf16 [rows, 3 D]: hi = bf16(v), lo = bf16(v - hi); which 0: (hi | hi | lo), 1: (hi | lo | hi)
__global__ void k_split3(const float* in, __nv_bfloat16* out, int64_t rows, int D, int which) {
  const int64_t n = rows * D;
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x) {
    const int64_t r = i / D;
    const int d = int(i % D);
    const float v = in[i];
    const __nv_bfloat16 hi = __float2bfloat16_rn(v);
    const __nv_bfloat16 lo = __float2bfloat16_rn(__fsub_rn(v, __bfloat162float(hi)));
    __nv_bfloat16* o = out + r * 3 * D;
    o[d] = hi;
    o[D + d] = which ? lo : hi;
    o[2 * D + d] = which ? hi : lo;
  }
}

int grid_for(int64_t n, int threads) {
  return int(std::max<int64_t>(1, std::min<int64_t>((n + threads - 1) / threads, int64_t(sm_count()) * 16)));
}

}  // namespace

void launch_finalize(const FinalizeArgs& a, cudaStream_t st) {
  if (a.rows <= 0) return;
  k_ce_finalize_rows<<<(a.rows + 31) / 32, 32 * kFinWarps, 0, st>>>(a);
  NM_CUDA(cudaGetLastError());
}

void launch_chunk_loss(const float* loss_tok, const float* weight, int rows, float* out, cudaStream_t st) {
  k_ce_chunk_loss<<<1, 1024, 0, st>>>(loss_tok, weight, rows, out);
  NM_CUDA(cudaGetLastError());
}

void launch_dlogits_inplace(const DzArgs& a, cudaStream_t st) {
  if (a.rows <= 0) return;
  // 16-byte vector accesses on every row of the store
  NM_REQUIRE(reinterpret_cast<uintptr_t>(a.store) % 16 == 0 && a.ldS % 8 == 0,
             "dlogits: the store must be 16-byte aligned with a row pitch that is a multiple of 8 elements");
  if (a.store_f32) {
    k_ce_dlogits_f32<<<std::min(a.rows, sm_count() * 8), 256, 0, st>>>(a);
  } else {
    const int npieces = int((a.V + 7) / 8);
    const int gx = (npieces + 255) / 256;
    const int groups = (a.rows + kDzRows - 1) / kDzRows;
    const int gy = std::max(1, std::min(groups, std::max(1, sm_count() * 16 / gx)));
    k_ce_dlogits_bf16<<<dim3(gx, gy), 256, 0, st>>>(a);
  }
  NM_CUDA(cudaGetLastError());
}

void launch_finish_microbatch(float* dw, float* dw_mb, int64_t n, cudaStream_t st) {
  if (n <= 0) return;
  k_finish_microbatch<<<grid_for(n, 256), 256, 0, st>>>(dw, dw_mb, n);
  NM_CUDA(cudaGetLastError());
}

void launch_zero_cols(void* x, int64_t rows, int D, int from, cudaStream_t st) {
  if (rows <= 0 || from >= D) return;
  k_zero_cols_bf16<<<grid_for(rows * (D - from), 256), 256, 0, st>>>(static_cast<__nv_bfloat16*>(x), rows, D, from);
  NM_CUDA(cudaGetLastError());
}

void launch_sum_scale(const float* w, int64_t n, float mult, float* out, cudaStream_t st) {
  k_sum_scale<<<1, 1024, 0, st>>>(w, n, mult, out);
  NM_CUDA(cudaGetLastError());
}

void launch_f32_to_bf16(const float* in, void* out, int64_t n, cudaStream_t st) {
  if (n <= 0) return;
  k_f32_to_bf16<<<grid_for(n, 256), 256, 0, st>>>(in, static_cast<__nv_bfloat16*>(out), n);
  NM_CUDA(cudaGetLastError());
}
void launch_bf16_to_f32(const void* in, float* out, int64_t n, cudaStream_t st) {
  if (n <= 0) return;
  k_bf16_to_f32<<<grid_for(n, 256), 256, 0, st>>>(static_cast<const __nv_bfloat16*>(in), out, n);
  NM_CUDA(cudaGetLastError());
}
void launch_split3(const float* in, void* out, int64_t rows, int D, int which, cudaStream_t st) {
  if (rows <= 0) return;
  k_split3<<<grid_for(rows * D, 256), 256, 0, st>>>(in, static_cast<__nv_bfloat16*>(out), rows, D, which);
  NM_CUDA(cudaGetLastError());
}

}  // namespace nm::ce
