// RMSNorm forward and backward (+ residual add, + gain-gradient partials) in bf16 storage, for the readout head.
// One warp per row; a lane owns the 16-byte pieces lane, lane + 32, ... of the row, so a row of D <= 8192 stays in
// registers between the reduction and the output pass.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "ew_rows.cuh"

namespace nm::ew {
namespace {

template <bool LEV>
__global__ void __launch_bounds__(kRowWarps * 32) k_rmsnorm_fwd(const __nv_bfloat16* __restrict__ x,
                                                             const __nv_bfloat16* __restrict__ gain,
                                                             __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                                             int64_t T, int D, float eps) {
  const int lane = threadIdx.x & 31;
  const int pieces = D / 8;
  for (int64_t row = blockIdx.x * int64_t(kRowWarps) + (threadIdx.x >> 5); row < T; row += int64_t(gridDim.x) * kRowWarps) {
    const __nv_bfloat16* xr = x + row * D;
    float ss = 0.f;
    for (int pc = lane; pc < pieces; pc += 32) {
      float f[8];
      load8(xr + pc * 8, f);
#pragma unroll
      for (int e = 0; e < 8; ++e) ss = fmaf(f[e], f[e], ss);
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(__fdiv_rn(ss, float(D)) + eps);
    if (rstd && lane == 0) rstd[row] = r;
    if (y) {
      for (int pc = lane; pc < pieces; pc += 32) {
        float f[8], g[8], o[8];
        load8(xr + pc * 8, f);
        load8(gain + pc * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = LEV ? __fmul_rn(g[e], rb(__fmul_rn(f[e], r))) : g[e] * (f[e] * r);
        store8(y + row * D + pc * 8, o);
      }
    }
  }
}

// One CTA per part of consecutive rows; warp w takes rows r0 + w, r0 + w + kRowWarps, ... and keeps its gain-gradient
// contributions in registers; the warps' sums are then added in warp order through shared memory.
template <bool LEV, int NP>   // NP: 16-byte pieces a lane may own (D <= NP * 256)
__global__ void __launch_bounds__(kRowWarps * 32) k_rmsnorm_bwd_add(const __nv_bfloat16* __restrict__ dy,
                                                                 const __nv_bfloat16* __restrict__ x,
                                                                 const __nv_bfloat16* __restrict__ gain,
                                                                 const float* __restrict__ rstd,
                                                                 const __nv_bfloat16* dres, __nv_bfloat16* dx,
                                                                 float* __restrict__ partial, int64_t T, int D,
                                                                 float eps, int64_t parts) {
  extern __shared__ float sred[];   // [kRowWarps, D]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pieces = D / 8;
  const int my = (pieces - lane + 31) / 32;   // pieces this lane owns
  for (int64_t p = blockIdx.x; p < parts; p += gridDim.x) {
    const int64_t r0 = p * T / parts, r1 = (p + 1) * T / parts;
    float dg[NP][8];
#pragma unroll
    for (int i = 0; i < NP; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) dg[i][e] = 0.f;
    for (int64_t row = r0 + warp; row < r1; row += kRowWarps) {
      const int64_t off = row * D;
      float s_xx = 0.f, s_xa = 0.f;
      for (int i = 0; i < my; ++i) {
        const int c0 = (lane + 32 * i) * 8;
        float xf[8], dyf[8], g[8];
        load8(x + off + c0, xf);
        load8(dy + off + c0, dyf);
        load8(gain + c0, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float a = LEV ? rb(__fmul_rn(g[e], dyf[e])) : g[e] * dyf[e];
          s_xx = fmaf(xf[e], xf[e], s_xx);
          s_xa = fmaf(xf[e], a, s_xa);
        }
      }
      s_xx = warp_sum(s_xx);
      s_xa = warp_sum(s_xa);
      const float ms = __fdiv_rn(s_xx, float(D));
      const float r = rstd ? __ldg(rstd + row) : rsqrtf(ms + eps);
      const float c = __fdiv_rn(__fmul_rn(s_xa, __fmul_rn(-0.5f, __fdiv_rn(r, ms + eps))), float(D));
#pragma unroll
      for (int i = 0; i < NP; ++i) {
        if (i < my) {
          const int c0 = (lane + 32 * i) * 8;
          float xf[8], dyf[8], g[8], d[8];
          load8(x + off + c0, xf);
          load8(dy + off + c0, dyf);
          load8(gain + c0, g);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float a = LEV ? rb(__fmul_rn(g[e], dyf[e])) : g[e] * dyf[e];
            d[e] = LEV ? __fadd_rn(__fmul_rn(a, r), __fmul_rn(c, __fmul_rn(2.f, xf[e]))) : fmaf(a, r, c * (2.f * xf[e]));
            dg[i][e] += LEV ? rb(__fmul_rn(dyf[e], rb(__fmul_rn(xf[e], r)))) : dyf[e] * (xf[e] * r);
          }
          if (dres) {
            float q[8];
            load8(dres + off + c0, q);
#pragma unroll
            for (int e = 0; e < 8; ++e) d[e] = LEV ? __fadd_rn(q[e], rb(d[e])) : q[e] + d[e];
          }
          store8(dx + off + c0, d);
        }
      }
    }
    if (partial) {
#pragma unroll
      for (int i = 0; i < NP; ++i)
        if (i < my) {
          const int c0 = (lane + 32 * i) * 8;
#pragma unroll
          for (int e = 0; e < 8; ++e) sred[warp * D + c0 + e] = dg[i][e];
        }
      __syncthreads();
      for (int d = threadIdx.x; d < D; d += kRowWarps * 32) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kRowWarps; ++w) s = __fadd_rn(s, sred[w * D + d]);
        partial[p * D + d] = s;
      }
      __syncthreads();
    }
  }
}

}  // namespace

int64_t norm_partial_rows(int64_t T) {
  const int64_t by_rows = std::max<int64_t>(1, (T + 15) / 16);
  return std::min<int64_t>(std::min<int64_t>(1024, by_rows), int64_t(4) * ce::sm_count());
}

void rmsnorm_fwd(const bf16_t* x, const bf16_t* gain, bf16_t* y, float* rstd, int64_t T, int D, float eps,
                 cudaStream_t st, Rounding r) {
  NM_REQUIRE(x && gain && T >= 0 && D > 0 && D % 8 == 0, "rmsnorm_fwd: x, gain, D % 8 == 0");
  NM_REQUIRE(aligned16(x, gain, y), "rmsnorm_fwd: x, gain, y must be 16-byte aligned");
  if (T == 0) return;
  const int grid = int(std::min<int64_t>((T + kRowWarps - 1) / kRowWarps, int64_t(ce::sm_count()) * 8));
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gain);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  if (r == Rounding::Levanter) k_rmsnorm_fwd<true><<<grid, kRowWarps * 32, 0, st>>>(X, G, Y, rstd, T, D, eps);
  else k_rmsnorm_fwd<false><<<grid, kRowWarps * 32, 0, st>>>(X, G, Y, rstd, T, D, eps);
  NM_CUDA(cudaGetLastError());
}

void rmsnorm_bwd_add(const bf16_t* dy, const bf16_t* x, const bf16_t* gain, const float* rstd, const bf16_t* dres,
                     bf16_t* dx, float* dgain_partial, int64_t T, int D, float eps, cudaStream_t st, Rounding r) {
  NM_REQUIRE(dy && x && gain && dx && T >= 0 && D > 0 && D % 8 == 0, "rmsnorm_bwd_add: dy, x, gain, dx, D % 8 == 0");
  NM_REQUIRE(aligned16(dy, x, gain, dres, dx, dgain_partial), "rmsnorm_bwd_add: every pointer must be 16-byte aligned");
  NM_REQUIRE(D <= kMaxPieces * 32 * 8, "rmsnorm_bwd_add: D <= 8192");
  if (T == 0) return;
  const int64_t parts = norm_partial_rows(T);
  const size_t smem = size_t(kRowWarps) * D * sizeof(float);
  const bool lev = r == Rounding::Levanter;
  auto kern = D <= 512    ? (lev ? k_rmsnorm_bwd_add<true, 2> : k_rmsnorm_bwd_add<false, 2>)
              : D <= 2048 ? (lev ? k_rmsnorm_bwd_add<true, 8> : k_rmsnorm_bwd_add<false, 8>)
                          : (lev ? k_rmsnorm_bwd_add<true, kMaxPieces> : k_rmsnorm_bwd_add<false, kMaxPieces>);
  NM_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
  kern<<<int(parts), kRowWarps * 32, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(dy),
                                              reinterpret_cast<const __nv_bfloat16*>(x),
                                              reinterpret_cast<const __nv_bfloat16*>(gain), rstd,
                                              reinterpret_cast<const __nv_bfloat16*>(dres),
                                              reinterpret_cast<__nv_bfloat16*>(dx), dgain_partial, T, D, eps, parts);
  NM_CUDA(cudaGetLastError());
}

}  // namespace nm::ew
