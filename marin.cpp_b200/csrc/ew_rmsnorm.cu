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

// One CTA per part of consecutive rows (the partition of norm_partial_rows), row groups as described in ew_rows.cuh:
// a thread loads its pieces of dy, x (and the residual gradient) once, the group reduces sum x^2 and sum x a, and the
// same registers feed the output pass. Gain-gradient sums stay in the owning thread's registers for the whole part.
template <bool LEV, int PP>
__global__ void __launch_bounds__(kGroupThreads, PP == 1 ? 4 : 1) k_rmsnorm_bwd_add(const __nv_bfloat16* __restrict__ dy,
                                                                const __nv_bfloat16* __restrict__ x,
                                                                const __nv_bfloat16* __restrict__ gain,
                                                                const float* __restrict__ rstd,
                                                                const __nv_bfloat16* dres, __nv_bfloat16* dx,
                                                                float* __restrict__ partial, int64_t T, int D,
                                                                float eps, int64_t parts, int G) {
  __shared__ float red[2 * 8 * 2];
  __shared__ float gsm[kGroupThreads * 8];
  const RowGroup rg = row_group(G);
  const int pieces = D / 8;
  int flip = 0;
  uint4 gq[PP];
#pragma unroll
  for (int i = 0; i < PP; ++i) {
    const int pc = rg.tg + i * rg.G;
    gq[i] = pc < pieces ? ldg16(gain + pc * 8) : make_uint4(0u, 0u, 0u, 0u);
  }
  for (int64_t p = blockIdx.x; p < parts; p += gridDim.x) {
    const int64_t r0 = p * T / parts, r1 = (p + 1) * T / parts;
    float dg[PP][8];
#pragma unroll
    for (int i = 0; i < PP; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) dg[i][e] = 0.f;
    // every group runs the same number of iterations (the group reduction is a barrier of the group only, but the
    // gain reduction at the end is a barrier of the CTA)
    for (int64_t base = r0; base < r1; base += rg.groups) {
      const int64_t row = base + rg.group;
      const bool on = row < r1;
      const int64_t off = row * D;
      uint4 xq[PP], dq[PP], rq[PP];
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        const int pc = rg.tg + i * rg.G;
        const bool in = on && pc < pieces;
        xq[i] = in ? ldg16(x + off + pc * 8) : make_uint4(0u, 0u, 0u, 0u);
        dq[i] = in ? ldg16(dy + off + pc * 8) : make_uint4(0u, 0u, 0u, 0u);
        rq[i] = (in && dres) ? ldg16(dres + off + pc * 8) : make_uint4(0u, 0u, 0u, 0u);
      }
      float sums[2] = {0.f, 0.f};   // sum x^2, sum x a
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        float xf[8], dyf[8], g[8];
        unpack8(xq[i], xf);
        unpack8(dq[i], dyf);
        unpack8(gq[i], g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sums[0] = fmaf(xf[e], xf[e], sums[0]);
          sums[1] = fmaf(xf[e], norm_a<LEV>(g[e], dyf[e]), sums[1]);
        }
      }
      group_sum<2>(sums, rg, red, flip);
      if (!on) continue;
      const float ms = __fdiv_rn(sums[0], float(D));
      const float r = rstd ? __ldg(rstd + row) : rsqrtf(ms + eps);
      const float c2 = norm_c2(sums[1], r, ms, eps, D);
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        const int pc = rg.tg + i * rg.G;
        if (pc < pieces) {
          float xf[8], dyf[8], g[8], d[8];
          unpack8(xq[i], xf);
          unpack8(dq[i], dyf);
          unpack8(gq[i], g);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            d[e] = norm_dx<LEV>(norm_a<LEV>(g[e], dyf[e]), r, c2, xf[e]);
            dg[i][e] += norm_gc<LEV>(dyf[e], xf[e], r);
          }
          if (dres) {
            float q[8];
            unpack8(rq[i], q);
#pragma unroll
            for (int e = 0; e < 8; ++e) d[e] = LEV ? __fadd_rn(q[e], rb(d[e])) : q[e] + d[e];
          }
          *reinterpret_cast<uint4*>(dx + off + pc * 8) = pack8(d);
        }
      }
    }
    if (partial) write_gain_partial<PP>(dg, rg, pieces, gsm, partial + p * D);
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
  NM_REQUIRE(D <= kGroupThreads * 4 * 8, "rmsnorm_bwd_add: D <= 8192");
  if (T == 0) return;
  const int64_t parts = norm_partial_rows(T);
  const bool lev = r == Rounding::Levanter;
  const int pieces = D / 8;
  const int pp = pieces <= kGroupThreads ? 1 : pieces <= 2 * kGroupThreads ? 2 : 4;
  const int G = group_threads_for(pieces, pp);
  auto kern = pp == 1   ? (lev ? k_rmsnorm_bwd_add<true, 1> : k_rmsnorm_bwd_add<false, 1>)
              : pp == 2 ? (lev ? k_rmsnorm_bwd_add<true, 2> : k_rmsnorm_bwd_add<false, 2>)
                        : (lev ? k_rmsnorm_bwd_add<true, 4> : k_rmsnorm_bwd_add<false, 4>);
  kern<<<int(parts), kGroupThreads, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(dy),
                                            reinterpret_cast<const __nv_bfloat16*>(x),
                                            reinterpret_cast<const __nv_bfloat16*>(gain), rstd,
                                            reinterpret_cast<const __nv_bfloat16*>(dres),
                                            reinterpret_cast<__nv_bfloat16*>(dx), dgain_partial, T, D, eps, parts, G);
  NM_CUDA(cudaGetLastError());
}

}  // namespace nm::ew
