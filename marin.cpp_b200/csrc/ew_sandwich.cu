// The sandwich tail around a residual add, forward and backward, in bf16 storage: optional post-norm of the branch
// output, residual add, and the next pre-norm (for the last layer: the final norm whose output feeds the LM head and
// whose input gradient is what the fused CE's dX flows into). Semantics follow the reference's
// src/kernels/elementwise/rmsnorm_kernels.cuh:100-235 (k_sandwich_fwd / k_sandwich_bwd):
//   forward   y = g_post ? norm(branch; g_post) : branch;  x_out = bf16(x_in + y);  a_next = norm(x_out; g_next)
//   backward  dx_mid = dx_out + norm_next_bwd(da_next);  dx_in = dx_mid;  dbranch = g_post ? norm_post_bwd(dx_mid) : dx_mid
// with the levanter rounding points of ew_api.hpp (or f32 chains under accurate rounding). Forward: one warp per row;
// backward: the row-group geometry of ew_rows.cuh.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "ew_rows.cuh"

namespace nm::ew {
namespace {

template <bool LEV>
__global__ void __launch_bounds__(kRowWarps * 32) k_sandwich_fwd(const __nv_bfloat16* __restrict__ branch,
                                                                 const __nv_bfloat16* __restrict__ x_in,
                                                                 const __nv_bfloat16* __restrict__ g_post,
                                                                 const __nv_bfloat16* __restrict__ g_next,
                                                                 __nv_bfloat16* __restrict__ x_out,
                                                                 __nv_bfloat16* __restrict__ a_next,
                                                                 float* __restrict__ rstd_post,
                                                                 float* __restrict__ rstd_next, int64_t T, int D,
                                                                 float eps) {
  const int lane = threadIdx.x & 31;
  const int pieces = D / 8;
  for (int64_t row = blockIdx.x * int64_t(kRowWarps) + (threadIdx.x >> 5); row < T;
       row += int64_t(gridDim.x) * kRowWarps) {
    const int64_t off = row * D;
    float r_p = 0.f;
    if (g_post) {
      float ss = 0.f;
      for (int pc = lane; pc < pieces; pc += 32) {
        float b[8];
        load8(branch + off + pc * 8, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) ss = fmaf(b[e], b[e], ss);
      }
      r_p = rsqrtf(__fdiv_rn(warp_sum(ss), float(D)) + eps);
      if (rstd_post && lane == 0) rstd_post[row] = r_p;
    }
    // x_out = round(x_in + y); its sum of squares is taken over the rounded values
    float sx = 0.f;
    for (int pc = lane; pc < pieces; pc += 32) {
      float b[8], xi[8], xo[8];
      load8(branch + off + pc * 8, b);
      load8(x_in + off + pc * 8, xi);
      if (g_post) {
        float g[8];
        load8(g_post + pc * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float y = norm_y<LEV>(g[e], b[e], r_p);
          xo[e] = rb(LEV ? __fadd_rn(xi[e], rb(y)) : xi[e] + y);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) xo[e] = rb(__fadd_rn(xi[e], b[e]));
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) sx = fmaf(xo[e], xo[e], sx);
      store8(x_out + off + pc * 8, xo);
    }
    const float r_n = rsqrtf(__fdiv_rn(warp_sum(sx), float(D)) + eps);
    if (rstd_next && lane == 0) rstd_next[row] = r_n;
    if (a_next) {
      for (int pc = lane; pc < pieces; pc += 32) {   // this lane re-reads the pieces it has just written
        float xo[8], g[8], o[8];
        load8(x_out + off + pc * 8, xo);
        load8(g_next + pc * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = norm_y<LEV>(g[e], xo[e], r_n);
        store8(a_next + off + pc * 8, o);
      }
    }
  }
}

// One CTA per part of consecutive rows (the partition of norm_partial_rows), row groups as described in ew_rows.cuh.
// A thread loads its pieces of x_out, da_next, dx_out and branch once; the group reduces sum x_out^2, sum x_out a and
// sum branch^2 together, the middle gradient dx_mid is formed and stored, the group reduces sum branch a_post, and
// the branch gradient follows from the registers that are still there. Gain-gradient sums of both norms stay in the
// owning thread's registers for the whole part.
template <bool LEV, int PP>
__global__ void __launch_bounds__(kGroupThreads, PP == 1 ? 4 : 1) k_sandwich_bwd(const __nv_bfloat16* dx_out,
                                                             const __nv_bfloat16* __restrict__ da_next,
                                                             const __nv_bfloat16* __restrict__ x_out,
                                                             const __nv_bfloat16* __restrict__ g_next,
                                                             const float* __restrict__ rstd_next,
                                                             const __nv_bfloat16* __restrict__ branch,
                                                             const __nv_bfloat16* __restrict__ g_post,
                                                             const float* __restrict__ rstd_post,
                                                             __nv_bfloat16* dx_in, __nv_bfloat16* dbranch,
                                                             float* __restrict__ pg_next,
                                                             float* __restrict__ pg_post, int64_t T, int D,
                                                             float eps, int64_t parts, int G) {
  __shared__ float red[2 * 8 * 3];    // the three-value reduction of every row
  __shared__ float red1[2 * 8 * 1];   // the one-value reduction that follows it: buffers of its own, flips of its own
  __shared__ float gsm[kGroupThreads * 8];
  const RowGroup rg = row_group(G);
  const int pieces = D / 8;
  const bool post = g_post != nullptr;
  const uint4 zero4 = make_uint4(0u, 0u, 0u, 0u);
  int flip = 0, flip1 = 0;
  uint4 gnq[PP], gpq[PP];
#pragma unroll
  for (int i = 0; i < PP; ++i) {
    const int pc = rg.tg + i * rg.G;
    gnq[i] = pc < pieces ? ldg16(g_next + pc * 8) : zero4;
    gpq[i] = (post && pc < pieces) ? ldg16(g_post + pc * 8) : zero4;
  }
  for (int64_t p = blockIdx.x; p < parts; p += gridDim.x) {
    const int64_t r0 = p * T / parts, r1 = (p + 1) * T / parts;
    float dgn[PP][8], dgp[PP][8];
#pragma unroll
    for (int i = 0; i < PP; ++i)
#pragma unroll
      for (int e = 0; e < 8; ++e) dgn[i][e] = dgp[i][e] = 0.f;
    for (int64_t base = r0; base < r1; base += rg.groups) {
      const int64_t row = base + rg.group;
      const bool on = row < r1;
      const int64_t off = row * D;
      uint4 xq[PP], aq[PP], oq[PP], bq[PP];
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        const int pc = rg.tg + i * rg.G;
        const bool in = on && pc < pieces;
        xq[i] = in ? ldg16(x_out + off + pc * 8) : zero4;
        aq[i] = in ? ldg16(da_next + off + pc * 8) : zero4;
        oq[i] = in ? ldg16(dx_out + off + pc * 8) : zero4;
        bq[i] = (in && post) ? ldg16(branch + off + pc * 8) : zero4;
      }
      float sums[3] = {0.f, 0.f, 0.f};   // sum x_out^2, sum x_out a_next, sum branch^2
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        float xo[8], da[8], g[8], b[8];
        unpack8(xq[i], xo);
        unpack8(aq[i], da);
        unpack8(gnq[i], g);
        unpack8(bq[i], b);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          sums[0] = fmaf(xo[e], xo[e], sums[0]);
          sums[1] = fmaf(xo[e], norm_a<LEV>(g[e], da[e]), sums[1]);
          sums[2] = fmaf(b[e], b[e], sums[2]);
        }
      }
      group_sum<3>(sums, rg, red, flip);
      float r_n = 0.f, c2n = 0.f;
      if (on) {
        const float ms_n = __fdiv_rn(sums[0], float(D));
        r_n = rstd_next ? __ldg(rstd_next + row) : rsqrtf(ms_n + eps);
        c2n = norm_c2(sums[1], r_n, ms_n, eps, D);
      }
      // the middle gradient: stored as dx_in, kept (rounded to bf16, as stored) for the post-norm backward
      uint4 mq[PP];
      float bap[1] = {0.f};
#pragma unroll
      for (int i = 0; i < PP; ++i) {
        const int pc = rg.tg + i * rg.G;
        mq[i] = zero4;
        if (on && pc < pieces) {
          float xo[8], da[8], g[8], dxo[8], dxm[8];
          unpack8(xq[i], xo);
          unpack8(aq[i], da);
          unpack8(gnq[i], g);
          unpack8(oq[i], dxo);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float a = norm_a<LEV>(g[e], da[e]);
            const float dxn = norm_dx<LEV>(a, r_n, c2n, xo[e]);
            dgn[i][e] += norm_gc<LEV>(da[e], xo[e], r_n);
            dxm[e] = rb(LEV ? __fadd_rn(dxo[e], rb(dxn)) : dxo[e] + dxn);
          }
          mq[i] = pack8(dxm);
          *reinterpret_cast<uint4*>(dx_in + off + pc * 8) = mq[i];
          if (post) {
            float b[8], gp[8];
            unpack8(bq[i], b);
            unpack8(gpq[i], gp);
#pragma unroll
            for (int e = 0; e < 8; ++e) bap[0] = fmaf(b[e], norm_a<LEV>(gp[e], dxm[e]), bap[0]);
          } else if (dbranch != dx_in) {
            *reinterpret_cast<uint4*>(dbranch + off + pc * 8) = mq[i];
          }
        }
      }
      if (post) {   // uniform over the CTA
        group_sum<1>(bap, rg, red1, flip1);
        if (on) {
          const float ms_p = __fdiv_rn(sums[2], float(D));
          const float r_p = rstd_post ? __ldg(rstd_post + row) : rsqrtf(ms_p + eps);
          const float c2p = norm_c2(bap[0], r_p, ms_p, eps, D);
#pragma unroll
          for (int i = 0; i < PP; ++i) {
            const int pc = rg.tg + i * rg.G;
            if (pc < pieces) {
              float b[8], gp[8], dxm[8], db[8];
              unpack8(bq[i], b);
              unpack8(gpq[i], gp);
              unpack8(mq[i], dxm);
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float ap = norm_a<LEV>(gp[e], dxm[e]);
                db[e] = norm_dx<LEV>(ap, r_p, c2p, b[e]);
                dgp[i][e] += norm_gc<LEV>(dxm[e], b[e], r_p);
              }
              *reinterpret_cast<uint4*>(dbranch + off + pc * 8) = pack8(db);
            }
          }
        }
      }
    }
    if (pg_next) write_gain_partial<PP>(dgn, rg, pieces, gsm, pg_next + p * D);
    if (pg_post && post) write_gain_partial<PP>(dgp, rg, pieces, gsm, pg_post + p * D);
  }
}

}  // namespace

void sandwich_tail_fwd(const bf16_t* branch, const bf16_t* x_in, const bf16_t* g_post, const bf16_t* g_next,
                       bf16_t* x_out, bf16_t* a_next, float* rstd_post, float* rstd_next, int64_t T, int D, float eps,
                       cudaStream_t st, Rounding r) {
  NM_REQUIRE(branch && x_in && g_next && x_out && T >= 0 && D > 0 && D % 8 == 0,
             "sandwich_tail_fwd: branch, x_in, g_next, x_out required; D % 8 == 0");
  NM_REQUIRE(aligned16(branch, x_in, g_post, g_next, x_out, a_next), "sandwich_tail_fwd: every row pointer must be "
                                                                     "16-byte aligned");
  if (T == 0) return;
  const int grid = int(std::min<int64_t>((T + kRowWarps - 1) / kRowWarps, int64_t(ce::sm_count()) * 8));
  auto B = [](const bf16_t* p) { return reinterpret_cast<const __nv_bfloat16*>(p); };
  auto M = [](bf16_t* p) { return reinterpret_cast<__nv_bfloat16*>(p); };
  if (r == Rounding::Levanter)
    k_sandwich_fwd<true><<<grid, kRowWarps * 32, 0, st>>>(B(branch), B(x_in), B(g_post), B(g_next), M(x_out), M(a_next),
                                                          rstd_post, rstd_next, T, D, eps);
  else
    k_sandwich_fwd<false><<<grid, kRowWarps * 32, 0, st>>>(B(branch), B(x_in), B(g_post), B(g_next), M(x_out),
                                                           M(a_next), rstd_post, rstd_next, T, D, eps);
  NM_CUDA(cudaGetLastError());
}

void sandwich_tail_bwd(const bf16_t* dx_out, const bf16_t* da_next, const bf16_t* x_out, const bf16_t* g_next,
                       const float* rstd_next, const bf16_t* branch, const bf16_t* g_post, const float* rstd_post,
                       bf16_t* dx_in, bf16_t* dbranch, float* pg_next, float* pg_post, int64_t T, int D, float eps,
                       cudaStream_t st, Rounding r) {
  NM_REQUIRE(dx_out && da_next && x_out && g_next && dx_in && dbranch && T >= 0 && D > 0 && D % 8 == 0,
             "sandwich_tail_bwd: dx_out, da_next, x_out, g_next, dx_in, dbranch required; D % 8 == 0");
  NM_REQUIRE(aligned16(dx_out, da_next, x_out, g_next, branch, g_post, dx_in, dbranch, pg_next, pg_post),
             "sandwich_tail_bwd: every row pointer must be 16-byte aligned");
  NM_REQUIRE(!g_post || branch, "sandwich_tail_bwd: a post-norm needs the branch output");
  NM_REQUIRE(D <= kGroupThreads * 4 * 8, "sandwich_tail_bwd: D <= 8192");
  if (T == 0) return;
  const int64_t parts = norm_partial_rows(T);
  const bool lev = r == Rounding::Levanter;
  const int pieces = D / 8;
  const int pp = pieces <= kGroupThreads ? 1 : pieces <= 2 * kGroupThreads ? 2 : 4;
  const int G = group_threads_for(pieces, pp);
  auto kern = pp == 1   ? (lev ? k_sandwich_bwd<true, 1> : k_sandwich_bwd<false, 1>)
              : pp == 2 ? (lev ? k_sandwich_bwd<true, 2> : k_sandwich_bwd<false, 2>)
                        : (lev ? k_sandwich_bwd<true, 4> : k_sandwich_bwd<false, 4>);
  auto B = [](const bf16_t* p) { return reinterpret_cast<const __nv_bfloat16*>(p); };
  auto M = [](bf16_t* p) { return reinterpret_cast<__nv_bfloat16*>(p); };
  kern<<<int(parts), kGroupThreads, 0, st>>>(B(dx_out), B(da_next), B(x_out), B(g_next), rstd_next, B(branch), B(g_post),
                                            rstd_post, M(dx_in), M(dbranch), pg_next, pg_post, T, D, eps, parts, G);
  NM_CUDA(cudaGetLastError());
}

}  // namespace nm::ew
