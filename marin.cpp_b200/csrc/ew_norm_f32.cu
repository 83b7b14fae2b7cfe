// f32-storage forms of the RMSNorm pair and the sandwich tails (the reference instantiates its norm kernels for float
// storage as well, src/kernels/elementwise/rmsnorm_kernels.cuh:297-304, and its tests use them to separate math errors
// from rounding: rel <= 1e-6 against float64, tests/s3/test_rmsnorm.py:4). f32 throughout, nothing rounded on the way,
// so both rounding modes share these kernels. Not a hot path (the model stores bf16): one warp per row (forward) or per
// part of rows (backward, so that a part's gain-gradient sums have one owner and a fixed order), rows re-read from L2
// for the second pass.
#include <cuda_runtime.h>

#include <algorithm>
#include <string>

#include "ce_internal.hpp"
#include "ew_api.hpp"
#include "ew_rows.cuh"

namespace nm::ew {
namespace {

__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

// sum over the row of f(piece) with lanes striding over the float4 pieces
template <class F>
__device__ __forceinline__ float row_sum4(int D, int lane, F f) {
  float s = 0.f;
  for (int c = lane * 4; c < D; c += 128) s += f(c);
  return warp_sum(s);
}

__global__ void __launch_bounds__(256) k_rmsnorm_fwd_f32(const float* __restrict__ x, const float* __restrict__ gain,
                                                         float* __restrict__ y, float* __restrict__ rstd, int64_t T, int D,
                                                         float eps) {
  const int lane = threadIdx.x & 31;
  for (int64_t row = blockIdx.x * 8ll + (threadIdx.x >> 5); row < T; row += gridDim.x * 8ll) {
    const float* xr = x + row * D;
    const float ss = row_sum4(D, lane, [&](int c) { const float4 v = ld4(xr + c); return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; });
    const float r = rsqrtf(__fdiv_rn(ss, float(D)) + eps);
    if (rstd && lane == 0) rstd[row] = r;
    if (!y) continue;
    for (int c = lane * 4; c < D; c += 128) {
      const float4 v = ld4(xr + c), g = ld4(gain + c);
      st4(y + row * D + c, make_float4(g.x * (v.x * r), g.y * (v.y * r), g.z * (v.z * r), g.w * (v.w * r)));
    }
  }
}

__global__ void __launch_bounds__(256) k_sandwich_fwd_f32(const float* __restrict__ branch, const float* x_in,
                                                          const float* __restrict__ g_post, const float* __restrict__ g_next,
                                                          float* x_out, float* __restrict__ a_next,
                                                          float* __restrict__ rstd_post, float* __restrict__ rstd_next,
                                                          int64_t T, int D, float eps) {
  const int lane = threadIdx.x & 31;
  for (int64_t row = blockIdx.x * 8ll + (threadIdx.x >> 5); row < T; row += gridDim.x * 8ll) {
    const int64_t off = row * D;
    float r_p = 0.f;
    if (g_post) {
      const float sb = row_sum4(D, lane, [&](int c) { const float4 v = ld4(branch + off + c); return v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w; });
      r_p = rsqrtf(__fdiv_rn(sb, float(D)) + eps);
      if (rstd_post && lane == 0) rstd_post[row] = r_p;
    }
    float sx = 0.f;
    for (int c = lane * 4; c < D; c += 128) {
      float4 b = ld4(branch + off + c);
      const float4 xi = ld4(x_in + off + c);
      if (g_post) {
        const float4 g = ld4(g_post + c);
        b = make_float4(g.x * (b.x * r_p), g.y * (b.y * r_p), g.z * (b.z * r_p), g.w * (b.w * r_p));
      }
      const float4 xo = make_float4(xi.x + b.x, xi.y + b.y, xi.z + b.z, xi.w + b.w);
      sx += xo.x * xo.x + xo.y * xo.y + xo.z * xo.z + xo.w * xo.w;
      st4(x_out + off + c, xo);
    }
    const float r_n = rsqrtf(__fdiv_rn(warp_sum(sx), float(D)) + eps);
    if (rstd_next && lane == 0) rstd_next[row] = r_n;
    if (!a_next) continue;
    __syncwarp();
    for (int c = lane * 4; c < D; c += 128) {   // this lane re-reads the pieces it has just written
      const float4 xo = ld4(x_out + off + c), g = ld4(g_next + c);
      st4(a_next + off + c, make_float4(g.x * (xo.x * r_n), g.y * (xo.y * r_n), g.z * (xo.z * r_n), g.w * (xo.w * r_n)));
    }
  }
}

// One warp per part of rows. dx_mid = dx_out (0 when null) + norm_next_bwd(da_next); dx_in = dx_mid; with a post-norm
// dbranch = norm_post_bwd(dx_mid) over the branch output, else dbranch = dx_mid (skipped when it is dx_in). The warp's
// gain-gradient sums of both norms live in shared memory ([2][D] f32, one owner per column: no atomics, fixed order).
__global__ void __launch_bounds__(32) k_sandwich_bwd_f32(const float* dx_out, const float* __restrict__ da_next,
                                                         const float* __restrict__ x_out, const float* __restrict__ g_next,
                                                         const float* __restrict__ rstd_next,
                                                         const float* __restrict__ branch, const float* __restrict__ g_post,
                                                         const float* __restrict__ rstd_post, float* dx_in, float* dbranch,
                                                         float* __restrict__ pg_next, float* __restrict__ pg_post, int64_t T,
                                                         int D, float eps, int64_t parts) {
  extern __shared__ float acc[];   // [2][D]
  const int lane = threadIdx.x;
  const bool post = g_post != nullptr;
  for (int64_t p = blockIdx.x; p < parts; p += gridDim.x) {
    for (int c = lane; c < 2 * D; c += 32) acc[c] = 0.f;
    __syncwarp();
    const int64_t r0 = p * T / parts, r1 = (p + 1) * T / parts;
    for (int64_t row = r0; row < r1; ++row) {
      const int64_t off = row * D;
      float sxx = 0.f, sxa = 0.f;
      for (int c = lane * 4; c < D; c += 128) {
        const float4 x = ld4(x_out + off + c), d = ld4(da_next + off + c), g = ld4(g_next + c);
        sxx += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
        sxa += x.x * (g.x * d.x) + x.y * (g.y * d.y) + x.z * (g.z * d.z) + x.w * (g.w * d.w);
      }
      sxx = warp_sum(sxx), sxa = warp_sum(sxa);
      const float ms_n = __fdiv_rn(sxx, float(D));
      const float r_n = rstd_next ? __ldg(rstd_next + row) : rsqrtf(ms_n + eps);
      const float c2n = norm_c2(sxa, r_n, ms_n, eps, D, 0.f);
      float sbb = 0.f, sba = 0.f;
      for (int c = lane * 4; c < D; c += 128) {
        const float4 x = ld4(x_out + off + c), d = ld4(da_next + off + c), g = ld4(g_next + c);
        float4 m = dx_out ? ld4(dx_out + off + c) : make_float4(0.f, 0.f, 0.f, 0.f);
        m.x += fmaf(g.x * d.x, r_n, c2n * x.x), m.y += fmaf(g.y * d.y, r_n, c2n * x.y);
        m.z += fmaf(g.z * d.z, r_n, c2n * x.z), m.w += fmaf(g.w * d.w, r_n, c2n * x.w);
        acc[c] += d.x * (x.x * r_n), acc[c + 1] += d.y * (x.y * r_n);
        acc[c + 2] += d.z * (x.z * r_n), acc[c + 3] += d.w * (x.w * r_n);
        st4(dx_in + off + c, m);
        if (post) {
          const float4 b = ld4(branch + off + c), gp = ld4(g_post + c);
          sbb += b.x * b.x + b.y * b.y + b.z * b.z + b.w * b.w;
          sba += b.x * (gp.x * m.x) + b.y * (gp.y * m.y) + b.z * (gp.z * m.z) + b.w * (gp.w * m.w);
        } else if (dbranch != dx_in) {
          st4(dbranch + off + c, m);
        }
      }
      if (!post) continue;
      sbb = warp_sum(sbb), sba = warp_sum(sba);
      const float ms_p = __fdiv_rn(sbb, float(D));
      const float r_p = rstd_post ? __ldg(rstd_post + row) : rsqrtf(ms_p + eps);
      const float c2p = norm_c2(sba, r_p, ms_p, eps, D, 0.f);
      __syncwarp();
      for (int c = lane * 4; c < D; c += 128) {   // this lane re-reads the pieces of dx_mid it has just written
        const float4 m = ld4(dx_in + off + c), b = ld4(branch + off + c), gp = ld4(g_post + c);
        st4(dbranch + off + c, make_float4(fmaf(gp.x * m.x, r_p, c2p * b.x), fmaf(gp.y * m.y, r_p, c2p * b.y),
                                           fmaf(gp.z * m.z, r_p, c2p * b.z), fmaf(gp.w * m.w, r_p, c2p * b.w)));
        acc[D + c] += m.x * (b.x * r_p), acc[D + c + 1] += m.y * (b.y * r_p);
        acc[D + c + 2] += m.z * (b.z * r_p), acc[D + c + 3] += m.w * (b.w * r_p);
      }
    }
    __syncwarp();
    for (int c = lane; c < D; c += 32) {
      if (pg_next) pg_next[p * D + c] = acc[c];
      if (pg_post && post) pg_post[p * D + c] = acc[D + c];
    }
    __syncwarp();
  }
}

int fwd_grid(int64_t T) { return int(std::min<int64_t>((T + 7) / 8, int64_t(ce::sm_count()) * 8)); }

void check(const char* who, int64_t T, int D) {
  NM_REQUIRE(T >= 0 && D > 0 && D % 8 == 0 && D <= 8192, std::string(who) + ": T >= 0, D % 8 == 0, D <= 8192");
}

}  // namespace

void rmsnorm_fwd_f32(const float* x, const float* gain, float* y, float* rstd, int64_t T, int D, float eps,
                     cudaStream_t st) {
  check("rmsnorm_fwd (f32 storage)", T, D);
  NM_REQUIRE(x && gain && aligned16(x, gain, y), "rmsnorm_fwd (f32 storage): x, gain required; 16-byte aligned rows");
  if (T == 0) return;
  k_rmsnorm_fwd_f32<<<fwd_grid(T), 256, 0, st>>>(x, gain, y, rstd, T, D, eps);
  NM_CUDA(cudaGetLastError());
}

void sandwich_tail_fwd_f32(const float* branch, const float* x_in, const float* g_post, const float* g_next, float* x_out,
                           float* a_next, float* rstd_post, float* rstd_next, int64_t T, int D, float eps,
                           cudaStream_t st) {
  check("sandwich_tail_fwd (f32 storage)", T, D);
  NM_REQUIRE(branch && x_in && g_next && x_out && aligned16(branch, x_in, g_post, g_next, x_out, a_next),
             "sandwich_tail_fwd (f32 storage): branch, x_in, g_next, x_out required; 16-byte aligned rows");
  if (T == 0) return;
  k_sandwich_fwd_f32<<<fwd_grid(T), 256, 0, st>>>(branch, x_in, g_post, g_next, x_out, a_next, rstd_post, rstd_next, T, D,
                                                  eps);
  NM_CUDA(cudaGetLastError());
}

void sandwich_tail_bwd_f32(const float* dx_out, const float* da_next, const float* x_out, const float* g_next,
                           const float* rstd_next, const float* branch, const float* g_post, const float* rstd_post,
                           float* dx_in, float* dbranch, float* pg_next, float* pg_post, int64_t T, int D, float eps,
                           cudaStream_t st) {
  check("norm backward (f32 storage)", T, D);
  NM_REQUIRE(da_next && x_out && g_next && dx_in && dbranch, "norm backward (f32 storage): gradient, input, gain and outputs required");
  NM_REQUIRE(!g_post || branch, "norm backward (f32 storage): a post-norm needs the branch output");
  NM_REQUIRE(aligned16(dx_out, da_next, x_out, g_next, branch, g_post, dx_in, dbranch),
             "norm backward (f32 storage): every row pointer must be 16-byte aligned");
  if (T == 0) return;
  const int64_t parts = norm_partial_rows(T);
  const int smem = 2 * D * int(sizeof(float));
  NM_CUDA(cudaFuncSetAttribute(k_sandwich_bwd_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  k_sandwich_bwd_f32<<<int(parts), 32, smem, st>>>(dx_out, da_next, x_out, g_next, rstd_next, branch, g_post, rstd_post,
                                                   dx_in, dbranch, pg_next, pg_post, T, D, eps, parts);
  NM_CUDA(cudaGetLastError());
}

void rmsnorm_bwd_add_f32(const float* dy, const float* x, const float* gain, const float* rstd, const float* dres, float* dx,
                         float* dgain_partial, int64_t T, int D, float eps, cudaStream_t st) {
  // the next-norm half of the sandwich backward: dx = dres + norm_bwd(dy), no post-norm, no separate branch gradient
  sandwich_tail_bwd_f32(dres, dy, x, gain, rstd, nullptr, nullptr, nullptr, dx, dx, dgain_partial, nullptr, T, D, eps, st);
}

}  // namespace nm::ew
