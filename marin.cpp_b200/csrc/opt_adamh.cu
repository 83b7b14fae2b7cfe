// AdamH update of the LM head over the element ranges a rank owns (ZeRO-1), as two streaming passes plus scalar
// reductions. The reference runs it as three passes over the owned slices (src/kernels/optim/optk_adam.cu:84-221:
// moments + sum p^2 + sum a^2, then sum w^2, then apply); here pass 1 also accumulates sum p a, so that
//     sum w^2 = sum p^2 - 2 c sum p a + c^2 sum a^2,   c = eta n / max(m, 1e-10),   w = p - c a
// is known without reading p, mu, nu a second time: 24 + 18 = 42 bytes per element instead of 24 + 12 + 18 = 54.
// Element arithmetic keeps the reference's operation order with explicitly rounded f32 operations
// (optk_adam.cu:19-26,178-199): mu, nu come out bit-identical; p differs only through the norms' summation order.
// Norms are f64 sums of f32-rounded squares, rounded to f32 once before the f32 square root (optk_common.cuh:28-30).
// All kernels are HBM-bound streaming kernels: float4 accesses, 256 threads, grid (blocks per range, ranges).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "opt_internal.hpp"

namespace nm::opt {
namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float dvd(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float norm_of(double sumsq) { return __fsqrt_rn(static_cast<float>(sumsq)); }
__device__ __forceinline__ double sq(float x) { return static_cast<double>(mul(x, x)); }
__device__ __forceinline__ float fmax_nan(float a, float b) { return (a != a || a > b) ? a : b; }

// fixed-order block sum (butterfly inside each warp, then warp 0 over the warp sums); valid in thread 0
__device__ __forceinline__ double block_sum(double v) {
  __shared__ double ws[kThreads / 32];
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) ws[w] = v;
  __syncthreads();
  double s = lane < kThreads / 32 ? ws[lane] : 0.0;
  if (w == 0)
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  return s;
}

struct Clip {
  bool on;
  float gn, max_norm;
};
// clip_mode 0: none; 1: the caller's (clip_gn, clip); 2: gn from the global sum of squares in scal[kSumG]
__device__ __forceinline__ Clip clip_of(const Hyper& h, const double* scal) {
  if (h.clip_mode == 1) return Clip{h.clip != 0, h.clip_gn, h.max_norm};
  if (h.clip_mode == 2) {
    const float gn = norm_of(scal[kSumG]);
    return Clip{!(gn < h.max_norm), gn, h.max_norm};   // optax clips unless gn < max (equality clips too)
  }
  return Clip{false, 1.f, 1.f};
}
__device__ __forceinline__ float clipped(float g, const Hyper& h, const Clip& c) {
  const float gi = mul(g, h.grad_scale);
  return c.on ? mul(dvd(gi, c.gn), c.max_norm) : gi;
}
__device__ __forceinline__ float adam_dir(float mu, float nu, const Hyper& h) {
  return dvd(mu, mul(h.bc1, add(__fsqrt_rn(dvd(nu, h.bc2)), h.eps)));
}

// A range is walked in float4 units when every pointer it touches (already offset to the range) is 16-byte aligned
// (the bf16 copy 8-byte); the last len % 4 elements, or the whole range otherwise, go one by one.
struct Walk {
  int64_t quads, len;
};
__device__ __forceinline__ bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
__device__ __forceinline__ bool al8(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 7) == 0; }
__device__ __forceinline__ Walk walk_of(const Ranges& r, int y, bool aligned) {
  return Walk{aligned ? r.len[y] >> 2 : 0, r.len[y]};
}

// ------------------------------------------------------------------------------------------------ sum of g^2
__global__ void __launch_bounds__(kThreads) k_sumsq(const float* __restrict__ g, Ranges r, float grad_scale,
                                                    double* __restrict__ partial) {
  const int y = blockIdx.y;
  const float* gp = g + r.goff[y];
  const Walk wk = walk_of(r, y, al16(gp));
  double s = 0.0;
  const int64_t stride = int64_t(gridDim.x) * kThreads, i0 = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  for (int64_t q = i0; q < wk.quads; q += stride) {
    const float4 v = reinterpret_cast<const float4*>(gp)[q];
    s += sq(mul(v.x, grad_scale)) + sq(mul(v.y, grad_scale)) + sq(mul(v.z, grad_scale)) + sq(mul(v.w, grad_scale));
  }
  for (int64_t i = wk.quads * 4 + i0; i < wk.len; i += stride) s += sq(mul(gp[i], grad_scale));
  s = block_sum(s);
  if (threadIdx.x == 0) partial[int64_t(y) * gridDim.x + blockIdx.x] = s;
}

// out[j] (+)= sum_i partial[i * width + j], one block, fixed order
__global__ void __launch_bounds__(kThreads) k_sum_partials(const double* __restrict__ partial, int n, int width,
                                                           double* __restrict__ out, int accumulate) {
  for (int j = 0; j < width; ++j) {
    double s = 0.0;
    for (int i = threadIdx.x; i < n; i += kThreads) s += partial[int64_t(i) * width + j];
    s = block_sum(s);
    if (threadIdx.x == 0) out[j] = accumulate ? out[j] + s : s;
  }
}

// ------------------------------------------------------------------------------------------------ pass 1
__global__ void __launch_bounds__(kThreads) k_adamh_moments(Ranges r, const float* __restrict__ g,
                                                            const float* __restrict__ p, float* __restrict__ mu,
                                                            float* __restrict__ nu, Hyper h,
                                                            const double* __restrict__ scal,
                                                            double* __restrict__ partial) {
  const int y = blockIdx.y;
  const Clip cl = clip_of(h, scal);
  const float* gp = g + r.goff[y];
  const float* pp = p + r.coff[y];
  float* mp = mu + r.coff[y];
  float* vp = nu + r.coff[y];
  const Walk wk = walk_of(r, y, al16(gp) && al16(pp) && al16(mp) && al16(vp));
  double spp = 0.0, saa = 0.0, spa = 0.0;
  auto elem = [&](float gv, float pv, float& m, float& v) {
    const float gi = clipped(gv, h, cl);
    m = add(mul(h.one_minus_b1, gi), mul(h.b1, m));
    v = add(mul(h.one_minus_b2, mul(gi, gi)), mul(h.b2, v));
    const float a = adam_dir(m, v, h);
    spp += sq(pv);
    saa += sq(a);
    spa = fma(static_cast<double>(pv), static_cast<double>(a), spa);
  };
  const int64_t stride = int64_t(gridDim.x) * kThreads, i0 = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  for (int64_t q = i0; q < wk.quads; q += stride) {
    const float4 G = reinterpret_cast<const float4*>(gp)[q], P = reinterpret_cast<const float4*>(pp)[q];
    float4 M = reinterpret_cast<const float4*>(mp)[q], V = reinterpret_cast<const float4*>(vp)[q];
    elem(G.x, P.x, M.x, V.x);
    elem(G.y, P.y, M.y, V.y);
    elem(G.z, P.z, M.z, V.z);
    elem(G.w, P.w, M.w, V.w);
    reinterpret_cast<float4*>(mp)[q] = M;
    reinterpret_cast<float4*>(vp)[q] = V;
  }
  for (int64_t i = wk.quads * 4 + i0; i < wk.len; i += stride) {
    float m = mp[i], v = vp[i];
    elem(gp[i], pp[i], m, v);
    mp[i] = m;
    vp[i] = v;
  }
  spp = block_sum(spp);
  saa = block_sum(saa);
  spa = block_sum(spa);
  if (threadIdx.x == 0) {
    double* o = partial + (int64_t(y) * gridDim.x + blockIdx.x) * 3;
    o[0] = spp, o[1] = saa, o[2] = spa;
  }
}

// ------------------------------------------------------------------------------------------------ pass 2 (apply)
__global__ void __launch_bounds__(kThreads) k_adamh_apply(Ranges r, float* __restrict__ p,
                                                          const float* __restrict__ mu, const float* __restrict__ nu,
                                                          __nv_bfloat16* __restrict__ w16, Hyper h,
                                                          const double* __restrict__ scal) {
  const int y = blockIdx.y;
  // the tensor's norms, from the sums over every rank's ranges
  const float n = norm_of(scal[kSumPP]);
  const float m_floor = fmax_nan(norm_of(scal[kSumAA]), 1e-10f);
  const double c = static_cast<double>(h.eta) * static_cast<double>(n) / static_cast<double>(m_floor);
  const double ww = scal[kSumPP] - 2.0 * c * scal[kSumPA] + c * c * scal[kSumAA];
  const float nw = norm_of(ww);
  float* pp = p + r.coff[y];
  const float* mp = mu + r.coff[y];
  const float* vp = nu + r.coff[y];
  __nv_bfloat16* wp = w16 ? w16 + r.goff[y] : nullptr;
  const Walk wk = walk_of(r, y, al16(pp) && al16(mp) && al16(vp) && (!wp || al8(wp)));
  auto elem = [&](float pv, float m, float v) {
    const float a = adam_dir(m, v, h);
    const float w = sub(pv, dvd(mul(mul(h.eta, a), n), m_floor));
    const float u = sub(mul(dvd(w, nw), n), pv);
    return add(pv, u);                                   // p + (target - p), as the reference applies updates
  };
  const int64_t stride = int64_t(gridDim.x) * kThreads, i0 = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  for (int64_t q = i0; q < wk.quads; q += stride) {
    float4 P = reinterpret_cast<const float4*>(pp)[q];
    const float4 M = reinterpret_cast<const float4*>(mp)[q], V = reinterpret_cast<const float4*>(vp)[q];
    P.x = elem(P.x, M.x, V.x);
    P.y = elem(P.y, M.y, V.y);
    P.z = elem(P.z, M.z, V.z);
    P.w = elem(P.w, M.w, V.w);
    reinterpret_cast<float4*>(pp)[q] = P;
    if (wp) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(P.x, P.y), hi = __floats2bfloat162_rn(P.z, P.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo);
      o.y = *reinterpret_cast<const uint32_t*>(&hi);
      reinterpret_cast<uint2*>(wp)[q] = o;
    }
  }
  for (int64_t i = wk.quads * 4 + i0; i < wk.len; i += stride) {
    const float pv = elem(pp[i], mp[i], vp[i]);
    pp[i] = pv;
    if (wp) wp[i] = __float2bfloat16_rn(pv);
  }
}

// ------------------------------------------------------------------------------------------------ plain Adam
// The reference's Adam rule (optk_adam.cu:38-82) for the tensors beside the head (the final norm's gain): moments as
// above, u = ((-lr) a), p = p + u; no projection, so one pass.
__global__ void __launch_bounds__(kThreads) k_adam(Ranges r, const float* __restrict__ g, float* __restrict__ p,
                                                   float* __restrict__ mu, float* __restrict__ nu,
                                                   __nv_bfloat16* __restrict__ w16, Hyper h,
                                                   const double* __restrict__ scal) {
  const int y = blockIdx.y;
  const Clip cl = clip_of(h, scal);
  const float neg_lr = -h.eta;
  const float* gp = g + r.goff[y];
  float* pp = p + r.coff[y];
  float* mp = mu + r.coff[y];
  float* vp = nu + r.coff[y];
  __nv_bfloat16* wp = w16 ? w16 + r.goff[y] : nullptr;
  const Walk wk = walk_of(r, y, al16(gp) && al16(pp) && al16(mp) && al16(vp) && (!wp || al8(wp)));
  auto elem = [&](float gv, float& pv, float& m, float& v) {
    const float gi = clipped(gv, h, cl);
    m = add(mul(h.one_minus_b1, gi), mul(h.b1, m));
    v = add(mul(h.one_minus_b2, mul(gi, gi)), mul(h.b2, v));
    pv = add(pv, mul(neg_lr, adam_dir(m, v, h)));
  };
  const int64_t stride = int64_t(gridDim.x) * kThreads, i0 = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  for (int64_t q = i0; q < wk.quads; q += stride) {
    const float4 G = reinterpret_cast<const float4*>(gp)[q];
    float4 P = reinterpret_cast<const float4*>(pp)[q], M = reinterpret_cast<const float4*>(mp)[q],
           V = reinterpret_cast<const float4*>(vp)[q];
    elem(G.x, P.x, M.x, V.x);
    elem(G.y, P.y, M.y, V.y);
    elem(G.z, P.z, M.z, V.z);
    elem(G.w, P.w, M.w, V.w);
    reinterpret_cast<float4*>(pp)[q] = P;
    reinterpret_cast<float4*>(mp)[q] = M;
    reinterpret_cast<float4*>(vp)[q] = V;
    if (wp) {
      const __nv_bfloat162 lo = __floats2bfloat162_rn(P.x, P.y), hi = __floats2bfloat162_rn(P.z, P.w);
      uint2 o;
      o.x = *reinterpret_cast<const uint32_t*>(&lo);
      o.y = *reinterpret_cast<const uint32_t*>(&hi);
      reinterpret_cast<uint2*>(wp)[q] = o;
    }
  }
  for (int64_t i = wk.quads * 4 + i0; i < wk.len; i += stride) {
    float pv = pp[i], m = mp[i], v = vp[i];
    elem(gp[i], pv, m, v);
    pp[i] = pv, mp[i] = m, vp[i] = v;
    if (wp) wp[i] = __float2bfloat16_rn(pv);
  }
}

// ------------------------------------------------------------------------------------------------ row blocks
// The one-tensor entry points with a row partition (reference src/optim/capi_optim.cpp:103-128, optk_adam.cu:28-31,
// 84-221 with sl.block >= 0): every row belongs to a block; a block has its own learning-rate multiplier, may be
// frozen (its rows keep p, mu, nu and enter no norm), and AdamH takes its norms over the block's rows instead of the
// whole tensor. One CUDA block walks whole rows (a row's block id is uniform), writes the row's f64 sums, and a second
// kernel adds the rows of each block in ascending row order per thread, then by the fixed tree: deterministic.
__device__ __forceinline__ bool blk_frozen(const BlockTab& bt, int b) { return bt.frozen && bt.frozen[b] != 0; }
__device__ __forceinline__ float blk_lr(const BlockTab& bt, int b, float lr) {
  return mul(mul(lr, 1.0f), bt.lr_mult ? bt.lr_mult[b] : 1.0f);   // lr * lr_scale * block multiplier
}

__global__ void __launch_bounds__(kThreads) k_blk_adamh_moments(const float* __restrict__ g, const float* __restrict__ p,
                                                                float* __restrict__ mu, float* __restrict__ nu,
                                                                int64_t rows, int64_t cols, Hyper h, BlockTab bt,
                                                                double* __restrict__ row_partial) {
  const Clip cl = clip_of(h, nullptr);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int b = bt.block_of_row[row];
    double spp = 0.0, saa = 0.0, spa = 0.0;
    if (!blk_frozen(bt, b)) {
      const int64_t o = row * cols;
      for (int64_t c = threadIdx.x; c < cols; c += kThreads) {
        const float gi = clipped(g[o + c], h, cl);
        const float m = add(mul(h.one_minus_b1, gi), mul(h.b1, mu[o + c]));
        const float v = add(mul(h.one_minus_b2, mul(gi, gi)), mul(h.b2, nu[o + c]));
        mu[o + c] = m;
        nu[o + c] = v;
        const float a = adam_dir(m, v, h), pv = p[o + c];
        spp += sq(pv);
        saa += sq(a);
        spa = fma(static_cast<double>(pv), static_cast<double>(a), spa);
      }
    }
    spp = block_sum(spp);
    saa = block_sum(saa);
    spa = block_sum(spa);
    if (threadIdx.x == 0) {
      row_partial[row * 3] = spp, row_partial[row * 3 + 1] = saa, row_partial[row * 3 + 2] = spa;
    }
  }
}

__global__ void __launch_bounds__(kThreads) k_blk_reduce(const double* __restrict__ row_partial,
                                                         const int32_t* __restrict__ block_of_row, int64_t rows,
                                                         double* __restrict__ blk_scal) {
  const int b = blockIdx.x;
  double s[3] = {0.0, 0.0, 0.0};
  for (int64_t row = threadIdx.x; row < rows; row += kThreads)
    if (block_of_row[row] == b) {
      s[0] += row_partial[row * 3], s[1] += row_partial[row * 3 + 1], s[2] += row_partial[row * 3 + 2];
    }
  for (int j = 0; j < 3; ++j) {
    const double t = block_sum(s[j]);
    if (threadIdx.x == 0) blk_scal[b * 3 + j] = t;
  }
}

__global__ void __launch_bounds__(kThreads) k_blk_adamh_apply(float* __restrict__ p, const float* __restrict__ mu,
                                                              const float* __restrict__ nu,
                                                              __nv_bfloat16* __restrict__ w16, int64_t rows, int64_t cols,
                                                              Hyper h, BlockTab bt, const double* __restrict__ blk_scal) {
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int b = bt.block_of_row[row];
    const int64_t o = row * cols;
    if (blk_frozen(bt, b)) continue;          // p, mu, nu and the bf16 copy keep their values
    const double pp = blk_scal[b * 3], aa = blk_scal[b * 3 + 1], pa = blk_scal[b * 3 + 2];
    const float eta = blk_lr(bt, b, h.eta);
    const float n = norm_of(pp);
    const float m_floor = fmax_nan(norm_of(aa), 1e-10f);
    const double c_ = static_cast<double>(eta) * static_cast<double>(n) / static_cast<double>(m_floor);
    const float nw = norm_of(pp - 2.0 * c_ * pa + c_ * c_ * aa);
    for (int64_t c = threadIdx.x; c < cols; c += kThreads) {
      const float pv = p[o + c];
      const float a = adam_dir(mu[o + c], nu[o + c], h);
      const float w = sub(pv, dvd(mul(mul(eta, a), n), m_floor));
      const float pn = add(pv, sub(mul(dvd(w, nw), n), pv));
      p[o + c] = pn;
      if (w16) w16[o + c] = __float2bfloat16_rn(pn);
    }
  }
}

__global__ void __launch_bounds__(kThreads) k_blk_adam(const float* __restrict__ g, float* __restrict__ p,
                                                       float* __restrict__ mu, float* __restrict__ nu,
                                                       __nv_bfloat16* __restrict__ w16, int64_t rows, int64_t cols,
                                                       Hyper h, BlockTab bt) {
  const Clip cl = clip_of(h, nullptr);
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const int b = bt.block_of_row[row];
    const int64_t o = row * cols;
    if (blk_frozen(bt, b)) continue;          // p, mu, nu and the bf16 copy keep their values
    const float neg_lr = -blk_lr(bt, b, h.eta);
    for (int64_t c = threadIdx.x; c < cols; c += kThreads) {
      const float gi = clipped(g[o + c], h, cl);
      const float m = add(mul(h.one_minus_b1, gi), mul(h.b1, mu[o + c]));
      const float v = add(mul(h.one_minus_b2, mul(gi, gi)), mul(h.b2, nu[o + c]));
      mu[o + c] = m;
      nu[o + c] = v;
      const float pv = add(p[o + c], mul(neg_lr, adam_dir(m, v, h)));
      p[o + c] = pv;
      if (w16) w16[o + c] = __float2bfloat16_rn(pv);
    }
  }
}

// master copy from the bf16 replica: p[compact] = f32(w16[global]) over the owned ranges
__global__ void __launch_bounds__(kThreads) k_master_from_bf16(Ranges r, const __nv_bfloat16* __restrict__ w16,
                                                               float* __restrict__ p) {
  const int y = blockIdx.y;
  const int64_t stride = int64_t(gridDim.x) * kThreads, i0 = int64_t(blockIdx.x) * kThreads + threadIdx.x;
  for (int64_t i = i0; i < r.len[y]; i += stride) p[r.coff[y] + i] = __bfloat162float(w16[r.goff[y] + i]);
}

int blocks_for(const Ranges& r) {
  int64_t longest = 1;
  for (int i = 0; i < r.n; ++i) longest = longest > r.len[i] ? longest : r.len[i];
  const int64_t want = (longest / 4 + kThreads * 4 - 1) / (kThreads * 4);          // about 4 quads per thread
  const int64_t cap = std::max<int64_t>(1, int64_t(kMaxBlocksTotal) / std::max(1, r.n));
  return int(std::max<int64_t>(1, std::min(want, cap)));
}

}  // namespace

int partial_blocks(const Ranges& r) { return blocks_for(r) * r.n; }

void launch_sumsq(const float* g, const Ranges& r, float grad_scale, double* partial, double* out, bool accumulate,
                  cudaStream_t st) {
  if (r.n <= 0) return;
  const int bx = blocks_for(r);
  k_sumsq<<<dim3(bx, r.n), kThreads, 0, st>>>(g, r, grad_scale, partial);
  NM_CUDA(cudaGetLastError());
  k_sum_partials<<<1, kThreads, 0, st>>>(partial, bx * r.n, 1, out, accumulate ? 1 : 0);
  NM_CUDA(cudaGetLastError());
}

void launch_moments(const Ranges& r, const float* g, const float* p, float* mu, float* nu, const Hyper& h,
                    double* scal, double* partial, cudaStream_t st) {
  if (r.n <= 0) return;
  const int bx = blocks_for(r);
  k_adamh_moments<<<dim3(bx, r.n), kThreads, 0, st>>>(r, g, p, mu, nu, h, scal, partial);
  NM_CUDA(cudaGetLastError());
  k_sum_partials<<<1, kThreads, 0, st>>>(partial, bx * r.n, 3, scal + kSumPP, 0);
  NM_CUDA(cudaGetLastError());
}

void launch_apply(const Ranges& r, float* p, const float* mu, const float* nu, void* w16, const Hyper& h,
                  const double* scal, cudaStream_t st) {
  if (r.n <= 0) return;
  k_adamh_apply<<<dim3(blocks_for(r), r.n), kThreads, 0, st>>>(r, p, mu, nu, static_cast<__nv_bfloat16*>(w16), h, scal);
  NM_CUDA(cudaGetLastError());
}

void launch_adam(const Ranges& r, const float* g, float* p, float* mu, float* nu, void* w16, const Hyper& h,
                 const double* scal, cudaStream_t st) {
  if (r.n <= 0) return;
  k_adam<<<dim3(blocks_for(r), r.n), kThreads, 0, st>>>(r, g, p, mu, nu, static_cast<__nv_bfloat16*>(w16), h, scal);
  NM_CUDA(cudaGetLastError());
}

namespace {
int row_grid(int64_t rows) { return int(std::min<int64_t>(rows, int64_t(kMaxBlocksTotal))); }
}  // namespace

void launch_blk_adamh(const float* g, float* p, float* mu, float* nu, void* w16, int64_t rows, int64_t cols,
                      const Hyper& h, const BlockTab& bt, double* row_partial, double* blk_scal, cudaStream_t st) {
  k_blk_adamh_moments<<<row_grid(rows), kThreads, 0, st>>>(g, p, mu, nu, rows, cols, h, bt, row_partial);
  NM_CUDA(cudaGetLastError());
  k_blk_reduce<<<bt.n_blocks, kThreads, 0, st>>>(row_partial, bt.block_of_row, rows, blk_scal);
  NM_CUDA(cudaGetLastError());
  k_blk_adamh_apply<<<row_grid(rows), kThreads, 0, st>>>(p, mu, nu, static_cast<__nv_bfloat16*>(w16), rows, cols, h, bt,
                                                         blk_scal);
  NM_CUDA(cudaGetLastError());
}

void launch_blk_adam(const float* g, float* p, float* mu, float* nu, void* w16, int64_t rows, int64_t cols,
                     const Hyper& h, const BlockTab& bt, cudaStream_t st) {
  k_blk_adam<<<row_grid(rows), kThreads, 0, st>>>(g, p, mu, nu, static_cast<__nv_bfloat16*>(w16), rows, cols, h, bt);
  NM_CUDA(cudaGetLastError());
}

void launch_master_from_bf16(const Ranges& r, const void* w16, float* p, cudaStream_t st) {
  if (r.n <= 0) return;
  k_master_from_bf16<<<dim3(blocks_for(r), r.n), kThreads, 0, st>>>(r, static_cast<const __nv_bfloat16*>(w16), p);
  NM_CUDA(cudaGetLastError());
}

}  // namespace nm::opt
