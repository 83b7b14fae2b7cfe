// Row and streaming kernels of the fused linear cross-entropy (plain SIMT, HBM- or latency-bound): the merge of the
// per-tile softmax partials, the in-place rewrite of the logits store as the normalised gradient, the fixed-order loss
// and weight reductions, and the small helpers of the strict dW mode, the readout head and the f32-io path.
// Counterparts in the reference: k_ce_finalize_rows, k_ce_chunk_loss, k_ce_dlogits_bf16 / _f32
// (src/kernels/cross_entropy/ce_logits.cu:220-318) and ce_small.cu:22-61.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>

#include "ce_grad_math.cuh"
#include "ce_internal.hpp"
#include "ce_umma.cuh"
#include "ptx.cuh"

namespace nm::ce {
namespace {

// ------------------------------------------------------------------------------------------------ finalize
// 32 rows per CTA (lane = row), 8 warps: warp w merges the tile partials of segment w of the vocabulary in ascending
// order (m_w = max_i m_i, s_w = sum_i s_i exp(m_i - m_w)); warp 0 then merges the 8 segments in ascending order:
// M = max_w m_w (0 when not finite), S = sum_w s_w exp(m_w - M), lse = log S + M. The order depends only on the
// number of tiles, so lse and the loss do not depend on the chunk size or the launch geometry.
// loss = lse - z[target] + L lse^2 for a row that counts, else 0. A gradient call also gets the row's packed factors
// of the normalised gradient: b = weight (0 for an ignored target), a = b (1 + 2 L lse), e = -lse log2e, the target.
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
  if (p.rowf) {
    const float b = valid ? wt : 0.f;
    const float a = (p.z_loss != 0.f) ? __fmul_rn(b, __fmaf_rn(2.f * p.z_loss, lse, 1.f)) : b;
    p.rowf[r] = RowFactors{gradmath::exponent_of(lse), a, b, valid ? tg : -1};
  }
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
// The stand-alone rewrite of a chunk's logits store as n = a p - b onehot(target) (element math: ce_grad_math.cuh),
// used when the gradient contractions do not form n themselves (hidden sizes where that costs more than it saves, the
// f32 store, the f32-io path, and the nm_ce_dlogits entry point; the reference's counterpart is the pass of
// src/kernels/cross_entropy/ce_logits.cu:262-318).
//
// bf16 store: a TMA pipeline. The store is cut into tiles of 32 rows x 256 columns (16 KiB); each persistent CTA walks
// its tiles through a ring of four shared-memory slots: one thread keeps three tile loads in flight
// (cp.async.bulk.tensor -> mbarrier), all 256 threads rewrite the landed tile in place in shared memory (four 16-byte
// pieces each, eight threads side by side on one row so that shared-memory accesses are conflict-free), and the same
// thread sends the slot back to where it came from with a TMA store; a slot is refilled once the store that last
// read it has drained. Global traffic is whole 512-byte row segments in both directions and no thread ever waits on
// its own global load. The tensor map spans the padded row (ldS columns), so the padding columns are written as 0.
constexpr int kDzTileRows = 32, kDzTileCols = 256, kDzSlots = 4, kDzThreads = 256;
constexpr int kDzTileBytes = kDzTileRows * kDzTileCols * 2;
constexpr int kDzSmem = kDzSlots * kDzTileBytes + 128 /*alignment slack*/ + 64 /*barriers*/;

struct RowABE { float e, a, b; int tg; };
__device__ __forceinline__ RowABE row_factors(const DzArgs& p, int r) {
  if (r >= p.rows) return RowABE{0.f, 0.f, 0.f, -1};
  if (p.rowf) {
    const RowFactors f = p.rowf[r];
    return RowABE{f.e, f.a, f.b, f.target};
  }
  return RowABE{gradmath::exponent_of(p.lse[r]), p.ga[r], p.gb[r], p.targets[r]};
}

__global__ void __launch_bounds__(kDzThreads) k_ce_dlogits_tiles(const __grid_constant__ CUtensorMap tm, const DzArgs p,
                                                                uint32_t* status) {
  using namespace nm::ptx;
  extern __shared__ __align__(128) uint8_t dz_smem_raw[];
  const uint32_t raw = smem_u32(dz_smem_raw);
  const uint32_t base = (raw + 127u) & ~127u;
  const uint32_t bar0 = base + kDzSlots * kDzTileBytes;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int col_tiles = int((p.ldS + kDzTileCols - 1) / kDzTileCols);
  const int row_tiles = (p.rows + kDzTileRows - 1) / kDzTileRows;
  const int64_t total = int64_t(col_tiles) * row_tiles;
  const int64_t first = blockIdx.x;
  const int mine = first < total ? int((total - first + gridDim.x - 1) / gridDim.x) : 0;
  auto tile_xy = [&](int i, int& c0, int& r0) {
    const int64_t t = first + int64_t(i) * gridDim.x;
    c0 = int(t % col_tiles) * kDzTileCols;
    r0 = int(t / col_tiles) * kDzTileRows;
  };
  if (threadIdx.x == 0) {
    for (int s = 0; s < kDzSlots; ++s) mbar_init(bar0 + 8u * s, 1);
    abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  auto fetch = [&](int i) {                    // thread 0 only
    int c0, r0;
    tile_xy(i, c0, r0);
    const int s = i % kDzSlots;
    mbar_arrive_expect_tx(bar0 + 8u * s, kDzTileBytes);
    tma_load_2d(base + s * kDzTileBytes, &tm, bar0 + 8u * s, c0, r0);
  };
  if (threadIdx.x == 0) {
    prefetch_tmap(&tm);
    for (int i = 0; i < kDzSlots - 1 && i < mine; ++i) fetch(i);
  }
  const int trow = threadIdx.x >> 3, tcol = threadIdx.x & 7;
  for (int i = 0; i < mine; ++i) {
    const int s = i % kDzSlots;
    int c0, r0;
    tile_xy(i, c0, r0);
    const RowABE f = row_factors(p, r0 + trow);          // issued before the wait: its latency hides behind the tile's
    if (!mbar_wait<true>(bar0 + 8u * s, uint32_t(i / kDzSlots) & 1u, abort_flag, status, kErrTransformWait)) break;
    const uint32_t row_addr = base + s * kDzTileBytes + trow * (kDzTileCols * 2);
    uint4 v[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) v[q] = ld_shared_v4(row_addr + uint32_t(q * 8 + tcol) * 16u);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int col = c0 + (q * 8 + tcol) * 8;
      v[q] = gradmath::piece_bf16(v[q], f.e, f.a, f.b, f.tg - col, p.V - col);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) st_shared_v4(row_addr + uint32_t(q * 8 + tcol) * 16u, v[q].x, v[q].y, v[q].z, v[q].w);
    fence_proxy_async_smem();
    __syncthreads();
    if (threadIdx.x == 0) {
      tma_store_2d(&tm, base + s * kDzTileBytes, c0, r0);
      bulk_commit();
      if (i + kDzSlots - 1 < mine) {           // the slot tile i - 1 used: its store is the one before the latest
        bulk_wait_read<1>();
        fetch(i + kDzSlots - 1);
      }
    }
  }
  if (threadIdx.x == 0) {
    bulk_wait<0>();
    if (*abort_flag) __nanosleep(200000);      // an expired wait: let loads in flight land before the CTA leaves
  }
}

// f32 store: the bf16 result of a row is packed over the first half of the same row (leading dimension 2 ldS in bf16
// elements). One warp per row, 512 logits per step in ascending order: all of a step's loads are in registers before
// any of its stores is issued, and a step's stores (bytes [2 s, 2 s + 1024) of the row) only cover logits of this and
// earlier steps (bytes below 4 s + 2048), so nothing is overwritten before it has been read.
__global__ void __launch_bounds__(256) k_ce_dlogits_f32_rows(const DzArgs p) {
  const int lane = threadIdx.x & 31;
  const int warps = int(gridDim.x) * (blockDim.x >> 5);
  for (int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); r < p.rows; r += warps) {
    float* zr = static_cast<float*>(p.store) + int64_t(r) * p.ldS;
    __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(zr);
    const RowABE f = row_factors(p, r);
    for (int s0 = 0; s0 < p.ldS; s0 += 512) {
      float4 z[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = s0 + u * 128 + lane * 4;
        z[u] = v < p.ldS ? *reinterpret_cast<const float4*>(zr + v) : make_float4(0.f, 0.f, 0.f, 0.f);   // ldS % 8 == 0
      }
      __syncwarp();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int v = s0 + u * 128 + lane * 4;
        if (v < p.ldS) *reinterpret_cast<uint2*>(out + v) = gradmath::piece_f32(z[u], f.e, f.a, f.b, f.tg - v, p.V - v);
      }
      __syncwarp();
    }
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

// acc += src (the owned slices of a reduce-scattered gradient into a rank's packed accumulator)
__global__ void k_add_f32(float* __restrict__ acc, const float* __restrict__ src, int64_t n) {
  for (int64_t i = blockIdx.x * int64_t(blockDim.x) + threadIdx.x; i < n; i += int64_t(gridDim.x) * blockDim.x)
    acc[i] = __fadd_rn(acc[i], src[i]);
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
  NM_REQUIRE(a.rowf || (a.lse && a.ga && a.gb && a.targets), "dlogits: per-row factors (packed or as four arrays) needed");
  NM_REQUIRE(reinterpret_cast<uintptr_t>(a.store) % 16 == 0 && a.ldS % 8 == 0,
             "dlogits: the store must be 16-byte aligned with a row pitch that is a multiple of 8 elements");
  if (a.store_f32) {
    const int warps_per_cta = 8;
    const int grid = std::max(1, std::min((a.rows + warps_per_cta - 1) / warps_per_cta, sm_count() * 8));
    k_ce_dlogits_f32_rows<<<grid, 32 * warps_per_cta, 0, st>>>(a);
  } else {
    // one map for loads and stores: [rows, ldS] bf16, boxes of 32 rows x 256 columns, no swizzle
    const CUtensorMap tm = make_tmap(a.store, uint64_t(a.ldS), uint64_t(a.rows), a.ldS, kDzTileCols, kDzTileRows, false, 0);
    const int64_t tiles = ((a.ldS + kDzTileCols - 1) / kDzTileCols) * int64_t((a.rows + kDzTileRows - 1) / kDzTileRows);
    NM_CUDA(cudaFuncSetAttribute(k_ce_dlogits_tiles, cudaFuncAttributeMaxDynamicSharedMemorySize, kDzSmem));
    const int grid = int(std::max<int64_t>(1, std::min<int64_t>(tiles, int64_t(sm_count()) * 3)));
    k_ce_dlogits_tiles<<<grid, kDzThreads, kDzSmem, st>>>(tm, a, a.status);
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

void launch_add_f32(float* acc, const float* src, int64_t n, cudaStream_t st) {
  if (n <= 0) return;
  k_add_f32<<<grid_for(n, 256), 256, 0, st>>>(acc, src, n);
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
