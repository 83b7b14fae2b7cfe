// The three contractions of the fused linear cross-entropy as one warp-specialised, persistent tcgen05 kernel template
// for sm_100a:
//     logits  z[rows, V]   = x[rows, D]  W[V, D]^T      (A K-major, B K-major)   + online (max, sum exp) epilogue
//     dX      dx[rows, D]  = n[rows, V]  W[V, D]        (A K-major, B MN-major)  + scale / bf16 / accumulate epilogue
//     dW      dw[V, D]    += n[rows, V]^T x[rows, D]    (A MN-major, B MN-major) + f32 read-modify-write epilogue
// They replace the reference's k_ce_logits_stats / k_ce_logits_sm90 (src/kernels/cross_entropy/ce_logits.cu:25-215,
// ce_sm90.cu:364-495), k_ce_dgrad / k_ce_wgrad / k_ce_gemm_sm90 (ce_gemm.cu:38-392, ce_sm90.cu:558-764) and its
// cuBLASLt plans (ce_lt.cpp:47-219).
//
// One CTA per SM, 320 threads: warp 0 issues the TMA loads (one elected lane), warp 1 allocates TMEM and issues the
// UMMAs (one elected lane), warps 2-9 are the epilogue (thread = accumulator row = TMEM lane; two warps per lane
// quadrant, one for each 128-column half of the tile, so every scheduler has two epilogue warps to alternate between). Tiles are 128 x 256
// (M x N) with K blocks of 64 bf16 (one 128-byte swizzle row); operands arrive by TMA into a 4-stage ring of
// SWIZZLE_128B tiles; the f32 accumulator lives in TMEM, two buffers of 256 columns, so the epilogue of tile i runs
// while the UMMAs of tile i + 1 are issued. TMEM loads are software-pipelined (the next 32 columns load while the
// current 32 are processed). The bf16 logits store and the f32 dW accumulation leave through shared memory: each
// epilogue warp packs its 32 rows into a 128-byte-swizzled 4 KiB staging tile and one lane issues a TMA store (logits)
// or a TMA reduce-add (dW += tile, the addition done at L2), so global traffic is full lines and the dW update needs no
// read. Every mbarrier wait is bounded (ptx.cuh mbar_wait).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>
#include <string>
#include <type_traits>

#include "ce_internal.hpp"
#include "ptx.cuh"

namespace nm::ce {
namespace {

using namespace nm::ptx;

constexpr int BM = 128, BN = 256, BK = 64, UK = 16;
// NCTA = 1: one CTA per tile of 128 x 256. NCTA = 2: a pair of CTAs (a cluster of two on one TPC) per tile of
// 256 x 256; each CTA stages its own 128 rows of A and its own 128 columns of B, the leader issues one UMMA of M = 256
// over both CTAs' shared memory, and each CTA keeps the accumulator of its own 128 rows in its own TMEM: the B
// operand crosses L2 -> shared memory once per pair instead of once per CTA.
constexpr int kABytes = BM * BK * 2;            // 16 KiB
__host__ __device__ constexpr int b_bytes(int ncta) { return BN / ncta * BK * 2; }                 // 32 / 16 KiB
__host__ __device__ constexpr int stage_bytes(int ncta) { return kABytes + b_bytes(ncta); }        // 48 / 32 KiB
__host__ __device__ constexpr int num_stages(int ncta) { return ncta == 2 ? 6 : 4; }
constexpr int kBoxBytesMN = 64 * BK * 2;        // one MN-major box: 64 k-rows of 128 bytes = 8 KiB
constexpr int kTmemCols = 512;
constexpr int kEpiWarps = 8;
constexpr int kThreads = 64 + 32 * kEpiWarps;
enum Epi : int { kEpiLogits = 0, kEpiDx = 1, kEpiDw = 2, kEpiTest = 3 };

// epilogue staging: one 32-row x 128-byte tile per epilogue warp, only for the epilogues that leave through TMA; the
// logits epilogue adds 1 KiB where the two column halves of a row meet to merge their (max, sum exp)
constexpr int kEpiBufBytes = 32 * 128;
constexpr int kMergeBytes = BM * 8;
__host__ __device__ constexpr int epi_stage_bytes(int epi) {
  return (epi == kEpiLogits || epi == kEpiDw) ? kEpiWarps * kEpiBufBytes + (epi == kEpiLogits ? kMergeBytes : 0) : 0;
}
constexpr int smem_bytes(int epi, int ncta) {
  return num_stages(ncta) * stage_bytes(ncta) + epi_stage_bytes(epi) + 1024 /*alignment slack*/ + 256 /*barriers*/;
}

struct GemmParams {
  int M, N, K;              // extents of this launch: accumulator rows, columns, contraction length
  int m_off;                // first A coordinate along M (dW vocabulary range start)
  int num_m, num_n;         // tiles (of 128 * NCTA rows, 256 columns)
  int m_inner;              // 1: consecutive tile indices walk M first (logits), 0: N first
  int m_group;              // m_inner only: M tiles are walked in groups of this many (all N tiles of a group before
                            // the next group), so that the A rows of a group stay in L2 while B streams past
  int a_3d, b_3d;           // an MN-major operand whose M / N extent is a multiple of 64 is described by a 3-D tensor
                            // map (64 contiguous, K, groups of 64): one TMA instruction per stage instead of 2 or 4
  uint32_t* status;
  // logits
  void* store; int64_t ldS; int store_f32;
  float* tmax; float* tsum; int64_t ldT; float* zt; const int32_t* targets; const float* bias;
  // dX
  const float* scale; const void* dx_old; void* dx_out; int acc_mode; int out_f32; int64_t ldo;
  // dW
  float* dw; int round_bf16;
  // test
  float* c; int64_t ldc;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ float round_bf16f(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// ---------------------------------------------------------------------------------------------- epilogues
// One call handles the 32 accumulator columns [col0, col0 + 32) of row `grow` held in v[].
struct LogitsRowState {
  float m, s, zt;
  bool hit;
};

__device__ __forceinline__ void epi_logits_chunk(const GemmParams& p, float* v, int grow, bool row_ok, int col0, int tg,
                                                 LogitsRowState& st) {
  const int V = p.N;
  const int ncols = min(32, V - col0);
  if (p.bias) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) v[j] += __ldg(p.bias + col0 + j);
  }
  if (p.store && p.store_f32 && row_ok) {   // f32 store: direct (the bf16 store leaves through the staging tile)
    float* o = static_cast<float*>(p.store) + int64_t(grow) * p.ldS + col0;
    if (ncols == 32) {
#pragma unroll
      for (int j = 0; j < 32; j += 4) *reinterpret_cast<float4*>(o + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)     // static indices only: a runtime index would move v[] to local memory
        if (j < ncols) o[j] = v[j];
    }
  }
  // online (max, sum exp): one rescale of the running sum per 32 columns
  constexpr float kLog2e = 1.4426950408889634f;
  float m_new, a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f, neg;
  if (ncols == 32) {                       // every chunk but the last of a ragged vocabulary: no column predicates
    float c0 = fmaxf(v[0], v[1]), c1 = fmaxf(v[2], v[3]), c2 = fmaxf(v[4], v[5]), c3 = fmaxf(v[6], v[7]);
#pragma unroll
    for (int j = 8; j < 32; j += 8) {
      c0 = fmaxf(c0, fmaxf(v[j], v[j + 1]));
      c1 = fmaxf(c1, fmaxf(v[j + 2], v[j + 3]));
      c2 = fmaxf(c2, fmaxf(v[j + 4], v[j + 5]));
      c3 = fmaxf(c3, fmaxf(v[j + 6], v[j + 7]));
    }
    m_new = fmaxf(st.m, fmaxf(fmaxf(c0, c1), fmaxf(c2, c3)));
    neg = -m_new * kLog2e;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      a0 += ex2_approx(fmaf(v[j], kLog2e, neg));
      a1 += ex2_approx(fmaf(v[j + 1], kLog2e, neg));
      a2 += ex2_approx(fmaf(v[j + 2], kLog2e, neg));
      a3 += ex2_approx(fmaf(v[j + 3], kLog2e, neg));
    }
  } else {
    float cm = -INFINITY;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols) cm = fmaxf(cm, v[j]);
    m_new = fmaxf(st.m, cm);
    neg = -m_new * kLog2e;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      a0 += (j < ncols) ? ex2_approx(fmaf(v[j], kLog2e, neg)) : 0.f;
      a1 += (j + 1 < ncols) ? ex2_approx(fmaf(v[j + 1], kLog2e, neg)) : 0.f;
      a2 += (j + 2 < ncols) ? ex2_approx(fmaf(v[j + 2], kLog2e, neg)) : 0.f;
      a3 += (j + 3 < ncols) ? ex2_approx(fmaf(v[j + 3], kLog2e, neg)) : 0.f;
    }
  }
  // st.m == -inf on the first chunk: ex2(-inf) = 0 and st.s = 0
  st.s = st.s * ex2_approx(fmaf(st.m, kLog2e, neg)) + ((a0 + a1) + (a2 + a3));
  st.m = m_new;
  if (tg >= col0 && tg < col0 + 32) {
    const int jt = tg - col0;
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j == jt) st.zt = v[j];
    st.hit = true;
  }
}

__device__ __forceinline__ void epi_dx_chunk(const GemmParams& p, const float* v, int grow, int col0, float scale) {
  const int D = p.N;
  const int ncols = min(32, D - col0);   // D % 8 == 0, so ncols is a multiple of 8
  if (p.out_f32) {
    float* o = static_cast<float*>(p.dx_out) + int64_t(grow) * p.ldo + col0;
    const float* old = static_cast<const float*>(p.dx_old) + int64_t(grow) * p.ldo + col0;
#pragma unroll
    for (int j = 0; j < 32; j += 4) {
      if (j < ncols) {
        float4 r = make_float4(v[j] * scale, v[j + 1] * scale, v[j + 2] * scale, v[j + 3] * scale);
        if (p.acc_mode) {
          const float4 q = *reinterpret_cast<const float4*>(old + j);
          r.x += q.x; r.y += q.y; r.z += q.z; r.w += q.w;
        }
        *reinterpret_cast<float4*>(o + j) = r;
      }
    }
    return;
  }
  __nv_bfloat16* o = static_cast<__nv_bfloat16*>(p.dx_out) + int64_t(grow) * p.ldo + col0;
  const __nv_bfloat16* old = static_cast<const __nv_bfloat16*>(p.dx_old) + int64_t(grow) * p.ldo + col0;
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    if (j < ncols) {
      float r[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) r[e] = v[j + e] * scale;
      if (p.acc_mode) {
        const uint4 q = *reinterpret_cast<const uint4*>(old + j);
        const uint32_t qq[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float o0 = bf_lo(qq[e]), o1 = bf_hi(qq[e]);
          if (p.acc_mode == 1) {   // levanter: bf16(old + f32(bf16(acc)))
            r[2 * e] = o0 + round_bf16f(r[2 * e]);
            r[2 * e + 1] = o1 + round_bf16f(r[2 * e + 1]);
          } else {                 // accurate: bf16(old + acc)
            r[2 * e] = o0 + r[2 * e];
            r[2 * e + 1] = o1 + r[2 * e + 1];
          }
        }
      }
      *reinterpret_cast<uint4*>(o + j) =
          make_uint4(pack2(r[0], r[1]), pack2(r[2], r[3]), pack2(r[4], r[5]), pack2(r[6], r[7]));
    }
  }
}

// Staging writers: this lane's row of a 32-row staging tile, 16-byte pieces XOR-swizzled with the row the way the
// tensor map's swizzle mode expects (the tile is 1024-byte aligned). f32: a 32-row x 128-byte tile (32 columns),
// SWIZZLE_128B: piece j of row r at r * 128 + ((j ^ (r & 7)) << 4).
// bf16: a 32-row x 64-byte tile (32 columns), SWIZZLE_64B: piece j of row r at r * 64 + ((j ^ ((r >> 1) & 3)) << 4).
__device__ __forceinline__ void stage_bf16_chunk(uint32_t buf, int lane, const float* v) {
#pragma unroll
  for (int j = 0; j < 4; ++j)
    st_shared_v4(buf + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4), pack2(v[8 * j], v[8 * j + 1]),
                 pack2(v[8 * j + 2], v[8 * j + 3]), pack2(v[8 * j + 4], v[8 * j + 5]), pack2(v[8 * j + 6], v[8 * j + 7]));
}
__device__ __forceinline__ void stage_f32_row(uint32_t buf, int lane, const float* v, float scale, bool round_bf16) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float r0 = v[4 * j] * scale, r1 = v[4 * j + 1] * scale, r2 = v[4 * j + 2] * scale, r3 = v[4 * j + 3] * scale;
    if (round_bf16) { r0 = round_bf16f(r0); r1 = round_bf16f(r1); r2 = round_bf16f(r2); r3 = round_bf16f(r3); }
    st_shared_v4(buf + lane * 128 + ((j ^ (lane & 7)) << 4), __float_as_uint(r0), __float_as_uint(r1),
                 __float_as_uint(r2), __float_as_uint(r3));
  }
}

// ---------------------------------------------------------------------------------------------- the kernel
template <int EPI, bool A_MN, bool B_MN, int NCTA>
__global__ void __launch_bounds__(kThreads, 1)
k_ce_umma(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
          const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;            // SWIZZLE_128B tiles need 1024-byte alignment
  uint8_t* smem = smem_raw + (base - raw);
  constexpr int kStages = num_stages(NCTA), kBBytes = b_bytes(NCTA), kStageBytes = stage_bytes(NCTA);
  constexpr int BMT = BM * NCTA;                           // accumulator rows of one tile (all CTAs of the pair)
  constexpr int BNC = BN / NCTA;                           // B columns this CTA stages
  const uint32_t sA = base, sB = base + kStages * kABytes;
  const uint32_t sEpi = base + kStages * kStageBytes;      // epilogue staging tiles (1024-byte aligned)
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes + epi_stage_bytes(EPI));
  const uint32_t bar0 = sEpi + epi_stage_bytes(EPI);
  auto full_bar = [&](int s) { return bar0 + 8u * s; };
  auto empty_bar = [&](int s) { return bar0 + 8u * (kStages + s); };
  auto tfull_bar = [&](int b) { return bar0 + 8u * (2 * kStages + b); };
  auto tempty_bar = [&](int b) { return bar0 + 8u * (2 * kStages + 2 + b); };
  auto mfull_bar = [&](int q) { return bar0 + 8u * (2 * kStages + 4 + q); };    // right half's (max, sum) written
  auto mempty_bar = [&](int q) { return bar0 + 8u * (2 * kStages + 8 + q); };   // left half has read them
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 12);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // pair mode: rank of this CTA in its pair (0 = leader), tiles are dealt to pairs
  const uint32_t rank = NCTA == 2 ? cluster_ctarank() : 0u;
  const int walker = NCTA == 2 ? int(blockIdx.x >> 1) : int(blockIdx.x);
  const int walkers = NCTA == 2 ? int(gridDim.x >> 1) : int(gridDim.x);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), NCTA * kEpiWarps); }
    for (int q = 0; q < 4; ++q) { mbar_init(mfull_bar(q), 1); mbar_init(mempty_bar(q), 1); }
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if constexpr (epi_stage_bytes(EPI) > 0) prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    if constexpr (NCTA == 2) {
      tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(tmem_slot), kTmemCols);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (NCTA == 2) cluster_sync_all();   // the peer's mbarriers are initialised before anything signals them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.num_m * p.num_n;
  const int k_blocks = (p.K + BK - 1) / BK;
  auto decode = [&](int tile, int& mi, int& ni) {
    if (p.m_inner) {
      const int per_group = p.m_group * p.num_n;
      const int g = tile / per_group, r = tile - g * per_group;
      const int gm = min(p.m_group, p.num_m - g * p.m_group);   // the last group may be smaller
      ni = r / gm;
      mi = g * p.m_group + (r - ni * gm);
    } else {
      ni = tile % p.num_n;
      mi = tile / p.num_n;
    }
  };

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      // L2 eviction hints, fixed per kernel: the logits kernel re-reads the x rows of a tile group for every
      // vocabulary tile and the dW kernel re-reads the whole x chunk for every vocabulary tile (keep: evict last)
      constexpr int kAPol = EPI == kEpiLogits ? 2 : 0;
      constexpr int kBPol = EPI == kEpiDw ? 2 : 0;
      const uint64_t pol_last = l2_policy_evict_last();
      // pair mode: the bytes of both CTAs are counted on the leader's barrier, which only the leader arms
      // (the policy is a compile-time constant: a run-time choice here costs the producer about a tenth of its rate)
      auto ld2 = [&](uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, auto keep) {
        if constexpr (NCTA == 2) {
          if constexpr (decltype(keep)::value) tma_pair_load_2d_hint(dst, tm, bar, c0, c1, pol_last);
          else tma_pair_load_2d(dst, tm, bar, c0, c1);
        } else {
          if constexpr (decltype(keep)::value) tma_load_2d_hint(dst, tm, bar, c0, c1, pol_last);
          else tma_load_2d(dst, tm, bar, c0, c1);
        }
      };
      auto ld3 = [&](uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1, int c2, auto keep) {
        if constexpr (NCTA == 2) {
          if constexpr (decltype(keep)::value) tma_pair_load_3d_hint(dst, tm, bar, c0, c1, c2, pol_last);
          else tma_pair_load_3d(dst, tm, bar, c0, c1, c2);
        } else {
          if constexpr (decltype(keep)::value) tma_load_3d_hint(dst, tm, bar, c0, c1, c2, pol_last);
          else tma_load_3d(dst, tm, bar, c0, c1, c2);
        }
      };
      constexpr std::bool_constant<kAPol == 2> keepA{};
      constexpr std::bool_constant<kBPol == 2> keepB{};
      for (int tile = walker; tile < num_tiles && ok; tile += walkers) {
        int mi, ni;
        decode(tile, mi, ni);
        const int m0 = p.m_off + mi * BMT + int(rank) * BM, n0 = ni * BN + int(rank) * BNC;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait<true>(empty_bar(stage), phase ^ 1u, abort_flag, p.status, kErrProducerWait)) { ok = false; break; }
          const uint32_t bar = NCTA == 2 ? mapa_shared(full_bar(stage), 0) : full_bar(stage);
          if (rank == 0) mbar_arrive_expect_tx(full_bar(stage), NCTA * kStageBytes);
          const uint32_t a_dst = sA + stage * kABytes, b_dst = sB + stage * kBBytes;
          const int k0 = kb * BK;
          if constexpr (A_MN) {
            if (p.a_3d) {
              ld3(a_dst, &tmA, bar, 0, k0, m0 >> 6, keepA);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j) ld2(a_dst + j * kBoxBytesMN, &tmA, bar, m0 + j * 64, k0, keepA);
            }
          } else {
            ld2(a_dst, &tmA, bar, k0, m0, keepA);
          }
          if constexpr (B_MN) {
            if (p.b_3d) {
              ld3(b_dst, &tmB, bar, 0, k0, n0 >> 6, keepB);
            } else {
#pragma unroll
              for (int j = 0; j < BNC / 64; ++j) ld2(b_dst + j * kBoxBytesMN, &tmB, bar, n0 + j * 64, k0, keepB);
            }
          } else {
            ld2(b_dst, &tmB, bar, k0, n0, keepB);
          }
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ------------------------------------------------------------------ UMMA issuer (pair mode: the leader only)
      constexpr uint32_t idesc = idesc_bf16_f32(BMT, BN, A_MN, B_MN);
      int stage = 0; uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = walker; tile < num_tiles && ok; tile += walkers, ++it) {
        const int b = it & 1;
        if (!mbar_wait(tempty_bar(b), ((it >> 1) & 1u) ^ 1u, abort_flag, p.status, kErrTmemFreeWait)) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + uint32_t(b * BN);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, abort_flag, p.status, kErrMmaWait)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_src = sA + stage * kABytes, b_src = sB + stage * kBBytes;
#pragma unroll
          for (int k = 0; k < BK / UK; ++k) {
            // K-major: 16 bf16 = 32 bytes further along the 128-byte row; MN-major: 16 k-rows = 2048 bytes further
            const uint64_t ad = A_MN ? smem_desc_sw128(a_src + k * (UK * 128), kBoxBytesMN, 1024)
                                     : smem_desc_sw128(a_src + k * (UK * 2), 16, 1024);
            const uint64_t bd = B_MN ? smem_desc_sw128(b_src + k * (UK * 128), kBoxBytesMN, 1024)
                                     : smem_desc_sw128(b_src + k * (UK * 2), 16, 1024);
            if constexpr (NCTA == 2) umma_pair_bf16(d_tmem, ad, bd, idesc, (kb | k) != 0);
            else umma_bf16(d_tmem, ad, bd, idesc, (kb | k) != 0);
          }
          // the stage is free again once these UMMAs have read it (pair mode: in both CTAs)
          if constexpr (NCTA == 2) umma_pair_commit(empty_bar(stage), 3);
          else umma_commit(empty_bar(stage));
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (ok) {                            // accumulator of this tile complete
          if constexpr (NCTA == 2) umma_pair_commit(tfull_bar(b), 3);
          else umma_commit(tfull_bar(b));
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- epilogue (warps 2-9)
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int half = (warp - 2) >> 2;          // which 128 columns of the 256-column tile this warp handles
    const int r_local = quad * 32 + lane;
    const uint32_t stg = sEpi + uint32_t(warp - 2) * kEpiBufBytes;       // this warp's staging tile(s)
    uint32_t n_bulk = 0;                        // TMA stores this warp has issued (logits: staging half = n_bulk & 1)
    float2* merge = reinterpret_cast<float2*>(smem + kStages * kStageBytes + kEpiWarps * kEpiBufBytes);
    float scale = 1.f;
    if constexpr (EPI == kEpiDx || EPI == kEpiDw) scale = p.scale ? __ldg(p.scale) : 1.f;
    const bool staged_store = EPI == kEpiLogits && p.store != nullptr && !p.store_f32;
    const uint64_t store_policy = l2_policy_evict_first();   // the logits store is not read again by this kernel
    constexpr int kChunks = BN / 32 / 2;       // 32-column chunks per warp
    int it = 0;
    for (int tile = walker; tile < num_tiles; tile += walkers, ++it) {
      const int b = it & 1;
      int mi, ni;
      decode(tile, mi, ni);
      const int m0 = mi * BMT + int(rank) * BM, n0 = ni * BN;
      const int grow = m0 + r_local;
      const bool row_ok = grow < p.M;
      const bool warp_rows_ok = m0 + quad * 32 < p.M;          // any row of this warp inside the matrix
      if (!mbar_wait<true>(tfull_bar(b), (it >> 1) & 1u, abort_flag, p.status, kErrEpilogueWait)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(b * BN + half * (BN / 2));
      LogitsRowState st{-INFINITY, 0.f, 0.f, false};
      int tg = -1;
      if constexpr (EPI == kEpiLogits) tg = row_ok ? __ldg(p.targets + grow) : -1;

      // one 32-column chunk held in v[]; c counts the chunks of the whole tile (0 .. 7)
      auto process = [&](float* v, int c) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) return;               // uniform over the warp
        if constexpr (EPI == kEpiLogits) {
          epi_logits_chunk(p, v, grow, row_ok, col0, tg, st);
          if (staged_store && warp_rows_ok) {
            // one 32-column staging tile per chunk, two tiles per warp used alternately: the TMA store that last read
            // the tile about to be written must have finished reading it
            const uint32_t buf = stg + (n_bulk & 1u) * (kEpiBufBytes / 2);
            if (lane == 0) bulk_wait_read<1>();
            __syncwarp();
            stage_bf16_chunk(buf, lane, v);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {                   // rows and columns beyond the matrix are clipped by the tensor map
              tma_store_2d_hint(&tmC, buf, col0, m0 + quad * 32, store_policy);
              bulk_commit();
            }
            ++n_bulk;
          }
        } else if constexpr (EPI == kEpiDx) {
          if (row_ok) epi_dx_chunk(p, v, grow, col0, scale);
        } else if constexpr (EPI == kEpiDw) {
          if (warp_rows_ok) {
            if (lane == 0) bulk_wait_read<0>();
            __syncwarp();
            stage_f32_row(stg, lane, v, scale, p.round_bf16 != 0);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {                   // rows beyond the vocabulary are clipped by the tensor map
              tma_reduce_add_2d(&tmC, stg, col0, p.m_off + m0 + quad * 32);
              bulk_commit();
            }
          }
        } else {
          if (row_ok) {
            const int ncols = min(32, p.N - col0);
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (j < ncols) p.c[int64_t(grow) * p.ldc + col0 + j] = v[j];
          }
        }
      };

      // software pipeline over this warp's chunks: the next chunk's TMEM load is in flight while one is processed
      float va[32], vb[32];
      __syncwarp();
      tmem_ld32(taddr, va);
#pragma unroll 1
      for (int c = 0; c < kChunks; c += 2) {
        tmem_ld_wait(va);
        __syncwarp();
        tmem_ld32(taddr + uint32_t((c + 1) * 32), vb);
        process(va, half * kChunks + c);
        tmem_ld_wait(vb);
        if (c + 2 < kChunks) {
          __syncwarp();
          tmem_ld32(taddr + uint32_t((c + 2) * 32), va);
        }
        process(vb, half * kChunks + c + 1);
      }
      // the accumulator buffer may be overwritten by the UMMAs of the tile after next
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if constexpr (NCTA == 2) mbar_arrive_cluster(mapa_shared(tempty_bar(b), 0));   // the leader issues the UMMAs
        else mbar_arrive(tempty_bar(b));
      }
      if constexpr (EPI == kEpiLogits) {
        // the two halves of a row meet in shared memory; the left half merges (left, then right: a fixed order) and
        // writes the tile's partial. Hand-over by two mbarriers per quadrant, waited on with the bounded wait.
        if (st.hit) p.zt[grow] = st.zt;
        const uint32_t mphase = uint32_t(it) & 1u;
        if (half == 1) {
          if (!mbar_wait<true>(mempty_bar(quad), mphase ^ 1u, abort_flag, p.status, kErrEpilogueWait)) break;
          merge[r_local] = make_float2(st.m, st.s);
          __syncwarp();
          if (lane == 0) mbar_arrive(mfull_bar(quad));
        } else {
          if (!mbar_wait<true>(mfull_bar(quad), mphase, abort_flag, p.status, kErrEpilogueWait)) break;
          const float2 o = merge[r_local];
          __syncwarp();
          if (lane == 0) mbar_arrive(mempty_bar(quad));
          constexpr float kLog2e = 1.4426950408889634f;
          const float m = fmaxf(st.m, o.x);      // st.m is finite: the left half always holds at least one valid column
          const float neg = -m * kLog2e;
          const float s = st.s * ex2_approx(fmaf(st.m, kLog2e, neg)) + o.y * ex2_approx(fmaf(o.x, kLog2e, neg));
          if (row_ok) {
            p.tmax[int64_t(ni) * p.ldT + grow] = m;
            p.tsum[int64_t(ni) * p.ldT + grow] = s;
          }
        }
      }
    }
    if constexpr (epi_stage_bytes(EPI) > 0) {
      if (lane == 0) bulk_wait<0>();           // every staged store / reduction has been performed
      __syncwarp();
    }
  }

  // -------------------------------------------------------------------- teardown
  tc_fence_before();
  // pair mode: neither CTA may leave (or free TMEM) while the other can still signal its barriers or read its shared
  // memory; every wait above is bounded, so both CTAs reach this barrier
  if constexpr (NCTA == 2) cluster_sync_all();
  else __syncthreads();
  if (warp == 1) {
    __syncwarp();
    if (*abort_flag) __nanosleep(200000);   // an expired wait: let copies and UMMAs in flight land before TMEM goes
    tc_fence_after();
    if constexpr (NCTA == 2) tmem_dealloc_pair(tmem_base, kTmemCols);
    else tmem_dealloc(tmem_base, kTmemCols);
  }
}

// A wait that nothing satisfies, with a short limit: the bounded wait must give up, record its error bit and raise the
// CTA's abort flag, which the other threads (polling it as the kernel roles do) observe; the kernel then returns
// normally and the context stays usable. This is how the time-out path of mbar_wait is exercised on a GPU.
__global__ void __launch_bounds__(64) k_wait_timeout_probe(uint32_t* status, long long limit_cycles, int* saw_abort) {
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    abort_word = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    const bool ok = mbar_wait(smem_u32(&bar), 0, abort_flag, status, kErrEpilogueWait, limit_cycles);
    if (ok) atomicOr(status, 0x80000000u);                      // cannot happen: nobody arrives on the barrier
  } else if (threadIdx.x == 32) {
    // a second role, waiting on the same never-completed barrier with a long limit: it must leave through the abort
    const bool ok = mbar_wait<true>(smem_u32(&bar), 0, abort_flag, status, kErrProducerWait, limit_cycles * 1000);
    if (!ok && *abort_flag) *saw_abort = 1;
  }
  __syncthreads();
}

// ---------------------------------------------------------------------------------------------- host side
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static std::once_flag once;
  static EncodeFn fn = nullptr;
  static cudaError_t err = cudaSuccess;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (err == cudaSuccess && q == cudaDriverEntryPointSuccess) fn = reinterpret_cast<EncodeFn>(p);
  });
  if (!fn) {
    cudaGetLastError();
    throw DeviceError(std::string("fused CE: cuTensorMapEncodeTiled is not available from the CUDA driver (") +
                      cudaGetErrorString(err) + "); this library needs an sm_100a device and has no other path");
  }
  return fn;
}

// bf16 matrix with `inner` contiguous elements per row, `outer` rows, row pitch ld elements; box = (box_inner, box_outer)
CUtensorMap make_tmap(const void* base, uint64_t inner, uint64_t outer, int64_t ld, uint32_t box_inner,
                      uint32_t box_outer, bool f32 = false, bool swizzle64 = false) {
  const int esz = f32 ? 4 : 2;
  NM_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0, "fused CE: a TMA operand must be 16-byte aligned");
  NM_REQUIRE((ld * esz) % 16 == 0, "fused CE: a TMA operand's row pitch must be a multiple of 16 bytes");
  NM_REQUIRE(inner > 0 && outer > 0, "fused CE: empty TMA operand");
  CUtensorMap m;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {cuuint64_t(ld) * esz};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode_fn()(&m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw DeviceError("fused CE: cuTensorMapEncodeTiled failed with CUresult " + std::to_string(int(r)) + " (inner " +
                      std::to_string(inner) + ", outer " + std::to_string(outer) + ", ld " + std::to_string(ld) + ")");
  return m;
}
// K-major operand [rows, K]: box = 64 k x `rows_per_box` rows. MN-major operand [K, MN]: box = 64 mn x 64 k.
CUtensorMap tmap_kmajor(const void* base, int64_t rows, int64_t K, int64_t ld, int rows_per_box) {
  return make_tmap(base, uint64_t(K), uint64_t(rows), ld, BK, uint32_t(rows_per_box));
}
CUtensorMap tmap_mnmajor(const void* base, int64_t K, int64_t MN, int64_t ld) {
  return make_tmap(base, uint64_t(MN), uint64_t(K), ld, 64, BK);
}
// The same operand when MN % 64 == 0, as a 3-D tensor (64 contiguous, K rows of pitch ld, MN / 64 groups 64 elements
// apart): a box of (64, 64 k, `groups`) lands in shared memory as `groups` consecutive 64-k x 128-byte blocks, which
// is the layout the 2-D boxes are placed in one by one.
CUtensorMap tmap_mnmajor_3d(const void* base, int64_t K, int64_t MN, int64_t ld, int groups) {
  NM_REQUIRE(MN % 64 == 0, "fused CE: the 3-D operand map needs an extent that is a multiple of 64");
  NM_REQUIRE(reinterpret_cast<uintptr_t>(base) % 16 == 0 && (ld * 2) % 16 == 0, "fused CE: TMA operand alignment");
  CUtensorMap m;
  const cuuint64_t dims[3] = {64, cuuint64_t(K), cuuint64_t(MN / 64)};
  const cuuint64_t strides[2] = {cuuint64_t(ld) * 2, 128};
  const cuuint32_t box[3] = {64, BK, cuuint32_t(groups)};
  const cuuint32_t estr[3] = {1, 1, 1};
  const CUresult r = encode_fn()(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box,
                                 estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                 CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    throw DeviceError("fused CE: cuTensorMapEncodeTiled (3-D) failed with CUresult " + std::to_string(int(r)));
  return m;
}
CUtensorMap tmap_mn_a(const void* base, int64_t K, int64_t MN, int64_t ld, int& is3d) {
  is3d = MN % 64 == 0;
  return is3d ? tmap_mnmajor_3d(base, K, MN, ld, BM / 64) : tmap_mnmajor(base, K, MN, ld);
}
CUtensorMap tmap_mn_b(const void* base, int64_t K, int64_t MN, int64_t ld, int& is3d, int ncta) {
  is3d = MN % 64 == 0;
  return is3d ? tmap_mnmajor_3d(base, K, MN, ld, BN / ncta / 64) : tmap_mnmajor(base, K, MN, ld);
}

// epilogue staging tile as a tensor-map box: 32 rows x 32 columns (f32: 128-byte rows, SWIZZLE_128B; bf16: 64-byte
// rows, SWIZZLE_64B)
CUtensorMap tmap_epilogue(void* base, int64_t rows, int64_t cols, int64_t ld, bool f32) {
  return make_tmap(base, uint64_t(cols), uint64_t(rows), ld, 32, 32, f32, !f32);
}

template <int EPI, bool A_MN, bool B_MN, int NCTA>
void launch_n(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
              cudaStream_t st, int sm_reserve) {
  auto kernel = k_ce_umma<EPI, A_MN, B_MN, NCTA>;
  constexpr int kSmem = smem_bytes(EPI, NCTA);
  static_assert(kSmem <= 232448, "dynamic shared memory beyond the 227 KiB a CTA may use");
  NM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  const int tiles = p.num_m * p.num_n;
  const int walkers = std::max(1, (sm_count() - std::max(0, sm_reserve)) / NCTA);   // CTAs, or pairs of CTAs
  const int grid = NCTA * std::min(tiles, walkers);
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3(unsigned(grid));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = st;
  cudaLaunchAttribute attr{};
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = NCTA; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = NCTA == 2 ? 1 : 0;
  NM_CUDA(cudaLaunchKernelEx(&cfg, kernel, ta, tb, tc, p));
}
template <int EPI, bool A_MN, bool B_MN>
void launch(int ncta, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
            cudaStream_t st, int sm_reserve = 0) {
  if (ncta == 2) launch_n<EPI, A_MN, B_MN, 2>(ta, tb, tc, p, st, sm_reserve);
  else launch_n<EPI, A_MN, B_MN, 1>(ta, tb, tc, p, st, sm_reserve);
}

// CTAs per tile for the three contractions: 1, 2 (pair mode) or 0 = chosen per launch. Pairs finish a tile in fewer
// cycles but draw more power, and on the power-capped large shapes the kernels around them lose most of what the
// paired kernel gains. The choice follows interleaved measurements (both forms alternated inside one process):
//   dX, dW: pairs for short, narrow calls (hidden size up to 512, at most 16384 rows per chunk: the per-layer
//           readouts), 2.8 % of that step;
//   logits: pairs for hidden sizes 1024 .. 2048 on calls of at least 4096 rows (step - 1.7 % at 1024, - 0.9 % at
//           2048); at 512 the kernel is bound by its epilogue and pairs are slower, at 4096 the step got 2 % slower.
int g_ncta[3] = {0, 0, 0};
int ncta_for(int which, int rows, int D) {
  if (g_ncta[which] != 0) return g_ncta[which];
  if (which == 0) return (D >= 1024 && D <= 2048 && rows >= 4096) ? 2 : 1;
  return (D <= 512 && rows <= 16384) ? 2 : 1;
}

}  // namespace

void launch_logits(const LogitsArgs& a, cudaStream_t st) {
  if (a.rows <= 0) return;
  GemmParams p{};
  const int ncta = ncta_for(0, a.rows, a.D), bmt = BM * ncta;
  p.M = a.rows; p.N = a.V; p.K = a.D; p.m_off = 0;
  p.num_m = (a.rows + bmt - 1) / bmt; p.num_n = (a.V + BN - 1) / BN; p.m_inner = 1;
  // rows are walked in groups whose x tiles (group x 128 x D bf16) take about 16 MiB of L2: x is then read from HBM
  // once per launch and W once per group, instead of x once per vocabulary tile
  p.m_group = int(std::max<int64_t>(1, std::min<int64_t>(p.num_m, (int64_t(16) << 20) / (int64_t(bmt) * a.D * 2))));
  p.status = a.status;
  p.store = a.store; p.ldS = a.ldS; p.store_f32 = a.store_f32;
  p.tmax = a.tmax; p.tsum = a.tsum; p.ldT = a.ldT; p.zt = a.zt; p.targets = a.targets; p.bias = a.bias;
  const CUtensorMap ta = tmap_kmajor(a.x, a.rows, a.D, a.D, BM);
  const CUtensorMap tb = tmap_kmajor(a.w, a.V, a.D, a.D, BN / ncta);
  // the bf16 store leaves by TMA; without one (forward only, f32 store) the map is unused
  const CUtensorMap tc = (a.store && !a.store_f32) ? tmap_epilogue(a.store, a.rows, a.V, a.ldS, false) : ta;
  launch<kEpiLogits, false, false>(ncta, ta, tb, tc, p, st);
}

void launch_dgrad(const DgradArgs& a, cudaStream_t st) {
  if (a.rows <= 0) return;
  GemmParams p{};
  const int ncta = ncta_for(1, a.rows, a.D), bmt = BM * ncta;
  p.M = a.rows; p.N = a.D; p.K = a.V; p.m_off = 0;
  p.num_m = (a.rows + bmt - 1) / bmt; p.num_n = (a.D + BN - 1) / BN; p.m_inner = 0;
  p.m_group = 1;
  p.status = a.status;
  p.scale = a.scale; p.dx_old = a.dx_old; p.dx_out = a.dx_out; p.acc_mode = a.dx_old ? a.acc_mode : 0;
  p.out_f32 = a.out_f32; p.ldo = a.D;
  const CUtensorMap ta = tmap_kmajor(a.n, a.rows, a.V, a.ldn, BM);
  const CUtensorMap tb = tmap_mn_b(a.w, a.V, a.D, a.ldw, p.b_3d, ncta);
  launch<kEpiDx, false, true>(ncta, ta, tb, ta, p, st, a.sm_reserve);
}

void launch_wgrad(const WgradArgs& a, cudaStream_t st) {
  if (a.rows <= 0 || a.v1 <= a.v0) return;
  NM_REQUIRE(a.v0 % BM == 0 && (a.v1 % BM == 0 || a.v1 == a.V) && a.v1 <= a.V,
             "fused CE: a dW vocabulary range must start and end on multiples of 128 (or end at V)");
  GemmParams p{};
  const int ncta = ncta_for(2, a.rows, a.D), bmt = BM * ncta;
  p.M = a.v1 - a.v0; p.N = a.D; p.K = a.rows; p.m_off = a.v0;
  p.num_m = (p.M + bmt - 1) / bmt; p.num_n = (a.D + BN - 1) / BN; p.m_inner = 0;
  p.m_group = 1;
  p.status = a.status;
  p.scale = a.scale; p.dw = a.dw; p.round_bf16 = a.round_bf16;
  const CUtensorMap ta = tmap_mn_a(a.n, a.rows, a.V, a.ldn, p.a_3d);
  const CUtensorMap tb = tmap_mn_b(a.x, a.rows, a.D, a.ldx, p.b_3d, ncta);
  const CUtensorMap tc = tmap_epilogue(a.dw, a.V, a.D, a.D, true);
  launch<kEpiDw, true, true>(ncta, ta, tb, tc, p, st, a.sm_reserve);
}

void set_cta_pair(int logits, int dgrad, int wgrad) {
  const int v[3] = {logits, dgrad, wgrad};
  for (int i = 0; i < 3; ++i) g_ncta[i] = v[i] < 0 ? 0 : (v[i] ? 2 : 1);
}

void launch_wait_timeout_probe(uint32_t* status, long long limit_cycles, int* saw_abort, cudaStream_t st) {
  NM_REQUIRE(status && saw_abort, "wait probe: status and saw_abort required");
  NM_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000, "wait probe: limit of at most 2e6 cycles (about 1 ms)");
  k_wait_timeout_probe<<<1, 64, 0, st>>>(status, limit_cycles, saw_abort);
  NM_CUDA(cudaGetLastError());
}

void launch_test_gemm(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc, int M,
                      int N, int K, uint32_t* status, cudaStream_t st) {
  NM_REQUIRE((kind & ~4) >= 0 && (kind & ~4) <= 2, "test gemm: kind 0, 1 or 2, plus 4 for the CTA-pair form");
  NM_REQUIRE(M > 0 && N > 0 && K > 0, "test gemm: M, N, K > 0");
  const int ncta = (kind & 4) ? 2 : 1, bmt = BM * ncta;
  kind &= ~4;
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.m_off = 0;
  p.num_m = (M + bmt - 1) / bmt; p.num_n = (N + BN - 1) / BN;
  p.m_inner = kind == 0; p.m_group = 3;          // the grouped walk is exercised by the K-major test
  p.status = status; p.c = c; p.ldc = ldc;
  if (kind == 0) {
    const CUtensorMap ta = tmap_kmajor(a, M, K, lda, BM);
    launch<kEpiTest, false, false>(ncta, ta, tmap_kmajor(b, N, K, ldb, BN / ncta), ta, p, st);
  } else if (kind == 1) {
    const CUtensorMap ta = tmap_kmajor(a, M, K, lda, BM);
    launch<kEpiTest, false, true>(ncta, ta, tmap_mn_b(b, K, N, ldb, p.b_3d, ncta), ta, p, st);
  } else {
    const CUtensorMap ta = tmap_mn_a(a, K, M, lda, p.a_3d);
    launch<kEpiTest, true, true>(ncta, ta, tmap_mn_b(b, K, N, ldb, p.b_3d, ncta), ta, p, st);
  }
}

}  // namespace nm::ce
