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
#include <algorithm>
#include <atomic>
#include <mutex>
#include <string>
#include <type_traits>

#include "ce_umma.cuh"

namespace nm::ce {
namespace {
// NCTA = 1: one CTA per tile of 128 x 256. NCTA = 2: a pair of CTAs (a cluster of two on one TPC) per tile of
// 256 x 256; each CTA stages its own 128 rows of A and its own 128 columns of B, the leader issues one UMMA of M = 256
// over both CTAs' shared memory, and each CTA keeps the accumulator of its own 128 rows in its own TMEM: the B
// operand crosses L2 -> shared memory once per pair instead of once per CTA.
constexpr int kABytes = BM * BK * 2;            // 16 KiB
__host__ __device__ constexpr int b_bytes(int ncta) { return BN / ncta * BK * 2; }                 // 32 / 16 KiB
__host__ __device__ constexpr int stage_bytes(int ncta) { return kABytes + b_bytes(ncta); }        // 48 / 32 KiB
__host__ __device__ constexpr int num_stages(int ncta) { return ncta == 2 ? 6 : 4; }

// epilogue staging: one 32-row x 128-byte tile per epilogue warp, only for the epilogues that leave through TMA; the
// logits epilogue adds 1 KiB where the two column halves of a row meet to merge their (max, sum exp)
constexpr int kMergeBytes = BM * 8;
__host__ __device__ constexpr int epi_stage_bytes(int epi) {
  return (epi == kEpiLogits || epi == kEpiDw) ? kEpiWarps * kEpiBufBytes + (epi == kEpiLogits ? kMergeBytes : 0) : 0;
}
constexpr int smem_bytes(int epi, int ncta) {
  return num_stages(ncta) * stage_bytes(ncta) + epi_stage_bytes(epi) + 1024 /*alignment slack*/ + 256 /*barriers*/;
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
// The override is process-wide and may be set from any host thread while other threads are inside a call: atomics.
std::atomic<int> g_ncta[3] = {{0}, {0}, {0}};
int ncta_for(int which, int rows, int D) {
  const int forced = g_ncta[which].load(std::memory_order_relaxed);
  if (forced != 0) return forced;
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

// ce_grad_wide.cu
void launch_dgrad_wide(const DgradArgs& a, cudaStream_t st);
void launch_wgrad_wide(const WgradArgs& a, cudaStream_t st);
void launch_test_gemm_wide(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc,
                           int M, int N, int K, uint32_t* status, const RowFactors* rowf, cudaStream_t st);

void launch_dgrad(const DgradArgs& a, cudaStream_t st) {
  if (a.rows <= 0) return;
  NM_REQUIRE(a.wide || !a.rowf, "dX: forming the gradient inside the kernel needs the wide tile form");
  if (a.wide) return launch_dgrad_wide(a, st);
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
  NM_REQUIRE(a.wide || !a.rowf, "dW: forming the gradient inside the kernel needs the wide tile form");
  if (a.wide) return launch_wgrad_wide(a, st);
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
  for (int i = 0; i < 3; ++i) g_ncta[i].store(v[i] < 0 ? 0 : (v[i] ? 2 : 1), std::memory_order_relaxed);
}

void launch_wait_timeout_probe(uint32_t* status, long long limit_cycles, int* saw_abort, cudaStream_t st) {
  NM_REQUIRE(status && saw_abort, "wait probe: status and saw_abort required");
  NM_REQUIRE(limit_cycles > 0 && limit_cycles <= 2000000, "wait probe: limit of at most 2e6 cycles (about 1 ms)");
  k_wait_timeout_probe<<<1, 64, 0, st>>>(status, limit_cycles, saw_abort);
  NM_CUDA(cudaGetLastError());
}

void launch_test_gemm(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc, int M,
                      int N, int K, uint32_t* status, const RowFactors* rowf, cudaStream_t st) {
  NM_REQUIRE(M > 0 && N > 0 && K > 0, "test gemm: M, N, K > 0");
  if (kind & 8) {   // the wide pair kernels; + 16: A holds raw logits and is transformed with rowf
    NM_REQUIRE(((kind & 16) != 0) == (rowf != nullptr), "test gemm: kind + 16 goes with row factors");
    return launch_test_gemm_wide(kind & 3, a, lda, b, ldb, c, ldc, M, N, K, status, rowf, st);
  }
  NM_REQUIRE((kind & ~4) >= 0 && (kind & ~4) <= 2, "test gemm: kind 0, 1 or 2, plus 4 for the CTA-pair form");
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
