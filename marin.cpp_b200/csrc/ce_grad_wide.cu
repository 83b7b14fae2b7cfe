// The two gradient contractions of the fused linear cross-entropy on CTA pairs with one wide accumulator, and, in
// their fused form, with the normalised gradient formed inside the kernel:
//     dX   dx[rows, D]  = n[rows, V]  W[V, D]        A K-major  (256 rows per pair),  B MN-major
//     dW   dw[V, D]    += n[rows, V]^T x[rows, D]    A MN-major (256 vocabulary rows per pair), B MN-major
// where n = a p - b onehot(target), p = exp(z - lse), is what the reference forms either in a separate pass over the
// logits store (src/kernels/cross_entropy/ce_logits.cu:262-318) or, on Hopper, in transform warps ahead of its wgmma
// main loop (ce_sm90.cu:558-764). This is the sm_100a design of the second idea:
//
//   * A cluster of two CTAs (one TPC) owns a 256 x 512 output tile. Each CTA stages its own 128 rows of A and, for each
//     of the two 256-column halves of the tile, its own 128 columns of B; the leader issues tcgen05.mma cta_group::2
//     (M 256, N 256, K 16) twice per K step, into TMEM columns [0, 256) and [256, 512). The whole 512-column TMEM of
//     both SMs is one accumulator: the contraction is 10^4 .. 10^5 long, so an epilogue that does not overlap the next
//     tile costs about 1 % while every staged A block now feeds twice the math (half the L2 -> shared-memory traffic of
//     A per FLOP, and the re-streamed operand crosses HBM half as often as with 256-column tiles).
//   * Fused form (kXform): A arrives by TMA as RAW bf16 logits. The eight warps that are the epilogue at the end of a
//     tile spend the main loop as transform warps: when a stage's A block has landed they rewrite it in place, in the
//     swizzled layout the UMMA reads (the map is element-wise, so the layout is only needed to know each 16-byte
//     piece's row and columns), fence it to the async proxy and arrive on the leader's barrier the UMMA issuer waits
//     on. Per 64-deep K block a CTA evaluates 8192 exponentials against 1024 tensor cycles: half the SM's MUFU rate.
//     Neither the separate pass nor a second copy of the gradient exists; the logits store is read-only here, so tiles
//     that share A (the N tiles of a wide hidden size) simply transform it again.
//   * Plain form: A is already n (the in-place pass ran); the transform warps idle until the epilogue.
//
// Warp roles per CTA (704 threads): warp 0 TMA producer of B (one lane), warp 1 TMEM allocation + UMMA issue (one lane,
// leader CTA only), warp 2 TMA producer of A (one lane), warps 3-18 transform (four per scheduler), of which warps
// 3-10 are also the epilogue, warps 19-21 relays (one lane each, in the CTA that issues no UMMAs). A and B have rings of their own (6 and 4 or 3
// stages): measured with the arithmetic of the transform switched off, the fused form was no faster, i.e. what it
// costs is the longer way of an A block to the tensor core (load, wake the warps, their barrier, the relay, the
// issuer), and a deeper A ring is what hides that.
// Barriers: per A stage full_a (fused form: this CTA's A bytes; plain form: the leader's, for both CTAs), xformed (this
// CTA's 16 transform warps are done with the stage), peer_ready (leader: the other CTA's relay thread has seen its
// xformed and fenced), empty_a; per B stage full_b (leader: the B bytes of both CTAs), empty_b (the empties arrive in
// both CTAs through the multicast commit once the UMMAs have read the stage). The writes of the transform reach the
// tensor core through one fence.proxy.async per CTA and stage, executed by the thread that acquired the warps' barrier
// (the UMMA issuer in the leader, the relay thread in the other CTA), not by the 512 writers. No TMA load is multicast.
// Every wait is bounded.
#include <algorithm>
#include <atomic>
#include <type_traits>

#include "ce_grad_math.cuh"
#include "ce_umma.cuh"

namespace nm::ce {
namespace {

constexpr int kWideN = 512;                        // accumulator columns of a tile
constexpr int kXWarps = 16;                        // transform warps (the first kEpiWarps of them are also the epilogue)
constexpr int kFirstXWarp = 3;                     // warps 0, 1, 2: B producer, UMMA issuer / relay, A producer
constexpr int kRelays = 3;                         // relay warps (after the transform warps); stage s belongs to relay s % 3
constexpr int kWThreads = 32 * (kFirstXWarp + kXWarps + kRelays);
constexpr int kWABytes = BM * BK * 2;              // 16 KiB: this CTA's 128 rows (or vocabulary entries) x 64 k
constexpr int kWBHalfBytes = 128 * BK * 2;         // 16 KiB: this CTA's 128 of the 256 columns of one UMMA
constexpr int kWBBytes = 2 * kWBHalfBytes;         // both 256-column halves of the tile
// The two operands have rings of their own. A's way from HBM to the tensor core is the long one (HBM latency, then the
// transform and two barrier hand-overs before the UMMAs may read it), so its ring is the deeper; B comes out of L2
// and is consumed as it lands. dW gives one B stage to the staging tiles of its epilogue (its B operand, the x chunk,
// stays in L2).
__host__ __device__ constexpr int a_stages(int epi) { return 6; }
__host__ __device__ constexpr int b_stages(int epi) { return epi == kEpiDw ? 3 : 4; }
__host__ __device__ constexpr int wide_epi_bytes(int epi) { return epi == kEpiDw ? kEpiWarps * kEpiBufBytes : 0; }
constexpr int kWBarrierBytes = 512;
constexpr int wide_smem_bytes(int epi) {
  return a_stages(epi) * kWABytes + b_stages(epi) * kWBBytes + wide_epi_bytes(epi) + 1024 /*alignment slack*/ +
         kWBarrierBytes;
}

template <int EPI, bool A_MN, bool kXform>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kWThreads, 1)
k_ce_grad_wide(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  constexpr int kA = a_stages(EPI), kB = b_stages(EPI);
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  const uint32_t sA = base, sB = base + kA * kWABytes;
  const uint32_t sEpi = sB + kB * kWBBytes;
  const uint32_t bar0 = sEpi + wide_epi_bytes(EPI);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kA * kWABytes + kB * kWBBytes + wide_epi_bytes(EPI));
  // per A stage: full_a (fused: this CTA's bytes; plain: leader only, the bytes of both CTAs), xformed (this CTA's
  // transform warps are done), peer_ready (leader: the other CTA's relay has seen its xformed), empty_a
  auto full_a = [&](int s) { return bar0 + 8u * s; };
  auto xformed = [&](int s) { return bar0 + 8u * (kA + s); };
  auto peer_ready = [&](int s) { return bar0 + 8u * (2 * kA + s); };
  auto empty_a = [&](int s) { return bar0 + 8u * (3 * kA + s); };
  // per B stage: full_b (leader: the bytes of both CTAs), empty_b
  auto full_b = [&](int s) { return bar0 + 8u * (4 * kA + s); };
  auto empty_b = [&](int s) { return bar0 + 8u * (4 * kA + kB + s); };
  const uint32_t tfull = bar0 + 8u * (4 * kA + 2 * kB), tempty = tfull + 8u;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * kA + 2 * kB + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  static_assert((4 * kA + 2 * kB + 2) * 8 + 8 <= kWBarrierBytes, "barrier region too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int walker = int(blockIdx.x >> 1), walkers = int(gridDim.x >> 1);
  if (threadIdx.x == 0) {
    for (int s = 0; s < kA; ++s) {
      mbar_init(full_a(s), 1);
      mbar_init(xformed(s), kXWarps);
      mbar_init(peer_ready(s), 1);
      mbar_init(empty_a(s), 1);
    }
    for (int s = 0; s < kB; ++s) {
      mbar_init(full_b(s), 1);
      mbar_init(empty_b(s), 1);
    }
    mbar_init(tfull, 1);
    mbar_init(tempty, 2 * kEpiWarps);
    *abort_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
    if constexpr (EPI == kEpiDw) prefetch_tmap(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  cluster_sync_all();            // the peer's barriers exist before anything signals them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int num_tiles = p.num_m * p.num_n;
  const int k_blocks = (p.K + BK - 1) / BK;
  // consecutive tiles share their A rows and differ in the 512-column block of the output
  auto decode = [&](int tile, int& mi, int& ni) { ni = tile % p.num_n; mi = tile / p.num_n; };
  auto halves = [&](int ni) { return (p.N - ni * kWideN > BN) ? 2 : 1; };   // 256-column halves with any column in range

  if (warp == 0) {
    if (lane == 0) {
      // ------------------------------------------------------------------ B producer (both CTAs)
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      const uint64_t pol_last = l2_policy_evict_last();   // dW re-reads the whole x chunk for every vocabulary tile
      for (int tile = walker; tile < num_tiles && ok; tile += walkers) {
        int mi, ni;
        decode(tile, mi, ni);
        const int nh = halves(ni);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait<true>(empty_b(stage), phase ^ 1u, abort_flag, p.status, kErrProducerWait)) { ok = false; break; }
          const uint32_t lead = mapa_shared(full_b(stage), 0);
          if (rank == 0) mbar_arrive_expect_tx(full_b(stage), 2 * nh * kWBHalfBytes);
          const int k0 = kb * BK;
          for (int u = 0; u < nh; ++u) {
            const int n0 = ni * kWideN + u * BN + int(rank) * (BN / 2);
            const uint32_t dst = sB + stage * kWBBytes + u * kWBHalfBytes;
            if (p.b_3d) {
              if constexpr (EPI == kEpiDw) tma_pair_load_3d_hint(dst, &tmB, lead, 0, k0, n0 >> 6, pol_last);
              else tma_pair_load_3d(dst, &tmB, lead, 0, k0, n0 >> 6);
            } else {
#pragma unroll
              for (int j = 0; j < 2; ++j) {
                if constexpr (EPI == kEpiDw) tma_pair_load_2d_hint(dst + j * kBoxBytesMN, &tmB, lead, n0 + j * 64, k0, pol_last);
                else tma_pair_load_2d(dst + j * kBoxBytesMN, &tmB, lead, n0 + j * 64, k0);
              }
            }
          }
          if (++stage == kB) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 2) {
    if (lane == 0) {
      // ------------------------------------------------------------------ A producer (both CTAs)
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = walker; tile < num_tiles && ok; tile += walkers) {
        int mi, ni;
        decode(tile, mi, ni);
        const int m0 = p.m_off + mi * (2 * BM) + int(rank) * BM;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!mbar_wait<true>(empty_a(stage), phase ^ 1u, abort_flag, p.status, kErrProducerWait)) { ok = false; break; }
          const uint32_t a_dst = sA + stage * kWABytes;
          const int k0 = kb * BK;
          if constexpr (kXform) {
            // the bytes are counted on this CTA's own barrier: its transform warps wait there
            mbar_arrive_expect_tx(full_a(stage), kWABytes);
            if constexpr (A_MN) {
              if (p.a_3d) {
                tma_load_3d(a_dst, &tmA, full_a(stage), 0, k0, m0 >> 6);
              } else {
#pragma unroll
                for (int j = 0; j < BM / 64; ++j) tma_load_2d(a_dst + j * kBoxBytesMN, &tmA, full_a(stage), m0 + j * 64, k0);
              }
            } else {
              tma_load_2d(a_dst, &tmA, full_a(stage), k0, m0);
            }
          } else {
            // the bytes of both CTAs are counted on the leader's barrier, which only the leader arms
            const uint32_t lead = mapa_shared(full_a(stage), 0);
            if (rank == 0) mbar_arrive_expect_tx(full_a(stage), 2 * kWABytes);
            if constexpr (A_MN) {
              if (p.a_3d) {
                tma_pair_load_3d(a_dst, &tmA, lead, 0, k0, m0 >> 6);
              } else {
#pragma unroll
                for (int j = 0; j < BM / 64; ++j) tma_pair_load_2d(a_dst + j * kBoxBytesMN, &tmA, lead, m0 + j * 64, k0);
              }
            } else {
              tma_pair_load_2d(a_dst, &tmA, lead, k0, m0);
            }
          }
          if (++stage == kA) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && rank == 0) {
      // ------------------------------------------------------------------ UMMA issuer (leader CTA)
      constexpr uint32_t idesc = idesc_bf16_f32(2 * BM, BN, A_MN, true);
      int sa = 0, sb = 0; uint32_t pa = 0, pb = 0;
      int it = 0;
      bool ok = true, ahead = false;
      for (int tile = walker; tile < num_tiles && ok; tile += walkers, ++it) {
        int mi, ni;
        decode(tile, mi, ni);
        const int nh = halves(ni);
        // one accumulator: the epilogue of the previous tile must have drained it
        if (!mbar_wait_cluster(tempty, (uint32_t(it) & 1u) ^ 1u, abort_flag, p.status, kErrTmemFreeWait)) break;
        tc_fence_after();
        for (int kb = 0; kb < k_blocks; ++kb) {
          // `ahead`: all barriers of this K block were seen complete by the look-ahead of the previous iteration
          if (!ahead) {
            if constexpr (kXform) {
              if (!mbar_wait(xformed(sa), pa, abort_flag, p.status, kErrMmaWait)) { ok = false; break; }
              if (!mbar_wait_cluster(peer_ready(sa), pa, abort_flag, p.status, kErrMmaWait)) { ok = false; break; }
            } else {
              if (!mbar_wait(full_a(sa), pa, abort_flag, p.status, kErrMmaWait)) { ok = false; break; }
            }
            if (!mbar_wait(full_b(sb), pb, abort_flag, p.status, kErrMmaWait)) { ok = false; break; }
          }
          // this CTA's transform warps released their shared-memory writes on xformed; one proxy fence here, on the
          // path from those writes to the UMMAs, orders them before the tensor core's reads. The other CTA's relay
          // thread did the same for its half before it arrived on peer_ready.
          if constexpr (kXform) fence_proxy_async_smem();
          tc_fence_after();
          // Look ahead: test the next K block's barriers now, without blocking. A test is a shared-memory round trip
          // of about a hundred cycles (measured with clock64 in this thread: 90 - 110 each), and three of them in a row
          // between two K blocks let the queue of issued UMMAs (about a third of a K block deep) run dry. Issued here,
          // they return while the UMMAs below wait for queue slots.
          const int na = sa + 1 == kA ? 0 : sa + 1, nb = sb + 1 == kB ? 0 : sb + 1;
          const uint32_t npa = sa + 1 == kA ? pa ^ 1u : pa, npb = sb + 1 == kB ? pb ^ 1u : pb;
          bool next_ready = false;
          if (kb + 1 < k_blocks) {
            bool ra;
            if constexpr (kXform) ra = mbar_try_wait(xformed(na), npa) & mbar_try_wait_cluster(peer_ready(na), npa);
            else ra = mbar_try_wait(full_a(na), npa);
            next_ready = ra & mbar_try_wait(full_b(nb), npb);
          }
          const uint32_t a_src = sA + sa * kWABytes, b_src = sB + sb * kWBBytes;
          for (int u = 0; u < nh; ++u) {
#pragma unroll
            for (int k = 0; k < BK / UK; ++k) {
              const uint64_t ad = A_MN ? smem_desc_sw128(a_src + k * (UK * 128), kBoxBytesMN, 1024)
                                       : smem_desc_sw128(a_src + k * (UK * 2), 16, 1024);
              const uint64_t bd = smem_desc_sw128(b_src + u * kWBHalfBytes + k * (UK * 128), kBoxBytesMN, 1024);
              umma_pair_bf16(tmem_base + uint32_t(u * BN), ad, bd, idesc, (kb | k) != 0);
            }
          }
          // both stages are free again, in both CTAs, once these UMMAs have read them
          umma_pair_commit(empty_a(sa), 3);
          umma_pair_commit(empty_b(sb), 3);
          sa = na; pa = npa; sb = nb; pb = npb;
          ahead = next_ready;
        }
        ahead = false;
        if (ok) umma_pair_commit(tfull, 3);
      }
    }
  } else if (warp >= kFirstXWarp + kXWarps) {
    if (kXform && lane == 0 && rank == 1) {
      // ------------------------------------------------------------------ relays (the CTA that issues no UMMAs)
      // Its transform warps arrive on a barrier of their own CTA (a CTA-scope release is cheap). A relay thread waits
      // there, fences the writes towards the async proxy and tells the leader with a cluster-scope release, which
      // takes the issuing thread longer than a K block lasts: hence three relay threads in three warps, each
      // serving every third stage, so that their arrivals overlap.
      static_assert(a_stages(EPI) % kRelays == 0, "every stage must always meet the same relay");
      const int me = warp - (kFirstXWarp + kXWarps);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      for (int tile = walker; tile < num_tiles && ok; tile += walkers) {
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (stage % kRelays == me) {
            if (!mbar_wait(xformed(stage), phase, abort_flag, p.status, kErrTransformWait)) { ok = false; break; }
            fence_proxy_async_smem();
            mbar_arrive_cluster(mapa_shared(peer_ready(stage), 0));
          }
          if (++stage == kA) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- transform (16 warps) + epilogue (first 8)
    const int w16 = warp - kFirstXWarp;
    const bool drains = w16 < kEpiWarps;       // the first eight transform warps also drain the accumulator
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int colhalf = (w16 >> 2) & 1;        // which 256 columns of the tile this warp drains
    const int r_local = quad * 32 + lane;
    const uint32_t stg = sEpi + uint32_t(w16 & (kEpiWarps - 1)) * kEpiBufBytes;
    float scale = 1.f;
    if constexpr (EPI == kEpiDx || EPI == kEpiDw) scale = p.scale ? __ldg(p.scale) : 1.f;
    // transform geometry: 8 rows of the staged A block per warp, lane & 7 = row, lane >> 3 = which two of the eight
    // 16-byte pieces of that 128-byte row. Eight consecutive lanes touch eight different rows, so their swizzled
    // pieces fall into eight different bank groups.
    const int xq = lane >> 3;
    // K-major A (dX): 128 rows x 128 bytes, row = w16 * 8 + (lane & 7), fixed for the tile
    // MN-major A (dW): two boxes of 64 k-rows x 128 bytes; box = w16 >> 3, k-row = (w16 & 7) * 8 + (lane & 7)
    const int xrow = A_MN ? ((w16 & 7) * 8 + (lane & 7)) : (w16 * 8 + (lane & 7));
    const uint32_t xoff = A_MN ? uint32_t((w16 >> 3) * kBoxBytesMN + xrow * 128) : uint32_t(xrow * 128);
    const uint32_t piece0 = (uint32_t((xq * 2) ^ (xrow & 7)) << 4), piece1 = (uint32_t((xq * 2 + 1) ^ (xrow & 7)) << 4);
    const uint32_t lead_tempty = mapa_shared(tempty, 0);
    const uint64_t ll = gradmath::pack_f32x2(gradmath::kLog2e, gradmath::kLog2e);
    int stage = 0; uint32_t phase = 0;
    int it = 0;
    bool alive = true;
    for (int tile = walker; tile < num_tiles && alive; tile += walkers, ++it) {
      int mi, ni;
      decode(tile, mi, ni);
      const int m0 = mi * (2 * BM) + int(rank) * BM, n0 = ni * kWideN;
      if constexpr (kXform) {
        RowFactors rf{0.f, 0.f, 0.f, -1};
        if constexpr (!A_MN) {                 // dX: this thread's row of the store, for the whole tile
          const int grow = m0 + xrow;
          if (grow < p.M) rf = p.rowf[grow];
        } else {
          if (xrow < p.K) rf = p.rowf[xrow];   // dW: the row changes with every K block; the next one is prefetched
        }
        for (int kb = 0; kb < k_blocks; ++kb) {
          const int k0 = kb * BK;
          RowFactors nxt{0.f, 0.f, 0.f, -1};
          if constexpr (A_MN) {
            const int r = k0 + BK + xrow;
            if (kb + 1 < k_blocks && r < p.K) nxt = p.rowf[r];
          }
          if (!mbar_wait<true>(full_a(stage), phase, abort_flag, p.status, kErrTransformWait)) { alive = false; break; }
          const uint32_t row_addr = sA + stage * kWABytes + xoff;
          // first column of the store this thread's two pieces cover
          const int vbase = A_MN ? (p.m_off + m0 + (w16 >> 3) * 64 + xq * 16) : (k0 + xq * 16);
          const int tpos = rf.target - vbase;                       // 0 .. 15 when the target is among them
          const int limit = A_MN ? 16 : (p.K - vbase);              // dX: columns at or beyond V are zero
          // the row's target, when it lies in these 16 columns (one thread, one K block per row): its raw logit is
          // picked up before the pieces are rewritten and its value patched in afterwards
          const bool has_target = static_cast<unsigned>(tpos) < 16u;
          const uint32_t t_addr = row_addr + (tpos < 8 ? piece0 : piece1) + uint32_t(tpos & 7) * 2u;
          uint16_t t_raw = 0;
          if (has_target) t_raw = ld_shared_u16(t_addr);
          uint4 v0 = ld_shared_v4(row_addr + piece0), v1 = ld_shared_v4(row_addr + piece1);
          if (limit >= 16) {                   // uniform over the CTA except in the last K block of a ragged vocabulary
            const uint64_t ee = gradmath::pack_f32x2(rf.e, rf.e), aa = gradmath::pack_f32x2(rf.a, rf.a);
            v0 = gradmath::piece_bf16_plain2(v0, ll, ee, aa);
            v1 = gradmath::piece_bf16_plain2(v1, ll, ee, aa);
          } else {
            v0 = gradmath::piece_bf16(v0, rf.e, rf.a, 0.f, -1, limit);
            v1 = gradmath::piece_bf16(v1, rf.e, rf.a, 0.f, -1, limit - 8);
          }
          st_shared_v4(row_addr + piece0, v0.x, v0.y, v0.z, v0.w);
          st_shared_v4(row_addr + piece1, v1.x, v1.y, v1.z, v1.w);
          if (has_target) st_shared_u16(t_addr, gradmath::target_element(t_raw, rf.e, rf.a, rf.b));
          __syncwarp();
          if (lane == 0) mbar_arrive(xformed(stage));   // CTA-scope release of the warp's writes
          if constexpr (A_MN) rf = nxt;
          if (++stage == kA) { stage = 0; phase ^= 1u; }
        }
        if (!alive) break;
      }
      if (!drains) continue;

      // ---- epilogue of the tile: 256 columns per warp in chunks of 32 (the contraction is so long that nothing is
      // gained by overlapping the accumulator loads with the stores)
      const int grow = m0 + r_local;
      const bool row_ok = grow < p.M;
      const bool warp_rows_ok = m0 + quad * 32 < p.M;
      if (!mbar_wait<true>(tfull, uint32_t(it) & 1u, abort_flag, p.status, kErrEpilogueWait)) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + (uint32_t(quad * 32) << 16) + uint32_t(colhalf * BN);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        const int col0 = n0 + colhalf * BN + c * 32;
        if (col0 >= p.N) break;                // uniform over the warp
        float v[32];
        __syncwarp();
        tmem_ld32(taddr + uint32_t(c * 32), v);
        tmem_ld_wait(v);
        if constexpr (EPI == kEpiDx) {
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
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(lead_tempty);   // the leader's UMMA issuer may overwrite the accumulator
    }
    if constexpr (EPI == kEpiDw) {
      if (drains && lane == 0) bulk_wait<0>();  // every staged reduction has been performed
      __syncwarp();
    }
  }

  // -------------------------------------------------------------------- teardown
  tc_fence_before();
  // neither CTA may leave (or free TMEM) while the other can still signal its barriers or read its shared memory;
  // every wait above is bounded, so both CTAs reach this barrier
  cluster_sync_all();
  if (warp == 1) {
    __syncwarp();
    if (*abort_flag) __nanosleep(200000);   // an expired wait: let copies and UMMAs in flight land before TMEM goes
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
}

template <int EPI, bool A_MN, bool kXform>
void launch_wide(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p,
                 cudaStream_t st, int sm_reserve) {
  auto kernel = k_ce_grad_wide<EPI, A_MN, kXform>;
  constexpr int kSmem = wide_smem_bytes(EPI);
  static_assert(kSmem <= 232448, "dynamic shared memory beyond the 227 KiB a CTA may use");
  NM_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem));
  const int tiles = p.num_m * p.num_n;
  const int pairs = std::max(1, (sm_count() - std::max(0, sm_reserve)) / 2);
  const int grid = 2 * std::min(tiles, pairs);
  kernel<<<dim3(unsigned(grid)), dim3(kWThreads), kSmem, st>>>(ta, tb, tc, p);
  NM_CUDA(cudaGetLastError());
}

void fill_wide_tiles(GemmParams& p) {
  p.num_m = (p.M + 2 * BM - 1) / (2 * BM);
  p.num_n = (p.N + kWideN - 1) / kWideN;
  p.m_inner = 0;
  p.m_group = 1;
}

}  // namespace

void launch_dgrad_wide(const DgradArgs& a, cudaStream_t st) {
  if (a.rows <= 0) return;
  GemmParams p{};
  p.M = a.rows; p.N = a.D; p.K = a.V; p.m_off = 0;
  fill_wide_tiles(p);
  p.status = a.status;
  p.scale = a.scale; p.dx_old = a.dx_old; p.dx_out = a.dx_out; p.acc_mode = a.dx_old ? a.acc_mode : 0;
  p.out_f32 = a.out_f32; p.ldo = a.D;
  p.rowf = a.rowf;
  const CUtensorMap ta = tmap_kmajor(a.n, a.rows, a.V, a.ldn, BM);
  const CUtensorMap tb = tmap_mn_b(a.w, a.V, a.D, a.ldw, p.b_3d, 2);
  if (a.rowf) launch_wide<kEpiDx, false, true>(ta, tb, ta, p, st, a.sm_reserve);
  else launch_wide<kEpiDx, false, false>(ta, tb, ta, p, st, a.sm_reserve);
}

void launch_wgrad_wide(const WgradArgs& a, cudaStream_t st) {
  if (a.rows <= 0 || a.v1 <= a.v0) return;
  NM_REQUIRE(a.v0 % BM == 0 && (a.v1 % BM == 0 || a.v1 == a.V) && a.v1 <= a.V,
             "fused CE: a dW vocabulary range must start and end on multiples of 128 (or end at V)");
  GemmParams p{};
  p.M = a.v1 - a.v0; p.N = a.D; p.K = a.rows; p.m_off = a.v0;
  fill_wide_tiles(p);
  p.status = a.status;
  p.scale = a.scale; p.dw = a.dw; p.round_bf16 = a.round_bf16;
  p.rowf = a.rowf;
  const CUtensorMap ta = tmap_mn_a(a.n, a.rows, a.V, a.ldn, p.a_3d);
  const CUtensorMap tb = tmap_mn_b(a.x, a.rows, a.D, a.ldx, p.b_3d, 2);
  const CUtensorMap tc = tmap_epilogue(a.dw, a.V, a.D, a.D, true);
  if (a.rowf) launch_wide<kEpiDw, true, true>(ta, tb, tc, p, st, a.sm_reserve);
  else launch_wide<kEpiDw, true, false>(ta, tb, tc, p, st, a.sm_reserve);
}

// unit-test entry (see launch_test_gemm): kinds 1 (A K-major) and 2 (A MN-major), B MN-major, plain f32 output
void launch_test_gemm_wide(int kind, const void* a, int64_t lda, const void* b, int64_t ldb, float* c, int64_t ldc,
                           int M, int N, int K, uint32_t* status, const RowFactors* rowf, cudaStream_t st) {
  NM_REQUIRE(kind == 1 || kind == 2, "test gemm (wide): kind 1 or 2");
  GemmParams p{};
  p.M = M; p.N = N; p.K = K; p.m_off = 0;
  fill_wide_tiles(p);
  p.status = status; p.c = c; p.ldc = ldc; p.rowf = rowf;
  if (kind == 1) {
    const CUtensorMap ta = tmap_kmajor(a, M, K, lda, BM);
    const CUtensorMap tb = tmap_mn_b(b, K, N, ldb, p.b_3d, 2);
    if (rowf) launch_wide<kEpiTest, false, true>(ta, tb, ta, p, st, 0);
    else launch_wide<kEpiTest, false, false>(ta, tb, ta, p, st, 0);
  } else {
    const CUtensorMap ta = tmap_mn_a(a, K, M, lda, p.a_3d);
    const CUtensorMap tb = tmap_mn_b(b, K, N, ldb, p.b_3d, 2);
    if (rowf) launch_wide<kEpiTest, true, true>(ta, tb, ta, p, st, 0);
    else launch_wide<kEpiTest, true, false>(ta, tb, ta, p, st, 0);
  }
}

}  // namespace nm::ce
