// Small kernels on either side of the fused CE in a training step: the microbatch metadata that produces the CE's
// targets and weights from token rows (doc_meta), and the fixed-order reductions that consume its per-chunk losses and
// the norms' gain partials. Integer outputs are exact; float reductions have a summation order that depends only on
// the sizes. Reference: src/kernels/elementwise/doc_meta.cu:19-81 and reduce_cast.cu:72-104 (behaviour pinned by the
// numpy reference of tests/s3/test_misc.py:17-36).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <mutex>

#include "ce_internal.hpp"
#include "ew_api.hpp"

namespace nm::ew {
namespace {

// Where the row kernels whose waits are bounded (the norm backward kernels' batch ring) leave their error bits: one word
// per GPU, built into the library because those entry points take no workspace.
static __device__ uint32_t g_row_status_word[2];   // [0] the error bits, [1] scratch of the test probe
std::mutex g_row_status_mu;
uint32_t* g_row_status_ptr[kMaxDeviceOrdinals] = {};

constexpr int kMetaThreads = 256;

// One CTA per row. targets[p] = row[p + 1] (the last position wraps to row[0], weight 0), weight, pos; segment starts
// (position 0 and every position after an EOS) compacted in ascending order by walking the row in tiles of 256
// positions: a ballot per warp, an exclusive prefix over the 8 warps, a running base across tiles.
__global__ void __launch_bounds__(kMetaThreads) k_doc_meta_rows(const int32_t* __restrict__ tokens,
                                                                const uint8_t* __restrict__ row_valid, int S,
                                                                int32_t eos, int max_segs,
                                                                int32_t* __restrict__ targets,
                                                                float* __restrict__ weight, int32_t* __restrict__ pos,
                                                                int32_t* __restrict__ row_seg_start,
                                                                uint32_t* __restrict__ overflow) {
  __shared__ int warp_cnt[kMetaThreads / 32];
  const int r = blockIdx.x;
  const int64_t base = int64_t(r) * S;
  const int32_t* row = tokens + base;
  const float wv = (row_valid == nullptr || row_valid[r]) ? 1.f : 0.f;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int32_t* rs = row_seg_start + int64_t(r) * (max_segs + 1);
  int seg_base = 0;
  for (int p0 = 0; p0 < S; p0 += kMetaThreads) {
    const int p = p0 + threadIdx.x;
    bool start = false;
    if (p < S) {
      targets[base + p] = p + 1 < S ? row[p + 1] : row[0];
      weight[base + p] = p + 1 < S ? wv : 0.f;
      pos[base + p] = p;
      start = p == 0 || row[p - 1] == eos;
    }
    const unsigned m = __ballot_sync(0xffffffffu, start);
    if (lane == 0) warp_cnt[warp] = __popc(m);
    __syncthreads();
    int before = seg_base, total = 0;
#pragma unroll
    for (int w = 0; w < kMetaThreads / 32; ++w) {
      if (w < warp) before += warp_cnt[w];
      total += warp_cnt[w];
    }
    if (start) {
      const int idx = before + __popc(m & ((1u << lane) - 1u));
      if (idx < max_segs) rs[idx] = p;
    }
    seg_base += total;
    __syncthreads();
  }
  if (seg_base > max_segs && threadIdx.x == 0) *overflow = 1u;
  for (int i = min(seg_base, max_segs) + threadIdx.x; i <= max_segs; i += kMetaThreads) rs[i] = S;
}

// One CTA of 1024 threads: per-row segment counts, an exclusive scan over the rows (each thread scans a contiguous
// run of rows, then the runs are scanned through shared memory), the packed cu_seqlens (row offset r S + start), the
// segment count; entries past the count hold the total token count.
__global__ void __launch_bounds__(1024) k_doc_meta_pack(const int32_t* __restrict__ row_seg_start, int rows, int S,
                                                        int max_segs, int32_t* __restrict__ cu_seqlens,
                                                        int32_t* __restrict__ n_segments) {
  __shared__ int run_sum[1024];
  const int per = (rows + 1023) / 1024;
  const int r0 = min(rows, int(threadIdx.x) * per), r1 = min(rows, r0 + per);
  int mine = 0;
  for (int r = r0; r < r1; ++r) {
    const int32_t* rs = row_seg_start + int64_t(r) * (max_segs + 1);
    int c = 0;
    while (c < max_segs && rs[c] < S) ++c;
    mine += c;
  }
  run_sum[threadIdx.x] = mine;
  __syncthreads();
  // Hillis-Steele inclusive scan over the 1024 run sums (integers: order does not matter)
  for (int o = 1; o < 1024; o <<= 1) {
    const int v = int(threadIdx.x) >= o ? run_sum[threadIdx.x - o] : 0;
    __syncthreads();
    run_sum[threadIdx.x] += v;
    __syncthreads();
  }
  const int total = run_sum[1023];
  int off = run_sum[threadIdx.x] - mine;
  for (int r = r0; r < r1; ++r) {
    const int32_t* rs = row_seg_start + int64_t(r) * (max_segs + 1);
    for (int c = 0; c < max_segs && rs[c] < S; ++c) cu_seqlens[off++] = r * S + rs[c];
  }
  if (threadIdx.x == 0) *n_segments = total;
  const int32_t T = rows * S;
  for (int i = total + threadIdx.x; i <= rows * max_segs; i += 1024) cu_seqlens[i] = T;
}

// out[0] = sum(x[0..n)): 1024 thread-strided sequential f32 sums, then a binary tree (the order of the per-chunk loss
// reduction, ce_rows.cu).
__global__ void __launch_bounds__(1024) k_sum_fixed(const float* __restrict__ x, int64_t n, float* __restrict__ out) {
  __shared__ float red[1024];
  float s = 0.f;
  for (int64_t i = threadIdx.x; i < n; i += 1024) s = __fadd_rn(s, x[i]);
  red[threadIdx.x] = s;
  __syncthreads();
  for (int o = 512; o > 0; o >>= 1) {
    if (int(threadIdx.x) < o) red[threadIdx.x] = __fadd_rn(red[threadIdx.x], red[threadIdx.x + o]);
    __syncthreads();
  }
  if (threadIdx.x == 0) out[0] = red[0];
}

// out[col] (+)= sum over the nb partial rows: 8 row groups, group q sums rows [q nb / 8, (q + 1) nb / 8) in ascending
// order, then the 8 group sums are added in ascending q; optional bf16 rounding of the reduced value.
__global__ void __launch_bounds__(256) k_reduce_rows(const float* __restrict__ partial, int nb, int width,
                                                     float* __restrict__ out, bool accumulate, bool round_bf16) {
  __shared__ float sm[8][33];
  const int cx = threadIdx.x & 31, q = threadIdx.x >> 5;
  const int col = blockIdx.x * 32 + cx;
  const int b0 = int(int64_t(q) * nb / 8), b1 = int(int64_t(q + 1) * nb / 8);
  float s = 0.f;
  if (col < width)
    for (int b = b0; b < b1; ++b) s = __fadd_rn(s, partial[int64_t(b) * width + col]);
  sm[q][cx] = s;
  __syncthreads();
  if (q == 0 && col < width) {
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) t = __fadd_rn(t, sm[i][cx]);
    if (round_bf16) t = __bfloat162float(__float2bfloat16_rn(t));
    out[col] = accumulate ? __fadd_rn(out[col], t) : t;
  }
}

}  // namespace

void doc_meta(const int32_t* tokens, const uint8_t* row_valid, int rows, int S, int32_t eos, int max_segs,
              int32_t* targets, float* weight, int32_t* pos, int32_t* cu_seqlens, int32_t* n_segs,
              int32_t* row_seg_start, uint32_t* overflow, cudaStream_t st) {
  NM_REQUIRE(rows > 0 && S > 0 && max_segs > 0, "doc_meta: rows, S and max_segs_per_seq must be > 0");
  NM_REQUIRE(int64_t(rows) * S < (int64_t(1) << 31), "doc_meta: rows * S must fit int32 (cu_seqlens)");
  NM_REQUIRE(tokens && targets && weight && pos && cu_seqlens && n_segs && row_seg_start && overflow,
             "doc_meta: missing output");
  NM_REQUIRE(rows <= 16384, "doc_meta: at most 16384 rows per call");
  k_doc_meta_rows<<<rows, kMetaThreads, 0, st>>>(tokens, row_valid, S, eos, max_segs, targets, weight, pos,
                                                 row_seg_start, overflow);
  NM_CUDA(cudaGetLastError());
  k_doc_meta_pack<<<1, 1024, 0, st>>>(row_seg_start, rows, S, max_segs, cu_seqlens, n_segs);
  NM_CUDA(cudaGetLastError());
}

uint32_t* row_status_word() {
  const int dev = current_device_info().ordinal;
  std::lock_guard<std::mutex> lk(g_row_status_mu);
  if (!g_row_status_ptr[dev]) {
    void* p = nullptr;
    NM_CUDA(cudaGetSymbolAddress(&p, g_row_status_word));
    g_row_status_ptr[dev] = static_cast<uint32_t*>(p);
  }
  return g_row_status_ptr[dev];
}

uint32_t read_row_status(cudaStream_t st) {
  uint32_t word = 0;
  uint32_t* dev = row_status_word();
  NM_CUDA(cudaMemcpyAsync(&word, dev, sizeof(word), cudaMemcpyDeviceToHost, st));
  NM_CUDA(cudaStreamSynchronize(st));
  if (word != 0) NM_CUDA(cudaMemsetAsync(dev, 0, sizeof(word), st));
  return word;
}

void sum_fixed(const float* x, int64_t n, float* out, cudaStream_t st) {
  NM_REQUIRE(out && (x || n == 0) && n >= 0, "sum_fixed: x, out, n >= 0");
  k_sum_fixed<<<1, 1024, 0, st>>>(x, n, out);
  NM_CUDA(cudaGetLastError());
}

void reduce_partials_rows(const float* partial, int n_blocks, int width, float* out, bool accumulate, bool round_bf16,
                          cudaStream_t st) {
  NM_REQUIRE(partial && out && n_blocks >= 0 && width > 0, "reduce_partials_rows: partial, out, width > 0");
  k_reduce_rows<<<(width + 31) / 32, 256, 0, st>>>(partial, n_blocks, width, out, accumulate, round_bf16);
  NM_CUDA(cudaGetLastError());
}

}  // namespace nm::ew
