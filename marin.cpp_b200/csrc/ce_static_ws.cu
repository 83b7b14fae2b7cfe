// nm_ce_forward_noalloc: the forward (statistics + loss) half of the fused linear cross-entropy for callers that cannot
// supply or allocate a workspace. Its scratch (per-tile softmax partials, lse and per-row factors of one chunk) lives
// in a file-scope device array of fixed size that every GPU using this library holds from load to exit.
//
// Who needs this: code that runs where device allocation is off limits. Two cases seen with this library's host: (1) a
// trainer that makes one arena allocation up front and plans every buffer in it (the design of the reference's memory
// plan) has no spare region to hand to an evaluation or probe call that was not in the plan; (2) while any thread of
// the process has a stream capture open in the global or thread-local capture mode, cudaMalloc / cudaFree are not
// permitted, so a helper thread that wants a quick loss read-out cannot size and allocate a workspace on the spot.
//
// Rules of use:
//   * The first call on a device looks up the device address of the array (cudaGetSymbolAddress, with that device
//     current) and caches it; make that first call before any stream capture begins.
//   * All calls on a device share the one array and it keeps whatever the previous call left. The only word that must
//     start at zero, the wait-status word, is cleared on the stream at the start of every call; everything else is
//     written before it is read within a call.
//   * Two calls whose kernels may overlap on the same GPU (different streams, or different host threads) race on the
//     array. Serialise them.
//   * The scratch needed is 256 + 8 ceil(V / 256) chunk_rows + 12 chunk_rows bytes (each region rounded up to 256);
//     a call that needs more than kScratchBytes (16 MiB) is refused with NM_ERR_INVALID. At V = 128256 that allows
//     chunk_rows up to 4096.
// The entry point makes no allocation of any kind: no cudaMalloc / cudaFree, no allocating library call.
#include <cuda_runtime.h>

#include <mutex>
#include <string>

#include "capi_util.hpp"
#include "ce_internal.hpp"
#include "marincpp/capi_ce.h"

namespace nm::ce {
namespace {

constexpr size_t kScratchBytes = size_t(16) << 20;
static __device__ __align__(256) unsigned char g_ce_static_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_scratch_mu;
void* g_scratch_ptr[kMaxDevices] = {};

// The array's name is only a host-side handle; kernels need its device address, which differs per device.
void* scratch_of_current_device() {
  int dev = 0;
  NM_CUDA(cudaGetDevice(&dev));
  NM_REQUIRE(dev >= 0 && dev < kMaxDevices, "nm_ce_forward_noalloc: device index out of range");
  std::lock_guard<std::mutex> lk(g_scratch_mu);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    NM_CUDA(cudaGetSymbolAddress(&p, g_ce_static_scratch));
    NM_REQUIRE(p && reinterpret_cast<uintptr_t>(p) % 256 == 0, "nm_ce_forward_noalloc: scratch address not aligned");
    g_scratch_ptr[dev] = p;
  }
  return g_scratch_ptr[dev];
}

struct FwdScratch {
  uint32_t* status; float* tmax; float* tsum; float* lse; float* rowa; float* rowb;
  int NT; uint64_t bytes;
};

FwdScratch carve_fwd(int V, int chunk_rows, void* base) {
  FwdScratch w{};
  uint64_t off = 0;
  auto take = [&](uint64_t bytes) -> void* {
    off = uint64_t(round_up(int64_t(off), 256));
    void* p = base ? static_cast<uint8_t*>(base) + off : nullptr;
    off += bytes;
    return p;
  };
  w.NT = stats_tiles(V);
  w.status = static_cast<uint32_t*>(take(256));
  w.tmax = static_cast<float*>(take(uint64_t(w.NT) * chunk_rows * 4));
  w.tsum = static_cast<float*>(take(uint64_t(w.NT) * chunk_rows * 4));
  w.lse = static_cast<float*>(take(uint64_t(chunk_rows) * 4));
  w.rowa = static_cast<float*>(take(uint64_t(chunk_rows) * 4));
  w.rowb = static_cast<float*>(take(uint64_t(chunk_rows) * 4));
  w.bytes = uint64_t(round_up(int64_t(off), 256));
  return w;
}

void forward_noalloc(const void* x, const void* w, const int32_t* targets, const float* weight, float* loss_tok,
                     float* lse, float* loss_partial, int64_t T, int D, int V, int chunk_rows, float z_loss,
                     int32_t ignore_index, cudaStream_t st) {
  NM_REQUIRE(T >= 0 && D > 0 && V > 0, "nm_ce_forward_noalloc: T >= 0, D > 0, V > 0");
  NM_REQUIRE(D % 8 == 0, "nm_ce_forward_noalloc: D must be a multiple of 8");
  NM_REQUIRE(chunk_rows > 0, "nm_ce_forward_noalloc: chunk_rows must be positive");
  if (T == 0) return;
  NM_REQUIRE(x && w && targets && weight && loss_tok, "nm_ce_forward_noalloc: x, w, targets, weight and loss_tok are "
                                                      "required");
  const uint64_t need = carve_fwd(V, chunk_rows, nullptr).bytes;
  NM_REQUIRE(need <= kScratchBytes,
             "nm_ce_forward_noalloc: V = " + std::to_string(V) + " with chunk_rows = " + std::to_string(chunk_rows) +
                 " needs " + std::to_string(need) + " bytes of scratch, more than the built-in " +
                 std::to_string(kScratchBytes) + "; use a smaller chunk_rows, or nm_fused_linear_ce with a workspace");
  NM_REQUIRE(device_arch() >= 100, "nm_ce_forward_noalloc: sm_100a kernels only");
  const FwdScratch s = carve_fwd(V, chunk_rows, scratch_of_current_device());
  NM_CUDA(cudaMemsetAsync(s.status, 0, 4, st));   // the one word that must start at zero
  const int64_t n_chunks = (T + chunk_rows - 1) / chunk_rows;
  for (int64_t c = 0; c < n_chunks; ++c) {
    const int64_t r0 = c * chunk_rows;
    const int n = int(T - r0 < chunk_rows ? T - r0 : chunk_rows);
    const void* x_c = static_cast<const uint8_t*>(x) + r0 * D * 2;
    float* loss_c = loss_tok + r0;
    float* lse_c = lse ? lse + r0 : s.lse;
    LogitsArgs la{x_c, w, nullptr, targets + r0, n, D, V, nullptr, store_ld(V), false, s.tmax, s.tsum, chunk_rows,
                  loss_c, s.status};
    launch_logits(la, st);
    FinalizeArgs fa{s.tmax, s.tsum, chunk_rows, s.NT, loss_c, targets + r0, weight + r0, n, V, z_loss, ignore_index,
                    false, lse_c, loss_c, s.rowa, s.rowb};
    launch_finalize(fa, st);
    if (loss_partial) launch_chunk_loss(loss_c, weight + r0, n, loss_partial + c, st);
  }
}

}  // namespace
}  // namespace nm::ce

extern "C" int nm_ce_forward_noalloc(const void* x, const void* w, const int32_t* targets, const float* weight,
                                     float* loss_tok, float* lse, float* loss_partial, int64_t T, int D, int V,
                                     int chunk_rows, float z_loss_weight, int32_t ignore_index, void* stream) {
  return nm::capi_call([&] {
    nm::ce::forward_noalloc(x, w, targets, weight, loss_tok, lse, loss_partial, T, D, V, chunk_rows, z_loss_weight,
                            ignore_index, static_cast<cudaStream_t>(stream));
  });
}
