// NCCL communicator and the bucketed dW reducer (include/marincpp/comm.hpp). NCCL is resolved at run time from the
// libnccl.so.2 already loaded in the process (the one torch.distributed uses) or, failing that, the system one, so the
// library carries no link-time dependency on a particular NCCL build.
#include "marincpp/comm.hpp"

#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>
#include <nvtx3/nvToolsExt.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>

#include "ce_internal.hpp"

namespace nm {
namespace {

struct NcclApi {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;   // optional
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
  ncclResult_t (*GroupStart)() = nullptr;
  ncclResult_t (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  std::string error;
};

const NcclApi& nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) {
      api.error = std::string("libnccl.so.2 could not be loaded: ") + dlerror();
      return;
    }
    auto sym = [&](const char* name) -> void* {
      void* p = dlsym(h, name);
      if (!p && api.error.empty()) api.error = std::string("libnccl.so.2 lacks ") + name;
      return p;
    };
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(sym("ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(sym("ncclCommInitRank"));
    api.CommInitRankConfig =
        reinterpret_cast<decltype(api.CommInitRankConfig)>(dlsym(h, "ncclCommInitRankConfig"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(sym("ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(sym("ncclAllReduce"));
    api.ReduceScatter = reinterpret_cast<decltype(api.ReduceScatter)>(sym("ncclReduceScatter"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(sym("ncclAllGather"));
    api.GroupStart = reinterpret_cast<decltype(api.GroupStart)>(sym("ncclGroupStart"));
    api.GroupEnd = reinterpret_cast<decltype(api.GroupEnd)>(sym("ncclGroupEnd"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(sym("ncclGetErrorString"));
  });
  if (!api.error.empty()) throw DeviceError("comm: " + api.error);
  return api;
}

}  // namespace

int comm_sms() {
  static const int v = [] {
    const char* e = std::getenv("NM_COMM_SMS");
    if (!e || !*e) return kCommSms;
    const int n = std::atoi(e);
    return n < 4 ? 4 : (n > 64 ? 64 : n);
  }();
  return v;
}

void nccl_check(int err, const char* expr, const char* where) {
  if (err == 0) return;
  const char* s = nccl().GetErrorString ? nccl().GetErrorString(static_cast<ncclResult_t>(err)) : "?";
  throw DeviceError(std::string(where) + ": " + expr + " failed: NCCL error " + std::to_string(err) + " (" + s + ")");
}

static_assert(sizeof(ncclUniqueId) == 128, "the C ABI passes the NCCL unique id as 128 bytes");

void Comm::unique_id(void* id128_host) {
  NM_REQUIRE(id128_host, "comm: id buffer required");
  ncclUniqueId id;
  NM_NCCL(nccl().GetUniqueId(&id));
  std::memcpy(id128_host, &id, sizeof(id));
}

Comm::Comm(const void* id128_host, int nranks, int rank) : nranks_(nranks), rank_(rank) {
  NM_REQUIRE(id128_host, "comm: id required");
  NM_REQUIRE(nranks >= 1 && nranks <= kMaxGpus && rank >= 0 && rank < nranks, "comm: 1 <= nranks <= 8, 0 <= rank < nranks");
  NM_CUDA(cudaGetDevice(&device_));
  ncclUniqueId id;
  std::memcpy(&id, id128_host, sizeof(id));
  ncclComm_t c = nullptr;
  if (nccl().CommInitRankConfig) {
    // the collectives of this communicator run beside the persistent tcgen05 kernels, which leave kCommSms SMs free
    // while a reduction is in flight: cap NCCL at that many CTAs
    ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
    cfg.maxCTAs = comm_sms();
    NM_NCCL(nccl().CommInitRankConfig(&c, nranks, id, rank, &cfg));
  } else {
    NM_NCCL(nccl().CommInitRank(&c, nranks, id, rank));
  }
  comm_ = c;
  NM_CUDA(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
}

Comm::~Comm() {
  if (stream_) cudaStreamDestroy(stream_);
  if (comm_) nccl().CommDestroy(static_cast<ncclComm_t>(comm_));
}

namespace {
ncclDataType_t nccl_type(DType dt) {
  NM_REQUIRE(dt == DType::f32 || dt == DType::bf16 || dt == DType::f64, "comm: f32, bf16 or f64 elements");
  return dt == DType::f32 ? ncclFloat32 : (dt == DType::bf16 ? ncclBfloat16 : ncclFloat64);
}
}  // namespace

void Comm::allreduce_sum(void* buf, int64_t n, DType dt, cudaStream_t st) {
  if (n <= 0) return;
  NM_NCCL(nccl().AllReduce(buf, buf, size_t(n), nccl_type(dt), ncclSum, static_cast<ncclComm_t>(comm_), st));
}

void Comm::reduce_scatter_sum_f32(float* buf, int64_t count, cudaStream_t st) {
  if (count <= 0) return;
  NM_NCCL(nccl().ReduceScatter(buf, buf + int64_t(rank_) * count, size_t(count), ncclFloat32, ncclSum,
                               static_cast<ncclComm_t>(comm_), st));
}

void Comm::allgather(void* buf, int64_t count, DType dt, cudaStream_t st) {
  if (count <= 0) return;
  const char* base = static_cast<const char*>(buf);
  NM_NCCL(nccl().AllGather(base + int64_t(rank_) * count * int64_t(dtype_size(dt)), buf, size_t(count), nccl_type(dt),
                           static_cast<ncclComm_t>(comm_), st));
}

void Comm::group_start() { NM_NCCL(nccl().GroupStart()); }
void Comm::group_end() { NM_NCCL(nccl().GroupEnd()); }

int grad_bucket_ranges(int V, int n_buckets, std::vector<int>& v0, std::vector<int>& v1) {
  NM_REQUIRE(V > 0, "grad reducer: V > 0");
  NM_REQUIRE(n_buckets >= 1 && n_buckets <= 64, "grad reducer: 1 <= n_buckets <= 64");
  const int tiles = (V + ce::kTileM - 1) / ce::kTileM;
  const int nb = n_buckets < tiles ? n_buckets : tiles;
  v0.clear();
  v1.clear();
  int t0 = 0;
  for (int b = 0; b < nb; ++b) {
    const int t1 = t0 + (tiles - t0) / (nb - b);
    v0.push_back(t0 * ce::kTileM);
    v1.push_back(t1 * ce::kTileM < V ? t1 * ce::kTileM : V);
    t0 = t1;
  }
  v1.back() = V;
  return nb;
}

GradReducer::GradReducer(Comm& comm, float* grad, int V, int D, int n_buckets, DType reduce_dtype, void* staging,
                         bool to_owners)
    : comm_(comm), grad_(grad), V_(V), D_(D), dtype_(reduce_dtype), staging_(staging), to_owners_(to_owners) {
  NM_REQUIRE(grad && V > 0 && D > 0, "grad reducer: grad, V, D required");
  NM_REQUIRE(reduce_dtype == DType::f32 || (reduce_dtype == DType::bf16 && staging),
             "grad reducer: reduce dtype f32, or bf16 with a staging buffer");
  NM_REQUIRE(!to_owners || reduce_dtype == DType::f32, "grad reducer: the reduction to owners is f32");
  grad_bucket_ranges(V, n_buckets, v0_, v1_);
  if (to_owners)
    for (size_t b = 0; b < v0_.size(); ++b)
      NM_REQUIRE((int64_t(v1_[b] - v0_[b]) * D) % comm.nranks() == 0,
                 "grad reducer: with a reduction to owners every bucket's element count must divide by the rank count");
  ready_.resize(v0_.size());
  for (auto& e : ready_) NM_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
  NM_CUDA(cudaEventCreateWithFlags(&done_, cudaEventDisableTiming));
  NM_CUDA(cudaEventRecord(done_, comm_.stream()));
}

GradReducer::~GradReducer() {
  for (auto e : ready_) if (e) cudaEventDestroy(e);
  if (done_) cudaEventDestroy(done_);
}

void GradReducer::bucket_ready(int b, cudaStream_t compute) {
  NM_REQUIRE(b >= 0 && b < n_buckets(), "grad reducer: bucket index");
  cudaStream_t cs = comm_.stream();
  nvtxRangePushA(to_owners_ ? "ce.dw_bucket_reduce_scatter" : "ce.dw_bucket_allreduce");
  struct Pop { ~Pop() { nvtxRangePop(); } } pop;
  NM_CUDA(cudaEventRecord(ready_[b], compute));
  NM_CUDA(cudaStreamWaitEvent(cs, ready_[b], 0));
  float* g = grad_ + int64_t(v0_[b]) * D_;
  const int64_t n = int64_t(v1_[b] - v0_[b]) * D_;
  if (to_owners_) {
    comm_.reduce_scatter_sum_f32(g, n / comm_.nranks(), cs);
  } else if (dtype_ == DType::f32) {
    comm_.allreduce_sum(g, n, DType::f32, cs);
  } else {
    uint16_t* s = static_cast<uint16_t*>(staging_) + int64_t(v0_[b]) * D_;
    ce::launch_f32_to_bf16(g, s, n, cs);
    comm_.allreduce_sum(s, n, DType::bf16, cs);
    ce::launch_bf16_to_f32(s, g, n, cs);
  }
  NM_CUDA(cudaEventRecord(done_, cs));
}

void GradReducer::owned_range(int b, int64_t& offset, int64_t& len) const {
  NM_REQUIRE(b >= 0 && b < n_buckets(), "grad reducer: bucket index");
  const int64_t n = int64_t(v1_[b] - v0_[b]) * D_;
  len = to_owners_ ? n / comm_.nranks() : n;
  offset = int64_t(v0_[b]) * D_ + (to_owners_ ? int64_t(comm_.rank()) * len : 0);
}

void GradReducer::reduce_all(cudaStream_t compute) {
  for (int b = 0; b < n_buckets(); ++b) bucket_ready(b, compute);
}

void GradReducer::wait(cudaStream_t st) { NM_CUDA(cudaStreamWaitEvent(st, done_, 0)); }

int64_t GradReducer::owned_elems() const {
  int64_t total = 0;
  for (int b = 0; b < n_buckets(); ++b) {
    int64_t off, len;
    owned_range(b, off, len);
    total += len;
  }
  return total;
}

void GradReducer::microbatch_done(float* owned_acc, cudaStream_t st) {
  NM_REQUIRE(to_owners_, "grad reducer: microbatch_done goes with a reduction to owners");
  NM_REQUIRE(owned_acc != nullptr, "grad reducer: owned_acc required");
  wait(st);
  int64_t at = 0;
  for (int b = 0; b < n_buckets(); ++b) {
    int64_t off, len;
    owned_range(b, off, len);
    ce::launch_add_f32(owned_acc + at, grad_ + off, len, st);
    at += len;
  }
  NM_CUDA(cudaMemsetAsync(grad_, 0, size_t(V_) * size_t(D_) * sizeof(float), st));
  // the next microbatch's bucket reductions are enqueued behind events recorded on the compute stream after this
}

void GradReducer::owned_to_grad(const float* owned_acc, cudaStream_t st) {
  NM_REQUIRE(to_owners_, "grad reducer: owned_to_grad goes with a reduction to owners");
  NM_REQUIRE(owned_acc != nullptr, "grad reducer: owned_acc required");
  int64_t at = 0;
  for (int b = 0; b < n_buckets(); ++b) {
    int64_t off, len;
    owned_range(b, off, len);
    NM_CUDA(cudaMemcpyAsync(grad_ + off, owned_acc + at, size_t(len) * sizeof(float), cudaMemcpyDeviceToDevice, st));
    at += len;
  }
}

}  // namespace nm
