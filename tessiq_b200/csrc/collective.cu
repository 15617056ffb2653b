// Global reductions over the GPUs of one box: the per-GPU partial, the exchange, the finish.
//
// A reduction over every element of a tensor that is split over several GPUs is three steps per
// GPU, all on one stream and all behind this ABI: tq_reduce_partial_launch reduces the local part to
// a two-float partial, tq_allreduce_scalar combines the partials of all GPUs (NCCL over NVLink), and
// tq_reduce_finish_launch turns the combined partial into the result in the tensor's type. The
// partial of a sum is {sum in f32, 0}; the partial of a maximum is {maximum with a NaN replaced by
// -inf, 1 if a NaN was seen} and both words are combined with MAX (a minimum: {.., -1 if NaN} with
// MIN), because a collective's maximum does not promise to propagate NaN.
//
// NCCL is opened at run time (dlopen of libnccl.so.2: the copy the process already has, PyTorch's,
// or the system's), so the library has no link dependency on it and loads without it; only the
// tq_comm_* and tq_allreduce_scalar calls need it. One process per GPU makes its communicator with
// tq_comm_unique_id (one rank) + tq_comm_create (every rank, the id passed around by the host's own
// means); a single process that drives several GPUs makes them all with tq_comm_create_all.
//
// The reference has no multi-GPU execution (one target device per recipe,
// python/tessiq/recipe.py:117-161); this is what its recipes would shard under.
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>
#include <vector>

#include "common.h"
#include "reducers.h"

struct tq_comm {
  ncclComm_t comm;
  int32_t rank, world, device;
};

namespace tq {
namespace {

struct Nccl {
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

const Nccl& nccl() {
  static Nccl table = [] {
    Nccl t;
    void* handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
    if (handle == nullptr) handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (handle == nullptr) handle = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (handle == nullptr) return t;
    auto find = [&](const char* name, auto& slot) {
      slot = reinterpret_cast<std::remove_reference_t<decltype(slot)>>(dlsym(handle, name));
      return slot != nullptr;
    };
    t.ok = find("ncclGetUniqueId", t.GetUniqueId) & find("ncclCommInitRank", t.CommInitRank) & find("ncclCommInitAll", t.CommInitAll) &
           find("ncclCommDestroy", t.CommDestroy) & find("ncclAllReduce", t.AllReduce) & find("ncclGetErrorString", t.GetErrorString);
    return t;
  }();
  return table;
}

#define TQ_NCCL(call)                                                                                         \
  do {                                                                                                        \
    ncclResult_t tq_nccl_status_ = (call);                                                                    \
    if (tq_nccl_status_ != ncclSuccess) {                                                                     \
      return ::tq::fail(TQ_EXTERNAL, "%s failed: %s", #call, ::tq::nccl().GetErrorString(tq_nccl_status_));   \
    }                                                                                                         \
  } while (0)

// partial[0..1] -> out, in the tensor's type. sum: partial[0]; mean: partial[0] / count; amax / amin:
// NaN when the flag word is not zero, else partial[0].
template <typename T>
__global__ void reduce_finish_kernel(int op, const float* __restrict__ partial, T* __restrict__ out, double count) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float value = partial[0];
  if (op == TQ_MEAN) value = static_cast<float>(static_cast<double>(value) / count);
  if ((op == TQ_AMAX || op == TQ_AMIN) && partial[1] != 0.f) value = __int_as_float(0x7fc00000);
  out[0] = from_compute<T, float>(value);
}

}  // namespace
}  // namespace tq

extern "C" {

tq_status tq_comm_unique_id(void* id, size_t bytes) {
  TQ_REQUIRE(id != nullptr && bytes >= sizeof(ncclUniqueId), TQ_INVALID_ARGUMENT, "the id buffer must hold %zu bytes", sizeof(ncclUniqueId));
  TQ_REQUIRE(tq::nccl().ok, TQ_NOT_FOUND, "NCCL (libnccl.so.2) is not available in this process");
  TQ_NCCL(tq::nccl().GetUniqueId(static_cast<ncclUniqueId*>(id)));
  return TQ_OK;
}

tq_status tq_comm_create(const void* id, size_t bytes, int32_t rank, int32_t world, int32_t device, tq_comm** comm) {
  TQ_REQUIRE(comm != nullptr, TQ_INVALID_ARGUMENT, "comm out-pointer is null");
  TQ_REQUIRE(id != nullptr && bytes >= sizeof(ncclUniqueId), TQ_INVALID_ARGUMENT, "the id buffer must hold %zu bytes", sizeof(ncclUniqueId));
  TQ_REQUIRE(world >= 1 && rank >= 0 && rank < world, TQ_INVALID_ARGUMENT, "rank %d is not in a world of %d", rank, world);
  TQ_REQUIRE(tq::nccl().ok, TQ_NOT_FOUND, "NCCL (libnccl.so.2) is not available in this process");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  ncclUniqueId unique;
  memcpy(&unique, id, sizeof(unique));
  ncclComm_t made = nullptr;
  TQ_NCCL(tq::nccl().CommInitRank(&made, world, unique, rank));
  *comm = new tq_comm{made, rank, world, device};
  return TQ_OK;
}

tq_status tq_comm_create_all(const int32_t* devices, int32_t count, tq_comm** comms) {
  TQ_REQUIRE(devices != nullptr && comms != nullptr && count >= 1 && count <= 64, TQ_INVALID_ARGUMENT, "1 to 64 devices and as many comm slots");
  TQ_REQUIRE(tq::nccl().ok, TQ_NOT_FOUND, "NCCL (libnccl.so.2) is not available in this process");
  std::vector<int> list(devices, devices + count);
  std::vector<ncclComm_t> made(count, nullptr);
  TQ_NCCL(tq::nccl().CommInitAll(made.data(), count, list.data()));
  for (int i = 0; i < count; ++i) comms[i] = new tq_comm{made[i], i, count, devices[i]};
  return TQ_OK;
}

tq_status tq_comm_destroy(tq_comm* comm) {
  if (comm == nullptr) return TQ_OK;
  ncclComm_t held = comm->comm;
  delete comm;
  if (held != nullptr && tq::nccl().ok) TQ_NCCL(tq::nccl().CommDestroy(held));
  return TQ_OK;
}

int32_t tq_comm_rank(const tq_comm* comm) { return comm ? comm->rank : -1; }
int32_t tq_comm_world(const tq_comm* comm) { return comm ? comm->world : 0; }

tq_status tq_allreduce_scalar(tq_comm* comm, void* buffer, int64_t count, tq_dtype dtype, tq_reduce_op op, int32_t device, void* stream) {
  TQ_REQUIRE(comm != nullptr && comm->comm != nullptr, TQ_INVALID_ARGUMENT, "null communicator");
  TQ_REQUIRE(buffer != nullptr && count >= 0, TQ_INVALID_ARGUMENT, "null buffer or negative count");
  TQ_REQUIRE(device == comm->device, TQ_INVALID_ARGUMENT, "the communicator was made for device %d, not %d", comm->device, device);
  if (count == 0) return TQ_OK;
  ncclDataType_t type;
  switch (dtype) {
    case TQ_F32: type = ncclFloat32; break;
    case TQ_F64: type = ncclFloat64; break;
    case TQ_F16: type = ncclFloat16; break;
    case TQ_BF16: type = ncclBfloat16; break;
    case TQ_I32: type = ncclInt32; break;
    case TQ_I64: type = ncclInt64; break;
    default: return tq::fail(TQ_UNSUPPORTED, "no all-reduce for element type %s", tq::dtype_name(dtype));
  }
  ncclRedOp_t how;
  switch (op) {
    case TQ_SUM: how = ncclSum; break;
    case TQ_AMAX: how = ncclMax; break;
    case TQ_AMIN: how = ncclMin; break;
    default: return tq::fail(TQ_UNSUPPORTED, "an all-reduce sums, takes the maximum or the minimum; not operation %d", op);
  }
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  TQ_NCCL(tq::nccl().AllReduce(buffer, buffer, static_cast<size_t>(count), type, how, comm->comm, static_cast<cudaStream_t>(stream)));
  return TQ_OK;
}

tq_status tq_reduce_finish_launch(tq_reduce_op op, tq_dtype dtype, const void* partial, void* out, int64_t total_count, int32_t device,
                                  void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) { return tq_reduce_finish_launch(op, dtype, partial, out, total_count, d, s); });
  TQ_REQUIRE(op == TQ_SUM || op == TQ_MEAN || op == TQ_AMAX || op == TQ_AMIN, TQ_UNSUPPORTED, "no global finish for operation %d", op);
  TQ_REQUIRE(partial != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null partial or output");
  TQ_REQUIRE(op != TQ_MEAN || total_count > 0, TQ_INVALID_ARGUMENT, "a mean over no elements");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  const float* words = static_cast<const float*>(partial);
  const double count = static_cast<double>(total_count);
  switch (dtype) {
    case TQ_F32: tq::reduce_finish_kernel<float><<<1, 32, 0, cuda_stream>>>(op, words, static_cast<float*>(out), count); break;
    case TQ_F16: tq::reduce_finish_kernel<__half><<<1, 32, 0, cuda_stream>>>(op, words, static_cast<__half*>(out), count); break;
    case TQ_BF16: tq::reduce_finish_kernel<__nv_bfloat16><<<1, 32, 0, cuda_stream>>>(op, words, static_cast<__nv_bfloat16*>(out), count); break;
    default: return tq::fail(TQ_UNSUPPORTED, "the two-float partial serves f32, f16 and bf16 tensors, not %s", tq::dtype_name(dtype));
  }
  return tq::check_launch("reduce_finish_kernel");
}

}  // extern "C"
