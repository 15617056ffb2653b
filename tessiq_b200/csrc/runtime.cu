// Library-wide state: error slot, device selection, per-GPU streams, the bump arena and the
// device-side status word that bounded waits report through.
#include <atomic>
#include <mutex>
#include <vector>

#include "common.h"
#include "tcgen05.h"

namespace tq {

namespace {
thread_local std::string g_error = "";
std::mutex g_mutex;
constexpr int kMaxDevices = 64;
int g_sm_count[kMaxDevices] = {0};
int32_t* g_status_word[kMaxDevices] = {nullptr};
}  // namespace

void set_error(const char* text) { g_error = text ? text : ""; }

tq_status fail(tq_status code, const char* format, ...) {
  char buffer[1024];
  va_list args;
  va_start(args, format);
  vsnprintf(buffer, sizeof(buffer), format, args);
  va_end(args);
  g_error = buffer;
  return code;
}

tq_status use_device(int32_t device) {
  TQ_REQUIRE(device >= 0 && device < kMaxDevices, TQ_INVALID_ARGUMENT,
             "device ordinal %d is out of range", device);
  int current = -1;
  cudaError_t status = cudaGetDevice(&current);
  if (status != cudaSuccess) {
    return fail(TQ_EXTERNAL, "no usable CUDA device: %s", cudaGetErrorString(status));
  }
  if (current != device) TQ_CUDA(cudaSetDevice(device));
  return TQ_OK;
}

int sm_count(int32_t device) {
  if (device < 0 || device >= kMaxDevices) return 148;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_sm_count[device] == 0) {
    int value = 0;
    if (cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess ||
        value <= 0) {
      value = 148;
    }
    g_sm_count[device] = value;
  }
  return g_sm_count[device];
}

int32_t* device_status_word(int32_t device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_mutex);
  if (g_status_word[device] == nullptr) {
    int32_t* word = nullptr;
    if (cudaMalloc(&word, 256) != cudaSuccess) return nullptr;
    if (cudaMemset(word, 0, 256) != cudaSuccess) return nullptr;
    g_status_word[device] = word;
  }
  return g_status_word[device];
}

WaitStatus wait_status_for(int32_t device) {
  static std::atomic<unsigned> launches{0};
  int32_t* block = device_status_word(device);
  if (block == nullptr) return WaitStatus{nullptr};
  return WaitStatus{block + 8 + launches.fetch_add(1, std::memory_order_relaxed) % 56};
}

}  // namespace tq

namespace tq {
namespace {
constexpr int kStatusSelfTest = 0x53454c46;   // "SELF"

// One warp waits, for at most `polls` looks, on an mbarrier that expects two arrivals and gets one:
// the wait cannot complete. It gives up the way every bounded wait of this library does — the sticky
// code, the launch's abort word — and the kernel returns by itself. A second wait then shows that
// the abort word takes the launch's other waits out at their next look.
__global__ void bounded_wait_selftest_kernel(WaitStatus status, uint32_t polls, int* looks) {
  __shared__ uint64_t barrier;
  const uint32_t bar = smem_address(&barrier);
  if (threadIdx.x == 0) {
    status.begin();
    barrier_init(bar, 2);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    barrier_arrive(bar);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t spin = 0;
    bool done = false;
    for (; spin < polls; ++spin) {
      if (barrier_try_wait(bar, 0)) {
        done = true;
        break;
      }
    }
    if (!done) {
      atomicCAS(status.sticky(), 0, kStatusSelfTest);
      status.set_abort();
    }
    looks[0] = static_cast<int>(spin);
    // the library's own wait now leaves at its first look at the abort word (every 1024 polls)
    const long long before = clock64();
    const bool second = barrier_wait(bar, 0, status, kStatusSelfTest);
    looks[1] = second ? -1 : static_cast<int>((clock64() - before) >> 10);
  }
}
}  // namespace
}  // namespace tq

struct tq_recipe {
  std::vector<tq::Replay> steps;
};

namespace tq {
namespace {
thread_local tq_recipe* g_recording = nullptr;
}
bool recording() { return g_recording != nullptr; }
tq_status record(Replay step) {
  g_recording->steps.push_back(std::move(step));
  return TQ_OK;
}
}  // namespace tq

struct tq_arena {
  int32_t device;
  size_t bytes;
  char* base;
};

// One handle over several GPUs of one process: per GPU a non-blocking stream, an arena slice with a
// bump pointer, and an event for joins.
struct tq_runtime {
  struct Slot {
    int32_t device;
    cudaStream_t stream;
    cudaEvent_t event;
    tq_arena arena;
    size_t used;
  };
  std::vector<Slot> slots;
};

extern "C" {

int32_t tq_abi_version(void) { return 1000; }

const char* tq_last_error(void) { return tq::g_error.c_str(); }

int32_t tq_dtype_size(tq_dtype dtype) { return tq::dtype_size(dtype); }

int32_t tq_device_count(void) {
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  return count;
}

tq_status tq_stream_create(int32_t device, void** stream) {
  TQ_REQUIRE(stream != nullptr, TQ_INVALID_ARGUMENT, "stream out-pointer is null");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  cudaStream_t created = nullptr;
  TQ_CUDA(cudaStreamCreateWithFlags(&created, cudaStreamNonBlocking));
  *stream = created;
  return TQ_OK;
}

tq_status tq_stream_destroy(int32_t device, void* stream) {
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  TQ_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)));
  return TQ_OK;
}

tq_status tq_stream_synchronize(int32_t device, void* stream) {
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  TQ_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
  return TQ_OK;
}

tq_status tq_arena_create(int32_t device, size_t bytes, tq_arena** arena) {
  TQ_REQUIRE(arena != nullptr, TQ_INVALID_ARGUMENT, "arena out-pointer is null");
  TQ_REQUIRE(bytes > 0, TQ_INVALID_ARGUMENT, "an arena of 0 bytes");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  void* base = nullptr;
  cudaError_t status = cudaMalloc(&base, bytes);
  if (status == cudaErrorMemoryAllocation) {
    cudaGetLastError();
    return tq::fail(TQ_RESOURCE_EXHAUSTED, "device %d has no %zu bytes for an arena", device, bytes);
  }
  TQ_CUDA(status);
  *arena = new tq_arena{device, bytes, static_cast<char*>(base)};
  return TQ_OK;
}

tq_status tq_arena_destroy(tq_arena* arena) {
  if (arena == nullptr) return TQ_OK;
  tq::DeviceScope device_scope(arena->device);
  if (tq_status s = device_scope.status()) return s;
  cudaError_t status = cudaFree(arena->base);
  delete arena;
  TQ_CUDA(status);
  return TQ_OK;
}

tq_status tq_arena_at(const tq_arena* arena, size_t offset, size_t bytes, void** pointer) {
  TQ_REQUIRE(arena != nullptr && pointer != nullptr, TQ_INVALID_ARGUMENT, "null arena or pointer");
  TQ_REQUIRE(offset <= arena->bytes && bytes <= arena->bytes - offset, TQ_INVALID_ARGUMENT,
             "range [%zu, %zu) is outside an arena of %zu bytes", offset, offset + bytes,
             arena->bytes);
  *pointer = arena->base + offset;
  return TQ_OK;
}

size_t tq_arena_bytes(const tq_arena* arena) { return arena ? arena->bytes : 0; }

tq_status tq_runtime_create(const int32_t* devices, int32_t count, size_t arena_bytes_per_device, tq_runtime** runtime) {
  TQ_REQUIRE(runtime != nullptr, TQ_INVALID_ARGUMENT, "runtime out-pointer is null");
  TQ_REQUIRE(devices != nullptr && count >= 1 && count <= 64, TQ_INVALID_ARGUMENT, "between 1 and 64 devices");
  const int32_t visible = tq_device_count();
  for (int i = 0; i < count; ++i) {
    TQ_REQUIRE(devices[i] >= 0 && devices[i] < visible, TQ_INVALID_ARGUMENT, "device %d is not one of the %d visible GPUs", devices[i], visible);
    for (int j = 0; j < i; ++j) TQ_REQUIRE(devices[j] != devices[i], TQ_INVALID_ARGUMENT, "device %d is listed twice", devices[i]);
  }
  tq::DeviceScope restore(devices[0]);   // the loop below moves from GPU to GPU: the caller's device comes back at the end
  tq_runtime* made = new tq_runtime();
  for (int i = 0; i < count; ++i) {
    tq_runtime::Slot slot = {devices[i], nullptr, nullptr, {devices[i], 0, nullptr}, 0};
    tq_status status = tq::use_device(devices[i]);
    if (status == TQ_OK && cudaStreamCreateWithFlags(&slot.stream, cudaStreamNonBlocking) != cudaSuccess) status = tq::fail(TQ_EXTERNAL, "no stream on device %d", devices[i]);
    if (status == TQ_OK && cudaEventCreateWithFlags(&slot.event, cudaEventDisableTiming) != cudaSuccess) status = tq::fail(TQ_EXTERNAL, "no event on device %d", devices[i]);
    if (status == TQ_OK && arena_bytes_per_device > 0) {
      void* base = nullptr;
      if (cudaMalloc(&base, arena_bytes_per_device) != cudaSuccess) {
        cudaGetLastError();
        status = tq::fail(TQ_RESOURCE_EXHAUSTED, "device %d has no %zu bytes for its arena slice", devices[i], arena_bytes_per_device);
      } else {
        slot.arena.bytes = arena_bytes_per_device;
        slot.arena.base = static_cast<char*>(base);
      }
    }
    made->slots.push_back(slot);
    if (status != TQ_OK) {
      const std::string kept = tq_last_error();
      tq_runtime_destroy(made);
      tq::set_error(kept.c_str());
      return status;
    }
  }
  *runtime = made;
  return TQ_OK;
}

tq_status tq_runtime_destroy(tq_runtime* runtime) {
  if (runtime == nullptr) return TQ_OK;
  tq::DeviceScope restore(runtime->slots.empty() ? 0 : runtime->slots[0].device);
  for (tq_runtime::Slot& slot : runtime->slots) {
    if (tq::use_device(slot.device) != TQ_OK) continue;
    if (slot.stream != nullptr) {
      cudaStreamSynchronize(slot.stream);
      cudaStreamDestroy(slot.stream);
    }
    if (slot.event != nullptr) cudaEventDestroy(slot.event);
    if (slot.arena.base != nullptr) cudaFree(slot.arena.base);
  }
  delete runtime;
  return TQ_OK;
}

int32_t tq_runtime_device_count(const tq_runtime* runtime) { return runtime ? static_cast<int32_t>(runtime->slots.size()) : 0; }

#define TQ_SLOT(runtime, index)                                                                                       \
  TQ_REQUIRE((runtime) != nullptr && (index) >= 0 && (index) < static_cast<int32_t>((runtime)->slots.size()), TQ_INVALID_ARGUMENT, \
             "slot %d is not one of the runtime's devices", static_cast<int>(index))

tq_status tq_runtime_device(const tq_runtime* runtime, int32_t index, int32_t* device) {
  TQ_SLOT(runtime, index);
  TQ_REQUIRE(device != nullptr, TQ_INVALID_ARGUMENT, "device out-pointer is null");
  *device = runtime->slots[index].device;
  return TQ_OK;
}

tq_status tq_runtime_stream(const tq_runtime* runtime, int32_t index, void** stream) {
  TQ_SLOT(runtime, index);
  TQ_REQUIRE(stream != nullptr, TQ_INVALID_ARGUMENT, "stream out-pointer is null");
  *stream = runtime->slots[index].stream;
  return TQ_OK;
}

tq_status tq_runtime_alloc(tq_runtime* runtime, int32_t index, size_t bytes, void** pointer) {
  TQ_SLOT(runtime, index);
  TQ_REQUIRE(pointer != nullptr, TQ_INVALID_ARGUMENT, "pointer out-pointer is null");
  tq_runtime::Slot& slot = runtime->slots[index];
  const size_t start = (slot.used + 255) / 256 * 256;
  TQ_REQUIRE(start <= slot.arena.bytes && bytes <= slot.arena.bytes - start, TQ_RESOURCE_EXHAUSTED,
             "device %d's arena slice holds %zu bytes, %zu are taken and %zu more were asked for", slot.device, slot.arena.bytes, start, bytes);
  *pointer = slot.arena.base + start;
  slot.used = start + bytes;
  return TQ_OK;
}

tq_status tq_runtime_release(tq_runtime* runtime, int32_t index) {
  TQ_SLOT(runtime, index);
  runtime->slots[index].used = 0;
  return TQ_OK;
}

size_t tq_runtime_arena_used(const tq_runtime* runtime, int32_t index) {
  return (runtime != nullptr && index >= 0 && index < static_cast<int32_t>(runtime->slots.size())) ? runtime->slots[index].used : 0;
}

tq_status tq_runtime_join(tq_runtime* runtime, int32_t onto) {
  TQ_SLOT(runtime, onto);
  tq::DeviceScope restore(runtime->slots[onto].device);
  // what every other GPU's stream has queued so far happens before whatever `onto`'s stream gets next
  for (size_t i = 0; i < runtime->slots.size(); ++i) {
    if (static_cast<int32_t>(i) == onto) continue;
    tq_runtime::Slot& slot = runtime->slots[i];
    if (tq_status s = tq::use_device(slot.device)) return s;
    TQ_CUDA(cudaEventRecord(slot.event, slot.stream));
  }
  tq_runtime::Slot& target = runtime->slots[onto];
  if (tq_status s = tq::use_device(target.device)) return s;
  for (size_t i = 0; i < runtime->slots.size(); ++i) {
    if (static_cast<int32_t>(i) != onto) TQ_CUDA(cudaStreamWaitEvent(target.stream, runtime->slots[i].event, 0));
  }
  return TQ_OK;
}

tq_status tq_runtime_fork(tq_runtime* runtime, int32_t from) {
  TQ_SLOT(runtime, from);
  tq::DeviceScope restore(runtime->slots[from].device);
  // what `from`'s stream has queued so far happens before whatever the other GPUs' streams get next
  tq_runtime::Slot& source = runtime->slots[from];
  if (tq_status s = tq::use_device(source.device)) return s;
  TQ_CUDA(cudaEventRecord(source.event, source.stream));
  for (size_t i = 0; i < runtime->slots.size(); ++i) {
    if (static_cast<int32_t>(i) == from) continue;
    if (tq_status s = tq::use_device(runtime->slots[i].device)) return s;
    TQ_CUDA(cudaStreamWaitEvent(runtime->slots[i].stream, source.event, 0));
  }
  return TQ_OK;
}

tq_status tq_runtime_synchronize(tq_runtime* runtime) {
  TQ_REQUIRE(runtime != nullptr, TQ_INVALID_ARGUMENT, "null runtime");
  tq::DeviceScope restore(runtime->slots.empty() ? 0 : runtime->slots[0].device);
  for (tq_runtime::Slot& slot : runtime->slots) {
    if (tq_status s = tq::use_device(slot.device)) return s;
    TQ_CUDA(cudaStreamSynchronize(slot.stream));
  }
  return TQ_OK;
}

tq_status tq_recipe_create(tq_recipe** recipe) {
  TQ_REQUIRE(recipe != nullptr, TQ_INVALID_ARGUMENT, "recipe out-pointer is null");
  *recipe = new tq_recipe();
  return TQ_OK;
}

tq_status tq_recipe_destroy(tq_recipe* recipe) {
  TQ_REQUIRE(recipe == nullptr || tq::g_recording != recipe, TQ_INVALID_ARGUMENT, "the recipe is still recording");
  delete recipe;
  return TQ_OK;
}

tq_status tq_recipe_begin_recording(tq_recipe* recipe) {
  TQ_REQUIRE(recipe != nullptr, TQ_INVALID_ARGUMENT, "null recipe");
  TQ_REQUIRE(tq::g_recording == nullptr, TQ_INVALID_ARGUMENT, "this thread is already recording a recipe");
  tq::g_recording = recipe;
  return TQ_OK;
}

tq_status tq_recipe_end_recording(tq_recipe* recipe) {
  TQ_REQUIRE(recipe != nullptr && tq::g_recording == recipe, TQ_INVALID_ARGUMENT, "this thread is not recording that recipe");
  tq::g_recording = nullptr;
  return TQ_OK;
}

int64_t tq_recipe_steps(const tq_recipe* recipe) { return recipe ? static_cast<int64_t>(recipe->steps.size()) : 0; }

tq_status tq_recipe_run(const tq_recipe* recipe, int32_t device, void* stream) {
  TQ_REQUIRE(recipe != nullptr, TQ_INVALID_ARGUMENT, "null recipe");
  TQ_REQUIRE(tq::g_recording == nullptr, TQ_INVALID_ARGUMENT, "a recipe cannot run while this thread is recording");
  for (size_t i = 0; i < recipe->steps.size(); ++i) {
    if (tq_status s = recipe->steps[i](device, stream)) return s;   // the step's own message stays in tq_last_error
  }
  return TQ_OK;
}

tq_status tq_status_poll(int32_t device, void* stream, int32_t* device_status) {
  TQ_REQUIRE(device_status != nullptr, TQ_INVALID_ARGUMENT, "status out-pointer is null");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  int32_t* word = tq::device_status_word(device);
  TQ_REQUIRE(word != nullptr, TQ_RESOURCE_EXHAUSTED, "no device memory for the status word");
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  int32_t host = 0;
  TQ_CUDA(cudaMemcpyAsync(&host, word, sizeof(host), cudaMemcpyDeviceToHost, cuda_stream));
  TQ_CUDA(cudaStreamSynchronize(cuda_stream));
  if (host != 0) TQ_CUDA(cudaMemsetAsync(word, 0, 256, cuda_stream));   // the code, where it happened, and the abort words
  *device_status = host;
  return TQ_OK;
}

tq_status tq_selftest_bounded_wait(int32_t device, void* stream, int32_t polls, int32_t* looks) {
  TQ_REQUIRE(polls > 0 && polls <= (1 << 20), TQ_INVALID_ARGUMENT, "between 1 and 2^20 polls");
  TQ_REQUIRE(looks != nullptr, TQ_INVALID_ARGUMENT, "looks out-pointer is null");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  const tq::WaitStatus status = tq::wait_status_for(device);
  TQ_REQUIRE(status.abort != nullptr, TQ_RESOURCE_EXHAUSTED, "no device memory for the status word");
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  int* device_looks = tq::device_status_word(device) + 6;   // words of the status block that only a give-up's detail uses
  tq::bounded_wait_selftest_kernel<<<1, 32, 0, cuda_stream>>>(status, static_cast<uint32_t>(polls), device_looks);
  if (tq_status s = tq::check_launch("bounded_wait_selftest_kernel")) return s;
  TQ_CUDA(cudaMemcpyAsync(looks, device_looks, 2 * sizeof(int32_t), cudaMemcpyDeviceToHost, cuda_stream));
  TQ_CUDA(cudaStreamSynchronize(cuda_stream));
  return TQ_OK;
}

tq_status tq_status_detail(int32_t device, void* stream, int32_t* words, int32_t count) {
  TQ_REQUIRE(words != nullptr && count >= 0 && count <= 64, TQ_INVALID_ARGUMENT, "the status block holds 64 words");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  int32_t* word = tq::device_status_word(device);
  TQ_REQUIRE(word != nullptr, TQ_RESOURCE_EXHAUSTED, "no device memory for the status word");
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  TQ_CUDA(cudaMemcpyAsync(words, word, sizeof(int32_t) * count, cudaMemcpyDeviceToHost, cuda_stream));
  TQ_CUDA(cudaStreamSynchronize(cuda_stream));
  return TQ_OK;
}

}  // extern "C"
