// Shared host and device helpers of the tessiq_b200 kernel library.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <functional>
#include <string>

#include "tessiq_b200.h"

namespace tq {

// ---------------------------------------------------------------------------------------------
// Errors. Every entry point returns through fail()/ok(); the message goes to a thread-local slot.

void set_error(const char* text);
tq_status fail(tq_status code, const char* format, ...) __attribute__((format(printf, 2, 3)));

#define TQ_CUDA(call)                                                                         \
  do {                                                                                        \
    cudaError_t tq_cuda_status_ = (call);                                                     \
    if (tq_cuda_status_ != cudaSuccess) {                                                     \
      return ::tq::fail(TQ_EXTERNAL, "%s failed: %s", #call,                                  \
                        cudaGetErrorString(tq_cuda_status_));                                 \
    }                                                                                         \
  } while (0)

#define TQ_REQUIRE(condition, code, ...)                                                      \
  do {                                                                                        \
    if (!(condition)) return ::tq::fail(code, __VA_ARGS__);                                   \
  } while (0)

// Makes `device` current for the calling thread. Cheap when it already is.
tq_status use_device(int32_t device);

// Makes `device` current for the rest of the enclosing block and puts the caller's device back at
// its end: an entry point must not leave the thread on another GPU than it found it on (PyTorch
// and every other user of the runtime API take the thread's current device as theirs).
class DeviceScope {
 public:
  explicit DeviceScope(int32_t device) {
    if (cudaGetDevice(&previous_) != cudaSuccess) previous_ = -1;
    status_ = use_device(device);
  }
  // Whatever the block did in between (the runtime handle's calls walk over several GPUs), the thread
  // leaves on the device it came with.
  ~DeviceScope() {
    int now = -1;
    if (previous_ >= 0 && cudaGetDevice(&now) == cudaSuccess && now != previous_) cudaSetDevice(previous_);
  }
  DeviceScope(const DeviceScope&) = delete;
  DeviceScope& operator=(const DeviceScope&) = delete;
  tq_status status() const { return status_; }

 private:
  int previous_ = -1;
  tq_status status_ = TQ_OK;
};

// Number of SMs of `device` (cached).
int sm_count(int32_t device);

// Checks the launch that was just queued.
inline tq_status check_launch(const char* what) {
  cudaError_t status = cudaGetLastError();
  if (status != cudaSuccess) {
    return fail(TQ_EXTERNAL, "launching %s failed: %s", what, cudaGetErrorString(status));
  }
  return TQ_OK;
}

inline int dtype_size(tq_dtype dtype) {
  switch (dtype) {
    case TQ_F32: return 4;
    case TQ_F64: return 8;
    case TQ_F16: return 2;
    case TQ_BF16: return 2;
    case TQ_I32: return 4;
    case TQ_I64: return 8;
    case TQ_BOOL: return 1;
    default: return 0;
  }
}

inline const char* dtype_name(tq_dtype dtype) {
  switch (dtype) {
    case TQ_F32: return "f32";
    case TQ_F64: return "f64";
    case TQ_F16: return "f16";
    case TQ_BF16: return "bf16";
    case TQ_I32: return "i32";
    case TQ_I64: return "i64";
    case TQ_BOOL: return "bool";
    default: return "?";
  }
}

inline bool aligned_to(const void* pointer, size_t bytes) {
  return (reinterpret_cast<uintptr_t>(pointer) % bytes) == 0;
}

// Recipe recording (runtime.cu). While the calling thread records into a tq_recipe, every launch
// entry point hands a closure of itself to record() instead of launching; tq_recipe_run calls the
// closures in order with its own (device, stream).
using Replay = std::function<tq_status(int32_t device, void* stream)>;
bool recording();
tq_status record(Replay step);

#define TQ_RECORD_OR_RUN(...)                                                   \
  do {                                                                          \
    if (::tq::recording()) return ::tq::record(__VA_ARGS__);                    \
  } while (0)

// Device-side status block (one per device, 64 words, 256-byte aligned), written by kernels whose
// bounded waits give up. Word 0 is the sticky code tq_status_poll reads and clears; words 1-7 say
// where the wait was (tq_status_detail); words 8-63 are abort words. Each launch is handed one abort
// word (launches take them in turn); its first CTA clears the word when the kernel starts, a wait
// that gives up sets it, and the launch's other waits leave when they see it set. A later launch has
// another word, so a give-up nobody has polled yet does not make it bail out. The handle is one
// pointer: the sticky word is found by rounding the abort word's address down to the block.
int32_t* device_status_word(int32_t device);
struct WaitStatus {
  int* abort;
#ifdef __CUDACC__
  __device__ int* sticky() const { return reinterpret_cast<int*>(reinterpret_cast<uintptr_t>(abort) & ~static_cast<uintptr_t>(255)); }
  __device__ bool aborted() const { return *reinterpret_cast<volatile int*>(abort) != 0; }
  __device__ void set_abort() const { *reinterpret_cast<volatile int*>(abort) = 1; }
  // by one thread of the launch's first CTA, before the CTA's first wait
  __device__ void begin() const { *reinterpret_cast<volatile int*>(abort) = 0; }
#endif
};
// The status handle for one launch on `device`; `abort` is null when the block cannot be allocated.
WaitStatus wait_status_for(int32_t device);

// reduce.cu: per-slice (max, 1/sum-exp) [kind 0] or (mean, variance) [kind 1] of a packed
// [outer, reduce, inner] tensor, two floats per slice. Used by the transposed softmax / LayerNorm.
size_t slice_stats_workspace_bytes(int kind, tq_dtype dtype, long long outer, long long reduce, long long inner, int32_t device);
tq_status slice_stats_launch(int kind, tq_dtype dtype, const void* in, void* stats, long long outer, long long reduce,
                             long long inner, void* workspace, size_t workspace_bytes, int32_t device, cudaStream_t stream);

// pack.cu: out[b][c][r] = f(in[b][r][c]) for a packed in[batch, rows, cols] — the tiled transpose
// with a per-element normalisation. `kind` 0: exp(x - stats[c].max) * stats[c].inv_sum (softmax over
// rows); `kind` 1: (x - mean_c) * rsqrt(var_c + eps) * weight[r] + bias[r] (LayerNorm over rows).
// Declines (TQ_UNSUPPORTED) shapes that are not multiples of the 16-byte vector width.
tq_status transpose_normalize_launch(int kind, tq_dtype dtype, const void* in, void* out, const void* stats, const void* weight,
                                     const void* bias, long long batch, long long rows, long long cols, float eps, cudaStream_t stream);

// slabnorm.cu: the same result from ONE pass over HBM — a cluster of 8 CTAs keeps a slab of columns
// by all the rows in its shared memory. Sets `*handled` and launches when slab_takes() the shape (rows
// a multiple of 8 vectors, 8192 to 51200, cols a multiple of two vectors, at most 32 MiB in all) and
// the pointers are 16-byte aligned; otherwise launches nothing.
bool slab_takes(tq_dtype dtype, long long batch, long long rows, long long cols);
tq_status slab_normalize_launch(int kind, tq_dtype dtype, const void* in, void* out, const void* weight, const void* bias,
                                long long batch, long long rows, long long cols, float eps, cudaStream_t stream, bool* handled);

// panelnorm.cu: the same result from 1 read + 1 write of HBM for tensors far larger than L2 — one
// persistent kernel walks panels of columns (512 bytes of every row) that stay in L2 between their
// statistics visit and their normalising visit. Sets `*handled` and launches when panel_takes() the
// shape and the pointers are 16-byte aligned; otherwise launches nothing. `workspace` must hold
// panel_workspace_bytes (partials, final statistics, panel counters, flags and the work queue).
bool panel_takes(tq_dtype dtype, long long batch, long long rows, long long cols);
size_t panel_workspace_bytes(tq_dtype dtype, long long batch, long long rows, long long cols);
tq_status panel_normalize_launch(int kind, tq_dtype dtype, const void* in, void* out, const void* weight, const void* bias,
                                 long long batch, long long rows, long long cols, float eps, void* workspace, size_t workspace_bytes,
                                 int32_t device, cudaStream_t stream, bool* handled);

}  // namespace tq

// ---------------------------------------------------------------------------------------------
// Device helpers
#ifdef __CUDACC__

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace tq {

// Storage type -> the type arithmetic runs in.
template <typename T> struct Compute { using type = T; };
template <> struct Compute<__half> { using type = float; };
template <> struct Compute<__nv_bfloat16> { using type = float; };

template <typename T> __device__ __forceinline__ typename Compute<T>::type to_compute(T v) { return v; }
template <> __device__ __forceinline__ float to_compute<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_compute<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}

template <typename T, typename C> __device__ __forceinline__ T from_compute(C v) { return static_cast<T>(v); }
template <> __device__ __forceinline__ __half from_compute<__half, float>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_compute<__nv_bfloat16, float>(float v) {
  return __float2bfloat16_rn(v);
}

// Two neighbouring results rounded and packed with one conversion (`to` is 4-byte aligned for the 2-byte types).
__device__ __forceinline__ void store_pair(__nv_bfloat16* to, float2 y) { *reinterpret_cast<__nv_bfloat162*>(to) = __floats2bfloat162_rn(y.x, y.y); }
__device__ __forceinline__ void store_pair(__half* to, float2 y) { *reinterpret_cast<__half2*>(to) = __floats2half2_rn(y.x, y.y); }
template <typename T>
__device__ __forceinline__ void store_pair(T* to, float2 y) {
  to[0] = from_compute<T, float>(y.x);
  to[1] = from_compute<T, float>(y.y);
}

// A vector of N elements of T moved with one instruction when N*sizeof(T) is 4, 8 or 16 bytes.
template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
  T v[N];
};

// Streaming (read-once) load: bypasses L1 allocation so that the data does not evict reused lines.
template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_stream(const T* pointer) {
  Vec<T, N> out;
  constexpr int kBytes = sizeof(T) * N;
  if constexpr (kBytes == 16) {
    uint4 raw;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                 : "l"(pointer));
    *reinterpret_cast<uint4*>(&out) = raw;
  } else if constexpr (kBytes == 32) {
    uint4 lo, hi;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(lo.x), "=r"(lo.y), "=r"(lo.z), "=r"(lo.w)
                 : "l"(pointer));
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(hi.x), "=r"(hi.y), "=r"(hi.z), "=r"(hi.w)
                 : "l"(reinterpret_cast<const char*>(pointer) + 16));
    reinterpret_cast<uint4*>(&out)[0] = lo;
    reinterpret_cast<uint4*>(&out)[1] = hi;
  } else if constexpr (kBytes == 8) {
    uint2 raw;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];"
                 : "=r"(raw.x), "=r"(raw.y)
                 : "l"(pointer));
    *reinterpret_cast<uint2*>(&out) = raw;
  } else if constexpr (kBytes == 4) {
    uint32_t raw;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(raw) : "l"(pointer));
    *reinterpret_cast<uint32_t*>(&out) = raw;
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) out.v[i] = pointer[i];
  }
  return out;
}

// Streaming store (evict-first): the result is not read again by this kernel.
template <typename T, int N>
__device__ __forceinline__ void store_stream(T* pointer, const Vec<T, N>& value) {
  constexpr int kBytes = sizeof(T) * N;
  if constexpr (kBytes == 16) {
    __stcs(reinterpret_cast<uint4*>(pointer), *reinterpret_cast<const uint4*>(&value));
  } else if constexpr (kBytes == 32) {
    __stcs(reinterpret_cast<uint4*>(pointer), reinterpret_cast<const uint4*>(&value)[0]);
    __stcs(reinterpret_cast<uint4*>(pointer) + 1, reinterpret_cast<const uint4*>(&value)[1]);
  } else if constexpr (kBytes == 8) {
    __stcs(reinterpret_cast<uint2*>(pointer), *reinterpret_cast<const uint2*>(&value));
  } else if constexpr (kBytes == 4) {
    __stcs(reinterpret_cast<unsigned int*>(pointer), *reinterpret_cast<const unsigned int*>(&value));
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) pointer[i] = value.v[i];
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
  return v;
}

}  // namespace tq

#endif  // __CUDACC__
