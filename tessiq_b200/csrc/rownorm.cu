// Row kernels that need a statistic of the whole row before they can write it: softmax,
// LayerNorm, RMSNorm. The row is read from HBM once, kept in registers, and written once.
//
//   warp-per-row     rows of up to 32*VEC*8 elements: one warp holds a row; shuffles only.
//   cluster-per-row  wider rows: a thread-block cluster of 1, 2, 4 or 8 CTAs holds a row
//                    (256 threads x up to 8 vectors each per CTA). Statistics go warp shuffle ->
//                    shared memory -> distributed shared memory: every CTA writes its block value
//                    into each peer's slot array, one cluster barrier, every CTA folds the slots
//                    in rank order, so all CTAs hold the same bits.
//   loop-per-row     any width or alignment: one CTA streams the row three times (two for
//                    RMSNorm). The fallback for rows that are unaligned or beyond what a cluster
//                    can hold.
//   softmax-columns  softmax over an axis that is not the last one: one thread per column, an
//                    online max/sum pass and a write pass, coalesced along the kept axis.
//
// Semantics follow csrc/custom_ops/softmax/softmax.cu:19-61 (softmax), csrc/tessiq/codegen/
// norm.cpp:22-135 (LayerNorm: mean, then centred sum of squares, rstd = 1/sqrt(var+eps)) and
// csrc/custom_ops/rms_norm/rms_norm.cu:15-42, except that a NaN anywhere in a softmax row makes
// the row NaN, as aten::_softmax does on the reference's host device (the reference's own kernel
// drops NaN from the maximum).
#include <cooperative_groups.h>

#include <limits>

#include <cstdlib>

#include "common.h"

namespace cg = cooperative_groups;

namespace tq {
namespace {

constexpr int kBlock = 256;
constexpr int kWarps = kBlock / 32;
constexpr int kMaxCluster = 8;
constexpr int kMaxVectors = 8;

enum RowOp { kSoftmax = 0, kLayerNorm = 1, kRmsNorm = 2 };

struct RowArgs {
  const void* in;
  void* out;
  const void* weight;
  const void* bias;
  void* mean;
  void* rstd;
  long long rows;
  long long width;
  double eps;
  int stat_is_f32;  // mean/rstd are stored as float rather than as the input's type
};

template <typename C> __device__ __forceinline__ C math_exp(C v);
template <> __device__ __forceinline__ float math_exp<float>(float v) { return expf(v); }
template <> __device__ __forceinline__ double math_exp<double>(double v) { return exp(v); }
template <typename C> __device__ __forceinline__ C math_sqrt(C v);
template <> __device__ __forceinline__ float math_sqrt<float>(float v) { return sqrtf(v); }
template <> __device__ __forceinline__ double math_sqrt<double>(double v) { return sqrt(v); }

// NaN-propagating: the row's NaN must reach every element of the result.
template <typename C> __device__ __forceinline__ C nan_max(C a, C b) {
  if (a != a) return a;
  if (b != b) return b;
  return a > b ? a : b;
}
template <> __device__ __forceinline__ float nan_max<float>(float a, float b) {
  float r;
  asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

// 2^t by the special-function unit (2 ulp). softmax uses it as exp(x - m) = 2^((x - m) * log2e);
// the subtraction comes first so that the row's maximum maps to exactly 2^0 whatever its size.
__device__ __forceinline__ float exp2_approx(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}

// Element e of a vector, widened to the arithmetic type. For bf16 the widening is a shift or a
// mask of the packed 32-bit word, written as volatile asm so that the compiler repeats it in each
// pass over the row instead of keeping a widened copy of the whole row alive in registers.
template <typename T, int VEC>
__device__ __forceinline__ typename Compute<T>::type widen(const Vec<T, VEC>& x, int e) {
  return to_compute(x.v[e]);
}
template <int VEC>
__device__ __forceinline__ float widen(const Vec<__nv_bfloat16, VEC>& x, int e) {
  static_assert(VEC % 2 == 0, "bf16 vectors are handled as 32-bit pairs");
  const uint32_t word = reinterpret_cast<const uint32_t*>(&x)[e >> 1];
  uint32_t bits;
  if (e & 1) {
    asm volatile("and.b32 %0, %1, 0xffff0000;" : "=r"(bits) : "r"(word));
  } else {
    asm volatile("shl.b32 %0, %1, 16;" : "=r"(bits) : "r"(word));
  }
  return __uint_as_float(bits);
}

template <typename C, bool kMax> __device__ __forceinline__ C fold(C a, C b) {
  if constexpr (kMax) return nan_max(a, b);
  return a + b;
}

template <typename C, bool kMax> __device__ __forceinline__ C warp_fold(C v) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    v = fold<C, kMax>(v, __shfl_xor_sync(0xffffffffu, v, offset));
  }
  return v;
}

// Every thread of the CTA gets the CTA-wide result.
template <typename C, bool kMax, int WARPS = kWarps>
__device__ __forceinline__ C block_fold(C v, C* warp_scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_fold<C, kMax>(v);
  if (lane == 0) warp_scratch[warp] = v;
  __syncthreads();
  C total = warp_scratch[0];
#pragma unroll
  for (int w = 1; w < WARPS; ++w) total = fold<C, kMax>(total, warp_scratch[w]);
  __syncthreads();  // warp_scratch is reused by the next statistic
  return total;
}

// Every thread of every CTA of the cluster gets the cluster-wide result. `slots` is an array of
// kMaxCluster values in this CTA's shared memory that no other statistic uses.
template <typename C, bool kMax, int WARPS = kWarps>
__device__ __forceinline__ C cluster_fold(C v, C* warp_scratch, C* slots, int cluster) {
  v = block_fold<C, kMax, WARPS>(v, warp_scratch);
  if (cluster == 1) return v;
  cg::cluster_group group = cg::this_cluster();
  const unsigned rank = group.block_rank();
  if (threadIdx.x < cluster) {
    C* peer = group.map_shared_rank(slots, threadIdx.x);
    peer[rank] = v;
  }
  group.sync();
  C total = slots[0];
  for (int r = 1; r < cluster; ++r) total = fold<C, kMax>(total, slots[r]);
  return total;
}

template <typename T>
__device__ __forceinline__ void store_stat(void* pointer, long long row, float value, int is_f32) {
  if (pointer == nullptr) return;
  if (is_f32) {
    static_cast<float*>(pointer)[row] = value;
  } else {
    static_cast<T*>(pointer)[row] = from_compute<T, float>(value);
  }
}

// The arithmetic shared by the register-resident kernels. `x` holds this thread's vectors of the
// row exactly as loaded: half-precision rows stay packed (two elements per register) and are
// widened on the fly in every pass, so a thread keeps twice the bytes in flight per register.
// `first` + j * `step` is the index of vector j within the row; vectors at or beyond `vectors` do
// not exist. fold_row(value, is_max, stage) reduces a float over the whole row.
template <typename T, typename OutT, int VEC, int K, int OP, typename FoldFn>
__device__ __forceinline__ void finish_row(Vec<T, VEC> (&x)[K], int first, int step, int vectors,
                                           const RowArgs& args, long long row, bool writes_stats,
                                           FoldFn fold_row) {
  OutT* out_row = static_cast<OutT*>(args.out) + row * args.width;
  const float width = static_cast<float>(args.width);
  constexpr bool kKeepsFloats = sizeof(T) == 4;  // a float row can hold exp(x - max) in place
  if constexpr (OP == kSoftmax) {
    float local = -std::numeric_limits<float>::infinity();
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if (first + j * step < vectors) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) local = nan_max(local, widen(x[j], e));
      }
    }
    const float row_max = fold_row(local, /*is_max=*/true, 0);
    constexpr float kLog2e = 1.4426950408889634f;
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if (first + j * step < vectors) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float value = exp2_approx((widen(x[j], e) - row_max) * kLog2e);
          sum += value;
          if constexpr (kKeepsFloats) x[j].v[e] = from_compute<T, float>(value);
        }
      }
    }
    const float inverse = 1.f / fold_row(sum, /*is_max=*/false, 1);
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if (first + j * step < vectors) {
        Vec<OutT, VEC> y;
        auto result = [&](int e) {
          float value;
          if constexpr (kKeepsFloats) {
            value = widen(x[j], e);
          } else {
            value = exp2_approx((widen(x[j], e) - row_max) * kLog2e);
          }
          return value * inverse;
        };
        if constexpr (sizeof(OutT) == 2 && VEC % 2 == 0) {   // one conversion per pair of results
#pragma unroll
          for (int e = 0; e < VEC; e += 2) store_pair(&y.v[e], make_float2(result(e), result(e + 1)));
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) y.v[e] = from_compute<OutT, float>(result(e));
        }
        store_stream<OutT, VEC>(out_row + static_cast<long long>(first + j * step) * VEC, y);
      }
    }
  } else {
    float mean = 0.f;
    if constexpr (OP == kLayerNorm) {
      float sum = 0.f;
#pragma unroll
      for (int j = 0; j < K; ++j) {
        if (first + j * step < vectors) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) sum += widen(x[j], e);
        }
      }
      mean = fold_row(sum, false, 0) / width;
    }
    float squares = 0.f;
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if (first + j * step < vectors) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
          const float centred = widen(x[j], e) - mean;
          squares += centred * centred;
        }
      }
    }
    const float variance = fold_row(squares, false, 1) / width;
    const float rstd = 1.f / sqrtf(variance + static_cast<float>(args.eps));
    if (writes_stats) {
      if constexpr (OP == kLayerNorm) store_stat<T>(args.mean, row, mean, args.stat_is_f32);
      store_stat<T>(args.rstd, row, rstd, args.stat_is_f32);
    }
    const T* weight = static_cast<const T*>(args.weight);
    const T* bias = static_cast<const T*>(args.bias);
#pragma unroll
    for (int j = 0; j < K; ++j) {
      if (first + j * step < vectors) {
        const long long offset = static_cast<long long>(first + j * step) * VEC;
        Vec<T, VEC> w, b;
        if (weight) w = *reinterpret_cast<const Vec<T, VEC>*>(weight + offset);
        if (bias) b = *reinterpret_cast<const Vec<T, VEC>*>(bias + offset);
        Vec<OutT, VEC> y;
        auto result = [&](int e) {
          float value = (widen(x[j], e) - mean) * rstd;
          if (weight) value *= widen(w, e);
          if (bias) value += widen(b, e);
          return value;
        };
        if constexpr (sizeof(OutT) == 2 && VEC % 2 == 0) {   // one conversion per pair of results
#pragma unroll
          for (int e = 0; e < VEC; e += 2) store_pair(&y.v[e], make_float2(result(e), result(e + 1)));
        } else {
#pragma unroll
          for (int e = 0; e < VEC; ++e) y.v[e] = from_compute<OutT, float>(result(e));
        }
        store_stream<OutT, VEC>(out_row + offset, y);
      }
    }
  }
}

// One warp per row; 8 rows per CTA.
template <typename T, typename OutT, int VEC, int K, int OP>
__global__ void __launch_bounds__(kBlock) row_warp_kernel(RowArgs args) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (row >= args.rows) return;
  const int vectors = static_cast<int>(args.width / VEC);
  const T* in_row = static_cast<const T*>(args.in) + row * args.width;
  Vec<T, VEC> x[K];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    if (lane + j * 32 < vectors) x[j] = load_stream<T, VEC>(in_row + static_cast<long long>(lane + j * 32) * VEC);
  }
  auto fold_row = [](float value, bool is_max, int) {
    return is_max ? warp_fold<float, true>(value) : warp_fold<float, false>(value);
  };
  finish_row<T, OutT, VEC, K, OP>(x, lane, 32, vectors, args, row, lane == 0, fold_row);
}

// A cluster of `cluster` CTAs per row. blockIdx.x = row * cluster + rank.
template <typename T, typename OutT, int VEC, int K, int OP, int THREADS = kBlock>
__global__ void __launch_bounds__(THREADS) row_cluster_kernel(RowArgs args, int cluster) {
  __shared__ float warp_scratch[THREADS / 32];
  __shared__ float slots[2][kMaxCluster];
  const long long row = blockIdx.x / cluster;
  const int rank = static_cast<int>(blockIdx.x % cluster);
  const int vectors = static_cast<int>(args.width / VEC);
  const T* in_row = static_cast<const T*>(args.in) + row * args.width;
  const int first = rank * K * THREADS + threadIdx.x;
  Vec<T, VEC> x[K];
#pragma unroll
  for (int j = 0; j < K; ++j) {
    if (first + j * THREADS < vectors) {
      x[j] = load_stream<T, VEC>(in_row + static_cast<long long>(first + j * THREADS) * VEC);
    }
  }
  auto fold_row = [&](float value, bool is_max, int stage) {
    return is_max ? cluster_fold<float, true, THREADS / 32>(value, warp_scratch, slots[stage], cluster)
                  : cluster_fold<float, false, THREADS / 32>(value, warp_scratch, slots[stage], cluster);
  };
  finish_row<T, OutT, VEC, K, OP>(x, first, THREADS, vectors, args, row,
                                  rank == 0 && threadIdx.x == 0, fold_row);
}

// Any width, any alignment: one CTA per row, scalar loads, the row re-read for each statistic.
template <typename T, typename OutT, int OP>
__global__ void __launch_bounds__(kBlock) row_loop_kernel(RowArgs args) {
  using C = typename Compute<T>::type;  // float, or double for f64 rows
  __shared__ C warp_scratch[kWarps];
  const long long row = blockIdx.x;
  const long long width = args.width;
  const T* in_row = static_cast<const T*>(args.in) + row * width;
  OutT* out_row = static_cast<OutT*>(args.out) + row * width;
  if constexpr (OP == kSoftmax) {
    C local = -std::numeric_limits<C>::infinity();
    for (long long i = threadIdx.x; i < width; i += kBlock) local = nan_max<C>(local, to_compute(in_row[i]));
    const C row_max = block_fold<C, true>(local, warp_scratch);
    C sum = 0;
    for (long long i = threadIdx.x; i < width; i += kBlock) sum += math_exp<C>(to_compute(in_row[i]) - row_max);
    const C inverse = C(1) / block_fold<C, false>(sum, warp_scratch);
    for (long long i = threadIdx.x; i < width; i += kBlock) {
      out_row[i] = from_compute<OutT, C>(math_exp<C>(to_compute(in_row[i]) - row_max) * inverse);
    }
  } else {
    C mean = 0;
    if constexpr (OP == kLayerNorm) {
      C sum = 0;
      for (long long i = threadIdx.x; i < width; i += kBlock) sum += to_compute(in_row[i]);
      mean = block_fold<C, false>(sum, warp_scratch) / static_cast<C>(width);
    }
    C squares = 0;
    for (long long i = threadIdx.x; i < width; i += kBlock) {
      const C centred = to_compute(in_row[i]) - mean;
      squares += centred * centred;
    }
    const C variance = block_fold<C, false>(squares, warp_scratch) / static_cast<C>(width);
    const C rstd = C(1) / math_sqrt<C>(variance + static_cast<C>(args.eps));
    if (threadIdx.x == 0) {
      if constexpr (std::is_same_v<C, double>) {
        if (OP == kLayerNorm && args.mean) static_cast<double*>(args.mean)[row] = mean;
        if (args.rstd) static_cast<double*>(args.rstd)[row] = rstd;
      } else {
        if constexpr (OP == kLayerNorm) store_stat<T>(args.mean, row, mean, args.stat_is_f32);
        store_stat<T>(args.rstd, row, rstd, args.stat_is_f32);
      }
    }
    const T* weight = static_cast<const T*>(args.weight);
    const T* bias = static_cast<const T*>(args.bias);
    for (long long i = threadIdx.x; i < width; i += kBlock) {
      C value = (to_compute(in_row[i]) - mean) * rstd;
      if (weight) value *= to_compute(weight[i]);
      if (bias) value += to_compute(bias[i]);
      out_row[i] = from_compute<OutT, C>(value);
    }
  }
}

// softmax over the middle axis of [outer, extent, inner], inner > 1: a thread per (outer, inner)
// column; pass 1 keeps a running maximum and a sum rescaled whenever the maximum grows, pass 2
// writes. Loads and stores of a warp are contiguous along inner.
template <typename T, typename OutT>
__global__ void __launch_bounds__(kBlock)
softmax_columns_kernel(const T* __restrict__ in, OutT* __restrict__ out, long long outer,
                       long long extent, long long inner) {
  using C = typename Compute<T>::type;
  const long long column = static_cast<long long>(blockIdx.x) * kBlock + threadIdx.x;
  if (column >= outer * inner) return;
  const long long o = column / inner, i = column % inner;
  const T* base = in + o * extent * inner + i;
  OutT* target = out + o * extent * inner + i;
  C running_max = -std::numeric_limits<C>::infinity();
  C sum = 0;
  bool saw_nan = false;
  for (long long r = 0; r < extent; ++r) {
    const C x = to_compute(base[r * inner]);
    if (x != x) saw_nan = true;
    if (x > running_max) {
      // exp(-inf - finite) is 0, so the first element needs no special case.
      sum = sum * math_exp<C>(running_max - x) + C(1);
      running_max = x;
    } else {
      sum += math_exp<C>(x - running_max);
    }
  }
  if (saw_nan) sum = std::numeric_limits<C>::quiet_NaN();
  const C inverse = C(1) / sum;
  for (long long r = 0; r < extent; ++r) {
    const C x = to_compute(base[r * inner]);
    target[r * inner] = from_compute<OutT, C>(math_exp<C>(x - running_max) * inverse);
  }
}

// ---------------------------------------------------------------------------------------------
// Host dispatch

template <typename Kernel>
tq_status launch_rows(Kernel kernel, long long blocks, int cluster, cudaStream_t stream,
                      const RowArgs& args, const char* name, int threads = kBlock) {
  TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld rows are more than a grid holds", args.rows);
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(blocks));
  config.blockDim = dim3(threads);
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = cluster;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = cluster > 1 ? 1 : 0;
  TQ_CUDA(cudaLaunchKernelEx(&config, kernel, args, cluster));
  return check_launch(name);
}

template <typename T, typename OutT, int VEC, int OP>
tq_status run_vector(const RowArgs& args, cudaStream_t stream, bool* handled) {
  *handled = true;
  const long long vectors = args.width / VEC;
  if (vectors <= 32 * kMaxVectors) {
    const long long blocks = (args.rows + kWarps - 1) / kWarps;
    TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld rows are more than a grid holds", args.rows);
    const unsigned grid = static_cast<unsigned>(blocks);
    if (vectors <= 32) {
      row_warp_kernel<T, OutT, VEC, 1, OP><<<grid, kBlock, 0, stream>>>(args);
    } else if (vectors <= 64) {
      row_warp_kernel<T, OutT, VEC, 2, OP><<<grid, kBlock, 0, stream>>>(args);
    } else if (vectors <= 96) {   // 768-wide 2-byte rows (a GPT-2-small hidden state): 38 us against 43 with four slots, one empty
      row_warp_kernel<T, OutT, VEC, 3, OP><<<grid, kBlock, 0, stream>>>(args);
    } else if (vectors <= 128) {
      row_warp_kernel<T, OutT, VEC, 4, OP><<<grid, kBlock, 0, stream>>>(args);
    } else {
      row_warp_kernel<T, OutT, VEC, 8, OP><<<grid, kBlock, 0, stream>>>(args);
    }
    return check_launch("row_warp_kernel");
  }
  // Rows of 2049 to 4096 vectors: one CTA of 256 threads holding 16 vectors each, not a cluster of
  // two CTAs — a cluster launch costs more than it spreads (measured on B200, 4096 rows of 32768 bf16:
  // softmax 113 -> 104 us, LayerNorm 151 -> 117; 4096 x 16384 f32 softmax 93 -> 86; 128 threads x 32
  // vectors: 140 / 158 / 92).
  if (vectors > kBlock * kMaxVectors && vectors <= kBlock * 16) {
    return launch_rows(row_cluster_kernel<T, OutT, VEC, 16, OP>, args.rows, 1, stream, args, "row_cluster_kernel");
  }
  int cluster = 1;
  while (cluster < kMaxCluster && vectors > static_cast<long long>(kBlock) * kMaxVectors * cluster) cluster *= 2;
  if (vectors > static_cast<long long>(kBlock) * kMaxVectors * cluster) {
    *handled = false;  // wider than a cluster's registers
    return TQ_OK;
  }
  const long long per_cta = (vectors + cluster - 1) / cluster;
  const long long blocks = args.rows * cluster;
  // Few threads holding several vectors each beat many threads holding one: a row then costs
  // fewer shuffles and barriers per byte, and more rows are in flight per SM.
  // Measured on B200, 32768 rows of 4096 bf16 (512 vectors): 64 threads x 8 vectors 87.5 us (softmax) /
  // 94 (LayerNorm); 128 x 4: 99 / 101; 32 x 16: 96 / 110; 256 x 2: 121 / 156.
  if (cluster == 1 && per_cta <= 64 * 8) {
    return launch_rows(row_cluster_kernel<T, OutT, VEC, 8, OP, 64>, blocks, cluster, stream, args, "row_cluster_kernel", 64);
  }
  if (per_cta <= 128 * 4) {
    return launch_rows(row_cluster_kernel<T, OutT, VEC, 4, OP, 128>, blocks, cluster, stream, args, "row_cluster_kernel", 128);
  }
  if (per_cta <= kBlock * 4) return launch_rows(row_cluster_kernel<T, OutT, VEC, 4, OP>, blocks, cluster, stream, args, "row_cluster_kernel");
  return launch_rows(row_cluster_kernel<T, OutT, VEC, 8, OP>, blocks, cluster, stream, args, "row_cluster_kernel");
}

template <typename T, typename OutT, int OP>
tq_status run_rows(const RowArgs& args, cudaStream_t stream) {
  if constexpr (!std::is_same_v<T, double>) {
    constexpr int kVec = 16 / sizeof(T);
    constexpr size_t kOutBytes = sizeof(OutT) * kVec;
    const bool vectorisable =
        args.width % kVec == 0 && aligned_to(args.in, 16) && aligned_to(args.out, kOutBytes > 16 ? 16 : kOutBytes) &&
        (args.weight == nullptr || aligned_to(args.weight, 16)) &&
        (args.bias == nullptr || aligned_to(args.bias, 16));
    if (vectorisable) {
      bool handled = false;
      if (tq_status s = run_vector<T, OutT, kVec, OP>(args, stream, &handled)) return s;
      if (handled) return TQ_OK;
    }
  }
  TQ_REQUIRE(args.rows <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld rows are more than a grid holds", args.rows);
  row_loop_kernel<T, OutT, OP><<<static_cast<unsigned>(args.rows), kBlock, 0, stream>>>(args);
  return check_launch("row_loop_kernel");
}

template <typename T, typename OutT>
tq_status run_softmax(const void* in, void* out, long long outer, long long extent, long long inner,
                      cudaStream_t stream) {
  if (inner == 1) {
    RowArgs args = {};
    args.in = in;
    args.out = out;
    args.rows = outer;
    args.width = extent;
    return run_rows<T, OutT, kSoftmax>(args, stream);
  }
  const long long columns = outer * inner;
  const long long blocks = (columns + kBlock - 1) / kBlock;
  TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld softmax columns are more than a grid holds", columns);
  softmax_columns_kernel<T, OutT><<<static_cast<unsigned>(blocks), kBlock, 0, stream>>>(
      static_cast<const T*>(in), static_cast<OutT*>(out), outer, extent, inner);
  return check_launch("softmax_columns_kernel");
}

}  // namespace
}  // namespace tq

extern "C" {

tq_status tq_softmax_launch(tq_dtype dtype, tq_dtype out_dtype, const void* in, void* out,
                            int64_t outer, int64_t extent, int64_t inner, int32_t device,
                            void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) { return tq_softmax_launch(dtype, out_dtype, in, out, outer, extent, inner, d, s); });
  TQ_REQUIRE(outer >= 0 && extent >= 0 && inner >= 0, TQ_INVALID_ARGUMENT,
             "negative extent in [%lld, %lld, %lld]", (long long)outer, (long long)extent, (long long)inner);
  if (outer == 0 || extent == 0 || inner == 0) return TQ_OK;
  TQ_REQUIRE(in != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null input or output");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  if (dtype == TQ_F32 && out_dtype == TQ_F32) return tq::run_softmax<float, float>(in, out, outer, extent, inner, cuda_stream);
  if (dtype == TQ_BF16 && out_dtype == TQ_BF16) return tq::run_softmax<__nv_bfloat16, __nv_bfloat16>(in, out, outer, extent, inner, cuda_stream);
  if (dtype == TQ_F16 && out_dtype == TQ_F16) return tq::run_softmax<__half, __half>(in, out, outer, extent, inner, cuda_stream);
  if (dtype == TQ_BF16 && out_dtype == TQ_F32) return tq::run_softmax<__nv_bfloat16, float>(in, out, outer, extent, inner, cuda_stream);
  if (dtype == TQ_F16 && out_dtype == TQ_F32) return tq::run_softmax<__half, float>(in, out, outer, extent, inner, cuda_stream);
  if (dtype == TQ_F64 && out_dtype == TQ_F64) return tq::run_softmax<double, double>(in, out, outer, extent, inner, cuda_stream);
  return tq::fail(TQ_UNSUPPORTED, "softmax has no kernel for %s -> %s", tq::dtype_name(dtype), tq::dtype_name(out_dtype));
}

tq_status tq_layer_norm_launch(tq_dtype dtype, const void* in, const void* weight, const void* bias,
                               void* out, void* mean, void* rstd, tq_dtype stat_dtype, int64_t rows,
                               int64_t width, double eps, int32_t device, void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) {
    return tq_layer_norm_launch(dtype, in, weight, bias, out, mean, rstd, stat_dtype, rows, width, eps, d, s);
  });
  TQ_REQUIRE(rows >= 0 && width >= 0, TQ_INVALID_ARGUMENT, "negative extent in [%lld, %lld]", (long long)rows, (long long)width);
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(width > 0, TQ_UNSUPPORTED, "LayerNorm over no elements has no kernel");
  TQ_REQUIRE(in != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null input or output");
  TQ_REQUIRE(stat_dtype == dtype || (stat_dtype == TQ_F32 && dtype != TQ_F64), TQ_UNSUPPORTED,
             "LayerNorm statistics of type %s for %s rows have no kernel", tq::dtype_name(stat_dtype), tq::dtype_name(dtype));
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  tq::RowArgs args = {};
  args.in = in;
  args.out = out;
  args.weight = weight;
  args.bias = bias;
  args.mean = mean;
  args.rstd = rstd;
  args.rows = rows;
  args.width = width;
  args.eps = eps;
  args.stat_is_f32 = stat_dtype == TQ_F32 ? 1 : 0;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TQ_F32: return tq::run_rows<float, float, tq::kLayerNorm>(args, cuda_stream);
    case TQ_BF16: return tq::run_rows<__nv_bfloat16, __nv_bfloat16, tq::kLayerNorm>(args, cuda_stream);
    case TQ_F16: return tq::run_rows<__half, __half, tq::kLayerNorm>(args, cuda_stream);
    case TQ_F64: return tq::run_rows<double, double, tq::kLayerNorm>(args, cuda_stream);
    default: return tq::fail(TQ_UNSUPPORTED, "LayerNorm has no kernel for element type %s", tq::dtype_name(dtype));
  }
}

tq_status tq_rms_norm_launch(tq_dtype dtype, const void* in, const void* weight, void* out,
                             int64_t rows, int64_t width, double eps, int32_t device, void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) { return tq_rms_norm_launch(dtype, in, weight, out, rows, width, eps, d, s); });
  TQ_REQUIRE(rows >= 0 && width >= 0, TQ_INVALID_ARGUMENT, "negative extent in [%lld, %lld]", (long long)rows, (long long)width);
  if (rows == 0) return TQ_OK;
  TQ_REQUIRE(width > 0, TQ_UNSUPPORTED, "RMSNorm over no elements has no kernel");
  TQ_REQUIRE(in != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null input or output");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  tq::RowArgs args = {};
  args.in = in;
  args.out = out;
  args.weight = weight;
  args.rows = rows;
  args.width = width;
  args.eps = eps;
  args.stat_is_f32 = 1;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TQ_F32: return tq::run_rows<float, float, tq::kRmsNorm>(args, cuda_stream);
    case TQ_BF16: return tq::run_rows<__nv_bfloat16, __nv_bfloat16, tq::kRmsNorm>(args, cuda_stream);
    case TQ_F16: return tq::run_rows<__half, __half, tq::kRmsNorm>(args, cuda_stream);
    case TQ_F64: return tq::run_rows<double, double, tq::kRmsNorm>(args, cuda_stream);
    default: return tq::fail(TQ_UNSUPPORTED, "RMSNorm has no kernel for element type %s", tq::dtype_name(dtype));
  }
}

// softmax / LayerNorm over the last axis of the TRANSPOSED view of a packed in[batch, rows, cols]:
// out[b][c][:] = softmax(in[b][:, c]) (or LayerNorm with weight/bias over `rows`), out packed
// [batch, cols, rows]. Two launches: per-column statistics read in place (no packed copy is made),
// then a tiled transpose that normalises on the way: 3 passes over the data instead of the 4 of
// pack-then-rows. Scratch layout: [batch * cols] float2 statistics, then the reduction's scratch.
namespace {

size_t stats_bytes(long long batch, long long cols) { return (static_cast<size_t>(batch * cols) * 8 + 255) / 256 * 256; }

tq_status transposed_launch(int kind, tq_dtype dtype, const void* in, const void* weight, const void* bias, void* out,
                            int64_t batch, int64_t rows, int64_t cols, double eps, void* workspace, size_t workspace_bytes,
                            int32_t device, void* stream) {
  TQ_REQUIRE(batch >= 0 && rows >= 0 && cols >= 0, TQ_INVALID_ARGUMENT, "negative extent in [%lld, %lld, %lld]",
             (long long)batch, (long long)rows, (long long)cols);
  if (batch == 0 || cols == 0) return TQ_OK;
  TQ_REQUIRE(rows > 0, TQ_UNSUPPORTED, "a normalisation over no elements has no kernel");
  TQ_REQUIRE(in != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null input or output");
  TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_F16 || dtype == TQ_BF16, TQ_UNSUPPORTED,
             "the transposed normalisations have no kernel for element type %s", tq::dtype_name(dtype));
  const int vec = 16 / tq::dtype_size(dtype);
  TQ_REQUIRE(rows % vec == 0 && cols % vec == 0 && tq::aligned_to(in, 16) && tq::aligned_to(out, 16), TQ_UNSUPPORTED,
             "the transposed normalisations need extents that are multiples of %d and 16-byte-aligned tensors", vec);
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  const size_t stats = stats_bytes(batch, cols);
  const size_t reduce_scratch = tq::slice_stats_workspace_bytes(kind, dtype, batch, rows, cols, device);
  const size_t need = std::max(stats + reduce_scratch, tq::panel_workspace_bytes(dtype, batch, rows, cols));
  TQ_REQUIRE(workspace != nullptr && workspace_bytes >= need && tq::aligned_to(workspace, 16), TQ_INVALID_ARGUMENT,
             "this call needs %zu bytes of 16-byte-aligned scratch and was given %zu", need, workspace_bytes);
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  unsigned char* scratch = static_cast<unsigned char*>(workspace);
  bool handled = false;
  if (tq_status s = tq::slab_normalize_launch(kind, dtype, in, out, weight, bias, batch, rows, cols, static_cast<float>(eps), cuda_stream, &handled)) return s;
  if (handled) return TQ_OK;
  if (tq_status s = tq::panel_normalize_launch(kind, dtype, in, out, weight, bias, batch, rows, cols, static_cast<float>(eps), workspace,
                                               workspace_bytes, device, cuda_stream, &handled)) return s;
  if (handled) return TQ_OK;
  if (tq_status s = tq::slice_stats_launch(kind, dtype, in, scratch, batch, rows, cols, scratch + stats, reduce_scratch, device, cuda_stream)) return s;
  return tq::transpose_normalize_launch(kind, dtype, in, out, scratch, weight, bias, batch, rows, cols, static_cast<float>(eps), cuda_stream);
}

}  // namespace

tq_status tq_transposed_workspace_bytes(int32_t layer_norm, tq_dtype dtype, int64_t batch, int64_t rows, int64_t cols,
                                        int32_t device, size_t* bytes) {
  TQ_REQUIRE(bytes != nullptr, TQ_INVALID_ARGUMENT, "bytes out-pointer is null");
  TQ_REQUIRE(batch >= 0 && rows >= 0 && cols >= 0, TQ_INVALID_ARGUMENT, "negative extent");
  TQ_REQUIRE(tq::dtype_size(dtype) != 0, TQ_INVALID_ARGUMENT, "unknown element type %d", dtype);
  *bytes = 0;
  if (batch == 0 || cols == 0 || rows == 0) return TQ_OK;
  *bytes = std::max(stats_bytes(batch, cols) + tq::slice_stats_workspace_bytes(layer_norm ? 1 : 0, dtype, batch, rows, cols, device),
                    tq::panel_workspace_bytes(dtype, batch, rows, cols));
  return TQ_OK;
}

tq_status tq_transposed_passes(int32_t layer_norm, tq_dtype dtype, int64_t batch, int64_t rows, int64_t cols, int32_t device,
                               int32_t* passes) {
  (void)layer_norm;
  (void)device;
  TQ_REQUIRE(passes != nullptr, TQ_INVALID_ARGUMENT, "passes out-pointer is null");
  TQ_REQUIRE(batch >= 0 && rows >= 0 && cols >= 0, TQ_INVALID_ARGUMENT, "negative extent");
  TQ_REQUIRE(tq::dtype_size(dtype) != 0, TQ_INVALID_ARGUMENT, "unknown element type %d", dtype);
  *passes = tq::slab_takes(dtype, batch, rows, cols) ? 2 : 3;
  return TQ_OK;
}

tq_status tq_transposed_form(int32_t layer_norm, tq_dtype dtype, int64_t batch, int64_t rows, int64_t cols, int32_t device,
                             int32_t* form) {
  (void)layer_norm;
  (void)device;
  TQ_REQUIRE(form != nullptr, TQ_INVALID_ARGUMENT, "form out-pointer is null");
  TQ_REQUIRE(batch >= 0 && rows >= 0 && cols >= 0, TQ_INVALID_ARGUMENT, "negative extent");
  TQ_REQUIRE(tq::dtype_size(dtype) != 0, TQ_INVALID_ARGUMENT, "unknown element type %d", dtype);
  *form = tq::slab_takes(dtype, batch, rows, cols) ? TQ_TRANSPOSED_SLAB : tq::panel_takes(dtype, batch, rows, cols) ? TQ_TRANSPOSED_PANELS : TQ_TRANSPOSED_THREE_PASS;
  return TQ_OK;
}

tq_status tq_softmax_transposed_launch(tq_dtype dtype, const void* in, void* out, int64_t batch, int64_t rows, int64_t cols,
                                       void* workspace, size_t workspace_bytes, int32_t device, void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) {
    return tq_softmax_transposed_launch(dtype, in, out, batch, rows, cols, workspace, workspace_bytes, d, s);
  });
  return transposed_launch(0, dtype, in, nullptr, nullptr, out, batch, rows, cols, 0.0, workspace, workspace_bytes, device, stream);
}

tq_status tq_layer_norm_transposed_launch(tq_dtype dtype, const void* in, const void* weight, const void* bias, void* out,
                                          int64_t batch, int64_t rows, int64_t cols, double eps, void* workspace,
                                          size_t workspace_bytes, int32_t device, void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) {
    return tq_layer_norm_transposed_launch(dtype, in, weight, bias, out, batch, rows, cols, eps, workspace, workspace_bytes, d, s);
  });
  return transposed_launch(1, dtype, in, weight, bias, out, batch, rows, cols, eps, workspace, workspace_bytes, device, stream);
}

}  // extern "C"
