// softmax / LayerNorm over the last axis of a TRANSPOSED view, with the data read from HBM once.
//
//   in  packed [batch, rows, cols];  out packed [batch, cols, rows]
//   out[b][c][:] = softmax(in[b][:, c])    or    LayerNorm(in[b][:, c]) * weight[:] + bias[:]
//
// The statistics of a column need every row, so a plain kernel reads the data twice (statistics,
// then normalise). Here a cluster of 8 CTAs keeps a slab of columns — two 16-byte units per row, i.e.
// 8 four-byte or 16 two-byte columns, by ALL the rows — in its shared memory: each CTA holds an
// eighth of the rows (32 bytes per row, up to 200 KiB). The slab comes in with cp.async (no
// registers, everything in flight at once), the per-column statistics are combined thread -> warp ->
// CTA -> cluster (distributed shared memory), exactly two-pass (maximum then sum of exponentials;
// mean then centred squares), and the normalised values leave through V x V register transposes as
// whole 512-byte runs of the output rows. HBM traffic: every element read once and written once —
// what the operation on a packed tensor costs.
//
// Shared-memory layout: 16-byte unit u = row * 2 + half is stored at u ^ ((row / V) & 7), which keeps
// a unit inside its own 128-byte group and makes the transposing reads (consecutive lanes take
// consecutive groups of V rows) conflict-free.
//
// The reference reaches this operation as pack (csrc/tessiq/codegen/pack.cpp:41-94) followed by its
// softmax (csrc/custom_ops/softmax/softmax.cu:19-61) or LayerNorm (csrc/tessiq/codegen/norm.cpp:22-135)
// kernel: four passes over the data.
#include <cooperative_groups.h>

#include <cstdlib>
#include <mutex>

#include "common.h"

namespace cg = cooperative_groups;

namespace tq {
namespace {

constexpr int kSlabCluster = 8;
constexpr int kSlabThreads = 256;
constexpr int kSlabWarps = kSlabThreads / 32;
constexpr int kSlabRowsPerPass = kSlabThreads / 2;          // 128: two threads (the two halves) per row
constexpr size_t kSlabMaxDataBytes = 200 * 1024;

struct SlabArgs {
  const void* in;
  void* out;
  const void* weight;
  const void* bias;
  long long rows, cols;
  int rows_per_cta;
  float eps;
};

template <int V>
__device__ __forceinline__ uint32_t slab_unit(int row, int half) {
  return static_cast<uint32_t>((row * 2 + half) ^ ((row / V) & 7));
}

// Folds `value[V]` over every thread of the cluster that holds the same half of the columns:
// lanes of equal parity, the CTA's 8 warps, the cluster's 8 CTAs. `slots` is this CTA's
// [2 halves][V] exchange area (a different one per call site, so one cluster barrier suffices).
template <int V, bool kMax>
__device__ __forceinline__ void slab_fold(float (&value)[V], int half, float* warp_scratch, float* slots, cg::cluster_group& cluster) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int e = 0; e < V; ++e) {
#pragma unroll
    for (int offset = 2; offset < 32; offset <<= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, value[e], offset);
      value[e] = kMax ? fmaxf(value[e], other) : value[e] + other;
    }
  }
  if (lane < 2) {
#pragma unroll
    for (int e = 0; e < V; ++e) warp_scratch[(warp * 2 + lane) * V + e] = value[e];   // lane 0: half 0, lane 1: half 1
  }
  __syncthreads();
  if (threadIdx.x < 2 * V) {
    const int h = threadIdx.x / V, e = threadIdx.x % V;
    float total = warp_scratch[h * V + e];
    for (int w = 1; w < kSlabWarps; ++w) {
      const float other = warp_scratch[(w * 2 + h) * V + e];
      total = kMax ? fmaxf(total, other) : total + other;
    }
    slots[h * V + e] = total;
  }
  cluster.sync();
#pragma unroll
  for (int e = 0; e < V; ++e) {
    float total = *cluster.map_shared_rank(slots + half * V + e, 0);
    for (int r = 1; r < kSlabCluster; ++r) {
      const float other = *cluster.map_shared_rank(slots + half * V + e, r);
      total = kMax ? fmaxf(total, other) : total + other;
    }
    value[e] = total;
  }
}

// KIND 0: softmax, KIND 1: LayerNorm. grid = (cols / (2 V)) * batch clusters of 8 CTAs.
template <typename T, int KIND>
__global__ void __launch_bounds__(kSlabThreads, 1) slab_normalize_kernel(SlabArgs args) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  constexpr float kLog2e = 1.4426950408889634f;
  extern __shared__ __align__(128) unsigned char slab_smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = static_cast<int>(cluster.block_rank());
  const long long slab = blockIdx.x / kSlabCluster;
  const long long slabs_per_matrix = args.cols / (2 * V);
  const long long batch = slab / slabs_per_matrix;
  const long long c0 = (slab % slabs_per_matrix) * (2 * V);
  const int rows_here = args.rows_per_cta;
  const long long row0 = static_cast<long long>(rank) * rows_here;
  const T* source = static_cast<const T*>(args.in) + batch * args.rows * args.cols;
  T* target = static_cast<T*>(args.out) + batch * args.rows * args.cols;

  uint4* data = reinterpret_cast<uint4*>(slab_smem);                                  // rows_here * 2 units
  float* warp_scratch = reinterpret_cast<float*>(slab_smem + static_cast<size_t>(rows_here) * 32);   // [8 warps][2][V]
  float* slots_a = warp_scratch + kSlabWarps * 2 * V;                                 // [2][V], and three more like it
  float* slots_b = slots_a + 2 * V;
  float* slots_c = slots_b + 2 * V;

  // ---- the slab comes in: every 16-byte unit of this CTA's rows, all in flight at once ----------
  const int half = threadIdx.x & 1;
  const int first_row = threadIdx.x >> 1;
  for (int row = first_row; row < rows_here; row += kSlabRowsPerPass) {
    const uint32_t slot = static_cast<uint32_t>(__cvta_generic_to_shared(data + slab_unit<V>(row, half)));
    const T* from = source + (row0 + row) * args.cols + c0 + half * V;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(slot), "l"(from) : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  // from here to the last cluster barrier a thread reads only the units it copied itself

  float first[V], second[V];        // softmax: maximum, 1 / sum;  LayerNorm: mean, 1 / sqrt(variance + eps)
  if constexpr (KIND == 0) {
#pragma unroll
    for (int e = 0; e < V; ++e) first[e] = __int_as_float(0xff800000);   // -inf
    for (int row = first_row; row < rows_here; row += kSlabRowsPerPass) {
      const uint4 raw = data[slab_unit<V>(row, half)];
      const Vec<T, V> x = *reinterpret_cast<const Vec<T, V>*>(&raw);
#pragma unroll
      for (int e = 0; e < V; ++e) first[e] = fmaxf(first[e], to_compute(x.v[e]));
    }
    slab_fold<V, true>(first, half, warp_scratch, slots_a, cluster);
    // fmaxf drops a NaN, but exp2(NaN - max) below brings it into the sum: the whole column becomes NaN, as on the host
#pragma unroll
    for (int e = 0; e < V; ++e) second[e] = 0.f;
    for (int row = first_row; row < rows_here; row += kSlabRowsPerPass) {
      const uint4 raw = data[slab_unit<V>(row, half)];
      const Vec<T, V> x = *reinterpret_cast<const Vec<T, V>*>(&raw);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        float term;
        const float t = (to_compute(x.v[e]) - first[e]) * kLog2e;      // inf - inf = NaN: a column with +inf is NaN, as on the host
        asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(term) : "f"(t));
        second[e] += term;
      }
    }
    slab_fold<V, false>(second, half, warp_scratch, slots_b, cluster);
#pragma unroll
    for (int e = 0; e < V; ++e) second[e] = 1.0f / second[e];
  } else {
#pragma unroll
    for (int e = 0; e < V; ++e) first[e] = 0.f;
    for (int row = first_row; row < rows_here; row += kSlabRowsPerPass) {
      const uint4 raw = data[slab_unit<V>(row, half)];
      const Vec<T, V> x = *reinterpret_cast<const Vec<T, V>*>(&raw);
#pragma unroll
      for (int e = 0; e < V; ++e) first[e] += to_compute(x.v[e]);
    }
    slab_fold<V, false>(first, half, warp_scratch, slots_a, cluster);
    const float count = static_cast<float>(args.rows);
#pragma unroll
    for (int e = 0; e < V; ++e) {
      first[e] /= count;
      second[e] = 0.f;
    }
    for (int row = first_row; row < rows_here; row += kSlabRowsPerPass) {
      const uint4 raw = data[slab_unit<V>(row, half)];
      const Vec<T, V> x = *reinterpret_cast<const Vec<T, V>*>(&raw);
#pragma unroll
      for (int e = 0; e < V; ++e) {
        const float d = to_compute(x.v[e]) - first[e];
        second[e] = fmaf(d, d, second[e]);
      }
    }
    slab_fold<V, false>(second, half, warp_scratch, slots_b, cluster);
#pragma unroll
    for (int e = 0; e < V; ++e) second[e] = rsqrtf(second[e] / count + args.eps);
  }

  // Every thread now holds the statistics of ITS half's V columns; the writers below are grouped by
  // half per warp, so pass them through shared memory once.
  if (threadIdx.x < 2) {
#pragma unroll
    for (int e = 0; e < V; ++e) {
      slots_c[(half * V + e) * 2 + 0] = first[e];
      slots_c[(half * V + e) * 2 + 1] = second[e];
    }
  }
  __syncthreads();   // also: from here on threads read units other threads copied (each waited for its own)

  // ---- out: V x V blocks, transposed in registers; a warp writes 32 x 16 bytes of one output row --
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int out_half = warp & 1;
  float mean_or_max[V], scale_of[V];
#pragma unroll
  for (int e = 0; e < V; ++e) {
    mean_or_max[e] = slots_c[(out_half * V + e) * 2 + 0];
    scale_of[e] = slots_c[(out_half * V + e) * 2 + 1];
  }
  const int blocks_here = rows_here / V;
  for (int block = (warp >> 1) * 32 + lane; block < blocks_here; block += (kSlabWarps / 2) * 32) {
    Vec<T, V> rows_of[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const uint4 raw = data[slab_unit<V>(block * V + i, out_half)];
      rows_of[i] = *reinterpret_cast<const Vec<T, V>*>(&raw);
    }
    float gain[V], offset[V];     // LayerNorm: per row of the input (= per element of the output row)
    if constexpr (KIND == 1) {
      const long long r = row0 + static_cast<long long>(block) * V;
      Vec<T, V> w, b;
      if (args.weight != nullptr) w = *reinterpret_cast<const Vec<T, V>*>(static_cast<const T*>(args.weight) + r);
      if (args.bias != nullptr) b = *reinterpret_cast<const Vec<T, V>*>(static_cast<const T*>(args.bias) + r);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        gain[i] = args.weight != nullptr ? to_compute(w.v[i]) : 1.0f;
        offset[i] = args.bias != nullptr ? to_compute(b.v[i]) : 0.0f;
      }
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
      Vec<T, V> line;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float x = to_compute(rows_of[i].v[j]);
        float y;
        if constexpr (KIND == 0) {
          float term;
          const float t = (x - mean_or_max[j]) * kLog2e;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(term) : "f"(t));
          y = term * scale_of[j];
        } else {
          y = (x - mean_or_max[j]) * scale_of[j] * gain[i] + offset[i];
        }
        line.v[i] = from_compute<T, float>(y);
      }
      store_stream<T, V>(target + (c0 + out_half * V + j) * args.rows + row0 + static_cast<long long>(block) * V, line);
    }
  }
  cluster.sync();   // nobody leaves while a peer may still read its exchange slots
}

template <typename T, int KIND>
tq_status slab_launch(const SlabArgs& args, long long batch, cudaStream_t stream) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  const size_t smem = static_cast<size_t>(args.rows_per_cta) * 32 + (kSlabWarps * 2 * V + 3 * 2 * V + 2 * V) * sizeof(float) + 128;
  static std::mutex mutex;
  {
    std::lock_guard<std::mutex> lock(mutex);
    TQ_CUDA(cudaFuncSetAttribute(slab_normalize_kernel<T, KIND>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  }
  const long long clusters = (args.cols / (2 * V)) * batch;
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(clusters * kSlabCluster));
  config.blockDim = dim3(kSlabThreads);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = kSlabCluster;
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  TQ_CUDA(cudaLaunchKernelEx(&config, slab_normalize_kernel<T, KIND>, args));
  return check_launch("slab_normalize_kernel");
}

}  // namespace

// Whether a shape takes the one-pass kernel. Measured on B200: it wins (up to 2.7x for LayerNorm)
// while the tensor is at most 32 MiB, so that the 32-byte pieces of neighbouring slabs meet in L2, and
// the columns are long (from 8192 rows: 1024 per CTA); past that the pieces, a whole row of the
// tensor apart, each open a DRAM page of their own and the two-launch form is ahead.
bool slab_takes(tq_dtype dtype, long long batch, long long rows, long long cols) {
  const int size = dtype_size(dtype);
  if (size != 2 && size != 4) return false;
  const int v = 16 / size;
  if (rows % (kSlabCluster * v) != 0 || cols % (2 * v) != 0) return false;
  const long long rows_per_cta = rows / kSlabCluster;
  if (rows_per_cta < kSlabRowsPerPass || static_cast<size_t>(rows_per_cta) * 32 > kSlabMaxDataBytes) return false;
  if (batch != 0 && (rows < 8192 || batch * rows * cols * size > (32ll << 20))) return false;
  if (batch != 0 && (cols / (2 * v)) * batch * kSlabCluster > 0x7fffffffLL) return false;
  return true;
}

// Launches and sets `*handled` when slab_takes() and the pointers are 16-byte aligned; otherwise
// launches nothing and the caller runs its statistics-then-normalise pair.
tq_status slab_normalize_launch(int kind, tq_dtype dtype, const void* in, void* out, const void* weight, const void* bias,
                                long long batch, long long rows, long long cols, float eps, cudaStream_t stream, bool* handled) {
  *handled = false;
  if (!slab_takes(dtype, batch, rows, cols)) return TQ_OK;
  if (!aligned_to(in, 16) || !aligned_to(out, 16) || (weight != nullptr && !aligned_to(weight, 16)) || (bias != nullptr && !aligned_to(bias, 16))) return TQ_OK;
  const long long rows_per_cta = rows / kSlabCluster;
  SlabArgs args = {};
  args.in = in;
  args.out = out;
  args.weight = weight;
  args.bias = bias;
  args.rows = rows;
  args.cols = cols;
  args.rows_per_cta = static_cast<int>(rows_per_cta);
  args.eps = eps;
  *handled = true;
#define TQ_SLAB(T) return kind == 0 ? slab_launch<T, 0>(args, batch, stream) : slab_launch<T, 1>(args, batch, stream)
  switch (dtype) {
    case TQ_F32: TQ_SLAB(float);
    case TQ_F16: TQ_SLAB(__half);
    case TQ_BF16: TQ_SLAB(__nv_bfloat16);
    default: *handled = false; return TQ_OK;
  }
#undef TQ_SLAB
}

}  // namespace tq
