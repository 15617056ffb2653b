// Reductions over a packed [outer, reduce, inner] view: sum, mean, amax, amin, argmax.
//
// Three kernel shapes, chosen on the host by plan():
//   warp-per-slice   inner == 1, many slices of moderate length: each warp streams one slice with
//                    128-bit loads and finishes with shuffles; no shared memory, no barrier.
//   cta-per-slice    inner == 1, long or few slices: `split` CTAs stream one slice; warp shuffle,
//                    then shared memory, then distributed shared memory across the thread-block
//                    cluster, then (only when a slice spans more than one cluster) per-cluster
//                    partials in scratch memory that the last cluster to arrive combines.
//   columns          inner > 1: threads run along `inner` (coalesced), warps along `reduce`;
//                    the same cluster / scratch steps when `reduce` is split.
// No wait anywhere: the "last to arrive" step uses a ticket, not a spin.
//
// Semantics follow the reference's reduction kernels (csrc/tessiq/codegen/cuda_emitter.cpp:159-210):
// mean divides once after the sum, amax/amin propagate NaN. argmax returns the first index of the
// maximum with NaN counted as the maximum, which is what aten.argmax computes on the reference's
// host device.
#include <cooperative_groups.h>

#include <algorithm>
#include <cstdlib>
#include <limits>
#include <mutex>
#include <type_traits>

#include "common.h"
#include "reducers.h"
#include "tcgen05.h"

namespace cg = cooperative_groups;

namespace tq {
namespace {

constexpr int kBlock = 256;
constexpr int kWarps = kBlock / 32;
constexpr int kUnroll = 4;
constexpr int kMaxCluster = 8;
constexpr int kRingDepth = 8;   // columns kernel: rows in flight per thread (cp.async ring)

// ---------------------------------------------------------------------------------------------
// Reducers

template <typename T>
struct SumReducer {
  static constexpr bool kSeeded = false;   // no seed / step_seeded / set_count protocol (see MomentsReducer)
  using C = typename Compute<T>::type;
  using Acc = std::conditional_t<std::is_integral_v<C>, long long, C>;
  using Out = std::conditional_t<std::is_same_v<T, int>, long long, T>;
  __device__ static Acc identity() { return Acc(0); }
  __device__ static Acc lift(T v, long long) { return static_cast<Acc>(to_compute(v)); }
  __device__ static Acc combine(Acc a, Acc b) { return a + b; }
  __device__ static Acc shuffle(Acc a, int offset) { return shfl_xor(a, offset); }
  template <int VEC> using Local = Acc;
  template <int VEC> __device__ static Acc local_identity() { return identity(); }
  template <int VEC> __device__ static void step(Acc& local, T v, long long) { local += static_cast<Acc>(to_compute(v)); }
  template <int VEC> __device__ static void step_vector(Acc& local, const Vec<T, VEC>& x, long long) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) local += static_cast<Acc>(to_compute(x.v[e]));
  }
  template <int VEC> __device__ static Acc to_acc(Acc local) { return local; }
  __device__ static Out finish(Acc a, long long count, bool mean) {
    if constexpr (!std::is_integral_v<C>) {
      if (mean) a = a / static_cast<Acc>(count);
      return from_compute<Out, Acc>(a);
    } else {
      return static_cast<Out>(a);
    }
  }
};


template <typename C>
struct alignas(16) Indexed {
  C value;
  long long index;
};

template <typename T>
struct ArgmaxReducer {
  static constexpr bool kSeeded = false;   // no seed / step_seeded / set_count protocol (see MomentsReducer)
  using C = typename Compute<T>::type;
  using Acc = Indexed<C>;
  using Out = long long;
  __device__ static Acc identity() {
    Acc a;
    if constexpr (std::is_integral_v<C>) {
      a.value = std::numeric_limits<C>::lowest();
    } else {
      a.value = -std::numeric_limits<C>::infinity();
    }
    a.index = std::numeric_limits<long long>::max();
    return a;
  }
  __device__ static Acc lift(T v, long long index) {
    Acc a;
    a.value = to_compute(v);
    a.index = index;
    return a;
  }
  // A total order: NaN above everything, then the value, then the lower index.
  __device__ static Acc combine(Acc a, Acc b) {
    bool a_nan = false, b_nan = false;
    if constexpr (!std::is_integral_v<C>) {
      a_nan = a.value != a.value;
      b_nan = b.value != b.value;
    }
    bool take_b;
    if (a_nan || b_nan) {
      take_b = (a_nan && b_nan) ? (b.index < a.index) : b_nan;
    } else if (a.value == b.value) {
      take_b = b.index < a.index;
    } else {
      take_b = b.value > a.value;
    }
    return take_b ? b : a;
  }
  __device__ static Acc shuffle(Acc a, int offset) {
    Acc b;
    b.value = shfl_xor(a.value, offset);
    b.index = shfl_xor(a.index, offset);
    return b;
  }
  // Within one thread the positions only grow, so a strict comparison keeps the first of equal
  // values and the thread needs no index comparison. A thread looks at one vector at a time: the
  // vector's NaN-propagating maximum (packed two-at-a-time for the half types) is compared with
  // the best so far, and a vector that beats it is kept whole together with its position; which
  // element of the kept vector won is resolved once, at the end. Positions are kept in 32 bits
  // (the host declines longer slices). `!(m <= best)` is true for a larger value and for a NaN;
  // the second test freezes the state once `best` itself is a NaN.
  template <int VEC>
  struct Local {
    C best;
    unsigned base;
    Vec<T, VEC> winner;
  };
  static constexpr unsigned kNone = 0xffffffffu;
  template <int VEC> __device__ static Local<VEC> local_identity() {
    Local<VEC> l;
    l.best = identity().value;
    l.base = kNone;
#pragma unroll
    for (int e = 0; e < VEC; ++e) l.winner.v[e] = T();
    return l;
  }
  __device__ static bool beats(C value, C best) {
    if constexpr (std::is_integral_v<C>) {
      return value > best;
    } else {
      return !(value <= best) && (best == best);
    }
  }
  template <int VEC> __device__ static void step(Local<VEC>& local, T v, long long index) {
    const C value = to_compute(v);
    if (beats(value, local.best)) {
      local.best = value;
      local.base = static_cast<unsigned>(index);
#pragma unroll
      for (int e = 0; e < VEC; ++e) local.winner.v[e] = v;
    }
  }
  // (Testing once per row of V neighbouring columns whether any of them beats its best, as the softmax
  // statistics do, measured 123 us against 86 at [32768, 4096]: a column of random values has a new
  // maximum in about ln(n) of its n rows, and with 32 lanes x V columns per warp nearly every row has one
  // somewhere in the warp, so the rare path ran for every row.)
  template <int VEC> __device__ static C vector_max(const Vec<T, VEC>& x) {
    if constexpr (std::is_same_v<T, __nv_bfloat16> && VEC % 2 == 0) {
      const __nv_bfloat162* pairs = reinterpret_cast<const __nv_bfloat162*>(&x);
      __nv_bfloat162 m = pairs[0];
#pragma unroll
      for (int i = 1; i < VEC / 2; ++i) m = __hmax2_nan(m, pairs[i]);
      return ExtremeReducer<float, true>::combine(__low2float(m), __high2float(m));
    } else if constexpr (std::is_same_v<T, __half> && VEC % 2 == 0) {
      const __half2* pairs = reinterpret_cast<const __half2*>(&x);
      __half2 m = pairs[0];
#pragma unroll
      for (int i = 1; i < VEC / 2; ++i) m = __hmax2_nan(m, pairs[i]);
      return ExtremeReducer<float, true>::combine(__low2float(m), __high2float(m));
    } else {
      C m = to_compute(x.v[0]);
#pragma unroll
      for (int e = 1; e < VEC; ++e) m = ExtremeReducer<C, true>::combine(m, to_compute(x.v[e]));
      return m;
    }
  }
  template <int VEC> __device__ static void step_vector(Local<VEC>& local, const Vec<T, VEC>& x, long long index) {
    const C m = vector_max<VEC>(x);
    if (beats(m, local.best)) {
      local.best = m;
      local.base = static_cast<unsigned>(index);
      local.winner = x;
    }
  }
  template <int VEC> __device__ static Acc to_acc(const Local<VEC>& local) {
    Acc a;
    a.value = local.best;
    a.index = std::numeric_limits<long long>::max();
    if (local.base != kNone) {
      int offset = 0;
#pragma unroll
      for (int e = VEC - 1; e >= 0; --e) {
        const C w = to_compute(local.winner.v[e]);
        const bool same = (w == local.best) || (w != w && local.best != local.best);
        if (same) offset = e;
      }
      a.index = static_cast<long long>(local.base) + offset;
    }
    return a;
  }
  // No position was ever taken only if every element equals the identity (-inf, or the lowest
  // integer): the first of equal values is position 0.
  __device__ static Out finish(Acc a, long long, bool) {
    return a.index == std::numeric_limits<long long>::max() ? 0 : a.index;
  }
};



// The local part of a reduction over a tensor that is split over several GPUs (collective.cu): the
// result is a two-float partial that an all-reduce can combine. A sum's partial is {sum in f32, 0}
// (the f32 accumulator itself: a bf16 tensor's partial is not rounded to bf16 first).
template <typename T>
struct SumPartialReducer : SumReducer<T> {
  using Out = float2;
  using Acc = typename SumReducer<T>::Acc;
  __device__ static Out finish(Acc a, long long, bool) { return make_float2(static_cast<float>(a), 0.f); }
};

// A maximum's partial is {maximum with a NaN replaced by -inf, 1 if a NaN was seen}, to be combined
// with MAX on both words; a minimum's {minimum with a NaN replaced by +inf, -1 if a NaN was seen},
// combined with MIN: a collective's maximum does not promise to propagate NaN, the flag does.
template <typename T, bool kMax>
struct ExtremePartialReducer : ExtremeReducer<T, kMax> {
  using Out = float2;
  using Acc = typename ExtremeReducer<T, kMax>::Acc;
  __device__ static Out finish(Acc a, long long, bool) {
    const float value = static_cast<float>(a);
    if (value != value) return make_float2(kMax ? -std::numeric_limits<float>::infinity() : std::numeric_limits<float>::infinity(), kMax ? 1.f : -1.f);
    return make_float2(value, 0.f);
  }
};

// Reads a partial another CTA wrote, from L2 (never a stale L1 line).
template <typename A>
__device__ __forceinline__ A load_partial(const A* pointer) {
  if constexpr (sizeof(A) == 16) {
    uint4 raw = __ldcg(reinterpret_cast<const uint4*>(pointer));
    return *reinterpret_cast<A*>(&raw);
  } else if constexpr (sizeof(A) == 8) {
    unsigned long long raw = __ldcg(reinterpret_cast<const unsigned long long*>(pointer));
    return *reinterpret_cast<A*>(&raw);
  } else {
    static_assert(sizeof(A) == 4, "accumulators are 4, 8 or 16 bytes");
    unsigned raw = __ldcg(reinterpret_cast<const unsigned*>(pointer));
    return *reinterpret_cast<A*>(&raw);
  }
}

template <typename R>
__device__ __forceinline__ typename R::Acc warp_reduce(typename R::Acc a) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) a = R::combine(a, R::shuffle(a, offset));
  return a;
}

// All threads call; the result is valid on thread 0.
template <typename R>
__device__ __forceinline__ typename R::Acc block_reduce(typename R::Acc a, typename R::Acc* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  a = warp_reduce<R>(a);
  __syncthreads();  // scratch may still be read from an earlier use
  if (lane == 0) scratch[warp] = a;
  __syncthreads();
  if (warp == 0) {
    a = lane < kWarps ? scratch[lane] : R::identity();
    a = warp_reduce<R>(a);
  }
  return a;
}

// Folds elements [begin, end) of `row` into `acc`, `threads` threads cooperating, this one being
// `tid`. The span is cut into a scalar head up to the first 16-byte boundary, a body of VEC-wide
// streaming loads, and a scalar tail, so that any element-aligned pointer works.
template <typename T, typename R, int VEC>
__device__ __forceinline__ void fold_span(const T* __restrict__ row, long long begin, long long end,
                                          int tid, int threads, typename R::template Local<VEC>& acc) {
  if (begin >= end) return;
  const T* start = row + begin;
  long long head = 0;
  if constexpr (VEC > 1) {
    const unsigned misaligned =
        static_cast<unsigned>(reinterpret_cast<uintptr_t>(start) % (sizeof(T) * VEC)) / sizeof(T);
    head = misaligned ? (VEC - misaligned) : 0;
    if (head > end - begin) head = end - begin;
    if (tid < head) R::template step<VEC>(acc, start[tid], begin + tid);
  }
  const long long body = begin + head;
  const long long vectors = (end - body) / VEC;
  const T* vector_base = row + body;
  for (long long v = tid; v < vectors; v += static_cast<long long>(threads) * kUnroll) {
    Vec<T, VEC> x[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long vi = v + static_cast<long long>(u) * threads;
      if (vi < vectors) x[u] = load_stream<T, VEC>(vector_base + vi * VEC);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const long long vi = v + static_cast<long long>(u) * threads;
      if (vi < vectors) R::template step_vector<VEC>(acc, x[u], body + vi * VEC);
    }
  }
  const long long tail = body + vectors * VEC + tid;
  if (tail < end) R::template step<VEC>(acc, row[tail], tail);
}

// ---------------------------------------------------------------------------------------------
// Kernels

// One warp per slice. grid.x * kWarps >= outer.
template <typename T, typename R, int VEC>
__global__ void __launch_bounds__(kBlock)
reduce_warp_per_slice(const T* __restrict__ in, typename R::Out* __restrict__ out, long long outer,
                      long long reduce, int mean) {
  const int lane = threadIdx.x & 31;
  const long long slice = static_cast<long long>(blockIdx.x) * kWarps + (threadIdx.x >> 5);
  if (slice >= outer) return;
  typename R::template Local<VEC> local = R::template local_identity<VEC>();
  fold_span<T, R, VEC>(in + slice * reduce, 0, reduce, lane, 32, local);
  typename R::Acc acc = warp_reduce<R>(R::template to_acc<VEC>(local));
  if (lane == 0) out[slice] = R::finish(acc, reduce, mean != 0);
}

// `split` CTAs per slice, `cluster` of them in one thread-block cluster (cluster divides split).
// blockIdx.x = slice * split + part.
template <typename T, typename R, int VEC>
__global__ void __launch_bounds__(kBlock)
reduce_cta_per_slice(const T* __restrict__ in, typename R::Out* __restrict__ out, long long reduce,
                     int split, int cluster, int mean, typename R::Acc* __restrict__ partials,
                     unsigned* __restrict__ tickets) {
  using Acc = typename R::Acc;
  __shared__ Acc warp_scratch[kWarps];
  __shared__ Acc cluster_scratch[kMaxCluster];
  __shared__ bool is_last;

  const long long slice = blockIdx.x / split;
  const int part = static_cast<int>(blockIdx.x % split);
  // Parts are cut on multiples of the vector width so that only the first can be misaligned.
  long long chunk = (reduce + split - 1) / split;
  chunk = (chunk + VEC - 1) / VEC * VEC;
  const long long begin = static_cast<long long>(part) * chunk;
  long long end = begin + chunk;
  if (end > reduce) end = reduce;

  typename R::template Local<VEC> local = R::template local_identity<VEC>();
  fold_span<T, R, VEC>(in + slice * reduce, begin, end, threadIdx.x, kBlock, local);
  Acc acc = block_reduce<R>(R::template to_acc<VEC>(local), warp_scratch);

  if (cluster > 1) {
    cg::cluster_group group = cg::this_cluster();
    const unsigned rank = group.block_rank();
    if (threadIdx.x == 0) {
      Acc* leader = group.map_shared_rank(cluster_scratch, 0);
      leader[rank] = acc;
    }
    group.sync();
    if (rank != 0) return;
    if (threadIdx.x == 0) {
      acc = cluster_scratch[0];
      for (int j = 1; j < cluster; ++j) acc = R::combine(acc, cluster_scratch[j]);
    }
  }

  const int clusters = split / cluster;
  if (clusters == 1) {
    if (threadIdx.x == 0) out[slice] = R::finish(acc, reduce, mean != 0);
    return;
  }

  if (threadIdx.x == 0) {
    partials[slice * clusters + part / cluster] = acc;
    __threadfence();
    const unsigned ticket = atomicAdd(&tickets[slice], 1u);
    is_last = ticket == static_cast<unsigned>(clusters - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  Acc total = R::identity();
  for (int j = threadIdx.x; j < clusters; j += kBlock) {
    total = R::combine(total, load_partial(partials + slice * clusters + j));
  }
  total = block_reduce<R>(total, warp_scratch);
  if (threadIdx.x == 0) out[slice] = R::finish(total, reduce, mean != 0);
}

// inner > 1. Thread layout: tx = threadIdx.x % lanes_x runs along inner (VEC columns each),
// ty = threadIdx.x / lanes_x along reduce. grid = (column tiles, split, outer); the cluster, when
// there is one, runs along grid.y.
template <typename T, typename R, int VEC, bool RING>
__global__ void __launch_bounds__(kBlock, sizeof(typename R::Acc) > 8 ? 4 : 5)
reduce_columns(const T* __restrict__ in, typename R::Out* __restrict__ out, long long reduce,
               long long inner, int lanes_x, int split, int cluster, int mean,
               typename R::Acc* __restrict__ partials, unsigned* __restrict__ tickets) {
  using Acc = typename R::Acc;
  extern __shared__ __align__(16) unsigned char dynamic_smem[];
  Acc* rows_scratch = reinterpret_cast<Acc*>(dynamic_smem);              // [kBlock * VEC]
  Acc* cluster_scratch = rows_scratch + kBlock * VEC;                    // [lanes_x * VEC]
  __shared__ bool is_last;

  const int tx = threadIdx.x % lanes_x;
  const int ty = threadIdx.x / lanes_x;
  const int lanes_y = kBlock / lanes_x;
  const long long slice = blockIdx.z;
  const int part = blockIdx.y;
  const long long column = (static_cast<long long>(blockIdx.x) * lanes_x + tx) * VEC;
  const bool in_range = column < inner;

  long long chunk = (reduce + split - 1) / split;
  const long long begin = static_cast<long long>(part) * chunk;
  long long end = begin + chunk;
  if (end > reduce) end = reduce;

  typename R::template Local<1> local[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) local[e] = R::template local_identity<1>();

  if (in_range) {
    const T* base = in + slice * reduce * inner + column;
    constexpr int kBytes = static_cast<int>(sizeof(T)) * VEC;
    constexpr int UNROLL = kUnroll;
    if constexpr (RING && (kBytes == 4 || kBytes == 8 || kBytes == 16)) {
      // Each thread streams its own column vector through a private ring of kRingDepth slots in
      // shared memory with cp.async: the copies in flight cost no registers, so a thread keeps
      // kRingDepth - 1 rows (up to 112 bytes) on their way from HBM while it folds the oldest.
      // A slot is written and read by the same thread only, so no barrier is involved.
      // The loop is unrolled by the ring's depth, so slot addresses are constants, the source is a
      // pointer that advances by one stride, and the count is 32 bits: per row a wait, a shared
      // load, a copy, a commit and a pointer add besides the reducer's own work (the rolled form
      // with 64-bit index arithmetic spent 18 instructions per element on 4-byte moments and made
      // every 2-byte column reduction issue-bound).
      Vec<T, VEC>* ring = reinterpret_cast<Vec<T, VEC>*>(cluster_scratch + lanes_x * VEC) + threadIdx.x;     // slot d at + d * kBlock
      const uint32_t ring_address = static_cast<uint32_t>(__cvta_generic_to_shared(ring));
      constexpr uint32_t kSlotBytes = static_cast<uint32_t>(kBlock) * kBytes;
      const long long first = begin + ty;
      const int count = first < end ? static_cast<int>((end - first + lanes_y - 1) / lanes_y) : 0;   // the host keeps this below 2^31
      const T* source = base + first * inner;
      const long long stride = static_cast<long long>(lanes_y) * inner;
      long long ri = first;
      auto copy = [&](int slot) {
        if constexpr (kBytes == 16) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ring_address + slot * kSlotBytes), "l"(source) : "memory");
        } else {
          asm volatile("cp.async.ca.shared.global [%0], [%1], %2;" ::"r"(ring_address + slot * kSlotBytes), "l"(source), "n"(kBytes) : "memory");
        }
        source += stride;
      };
      if constexpr (R::kSeeded) {
        if (count > 0) {
          const Vec<T, VEC> x = load_stream<T, VEC>(source);
#pragma unroll
          for (int e = 0; e < VEC; ++e) R::template seed<1>(local[e], x.v[e]);
        }
      }
#pragma unroll
      for (int d = 0; d < kRingDepth - 1; ++d) {
        if (d < count) copy(d);
        asm volatile("cp.async.commit_group;" ::: "memory");   // one group per row, empty past the end
      }
      for (int i = 0; i < count; i += kRingDepth) {
#pragma unroll
        for (int d = 0; d < kRingDepth; ++d) {
          if (i + d < count) {
            asm volatile("cp.async.wait_group %0;" ::"n"(kRingDepth - 2) : "memory");   // row i + d has landed
            const Vec<T, VEC> x = ring[d * kBlock];
            if constexpr (R::kSeeded) {
#pragma unroll
              for (int e = 0; e < VEC; ++e) R::template step_seeded<1>(local[e], x.v[e]);
            } else if constexpr (has_column_step<R>::value) {
              R::template step_columns<VEC>(local, x, ri);
              ri += lanes_y;
            } else {
#pragma unroll
              for (int e = 0; e < VEC; ++e) R::template step<1>(local[e], x.v[e], ri);
              ri += lanes_y;
            }
            if (i + d + kRingDepth - 1 < count) copy((d + kRingDepth - 1) % kRingDepth);   // into the slot read one row ago
            asm volatile("cp.async.commit_group;" ::: "memory");
          }
        }
      }
      asm volatile("cp.async.wait_group 0;" ::: "memory");
      if constexpr (R::kSeeded) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) R::template set_count<1>(local[e], count);
      }
    } else {
      for (long long r = begin + ty; r < end; r += static_cast<long long>(lanes_y) * UNROLL) {
        Vec<T, VEC> x[UNROLL];
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long ri = r + static_cast<long long>(u) * lanes_y;
          if (ri < end) x[u] = load_stream<T, VEC>(base + ri * inner);
        }
#pragma unroll
        for (int u = 0; u < UNROLL; ++u) {
          const long long ri = r + static_cast<long long>(u) * lanes_y;
          if (ri < end) {
            if constexpr (has_column_step<R>::value) {
              R::template step_columns<VEC>(local, x[u], ri);
            } else {
#pragma unroll
              for (int e = 0; e < VEC; ++e) R::template step<1>(local[e], x[u].v[e], ri);
            }
          }
        }
      }
    }
  }

  // Across ty, through shared memory, in a fixed order.
  Acc acc[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) acc[e] = R::template to_acc<1>(local[e]);
#pragma unroll
  for (int e = 0; e < VEC; ++e) rows_scratch[(ty * lanes_x + tx) * VEC + e] = acc[e];
  __syncthreads();
  const bool holder = ty == 0;
  if (holder) {
    for (int y = 1; y < lanes_y; ++y) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        acc[e] = R::combine(acc[e], rows_scratch[(y * lanes_x + tx) * VEC + e]);
      }
    }
  }

  // Across the CTAs of the cluster: a reduce-scatter through distributed shared memory. The
  // tile's `items` accumulators are cut into `cluster` equal slices; every CTA sends slice q of
  // its accumulators to CTA q, one cluster barrier, and CTA q folds what it received in rank
  // order. Each CTA then owns items [rank * slice_items, (rank + 1) * slice_items) of the tile.
  const int items = lanes_x * VEC;
  const int slice_items = items / cluster;  // a multiple of VEC: cluster <= lanes_x, both powers of 2
  unsigned rank = 0;
  typename R::Out* out_row = out + slice * inner;
  const long long tile_column = static_cast<long long>(blockIdx.x) * items;
  const int clusters = split / cluster;
  const long long tile = slice * gridDim.x + blockIdx.x;
  Acc* tile_partials = partials + tile * clusters * items;

  if (cluster > 1) {
    cg::cluster_group group = cg::this_cluster();
    rank = group.block_rank();
    if (holder) {
      const int item = tx * VEC;
      Acc* owner = group.map_shared_rank(cluster_scratch, item / slice_items);
#pragma unroll
      for (int e = 0; e < VEC; ++e) owner[rank * slice_items + item % slice_items + e] = acc[e];
    }
    group.sync();
    // Thread t < slice_items now finishes item rank * slice_items + t.
    if (threadIdx.x < slice_items) {
      Acc total = cluster_scratch[threadIdx.x];
      for (int j = 1; j < cluster; ++j) total = R::combine(total, cluster_scratch[j * slice_items + threadIdx.x]);
      const int item = rank * slice_items + threadIdx.x;
      if (clusters == 1) {
        if (tile_column + item < inner) out_row[tile_column + item] = R::finish(total, reduce, mean != 0);
      } else {
        tile_partials[(part / cluster) * items + item] = total;
      }
    }
    if (clusters == 1) return;
  } else {
    if (clusters == 1) {
      if (holder && in_range) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) out_row[column + e] = R::finish(acc[e], reduce, mean != 0);
      }
      return;
    }
    if (holder) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) tile_partials[part * items + tx * VEC + e] = acc[e];
    }
  }

  // Across clusters: every CTA has written its share of its cluster's partial; the last CTA of
  // the tile to take a ticket folds the `clusters` partials of every item, all threads at work,
  // eight loads in flight each, in a fixed order.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned ticket = atomicAdd(&tickets[tile], 1u);
    is_last = ticket == static_cast<unsigned>(split - 1);
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int item = threadIdx.x; item < items; item += kBlock) {
    if (tile_column + item >= inner) continue;
    Acc total = R::identity();
    for (int j = 0; j < clusters; j += 4) {
      Acc batch[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (j + u < clusters) batch[u] = load_partial(tile_partials + static_cast<long long>(j + u) * items + item);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (j + u < clusters) total = R::combine(total, batch[u]);
      }
    }
    out_row[tile_column + item] = R::finish(total, reduce, mean != 0);
  }
}

// ---------------------------------------------------------------------------------------------
// inner > 1, large tensors: the persistent streaming form. The tensor is cut into panels of columns
// (512 bytes of every row) and a panel into units of 64 rows; a unit is one TMA tile (32 KiB). The
// units, panel after panel, are dealt out as one contiguous range per CTA (one CTA per SM), so every
// SM streams the same number of bytes (to within one unit) and a panel is shared by the few CTAs
// whose ranges meet it. One lane issues the tile loads into a ring of shared-memory stages; eight
// consumer warps fold the rows (warp w rows w, w + 8, ... of a unit, a lane 16 bytes of a row). Where
// a CTA's range leaves a panel it folds its eight warps' accumulators through shared memory and, if
// it is not the panel's only CTA, leaves one partial per column in scratch; the last CTA of the panel
// to take a ticket folds the partials in row order and writes the results. Replaces the thread-level
// loads of reduce_columns for the shapes where those leave the memory system short of requests:
// per 16 bytes a consumer spends a shared-memory load and the reducer's own work, nothing else.
// Consumer warps: eight, or sixteen for the softmax statistics of 2-byte elements, whose per-element work
// (a scaling, a test, an exponential, an add; 8 elements per 16 bytes) binds before HBM does with eight.
// Measured on B200 at [32768, 4096] bf16: softmax over the view's statistics + normalise 190 us with
// sixteen against 228 with eight (177 against 190 once the reducer stepped eight columns behind one
// test); argmax 63.5 us with sixteen against 58.6 with eight, the moments equal.
template <typename T, typename R>
constexpr int stream_consumers() { return (sizeof(T) == 2 && std::is_same_v<R, SoftmaxStatReducer<T>>) ? 16 : 8; }
constexpr int kStreamPieceBytes = 512;
constexpr int kStreamUnitRows = 64;
constexpr int kStreamStageBytes = kStreamUnitRows * kStreamPieceBytes;
constexpr int kStreamStages = 5;                 // with eight consumer warps; four with sixteen (their accumulators take the room)
constexpr int kStatusStreamData = 0x53544d31;    // "STM1": a unit's data never arrived
constexpr int kStatusStreamRing = 0x53544d32;    // "STM2": a stage was never handed back

struct StreamArgs {
  long long reduce, inner;
  long long units;            // outer * panels per slice * units per panel
  int units_per_panel;        // reduce / 64
  int panels_per_slice;       // inner / columns per panel
  int slots;                  // partial rows reserved per panel
  int mean;
  WaitStatus status;
};

// units * grid stays below 2^32 (the plan declines otherwise), so the kernel's divisions are 32-bit ones:
// a 64-bit division is about a hundred dependent instructions, and a segment's end runs six of them.
__device__ __forceinline__ long long stream_first_unit(long long cta, long long units, long long grid) {
  return static_cast<unsigned>(cta * units) / static_cast<unsigned>(grid);
}

// The CTA whose range holds `unit`.
__device__ __forceinline__ int stream_owner(long long unit, long long units, int grid) {
  long long c = static_cast<unsigned>(unit * grid) / static_cast<unsigned>(units);
  while (c + 1 < grid && stream_first_unit(c + 1, units, grid) <= unit) ++c;
  while (c > 0 && stream_first_unit(c, units, grid) > unit) --c;
  return static_cast<int>(c);
}

template <typename T, typename R>
__global__ void __launch_bounds__((stream_consumers<T, R>() + 1) * 32, 1)
reduce_columns_stream(const __grid_constant__ CUtensorMap map, const StreamArgs args, typename R::Out* __restrict__ out,
                      typename R::Acc* __restrict__ partials, unsigned* __restrict__ tickets) {
  using Acc = typename R::Acc;
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  constexpr int kColumns = 32 * V;
  constexpr int kStreamConsumers = stream_consumers<T, R>();
  constexpr int kStreamStages = kStreamConsumers == 8 ? 5 : 4;      // (hides the namespace's value)
  constexpr int kConsumerThreads = kStreamConsumers * 32;
  constexpr int kRowsPerWarp = kStreamUnitRows / kStreamConsumers;
  extern __shared__ __align__(128) unsigned char stream_smem[];
  __shared__ int is_last;
  unsigned char* ring = stream_smem;
  Acc* scratch = reinterpret_cast<Acc*>(ring + kStreamStages * kStreamStageBytes);   // [8 warps][columns]
  uint64_t* barriers = reinterpret_cast<uint64_t*>(scratch + kStreamConsumers * kColumns);
  const uint32_t full0 = smem_address(barriers), empty0 = full0 + 8 * kStreamStages;
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStreamStages; ++s) {
      barrier_init(full0 + 8 * s, 1);
      barrier_init(empty0 + 8 * s, kStreamConsumers);
    }
    if (blockIdx.x == 0) args.status.begin();
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int grid = static_cast<int>(gridDim.x), cta = static_cast<int>(blockIdx.x);
  const long long first = stream_first_unit(cta, args.units, grid), last = stream_first_unit(cta + 1, args.units, grid);
  const int upp = args.units_per_panel;
  int stage = 0;
  uint32_t phase = 0;

  if (warp == kStreamConsumers) {
    // ---- producer ---------------------------------------------------------------------------------
    if (lane == 0) {
      for (long long u = first; u < last; ++u) {
        const long long panel = static_cast<unsigned>(u) / static_cast<unsigned>(upp);
        const int unit = static_cast<int>(u - panel * upp);
        const long long slice = static_cast<unsigned>(panel) / static_cast<unsigned>(args.panels_per_slice);
        const int column = static_cast<int>(panel - slice * args.panels_per_slice) * kColumns;
        if (!barrier_wait(empty0 + 8 * stage, phase ^ 1, args.status, kStatusStreamRing)) break;
        barrier_expect_tx(full0 + 8 * stage, kStreamStageBytes);
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                         smem_address(ring) + stage * kStreamStageBytes),
                     "l"(&map), "r"(full0 + 8 * stage), "r"(column), "r"(static_cast<int>(slice * args.reduce + static_cast<long long>(unit) * kStreamUnitRows))
                     : "memory");
        if (++stage == kStreamStages) {
          stage = 0;
          phase ^= 1;
        }
      }
      // nothing may still be on its way into this CTA's shared memory when it leaves: the consumers
      // wait for every tile they were promised, and after a give-up the loads already issued are
      // waited for here (a stage that was never armed answers at once)
      if (args.status.aborted()) {
        for (int s = 0; s < kStreamStages; ++s) {
          const uint32_t parity = s < stage ? phase : phase ^ 1;
          for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
            if (barrier_try_wait(full0 + 8 * s, parity)) break;
          }
        }
      }
    }
    return;
  }

  // ---- consumers: a segment is the part of the CTA's range that lies in one panel --------------------
  bool alive = true;
  for (long long u = first; u < last && alive;) {
    const long long panel = static_cast<unsigned>(u) / static_cast<unsigned>(upp);
    const long long panel_first = panel * upp;
    long long segment_end = panel_first + upp;
    if (segment_end > last) segment_end = last;
    typename R::template Local<1> local[V];
#pragma unroll
    for (int e = 0; e < V; ++e) local[e] = R::template local_identity<1>();
    const long long segment_first = u;
    for (; u < segment_end; ++u) {
      if (!barrier_wait(full0 + 8 * stage, phase, args.status, kStatusStreamData)) {
        alive = false;
        break;
      }
      const Vec<T, V>* mine = reinterpret_cast<const Vec<T, V>*>(ring + static_cast<size_t>(stage) * kStreamStageBytes +
                                                                 static_cast<size_t>(warp) * kStreamPieceBytes) + lane;
      long long row = (u - panel_first) * kStreamUnitRows + warp;   // within the slice
      if constexpr (R::kSeeded) {
        if (u == segment_first) {
          const Vec<T, V> x = mine[0];
#pragma unroll
          for (int e = 0; e < V; ++e) R::template seed<1>(local[e], x.v[e]);
        }
      }
#pragma unroll
      for (int i = 0; i < kRowsPerWarp; ++i) {
        const Vec<T, V> x = mine[i * kStreamConsumers * (kStreamPieceBytes / 16)];
        if constexpr (has_column_step<R>::value) {
          R::template step_columns<V>(local, x, row);
        } else {
#pragma unroll
          for (int e = 0; e < V; ++e) {
            if constexpr (R::kSeeded) {
              R::template step_seeded<1>(local[e], x.v[e]);
            } else {
              R::template step<1>(local[e], x.v[e], row);
            }
          }
        }
        row += kStreamConsumers;
      }
      __syncwarp();
      if (lane == 0) barrier_arrive(empty0 + 8 * stage);
      if (++stage == kStreamStages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (!alive) break;
    if constexpr (R::kSeeded) {
#pragma unroll
      for (int e = 0; e < V; ++e) R::template set_count<1>(local[e], static_cast<int>(segment_end - segment_first) * kRowsPerWarp);
    }
    // the eight warps' accumulators meet in shared memory (the first barrier: everyone is done reading
    // what the previous segment left there), one thread per column folds them in warp order
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
#pragma unroll
    for (int e = 0; e < V; ++e) scratch[warp * kColumns + lane * V + e] = R::template to_acc<1>(local[e]);
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
    const int owner_first = stream_owner(panel_first, args.units, grid);
    const int owner_last = stream_owner(panel_first + upp - 1, args.units, grid);
    const int sharers = owner_last - owner_first + 1;
    const long long slice = static_cast<unsigned>(panel) / static_cast<unsigned>(args.panels_per_slice);
    typename R::Out* out_row = out + slice * args.inner + (panel - slice * args.panels_per_slice) * kColumns;
    Acc* panel_partials = partials + panel * args.slots * kColumns;
    for (int column = threadIdx.x; column < kColumns; column += kConsumerThreads) {
      Acc total = scratch[column];
#pragma unroll
      for (int w = 1; w < kStreamConsumers; ++w) total = R::combine(total, scratch[w * kColumns + column]);
      if (sharers == 1) {
        out_row[column] = R::finish(total, args.reduce, args.mean != 0);
      } else {
        panel_partials[(cta - owner_first) * kColumns + column] = total;
      }
    }
    if (sharers > 1) {
      // the last CTA of the panel to take a ticket folds the partials in CTA order, which is row order
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
      if (threadIdx.x == 0) is_last = atomicAdd(&tickets[panel], 1u) == static_cast<unsigned>(sharers - 1) ? 1 : 0;
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
      if (is_last) {
        __threadfence();
        for (int column = threadIdx.x; column < kColumns; column += kConsumerThreads) {
          Acc total = R::identity();
          for (int j = 0; j < sharers; j += 12) {
            Acc batch[12];
#pragma unroll
            for (int k = 0; k < 12; ++k) {
              if (j + k < sharers) batch[k] = load_partial(panel_partials + (j + k) * kColumns + column);
            }
#pragma unroll
            for (int k = 0; k < 12; ++k) {
              if (j + k < sharers) total = R::combine(total, batch[k]);
            }
          }
          out_row[column] = R::finish(total, args.reduce, args.mean != 0);
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host: the plan and the launch

enum class Shape { kWarpPerSlice, kCtaPerSlice, kColumns, kColumnStream };

struct Plan {
  Shape shape = Shape::kWarpPerSlice;
  int split = 1;      // CTAs per slice (or per column tile)
  int cluster = 1;    // CTAs per thread-block cluster; divides split
  int lanes_x = 32;   // columns kernel: threads along inner
  int vec = 1;        // columns kernel: elements per thread along inner
  bool ring = false;  // columns kernel: stream through the per-thread cp.async ring
  long long tiles = 0;        // ticketed outputs: slices, or outer * column tiles
  long long column_tiles = 0;
  size_t acc_bytes = 0;
  size_t partial_bytes = 0;   // scratch for partials (0 when one cluster covers a slice)
  size_t ticket_bytes = 0;
  // the streaming columns kernel
  int device = 0;
  int grid = 0;               // CTAs: one per SM
  long long units = 0;        // outer * panels per slice * units per panel
  int units_per_panel = 0;
  int panels_per_slice = 0;
  int slots = 0;              // partial rows per panel
};

// Whether the persistent streaming kernel takes a column reduction, and its tiling. Measured on B200
// at [32768, 4096] against reduce_columns: bf16 sum / mean / amax 51-52 us against 54-55, bf16 argmax
// 60 against 72, f32 argmax 93 against 103, bf16 moments (inside LayerNorm over a transposed view) 18 us
// less; f32 sum / mean / amax 89-91 us against 82-85, so those stay with reduce_columns. The streaming
// kernel moves 5.9-6.0 TB/s whatever the reducer until the reducer's instructions bind (bf16 argmax);
// what it loses is fixed: about 2 us until the first tile lands and 3 us for the last panel's fold.
bool plan_stream(Plan& p, tq_reduce_op op, tq_dtype dtype, long long outer, long long reduce, long long inner, int32_t device,
                 int vec_bytes_limit) {
  const int size = dtype_size(dtype);
  if (dtype != TQ_F32 && dtype != TQ_F16 && dtype != TQ_BF16) return false;
  if (!(size == 2 || op == TQ_ARGMAX || static_cast<int>(op) >= kOpSoftmaxStat)) return false;
  if (vec_bytes_limit != 16 || (inner * size) % kStreamPieceBytes != 0 || reduce % kStreamUnitRows != 0) return false;
  if (outer * reduce >= (1ll << 31) || inner >= (1ll << 31)) return false;   // TMA coordinates are 32 bits
  if (outer * reduce * inner * size < (64ll << 20)) return false;
  const int sms = sm_count(device);
  const long long panels = outer * (inner * size / kStreamPieceBytes);
  const long long units = panels * (reduce / kStreamUnitRows);
  if (units < 4ll * sms || panels > (1ll << 24)) return false;
  if (units * (sms + 1) >= (1ll << 32)) return false;   // the kernel divides unit x CTA products as 32-bit numbers
  p.shape = Shape::kColumnStream;
  p.device = device;
  p.grid = sms;
  p.units = units;
  p.units_per_panel = static_cast<int>(reduce / kStreamUnitRows);
  p.panels_per_slice = static_cast<int>(inner * size / kStreamPieceBytes);
  p.slots = static_cast<int>((p.units_per_panel + units / sms - 1) / (units / sms)) + 1;
  p.tiles = panels;
  const long long columns = kStreamPieceBytes / size;
  p.partial_bytes = (static_cast<size_t>(panels) * p.slots * columns * p.acc_bytes + 255) / 256 * 256;
  p.ticket_bytes = (static_cast<size_t>(panels) * sizeof(unsigned) + 255) / 256 * 256;
  return true;
}

int floor_pow2(long long v) {
  int p = 1;
  while (static_cast<long long>(p) * 2 <= v) p *= 2;
  return p;
}

Plan plan(tq_reduce_op op, tq_dtype dtype, long long outer, long long reduce, long long inner,
          int32_t device, int vec_bytes_limit) {
  Plan p;
  const int size = dtype_size(dtype);
  const int sms = sm_count(device);
  const long long target_ctas = static_cast<long long>(sms) * 4;
  p.acc_bytes = (op == TQ_ARGMAX || op == kOpMoments) ? 16 : 8;  // upper bound; every other Acc fits 8 bytes
  if (inner == 1) {
    const int vec = 16 / size;
    const long long slice_bytes = reduce * size;
    if (slice_bytes <= 4096 || (outer >= static_cast<long long>(sms) * 16 && slice_bytes <= 65536)) {
      p.shape = Shape::kWarpPerSlice;
      return p;
    }
    p.shape = Shape::kCtaPerSlice;
    long long want = (target_ctas + outer - 1) / outer;
    const long long per_pass = static_cast<long long>(kBlock) * vec * kUnroll;
    long long most = reduce / per_pass;
    if (most < 1) most = 1;
    if (want > most) want = most;
    if (want < 1) want = 1;
    if (want <= kMaxCluster) {
      p.split = floor_pow2(want);
      p.cluster = p.split;
    } else {
      if (want > 1024) want = 1024;
      p.split = static_cast<int>((want + kMaxCluster - 1) / kMaxCluster * kMaxCluster);
      p.cluster = kMaxCluster;
    }
    p.tiles = outer;
  } else {
    if (plan_stream(p, op, dtype, outer, reduce, inner, device, vec_bytes_limit)) return p;
    p.shape = Shape::kColumns;
    int vec = vec_bytes_limit / size;
    if (vec > 8) vec = 8;
    if (vec < 1) vec = 1;
    while (vec > 1 && inner % vec != 0) vec /= 2;
    if ((op == TQ_ARGMAX || op == kOpMoments) && vec > 4) vec = 4;  // their per-column state is large; 16-byte loads measured no better (argmax) or worse (moments)
    p.vec = vec;
    long long groups = (inner + vec - 1) / vec;
    // A warp reads 32 vectors (512 bytes) of one row; the CTA's 8 warps read 8 consecutive rows.
    // Measured on B200 at [32768, 4096]: 4-byte sums and extremes are fastest with plain unrolled
    // loads, 64 lanes along `inner` and one wave of CTAs; 2-byte types and argmax (whose state
    // costs registers) with the cp.async ring and 32 lanes.
    p.ring = (size <= 2 || op == TQ_ARGMAX || op >= kOpSoftmaxStat) && reduce < (1ll << 31);   // the ring counts a thread's rows in 32 bits
    int lanes = p.ring ? 32 : 64;
    while (lanes > 1 && lanes / 2 >= groups) lanes /= 2;
    p.lanes_x = lanes;
    p.column_tiles = (groups + lanes - 1) / lanes;
    const long long base_ctas = p.column_tiles * outer;
    // One or two waves of CTAs (all of a wave resident at once, equal work each).
    const int waves = (p.ring && !(op == TQ_ARGMAX && size <= 2)) ? 2 : 1;
    long long want = (target_ctas * waves + base_ctas - 1) / base_ctas;
    const long long per_pass = static_cast<long long>(kBlock / lanes) * kUnroll;
    long long most = reduce / per_pass;
    if (most < 1) most = 1;
    if (want > most) want = most;
    if (want < 1) want = 1;
    // The cluster's reduce-scatter gives every CTA a whole number of threads' accumulators.
    int max_cluster = kMaxCluster;
    while (max_cluster > lanes) max_cluster /= 2;
    if (want <= max_cluster) {
      p.split = floor_pow2(want);
      p.cluster = p.split;
    } else {
      if (want > 1024) want = 1024;
      p.split = static_cast<int>((want + max_cluster - 1) / max_cluster * max_cluster);
      p.cluster = max_cluster;
    }
    p.tiles = base_ctas;
  }
  const int clusters = p.split / p.cluster;
  if (clusters > 1) {
    const long long items = p.shape == Shape::kColumns ? p.lanes_x * p.vec : 1;
    p.partial_bytes = static_cast<size_t>(p.tiles) * clusters * items * p.acc_bytes;
    p.partial_bytes = (p.partial_bytes + 255) / 256 * 256;
    p.ticket_bytes = (static_cast<size_t>(p.tiles) * sizeof(unsigned) + 255) / 256 * 256;
  }
  return p;
}

template <typename Kernel, typename... Args>
tq_status launch_clustered(Kernel kernel, dim3 grid, dim3 cluster, size_t smem, cudaStream_t stream,
                           Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = dim3(kBlock);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = cluster.x;
  attribute[0].val.clusterDim.y = cluster.y;
  attribute[0].val.clusterDim.z = cluster.z;
  config.attrs = attribute;
  config.numAttrs = (cluster.x * cluster.y * cluster.z > 1) ? 1 : 0;
  TQ_CUDA(cudaLaunchKernelEx(&config, kernel, args...));
  return TQ_OK;
}

template <typename T, typename R>
tq_status run(const Plan& p, const void* in, void* out, long long outer, long long reduce,
              long long inner, bool mean, void* workspace, cudaStream_t stream) {
  using Acc = typename R::Acc;
  using Out = typename R::Out;
  static_assert(sizeof(Acc) <= 16, "accumulators are sized as at most 16 bytes in plan()");
  const T* input = static_cast<const T*>(in);
  Out* output = static_cast<Out*>(out);
  Acc* partials = static_cast<Acc*>(workspace);
  unsigned* tickets =
      reinterpret_cast<unsigned*>(static_cast<unsigned char*>(workspace) + p.partial_bytes);
  if (p.ticket_bytes) TQ_CUDA(cudaMemsetAsync(tickets, 0, p.ticket_bytes, stream));
  constexpr int kVec = 16 / sizeof(T);
  switch (p.shape) {
    case Shape::kWarpPerSlice: {
      const long long blocks = (outer + kWarps - 1) / kWarps;
      TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld slices are more than a grid holds", outer);
      reduce_warp_per_slice<T, R, kVec><<<static_cast<unsigned>(blocks), kBlock, 0, stream>>>(
          input, output, outer, reduce, mean ? 1 : 0);
      return check_launch("reduce_warp_per_slice");
    }
    case Shape::kCtaPerSlice: {
      const long long blocks = outer * p.split;
      TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld slices are more than a grid holds", outer);
      if (tq_status s = launch_clustered(reduce_cta_per_slice<T, R, kVec>,
                                         dim3(static_cast<unsigned>(blocks)), dim3(p.cluster), 0,
                                         stream, input, output, reduce, p.split, p.cluster,
                                         mean ? 1 : 0, partials, tickets)) {
        return s;
      }
      return check_launch("reduce_cta_per_slice");
    }
    case Shape::kColumns: {
      TQ_REQUIRE(outer <= 65535, TQ_UNSUPPORTED,
                 "a reduction with kept axes on both sides and %lld leading slices has no kernel", outer);
      dim3 grid(static_cast<unsigned>(p.column_tiles), p.split, static_cast<unsigned>(outer));
      auto go = [&](auto kernel, int vec) -> tq_status {
        const size_t smem = (static_cast<size_t>(kBlock) * vec + static_cast<size_t>(p.lanes_x) * vec) * sizeof(Acc) +
                            static_cast<size_t>(kRingDepth) * kBlock * vec * sizeof(T);
        if (smem > 40 * 1024) {
          TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(smem)));
        }
        if (tq_status s = launch_clustered(kernel, grid, dim3(1, p.cluster, 1), smem, stream, input,
                                           output, reduce, inner, p.lanes_x, p.split, p.cluster,
                                           mean ? 1 : 0, partials, tickets)) {
          return s;
        }
        return check_launch("reduce_columns");
      };
      constexpr int kColumnVec = kVec > 8 ? 8 : kVec;
      if (p.vec == 1) return p.ring ? go(reduce_columns<T, R, 1, true>, 1) : go(reduce_columns<T, R, 1, false>, 1);
      if constexpr (kColumnVec >= 2) {
        if (p.vec == 2) return p.ring ? go(reduce_columns<T, R, 2, true>, 2) : go(reduce_columns<T, R, 2, false>, 2);
      }
      if constexpr (kColumnVec >= 4) {
        if (p.vec == 4) return p.ring ? go(reduce_columns<T, R, 4, true>, 4) : go(reduce_columns<T, R, 4, false>, 4);
      }
      if constexpr (kColumnVec >= 8) {
        if (p.vec == 8) return p.ring ? go(reduce_columns<T, R, 8, true>, 8) : go(reduce_columns<T, R, 8, false>, 8);
      }
      return fail(TQ_INTERNAL, "no column kernel for %d elements per thread", p.vec);
    }
    case Shape::kColumnStream: {
      if constexpr (std::is_same_v<T, float> || std::is_same_v<T, __half> || std::is_same_v<T, __nv_bfloat16>) {
        constexpr int kColumns = kStreamPieceBytes / static_cast<int>(sizeof(T));
        EncodeTiled encode = encode_tiled();
        TQ_REQUIRE(encode != nullptr, TQ_EXTERNAL, "the CUDA driver does not provide cuTensorMapEncodeTiled");
        // in[outer * reduce, inner] as a two-axis map; a tile is one unit: 512 bytes of 64 consecutive rows
        CUtensorMap map;
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer * reduce)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(inner) * sizeof(T)};
        const cuuint32_t box[2] = {static_cast<cuuint32_t>(kColumns), static_cast<cuuint32_t>(kStreamUnitRows)};
        const cuuint32_t element_strides[2] = {1, 1};
        const CUtensorMapDataType type = std::is_same_v<T, float>    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                         : std::is_same_v<T, __half> ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                                     : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
        const CUresult encoded = encode(&map, type, 2, const_cast<T*>(input), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                        CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        TQ_REQUIRE(encoded == CUDA_SUCCESS, TQ_EXTERNAL, "cuTensorMapEncodeTiled refused the reduction's input (%d)", static_cast<int>(encoded));
        StreamArgs args = {};
        args.reduce = reduce;
        args.inner = inner;
        args.units = p.units;
        args.units_per_panel = p.units_per_panel;
        args.panels_per_slice = p.panels_per_slice;
        args.slots = p.slots;
        args.mean = mean ? 1 : 0;
        args.status = wait_status_for(p.device);
        TQ_REQUIRE(args.status.abort != nullptr, TQ_RESOURCE_EXHAUSTED, "no device memory for the status word");
        auto kernel = reduce_columns_stream<T, R>;
        constexpr int kConsumers = stream_consumers<T, R>();
        constexpr int kStages = kConsumers == 8 ? kStreamStages : 4;
        const size_t smem = static_cast<size_t>(kStages) * kStreamStageBytes + static_cast<size_t>(kConsumers) * kColumns * sizeof(Acc) + 2 * kStages * 8;
        TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
        kernel<<<static_cast<unsigned>(p.grid), (kConsumers + 1) * 32, smem, stream>>>(map, args, output, partials, tickets);
        return check_launch("reduce_columns_stream");
      } else {
        return fail(TQ_INTERNAL, "the streaming columns kernel was planned for an element type it does not serve");
      }
    }
  }
  return fail(TQ_INTERNAL, "unreachable reduction shape");
}

template <typename T>
tq_status run_op(tq_reduce_op op, const Plan& p, const void* in, void* out, long long outer,
                 long long reduce, long long inner, void* workspace, cudaStream_t stream) {
  switch (op) {
    case TQ_SUM: return run<T, SumReducer<T>>(p, in, out, outer, reduce, inner, false, workspace, stream);
    case TQ_MEAN: return run<T, SumReducer<T>>(p, in, out, outer, reduce, inner, true, workspace, stream);
    case TQ_AMAX: return run<T, ExtremeReducer<T, true>>(p, in, out, outer, reduce, inner, false, workspace, stream);
    case TQ_AMIN: return run<T, ExtremeReducer<T, false>>(p, in, out, outer, reduce, inner, false, workspace, stream);
    case TQ_ARGMAX: return run<T, ArgmaxReducer<T>>(p, in, out, outer, reduce, inner, false, workspace, stream);
    default: return fail(TQ_INVALID_ARGUMENT, "unknown reduction %d", op);
  }
}

tq_status validate(tq_reduce_op op, tq_dtype dtype, long long outer, long long reduce, long long inner) {
  TQ_REQUIRE(op >= TQ_SUM && op <= TQ_ARGMAX, TQ_INVALID_ARGUMENT, "unknown reduction %d", op);
  TQ_REQUIRE(dtype_size(dtype) != 0 && dtype != TQ_BOOL, TQ_UNSUPPORTED,
             "reductions have no kernel for element type %s", dtype_name(dtype));
  TQ_REQUIRE(outer >= 0 && reduce >= 0 && inner >= 0, TQ_INVALID_ARGUMENT,
             "negative extent in [%lld, %lld, %lld]", outer, reduce, inner);
  TQ_REQUIRE(reduce > 0, TQ_UNSUPPORTED, "a reduction over no elements has no kernel");
  TQ_REQUIRE(!(op == TQ_ARGMAX && reduce >= 0xffffffffLL), TQ_UNSUPPORTED,
             "argmax over %lld elements has no kernel (positions are kept in 32 bits)", reduce);
  TQ_REQUIRE(!(op == TQ_MEAN && (dtype == TQ_I32 || dtype == TQ_I64)), TQ_UNSUPPORTED,
             "mean of an integer tensor has no kernel");
  return TQ_OK;
}

// The columns kernel needs vector loads aligned in every row: inner * size and the base pointer
// must both be multiples of the vector's bytes.
int column_vec_bytes(const void* in, long long inner, int size) {
  int bytes = 16;
  while (bytes > size && (!aligned_to(in, bytes) || (inner * size) % bytes != 0)) bytes /= 2;
  return bytes;
}

template <typename T>
tq_status run_stats(int kind, const Plan& p, const void* in, void* out, long long outer, long long reduce,
                    long long inner, void* workspace, cudaStream_t stream) {
  if (kind == kOpSoftmaxStat) return run<T, SoftmaxStatReducer<T>>(p, in, out, outer, reduce, inner, false, workspace, stream);
  return run<T, MomentsReducer<T>>(p, in, out, outer, reduce, inner, false, workspace, stream);
}

// ---------------------------------------------------------------------------------------------
// Scratch that exists without anyone allocating it, for tq_reduce_launch_static.
//
// The array lives in the library's device image: every GPU that loads the library carries these
// bytes from load until the process exits. In host code the array's name is only a stand-in for
// the symbol, not a device address, so the host asks the runtime for the real address once per
// device (with that device current) and hands that pointer to the kernels.
constexpr size_t kStaticScratchBytes = TQ_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

std::mutex g_static_mutex;
void* g_static_address[64] = {nullptr};

// Looks the address up on first use for `device`, which must be current.
tq_status static_scratch_for(int32_t device, void** address) {
  TQ_REQUIRE(device >= 0 && device < 64, TQ_INVALID_ARGUMENT, "device ordinal %d is out of range", device);
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_address[device] == nullptr) {
    void* found = nullptr;
    const cudaError_t status = cudaGetSymbolAddress(&found, g_static_scratch);
    if (status != cudaSuccess || found == nullptr) {
      return fail(TQ_EXTERNAL, "cannot find the built-in scratch on device %d: %s", device,
                  cudaGetErrorString(status));
    }
    g_static_address[device] = found;
  }
  *address = g_static_address[device];
  return TQ_OK;
}

}  // namespace

// Per-slice statistics for the transposed softmax / LayerNorm (rownorm.cu): `kind` 0 writes
// (max, 1 / sum exp(x - max)), `kind` 1 writes (mean, biased variance), as two floats per slice,
// for a packed [outer, reduce, inner] input of a floating type (f32, f16, bf16).
size_t slice_stats_workspace_bytes(int kind, tq_dtype dtype, long long outer, long long reduce, long long inner, int32_t device) {
  size_t bytes = 0;
  const int op = kind == 0 ? kOpSoftmaxStat : kOpMoments;
  for (int limit = 16; limit >= dtype_size(dtype); limit /= 2) {
    const Plan p = plan(op, dtype, outer, reduce, inner, device, limit);
    if (p.partial_bytes + p.ticket_bytes > bytes) bytes = p.partial_bytes + p.ticket_bytes;
  }
  return bytes;
}

tq_status slice_stats_launch(int kind, tq_dtype dtype, const void* in, void* stats, long long outer, long long reduce,
                             long long inner, void* workspace, size_t workspace_bytes, int32_t device, cudaStream_t stream) {
  const int op = kind == 0 ? kOpSoftmaxStat : kOpMoments;
  const int size = dtype_size(dtype);
  const Plan p = plan(op, dtype, outer, reduce, inner, device, inner == 1 ? 16 : column_vec_bytes(in, inner, size));
  const size_t need = p.partial_bytes + p.ticket_bytes;
  TQ_REQUIRE(need == 0 || (workspace != nullptr && workspace_bytes >= need && aligned_to(workspace, 16)), TQ_INVALID_ARGUMENT,
             "the statistics pass needs %zu bytes of 16-byte-aligned scratch and was given %zu", need, workspace_bytes);
  switch (dtype) {
    case TQ_F32: return run_stats<float>(op, p, in, stats, outer, reduce, inner, workspace, stream);
    case TQ_F16: return run_stats<__half>(op, p, in, stats, outer, reduce, inner, workspace, stream);
    case TQ_BF16: return run_stats<__nv_bfloat16>(op, p, in, stats, outer, reduce, inner, workspace, stream);
    default: return fail(TQ_UNSUPPORTED, "slice statistics have no kernel for element type %s", dtype_name(dtype));
  }
}

}  // namespace tq

extern "C" {

tq_status tq_reduce_workspace_bytes(tq_reduce_op op, tq_dtype dtype, int64_t outer, int64_t reduce,
                                    int64_t inner, int32_t device, size_t* bytes) {
  TQ_REQUIRE(bytes != nullptr, TQ_INVALID_ARGUMENT, "bytes out-pointer is null");
  if (tq_status s = tq::validate(op, dtype, outer, reduce, inner)) return s;
  *bytes = 0;
  if (outer == 0 || inner == 0) return TQ_OK;
  // The input's alignment is unknown here and decides the vector width of the columns kernel,
  // which changes its tiling: answer with the largest need over the widths it may pick.
  for (int limit = 16; limit >= tq::dtype_size(dtype); limit /= 2) {
    tq::Plan p = tq::plan(op, dtype, outer, reduce, inner, device, limit);
    if (p.partial_bytes + p.ticket_bytes > *bytes) *bytes = p.partial_bytes + p.ticket_bytes;
  }
  return TQ_OK;
}

tq_status tq_reduce_launch(tq_reduce_op op, tq_dtype dtype, const void* in, void* out, int64_t outer,
                           int64_t reduce, int64_t inner, void* workspace, size_t workspace_bytes,
                           int32_t device, void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) {
    return tq_reduce_launch(op, dtype, in, out, outer, reduce, inner, workspace, workspace_bytes, d, s);
  });
  if (tq_status s = tq::validate(op, dtype, outer, reduce, inner)) return s;
  if (outer == 0 || inner == 0) return TQ_OK;
  TQ_REQUIRE(in != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null input or output");
  const int size = tq::dtype_size(dtype);
  TQ_REQUIRE(tq::aligned_to(in, size), TQ_INVALID_ARGUMENT, "input pointer is not aligned to its element type");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  tq::Plan p = tq::plan(op, dtype, outer, reduce, inner, device,
                        inner == 1 ? 16 : tq::column_vec_bytes(in, inner, size));
  const size_t need = p.partial_bytes + p.ticket_bytes;
  TQ_REQUIRE(need == 0 || (workspace != nullptr && workspace_bytes >= need), TQ_INVALID_ARGUMENT,
             "this reduction needs %zu bytes of scratch and was given %zu", need, workspace_bytes);
  TQ_REQUIRE(need == 0 || tq::aligned_to(workspace, 16), TQ_INVALID_ARGUMENT,
             "scratch memory must be 16-byte aligned");
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TQ_F32: return tq::run_op<float>(op, p, in, out, outer, reduce, inner, workspace, cuda_stream);
    case TQ_F64: return tq::run_op<double>(op, p, in, out, outer, reduce, inner, workspace, cuda_stream);
    case TQ_F16: return tq::run_op<__half>(op, p, in, out, outer, reduce, inner, workspace, cuda_stream);
    case TQ_BF16: return tq::run_op<__nv_bfloat16>(op, p, in, out, outer, reduce, inner, workspace, cuda_stream);
    case TQ_I32: return tq::run_op<int>(op, p, in, out, outer, reduce, inner, workspace, cuda_stream);
    case TQ_I64: return tq::run_op<long long>(op, p, in, out, outer, reduce, inner, workspace, cuda_stream);
    default: return tq::fail(TQ_UNSUPPORTED, "reductions have no kernel for element type %s", tq::dtype_name(dtype));
  }
}

tq_status tq_reduce_partial_launch(tq_reduce_op op, tq_dtype dtype, const void* in, void* partial, int64_t count, void* workspace,
                                   size_t workspace_bytes, int32_t device, void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) { return tq_reduce_partial_launch(op, dtype, in, partial, count, workspace, workspace_bytes, d, s); });
  TQ_REQUIRE(op == TQ_SUM || op == TQ_MEAN || op == TQ_AMAX || op == TQ_AMIN, TQ_UNSUPPORTED, "no global partial for operation %d", op);
  TQ_REQUIRE(dtype == TQ_F32 || dtype == TQ_F16 || dtype == TQ_BF16, TQ_UNSUPPORTED,
             "the two-float partial serves f32, f16 and bf16 tensors, not %s", tq::dtype_name(dtype));
  TQ_REQUIRE(count > 0, TQ_UNSUPPORTED, "a reduction over no elements has no kernel");
  TQ_REQUIRE(in != nullptr && partial != nullptr && tq::aligned_to(partial, 8), TQ_INVALID_ARGUMENT, "null input, or a partial that is not 8-byte aligned");
  const int size = tq::dtype_size(dtype);
  TQ_REQUIRE(tq::aligned_to(in, size), TQ_INVALID_ARGUMENT, "input pointer is not aligned to its element type");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  // the plan of the plain reduction over [1, count, 1]: same kernels, same scratch, another finish
  const tq::Plan p = tq::plan(op == TQ_MEAN ? TQ_SUM : op, dtype, 1, count, 1, device, 16);
  const size_t need = p.partial_bytes + p.ticket_bytes;
  TQ_REQUIRE(need == 0 || (workspace != nullptr && workspace_bytes >= need && tq::aligned_to(workspace, 16)), TQ_INVALID_ARGUMENT,
             "this reduction needs %zu bytes of 16-byte-aligned scratch (tq_reduce_workspace_bytes) and was given %zu", need, workspace_bytes);
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
#define TQ_PARTIAL(T)                                                                                                                      \
  switch (op) {                                                                                                                            \
    case TQ_AMAX: return tq::run<T, tq::ExtremePartialReducer<T, true>>(p, in, partial, 1, count, 1, false, workspace, cuda_stream);        \
    case TQ_AMIN: return tq::run<T, tq::ExtremePartialReducer<T, false>>(p, in, partial, 1, count, 1, false, workspace, cuda_stream);       \
    default: return tq::run<T, tq::SumPartialReducer<T>>(p, in, partial, 1, count, 1, false, workspace, cuda_stream);                        \
  }
  switch (dtype) {
    case TQ_F32: TQ_PARTIAL(float)
    case TQ_F16: TQ_PARTIAL(__half)
    default: TQ_PARTIAL(__nv_bfloat16)
  }
#undef TQ_PARTIAL
}

tq_status tq_reduce_launch_static(tq_reduce_op op, tq_dtype dtype, const void* in, void* out,
                                  int64_t outer, int64_t reduce, int64_t inner, int32_t device,
                                  void* stream) {
  // recorded like every other launch: the replay looks the built-in array up for the device it runs on
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) { return tq_reduce_launch_static(op, dtype, in, out, outer, reduce, inner, d, s); });
  if (tq_status s = tq::validate(op, dtype, outer, reduce, inner)) return s;
  if (outer == 0 || inner == 0) return TQ_OK;
  TQ_REQUIRE(in != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null input or output");
  const int size = tq::dtype_size(dtype);
  TQ_REQUIRE(tq::aligned_to(in, size), TQ_INVALID_ARGUMENT, "input pointer is not aligned to its element type");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  const tq::Plan p = tq::plan(op, dtype, outer, reduce, inner, device,
                              inner == 1 ? 16 : tq::column_vec_bytes(in, inner, size));
  const size_t need = p.partial_bytes + p.ticket_bytes;
  TQ_REQUIRE(need <= tq::kStaticScratchBytes, TQ_RESOURCE_EXHAUSTED,
             "this reduction needs %zu bytes of scratch; the built-in scratch of tq_reduce_launch_static holds %zu. "
             "Use tq_reduce_launch with caller-provided scratch for extents this large",
             need, tq::kStaticScratchBytes);
  void* scratch = nullptr;
  if (need != 0) {
    if (tq_status s = tq::static_scratch_for(device, &scratch)) return s;
  }
  // Partials are overwritten before they are read and the ticket words are cleared by the launch
  // itself (a memset node on `stream`), so whatever the previous call left behind does not matter.
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case TQ_F32: return tq::run_op<float>(op, p, in, out, outer, reduce, inner, scratch, cuda_stream);
    case TQ_F64: return tq::run_op<double>(op, p, in, out, outer, reduce, inner, scratch, cuda_stream);
    case TQ_F16: return tq::run_op<__half>(op, p, in, out, outer, reduce, inner, scratch, cuda_stream);
    case TQ_BF16: return tq::run_op<__nv_bfloat16>(op, p, in, out, outer, reduce, inner, scratch, cuda_stream);
    case TQ_I32: return tq::run_op<int>(op, p, in, out, outer, reduce, inner, scratch, cuda_stream);
    case TQ_I64: return tq::run_op<long long>(op, p, in, out, outer, reduce, inner, scratch, cuda_stream);
    default: return tq::fail(TQ_UNSUPPORTED, "reductions have no kernel for element type %s", tq::dtype_name(dtype));
  }
}

}  // extern "C"
