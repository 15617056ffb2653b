// Reducers shared by the reduction kernels (reduce.cu) and the panel normalisation (panelnorm.cu):
// the NaN-propagating extreme, the online softmax statistics and the mergeable moments.
#pragma once

#include <limits>
#include <type_traits>

#include "common.h"

namespace tq {

template <typename C> __device__ __forceinline__ C shfl_xor(C v, int offset) {
  return __shfl_xor_sync(0xffffffffu, v, offset);
}


template <typename T, bool kMax>
struct ExtremeReducer {
  static constexpr bool kSeeded = false;   // no seed / step_seeded / set_count protocol (see MomentsReducer)
  using C = typename Compute<T>::type;
  using Acc = C;
  using Out = T;
  __device__ static Acc identity() {
    if constexpr (std::is_integral_v<C>) {
      return kMax ? std::numeric_limits<C>::lowest() : std::numeric_limits<C>::max();
    } else {
      return kMax ? -std::numeric_limits<C>::infinity() : std::numeric_limits<C>::infinity();
    }
  }
  __device__ static Acc lift(T v, long long) { return to_compute(v); }
  __device__ static Acc combine(Acc a, Acc b) {
    if constexpr (std::is_same_v<C, float>) {
      // One instruction: the NaN-propagating maximum / minimum of PTX.
      float r;
      if constexpr (kMax) {
        asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
      } else {
        asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
      }
      return r;
    } else {
      if constexpr (!std::is_integral_v<C>) {
        if (a != a) return a;
        if (b != b) return b;
      }
      if constexpr (kMax) return a > b ? a : b;
      return a < b ? a : b;
    }
  }
  __device__ static Acc shuffle(Acc a, int offset) { return shfl_xor(a, offset); }
  template <int VEC> using Local = Acc;
  template <int VEC> __device__ static Acc local_identity() { return identity(); }
  template <int VEC> __device__ static void step(Acc& local, T v, long long) { local = combine(local, to_compute(v)); }
  template <int VEC> __device__ static void step_vector(Acc& local, const Vec<T, VEC>& x, long long) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) local = combine(local, to_compute(x.v[e]));
  }
  template <int VEC> __device__ static Acc to_acc(Acc local) { return local; }
  __device__ static Out finish(Acc a, long long, bool) { return from_compute<Out, Acc>(a); }
};

// ---------------------------------------------------------------------------------------------
// Two statistics of a slice that later kernels normalise with (softmax and LayerNorm over a
// transposed view read their columns through the columns kernel below).

constexpr int kOpSoftmaxStat = 100;   // (max, 1 / sum exp(x - max)) per slice
constexpr int kOpMoments = 101;       // (mean, biased variance) per slice

struct alignas(8) MaxSum {
  float m;
  float s;
};

__device__ __forceinline__ float stat_exp2(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}

// Online softmax statistics: a running maximum and the sum of exp(x - maximum), rescaled whenever
// the maximum grows. Equal maxima (also -inf with -inf) need no rescaling, which keeps a slice of
// all -inf at (-inf, count) instead of NaN; a NaN makes the maximum and the sum NaN.
template <typename T>
struct SoftmaxStatReducer {
  static constexpr bool kSeeded = false;   // no seed / step_seeded / set_count protocol (see MomentsReducer)
  using C = float;
  using Acc = MaxSum;
  using Out = MaxSum;
  static constexpr float kLog2e = 1.4426950408889634f;
  __device__ static Acc identity() { return Acc{-std::numeric_limits<float>::infinity(), 0.f}; }
  __device__ static Acc combine(Acc a, Acc b) {
    const float m = ExtremeReducer<float, true>::combine(a.m, b.m);
    const float scale_a = a.m == m ? 1.f : stat_exp2((a.m - m) * kLog2e);
    const float scale_b = b.m == m ? 1.f : stat_exp2((b.m - m) * kLog2e);
    return Acc{m, a.s * scale_a + b.s * scale_b};
  }
  __device__ static Acc shuffle(Acc a, int offset) { return Acc{shfl_xor(a.m, offset), shfl_xor(a.s, offset)}; }
  template <int VEC> using Local = Acc;
  template <int VEC> __device__ static Acc local_identity() { return identity(); }
  // `m` is a reference point, not necessarily the maximum: softmax is exp(x - m) / sum exp(x - m) for
  // any m, so a thread keeps the first value it sees and only moves the reference (rescaling its
  // sum) when an element lies more than 2^kSlack above it — rare, and then a real branch. Per
  // element that leaves one FMA, one ex2 and one add (the exact running maximum with its
  // predicated rescale was 24 instructions per element and made this pass issue-bound). Terms are
  // at most 2^kSlack, far from overflow in f32; `combine` brings two references together exactly.
  static constexpr float kSlack = 32.f;
  template <int VEC> __device__ static void step(Acc& local, T v, long long) {
    const float x = to_compute(v);
    float t = (x - local.m) * kLog2e;
    if (!(t <= kSlack)) {                      // far above the reference, the first element (m = -inf), or a NaN
      if (x == -std::numeric_limits<float>::infinity()) {
        t = x;                                 // -inf before any finite value: contributes nothing, the reference stays
      } else {
        local.s *= stat_exp2(-t);              // exp2(-inf) = 0 for the first element; NaN for a NaN or a second +inf
        local.m = x;
        t = 0.f;
      }
    }
    local.s += stat_exp2(t);
  }
  template <int VEC> __device__ static void step_vector(Acc& local, const Vec<T, VEC>& x, long long) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) step<VEC>(local, x.v[e], 0);
  }
  // One row of V neighbouring columns, each with its own accumulator: the test for "far above the
  // reference" is taken once for the V elements, so that the common path is V independent
  // subtract-scale / ex2 / add chains with no branch between them (with a branch per element the ex2
  // latency of every element was exposed, and the pass ran at that latency rather than at the memory's
  // rate). The rare path is the per-element step; both give the same bits as V calls of `step`.
  static constexpr bool kColumnStep = true;
  template <int V> __device__ static void step_columns(Acc (&local)[V], const Vec<T, V>& x, long long) {
    float t[V];
    bool near = true;
#pragma unroll
    for (int e = 0; e < V; ++e) {
      t[e] = (to_compute(x.v[e]) - local[e].m) * kLog2e;
      near = near && t[e] <= kSlack;
    }
    if (near) {
#pragma unroll
      for (int e = 0; e < V; ++e) local[e].s += stat_exp2(t[e]);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) step<1>(local[e], x.v[e], 0);
    }
  }
  template <int VEC> __device__ static Acc to_acc(Acc local) { return local; }
  // A slice whose maximum is +inf is NaN throughout (inf - inf), as the plain three-pass form gives.
  __device__ static Out finish(Acc a, long long, bool) {
    const float inverse = a.m == std::numeric_limits<float>::infinity() ? std::numeric_limits<float>::quiet_NaN() : 1.f / a.s;
    return Out{a.m, inverse};
  }
};

struct alignas(16) Moments {
  float n;
  float mean;
  float m2;
  float unused;
};

// Mean and sum of squared deviations. A thread sums (x - pivot) and (x - pivot)^2 with the first
// element it sees as the pivot (two FMAs per element, little cancellation over its few hundred
// elements); partial results are merged with the pairwise update of Chan et al., which is stable
// however the slice was cut.
template <typename T>
struct MomentsReducer {
  using C = float;
  using Acc = Moments;
  struct Out {
    float mean;
    float variance;
  };
  __device__ static Acc identity() { return Acc{0.f, 0.f, 0.f, 0.f}; }
  __device__ static Acc combine(Acc a, Acc b) {
    if (a.n == 0.f) return b;
    if (b.n == 0.f) return a;
    const float n = a.n + b.n;
    const float delta = b.mean - a.mean;
    return Acc{n, a.mean + delta * (b.n / n), a.m2 + b.m2 + delta * delta * (a.n * b.n / n), 0.f};
  }
  __device__ static Acc shuffle(Acc a, int offset) {
    return Acc{shfl_xor(a.n, offset), shfl_xor(a.mean, offset), shfl_xor(a.m2, offset), 0.f};
  }
  template <int VEC>
  struct Local {
    float pivot, s1, s2, n;
  };
  template <int VEC> __device__ static Local<VEC> local_identity() { return Local<VEC>{0.f, 0.f, 0.f, 0.f}; }
  template <int VEC> __device__ static void step(Local<VEC>& local, T v, long long) {
    const float x = to_compute(v);
    if (local.n == 0.f) local.pivot = x;
    const float d = x - local.pivot;
    local.s1 += d;
    local.s2 = fmaf(d, d, local.s2);
    local.n += 1.f;
  }
  template <int VEC> __device__ static void step_vector(Local<VEC>& local, const Vec<T, VEC>& x, long long) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) step<VEC>(local, x.v[e], 0);
  }
  // The columns kernel seeds the pivot with the thread's first value before its loop and sets the
  // count after it, which leaves a subtraction, an add and an FMA per element.
  static constexpr bool kSeeded = true;
  template <int VEC> __device__ static void seed(Local<VEC>& local, T v) { local.pivot = to_compute(v); }
  template <int VEC> __device__ static void step_seeded(Local<VEC>& local, T v) {
    const float d = to_compute(v) - local.pivot;
    local.s1 += d;
    local.s2 = fmaf(d, d, local.s2);
  }
  template <int VEC> __device__ static void set_count(Local<VEC>& local, int count) { local.n = static_cast<float>(count); }
  template <int VEC> __device__ static Acc to_acc(const Local<VEC>& local) {
    if (local.n == 0.f) return identity();
    const float shifted_mean = local.s1 / local.n;
    const float m2 = local.s2 - local.s1 * shifted_mean;
    return Acc{local.n, local.pivot + shifted_mean, m2 > 0.f || m2 != m2 ? m2 : 0.f, 0.f};
  }
  __device__ static Out finish(Acc a, long long, bool) { return Out{a.mean, a.m2 / a.n}; }
};

// Whether a reducer steps V neighbouring columns at once (step_columns above).
template <typename R, typename = void> struct has_column_step : std::false_type {};
template <typename R> struct has_column_step<R, std::void_t<decltype(R::kColumnStep)>> : std::bool_constant<R::kColumnStep> {};

}  // namespace tq
