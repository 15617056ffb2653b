// The fixed part of every fused elementwise kernel: storage types, conversions, 128-bit streaming
// loads and stores, the four operand readers, and the tile loop. The selector (fused.cu) appends
// the per-expression part — storage typedefs, `tq_body`, and the four `extern "C"` entry kernels —
// and compiles the whole with NVRTC for sm_100a. The text includes no header, so NVRTC needs no
// include path.
#pragma once

namespace tq {

inline constexpr const char* kFusedPrelude = R"TQ(
typedef unsigned short tq_bf16;   // storage only; arithmetic is in float
typedef unsigned short tq_f16;
typedef unsigned char tq_bool;

struct tq_bf16_tag { unsigned short bits; };
struct tq_f16_tag { unsigned short bits; };

#define TQ_DEV __device__ __forceinline__
#define TQ_BLOCK 256

struct tq_layout_t { int rank; long long sizes[8]; long long strides[8]; unsigned long long magics[8]; };   // magics: see tq_quotient

// ---- conversions between storage and compute types --------------------------------------
template <typename S> struct tq_storage;   // ::compute, ::load(S) -> compute, ::store(compute) -> S
template <> struct tq_storage<float> {
  typedef float compute; typedef float raw;
  static TQ_DEV float load(float v) { return v; }
  static TQ_DEV float store(float v) { return v; }
};
template <> struct tq_storage<double> {
  typedef double compute; typedef double raw;
  static TQ_DEV double load(double v) { return v; }
  static TQ_DEV double store(double v) { return v; }
};
template <> struct tq_storage<int> {
  typedef int compute; typedef int raw;
  static TQ_DEV int load(int v) { return v; }
  static TQ_DEV int store(int v) { return v; }
};
template <> struct tq_storage<long long> {
  typedef long long compute; typedef long long raw;
  static TQ_DEV long long load(long long v) { return v; }
  static TQ_DEV long long store(long long v) { return v; }
};
template <> struct tq_storage<tq_bool> {
  typedef bool compute; typedef unsigned char raw;
  static TQ_DEV bool load(unsigned char v) { return v != 0; }
  static TQ_DEV unsigned char store(bool v) { return v ? 1 : 0; }
};
TQ_DEV float tq_bf16_to_float(unsigned short bits) { return __uint_as_float(((unsigned)bits) << 16); }
TQ_DEV unsigned short tq_float_to_bf16(float v) {
  unsigned short bits;
  asm("cvt.rn.bf16.f32 %0, %1;" : "=h"(bits) : "f"(v));
  return bits;
}
TQ_DEV float tq_f16_to_float(unsigned short bits) {
  float v;
  asm("cvt.f32.f16 %0, %1;" : "=f"(v) : "h"(bits));
  return v;
}
TQ_DEV unsigned short tq_float_to_f16(float v) {
  unsigned short bits;
  asm("cvt.rn.f16.f32 %0, %1;" : "=h"(bits) : "f"(v));
  return bits;
}
template <> struct tq_storage<tq_bf16_tag> {
  typedef float compute; typedef unsigned short raw;
  static TQ_DEV float load(unsigned short v) { return tq_bf16_to_float(v); }
  static TQ_DEV unsigned short store(float v) { return tq_float_to_bf16(v); }
};
template <> struct tq_storage<tq_f16_tag> {
  typedef float compute; typedef unsigned short raw;
  static TQ_DEV float load(unsigned short v) { return tq_f16_to_float(v); }
  static TQ_DEV unsigned short store(float v) { return tq_float_to_f16(v); }
};
TQ_DEV float tq_round_bf16(float v) { return tq_bf16_to_float(tq_float_to_bf16(v)); }
TQ_DEV float tq_round_f16(float v) { return tq_f16_to_float(tq_float_to_f16(v)); }

// ---- math helpers ---------------------------------------------------------------------------
#define TQ_INF_F __int_as_float(0x7f800000)
#define TQ_NAN_F __int_as_float(0x7fc00000)
#define TQ_INF_D __longlong_as_double(0x7ff0000000000000LL)
#define TQ_NAN_D __longlong_as_double(0x7ff8000000000000LL)

// torch.maximum / torch.minimum propagate NaN.
template <typename C> TQ_DEV C tq_maximum(C a, C b) { return (a != a || b != b) ? (a + b) : (a > b ? a : b); }
template <typename C> TQ_DEV C tq_minimum(C a, C b) { return (a != a || b != b) ? (a + b) : (a < b ? a : b); }

// gelu(x, approximate="tanh") = 0.5 x (1 + tanh(k (x + 0.044715 x^3))), k = sqrt(2/pi).
TQ_DEV float tq_gelu_tanh_precise(float x) {
  const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}
// Hardware approximations with denormals flushed: one special-function instruction each, 2 ulp.
TQ_DEV float tq_exp2_ftz(float t) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(t));
  return r;
}
TQ_DEV float tq_rcp_ftz(float d) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
  return r;
}
TQ_DEV float tq_exp_fast(float x) { return tq_exp2_ftz(x * 1.4426950408889634f); }
TQ_DEV double tq_gelu_tanh_precise(double x) {
  const double inner = 0.7978845608028654 * (x + 0.044715 * x * x * x);
  return 0.5 * x * (1.0 + tanh(inner));
}

// ---- vector moves ------------------------------------------------------------------------
// Moves BYTES (1, 2, 4, 8 or a multiple of 16) between global memory and registers. Loads are
// streaming (no L1 allocation): every `same` operand is read exactly once.
template <int BYTES> TQ_DEV void tq_load_bytes(const void* source, void* target) {
  if (BYTES >= 16) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) {
      uint4 raw;
      asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                   : "=r"(raw.x), "=r"(raw.y), "=r"(raw.z), "=r"(raw.w)
                   : "l"((const char*)source + 16 * i));
      ((uint4*)target)[i] = raw;
    }
  } else if (BYTES == 8) {
    uint2 raw;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(raw.x), "=r"(raw.y) : "l"(source));
    *(uint2*)target = raw;
  } else if (BYTES == 4) {
    unsigned raw;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(raw) : "l"(source));
    *(unsigned*)target = raw;
  } else if (BYTES == 2) {
    *(unsigned short*)target = *(const unsigned short*)source;
  } else {
    *(unsigned char*)target = *(const unsigned char*)source;
  }
}
// Cached variant for broadcast operands, which many threads re-read.
template <int BYTES> TQ_DEV void tq_load_bytes_cached(const void* source, void* target) {
  if (BYTES >= 16) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) ((uint4*)target)[i] = __ldg((const uint4*)source + i);
  } else if (BYTES == 8) {
    *(uint2*)target = __ldg((const uint2*)source);
  } else if (BYTES == 4) {
    *(unsigned*)target = __ldg((const unsigned*)source);
  } else if (BYTES == 2) {
    *(unsigned short*)target = __ldg((const unsigned short*)source);
  } else {
    *(unsigned char*)target = __ldg((const unsigned char*)source);
  }
}
template <int BYTES> TQ_DEV void tq_store_bytes(void* target, const void* source) {
  if (BYTES >= 16) {
#pragma unroll
    for (int i = 0; i < BYTES / 16; ++i) __stcs((uint4*)target + i, ((const uint4*)source)[i]);
  } else if (BYTES == 8) {
    __stcs((uint2*)target, *(const uint2*)source);
  } else if (BYTES == 4) {
    __stcs((unsigned*)target, *(const unsigned*)source);
  } else if (BYTES == 2) {
    *(unsigned short*)target = *(const unsigned short*)source;
  } else {
    *(unsigned char*)target = *(const unsigned char*)source;
  }
}

template <typename S, int VEC> struct tq_raw_vec {
  typedef typename tq_storage<S>::raw raw;
  __align__(16) raw v[VEC];
};

// ---- operand readers ----------------------------------------------------------------------
// Each fills `out[VEC]` with the operand's values for output positions idx .. idx+VEC-1, all of
// which are in range. idx is a multiple of VEC. `fast` says the host checked that one vector move
// (or one broadcast element) covers the group.

template <typename S, int VEC, typename Index>
TQ_DEV void tq_read_same(const void* pointer, Index idx, typename tq_storage<S>::compute (&out)[VEC]) {
  typedef typename tq_storage<S>::raw raw;
  tq_raw_vec<S, VEC> x;
  tq_load_bytes<sizeof(raw) * VEC>((const raw*)pointer + idx, x.v);
#pragma unroll
  for (int e = 0; e < VEC; ++e) out[e] = tq_storage<S>::load(x.v[e]);
}

template <typename S, typename Index>
TQ_DEV typename tq_storage<S>::compute tq_read_one(const void* pointer, Index position) {
  typedef typename tq_storage<S>::raw raw;
  return tq_storage<S>::load(__ldg((const raw*)pointer + position));
}

// i / d without a division. For 32-bit indices the host passes magic = floor(2^64 / d) + 1 (2^64 - 1
// for d = 1): the high half of idx * magic is the quotient for every idx below 2^32 and every d below
// 2^32 (the excess of magic * d over 2^64 is at most d, so the error stays below 2^-32 <= 1 / d); the
// single correction step covers d = 1. A 32-bit `/` or `%` costs about sixteen instructions, three of
// them on the special-function unit that the exponentials of a fused chain need.
TQ_DEV unsigned tq_quotient(unsigned idx, unsigned divisor, unsigned long long magic) {
  unsigned q = (unsigned)__umul64hi(magic, (unsigned long long)idx);
  if (idx - q * divisor >= divisor) ++q;
  return q;
}
TQ_DEV long long tq_quotient(long long idx, long long divisor, unsigned long long) { return idx / divisor; }

// i % d: a row that repeats, such as a bias.
template <typename S, int VEC, typename Index>
TQ_DEV void tq_read_cycled(const void* pointer, Index idx, Index divisor, unsigned long long magic, bool fast,
                           typename tq_storage<S>::compute (&out)[VEC]) {
  typedef typename tq_storage<S>::raw raw;
  Index position = idx - tq_quotient(idx, divisor, magic) * divisor;
  if (VEC > 1 && fast) {
    tq_raw_vec<S, VEC> x;
    tq_load_bytes_cached<sizeof(raw) * VEC>((const raw*)pointer + position, x.v);
#pragma unroll
    for (int e = 0; e < VEC; ++e) out[e] = tq_storage<S>::load(x.v[e]);
  } else {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      out[e] = tq_read_one<S, Index>(pointer, position);
      if (++position == divisor) position = 0;
    }
  }
}

// i / d: one value per run of d outputs, such as an [N, 1] column.
template <typename S, int VEC, typename Index>
TQ_DEV void tq_read_repeated(const void* pointer, Index idx, Index divisor, unsigned long long magic, bool fast,
                             typename tq_storage<S>::compute (&out)[VEC]) {
  Index position = tq_quotient(idx, divisor, magic);
  if (VEC > 1 && fast) {
    const typename tq_storage<S>::compute value = tq_read_one<S, Index>(pointer, position);
#pragma unroll
    for (int e = 0; e < VEC; ++e) out[e] = value;
  } else {
    Index within = idx - position * divisor;
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      out[e] = tq_read_one<S, Index>(pointer, position);
      if (++within == divisor) { within = 0; ++position; }
    }
  }
}

template <typename Index>
TQ_DEV long long tq_unravel(const tq_layout_t& layout, Index idx) {
  long long offset = 0;
#pragma unroll
  for (int d = 7; d >= 0; --d) {
    if (d < layout.rank) {
      const Index extent = (Index)layout.sizes[d];
      const Index quotient = tq_quotient(idx, extent, layout.magics[d]);
      const Index coordinate = idx - quotient * extent;
      idx = quotient;
      offset += (long long)coordinate * layout.strides[d];
    }
  }
  return offset;
}

// A strided or oddly broadcast operand: the position unravelled over the output's extents.
template <typename S, int VEC, typename Index>
TQ_DEV void tq_read_strided(const void* pointer, Index idx, const tq_layout_t& layout, bool fast,
                            typename tq_storage<S>::compute (&out)[VEC]) {
  typedef typename tq_storage<S>::raw raw;
  if (VEC > 1 && fast) {
    tq_raw_vec<S, VEC> x;
    tq_load_bytes<sizeof(raw) * VEC>((const raw*)pointer + tq_unravel<Index>(layout, idx), x.v);
#pragma unroll
    for (int e = 0; e < VEC; ++e) out[e] = tq_storage<S>::load(x.v[e]);
  } else if (VEC > 1 && layout.rank > 0 && layout.sizes[layout.rank - 1] % VEC == 0) {
    // the vector's elements share every coordinate but the innermost (a tile starts on a multiple of VEC,
    // the innermost extent is one): one unravel, then steps of the innermost stride — a column slice, an
    // every-other-column view and a broadcast innermost axis (stride 0) all come here
    const long long first = tq_unravel<Index>(layout, idx);
    const long long step = layout.strides[layout.rank - 1];
#pragma unroll
    for (int e = 0; e < VEC; ++e) out[e] = tq_read_one<S, long long>(pointer, first + (long long)e * step);
  } else {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      out[e] = tq_read_one<S, long long>(pointer, tq_unravel<Index>(layout, idx + (Index)e));
    }
  }
}

template <typename S, int VEC, typename Index>
TQ_DEV void tq_write(void* pointer, Index idx, const typename tq_storage<S>::compute (&values)[VEC]) {
  typedef typename tq_storage<S>::raw raw;
  tq_raw_vec<S, VEC> y;
#pragma unroll
  for (int e = 0; e < VEC; ++e) y.v[e] = tq_storage<S>::store(values[e]);
  tq_store_bytes<sizeof(raw) * VEC>((raw*)pointer + idx, y.v);
}
)TQ";

}  // namespace tq
