// GEMM + bias + activation on the 5th-generation tensor cores (tcgen05), for sm_100a.
//
//   C[b] = act(op(A[b]) @ op(B[b]) + bias)      bf16 or f16 operands, f32 accumulation, one rounding
//
// One persistent CTA per SM walks 128 x 256 output tiles. Inside a CTA, ten warps have three jobs:
//
//   warp 0, one lane   producer: TMA loads (cp.async.bulk.tensor, 128-byte swizzle) of a
//                      128 x 64 slice of A and a 256 x 64 slice of B into a 3-stage ring in
//                      shared memory, each stage announced on an mbarrier by its byte count;
//   warp 1, one lane   issuer: for every stage four tcgen05.mma (128 x 256 x 16) accumulating in
//                      tensor memory; tcgen05.commit hands the stage back to the producer and, after
//                      the last slice of a tile, hands the accumulator to the epilogue;
//   warps 2..9         epilogue: tcgen05.ld of the f32 accumulator (each warp 32 lanes of tensor
//                      memory by half of the columns), + bias, activation in f32, one rounding, a
//                      regrouping through shared memory, whole-line 128-bit stores.
//
// Tensor memory holds two 128 x 256 f32 accumulators (all 512 columns), so the epilogue of tile i
// runs under the MMAs of tile i+1. Either operand may be K-major (row-major A, nn.Linear weight
// [n,k]) or MN-major (A stored [k,m]; B stored [k,n], the `A @ B` form): transposed operands are
// consumed in place through the shared-memory descriptor's major bit, never copied
// (csrc/tessiq/codegen/gemm.cpp:28-53 in the reference does the same through cuBLAS flags).
// No load uses cluster multicast. Every wait is bounded: a wait that gives up sets the device
// status word (see tq_status_poll) and the CTA leaves through the normal teardown, freeing its
// tensor memory.
//
// Replaces launch_gemm + the bias pre-fill (csrc/tessiq/codegen/blas.cpp:92-193,
// csrc/tessiq/codegen/gemm.cpp:186-199) and the custom ops gemm_bias_gelu_tanh
// (csrc/custom_ops/gemm_bias_gelu_tanh/gemm_bias_gelu_tanh.nvcc.cu:219-288) and gemm_bias_gelu
// (csrc/custom_ops/gemm_bias_gelu/gemm_bias_gelu.nvcc.cu:90-158).
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <type_traits>

#include "common.h"
#include "tcgen05.h"

namespace tq {
namespace {

constexpr int kTileM = 128;
constexpr int kTileN = 256;
constexpr int kTileK = 64;    // 64 two-byte elements = one 128-byte swizzle row
constexpr int kStages = 3;
constexpr int kMmaK = 16;
constexpr int kThreads = 320;           // producer warp, issuer warp, eight epilogue warps
constexpr int kEpilogueThreads = 256;
constexpr int kEpilogueWarps = kEpilogueThreads / 32;
constexpr int kStoreColumns = 64;       // columns an epilogue warp regroups at a time
constexpr uint32_t kStoreBytes = 32 * kStoreColumns * 2;   // 4 KiB of staging per epilogue warp
constexpr uint32_t kBytesA = kTileM * kTileK * 2;   // 16 KiB
constexpr uint32_t kBytesB = kTileN * kTileK * 2;   // 32 KiB
constexpr uint32_t kStageBytes = kBytesA + kBytesB;
constexpr uint32_t kChunkBytes = 64 * kTileK * 2;   // one 64-wide MN chunk of an MN-major operand: 8 KiB
constexpr uint32_t kTmemColumns = 512;

constexpr size_t kSmemBytes = 1024 /*alignment slack*/ + static_cast<size_t>(kStages) * kStageBytes +
                              2 * kTileN * sizeof(float) /*bias*/ + 256 /*barriers, tmem slot*/ + kEpilogueWarps * kStoreBytes;

enum WaitCode { kWaitEmpty = 101, kWaitFull = 102, kWaitTmemEmpty = 103, kWaitTmemFull = 104 };

struct GemmParams {
  int m, n, k, batch;
  int tiles_m, tiles_n;
  long long num_tiles;
  const void* bias;
  const void* residual;            // added after the activation, or null
  long long ldr, stride_r;
  void* c;
  long long ldc, stride_c;
  int activation;
  WaitStatus status;
};

// Instruction descriptor of tcgen05.mma kind::f16: f32 accumulator, A/B format (0 f16, 1 bf16),
// major bits (0 K-major, 1 MN-major), N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t instruction_descriptor(bool bf16, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(kTileN >> 3) << 17) |
         (static_cast<uint32_t>(kTileM >> 4) << 24);
}

__device__ __forceinline__ float activate(float v, int activation) {
  if (activation == TQ_ACT_GELU_TANH) {
    // 0.5 v (1 + tanh(k (v + 0.044715 v^3))) = v / (1 + exp(-2k (v + 0.044715 v^3)))
    return v * rcp_ftz(1.0f + exp2_ftz(-2.302208198144325f * (v + 0.044715f * v * v * v)));
  }
  if (activation == TQ_ACT_GELU_ERF) return 0.5f * v * (1.0f + erff(v * 0.70710678118654752440f));
  return v;
}

// A barrier of the eight epilogue warps (named barrier 1) that also returns whether `ok` held on every
// one of its threads, so that a bounded wait that gave up on one warp takes all of them out at once.
__device__ __forceinline__ bool epilogue_all(bool ok) {
  uint32_t all;
  asm volatile(
      "{\n\t.reg .pred mine, every;\n\t"
      "setp.ne.b32 mine, %1, 0;\n\t"
      "bar.red.and.pred every, 1, %2, mine;\n\t"
      "selp.u32 %0, 1, 0, every;\n\t}"
      : "=r"(all)
      : "r"(static_cast<uint32_t>(ok)), "n"(kEpilogueThreads)
      : "memory");
  return all != 0;
}

// The same on two elements at once with the .f32x2 forms of add, mul and fma, and with the
// activation a compile-time constant: the epilogue of a short-K product (12 k-blocks at K = 768) is
// what the CTA waits for, and it is bound by the instructions its eight warps issue.
template <int ACTIVATION>
__device__ __forceinline__ float2 activate_pair(float2 v) {
  if constexpr (ACTIVATION == TQ_ACT_GELU_TANH) {
    // v / (1 + exp2(v (c0 + c1 v^2))), c0 = -2 k log2(e) = -2.3022082, c1 = 0.044715 c0
    const float2 square = __fmul2_rn(v, v);
    const float2 inner = __ffma2_rn(square, make_float2(-0.10294324f, -0.10294324f), make_float2(-2.302208198144325f, -2.302208198144325f));
    const float2 t = __fmul2_rn(v, inner);
    const float2 denominator = __fadd2_rn(make_float2(exp2_ftz(t.x), exp2_ftz(t.y)), make_float2(1.0f, 1.0f));
    return __fmul2_rn(v, make_float2(rcp_ftz(denominator.x), rcp_ftz(denominator.y)));
  } else if constexpr (ACTIVATION == TQ_ACT_GELU_ERF) {
    // 0.5 v (1 + erf(v / sqrt 2)) = v Phi(v), Phi(v) = 1 - h for v >= 0 and h for v < 0, where
    // h = 0.5 erfc(|v| / sqrt 2) and erfc(z) = exp(-z^2) P(t), t = 1 / (1 + 0.3275911 z), P a polynomial
    // of degree 8 without a constant term fitted to erfc(z) exp(z^2) over 0 <= z <= 10 with a RELATIVE
    // error of 4e-7, so the negative tail keeps its digits (erff's branches cost 25 instructions per
    // element, this is 12). |v| is clamped at 14.2, where erfc has left the f32 range. As with the
    // erff form: +inf gives +inf, -inf gives NaN (inf * 0), NaN stays NaN, -0 stays -0.
    float2 a;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(a.x) : "f"(fabsf(v.x)), "f"(14.2f));
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(a.y) : "f"(fabsf(v.y)), "f"(14.2f));
    auto both = [](float c) { return make_float2(c, c); };
    const float2 denominator = __ffma2_rn(a, both(0.3275911f * 0.70710678118654752440f), both(1.0f));
    const float2 t = make_float2(rcp_ftz(denominator.x), rcp_ftz(denominator.y));
    const float2 exponent = __ffma2_rn(__fmul2_rn(a, a), both(-0.72134752044448170368f), both(-1.0f));   // log2(0.5 exp(-z^2)), z^2 = a^2 / 2
    const float2 decay = make_float2(exp2_ftz(exponent.x), exp2_ftz(exponent.y));
    float2 poly = __ffma2_rn(both(-0.140646293759346f), t, both(0.49450618028640747f));
    poly = __ffma2_rn(poly, t, both(-0.4017721116542816f));
    poly = __ffma2_rn(poly, t, both(0.4490189850330353f));
    poly = __ffma2_rn(poly, t, both(0.02793201059103012f));
    poly = __ffma2_rn(poly, t, both(0.2050340622663498f));
    poly = __ffma2_rn(poly, t, both(0.18088608980178833f));
    poly = __ffma2_rn(poly, t, both(0.18504123389720917f));
    const float2 h = __fmul2_rn(__fmul2_rn(poly, t), decay);
    const float2 upper = __ffma2_rn(h, both(-1.0f), both(1.0f));
    return __fmul2_rn(v, make_float2(v.x >= 0.0f ? upper.x : h.x, v.y >= 0.0f ? upper.y : h.y));
  } else {
    return v;
  }
}

// Eight consecutive columns of one row: accumulators + bias, activation, residual, one rounding.
template <typename T, int ACTIVATION, bool RESIDUAL>
__device__ __forceinline__ uint4 finish_unit(const uint32_t (&r0)[32], const uint32_t (&r1)[32], const float* bias, int unit, const uint4& residual) {
  Vec<T, 8> out;
  const Vec<T, 8> add = *reinterpret_cast<const Vec<T, 8>*>(&residual);
  const float4 bias_low = *reinterpret_cast<const float4*>(bias + unit * 8), bias_high = *reinterpret_cast<const float4*>(bias + unit * 8 + 4);
  const float bias_of[8] = {bias_low.x, bias_low.y, bias_low.z, bias_low.w, bias_high.x, bias_high.y, bias_high.z, bias_high.w};
#pragma unroll
  for (int e = 0; e < 8; e += 2) {
    const int j = unit * 8 + e;
    const float2 accumulator = make_float2(__uint_as_float(j < 32 ? r0[j] : r1[j - 32]), __uint_as_float(j < 32 ? r0[j + 1] : r1[j - 31]));
    float2 value = activate_pair<ACTIVATION>(__fadd2_rn(accumulator, make_float2(bias_of[e], bias_of[e + 1])));
    if constexpr (RESIDUAL) value = __fadd2_rn(value, make_float2(to_compute(add.v[e]), to_compute(add.v[e + 1])));
    out.v[e] = from_compute<T, float>(value.x);
    out.v[e + 1] = from_compute<T, float>(value.y);
  }
  return *reinterpret_cast<const uint4*>(&out);
}

// Tiles in groups of 16 rows of tiles, so that the CTAs running at one time share A and B slices
// in L2.
__device__ __forceinline__ void tile_coordinates(long long tile, const GemmParams& p, int& batch, int& tile_m, int& tile_n) {
  const long long per_batch = static_cast<long long>(p.tiles_m) * p.tiles_n;
  batch = static_cast<int>(tile / per_batch);
  const int t = static_cast<int>(tile % per_batch);
  constexpr int kGroup = 16;
  const int group_span = kGroup * p.tiles_n;
  const int group = t / group_span;
  const int first_m = group * kGroup;
  const int rows = min(kGroup, p.tiles_m - first_m);
  tile_m = first_m + (t % group_span) % rows;
  tile_n = (t % group_span) / rows;
}

// One epilogue warp's share of a 128 x 256 accumulator: the 32 rows of its tensor-memory lanes by
// the 128 columns of its half. Per 64 columns: tcgen05.ld (lane i holds row i), + bias, activation,
// one rounding, then the 32 x 64 block goes through 4 KiB of this warp's shared memory (16-byte
// units XOR-swizzled by row, conflict-free both ways) so that each store instruction writes four
// whole 128-byte lines of C instead of 32 scattered 16-byte pieces. A residual tile (added after
// the activation, before the one rounding) takes the same road the other way: whole lines from
// global memory into the staging block, then each thread picks up its own row.
template <typename T>
__device__ __forceinline__ void epilogue_rows(uint32_t tmem_accumulator, int quarter, int half, int lane, const float* bias_tile,
                                              T* c_tile, long long ldc, const T* residual_tile, long long ldr, int rows_left,
                                              int columns_left, int activation, unsigned char* staging, bool vector_ok) {
  const int row = quarter * 32 + lane;
  const uint32_t staging_address = smem_address(staging);
#pragma unroll 1
  for (int step = 0; step < (kTileN / 2) / kStoreColumns; ++step) {
    const int column0 = half * (kTileN / 2) + step * kStoreColumns;
    uint4 residual_words[8];
    if (residual_tile != nullptr && vector_ok) {      // issued before the tensor-memory load so the two latencies overlap
      const int unit = lane & 7;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = quarter * 32 + i * 4 + (lane >> 3);
        residual_words[i] = make_uint4(0, 0, 0, 0);
        if (r < rows_left && column0 + unit * 8 < columns_left) {
          residual_words[i] = __ldg(reinterpret_cast<const uint4*>(residual_tile + static_cast<long long>(r) * ldr + column0 + unit * 8));
        }
      }
    }
    uint32_t r0[32], r1[32];
    tmem_load_32(tmem_accumulator + column0 + (static_cast<uint32_t>(quarter * 32) << 16), r0);
    tmem_load_32(tmem_accumulator + column0 + 32 + (static_cast<uint32_t>(quarter * 32) << 16), r1);
    tmem_load_wait();
    if (vector_ok) {
      if (residual_tile != nullptr) {
        const int unit = lane & 7;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(staging_address + r * 128 + ((unit ^ (r & 7)) << 4)),
                       "r"(residual_words[i].x), "r"(residual_words[i].y), "r"(residual_words[i].z), "r"(residual_words[i].w)
                       : "memory");
        }
        __syncwarp();
      }
      auto finish = [&](auto activation_tag, auto residual_tag) {
        constexpr int kActivation = decltype(activation_tag)::value;
        constexpr bool kResidual = decltype(residual_tag)::value;
#pragma unroll
        for (int unit = 0; unit < 8; ++unit) {
          uint4 word = make_uint4(0, 0, 0, 0);
          if constexpr (kResidual) {
            asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(word.x), "=r"(word.y), "=r"(word.z), "=r"(word.w)
                         : "r"(staging_address + lane * 128 + ((unit ^ (lane & 7)) << 4))
                         : "memory");
          }
          word = finish_unit<T, kActivation, kResidual>(r0, r1, bias_tile + column0, unit, word);
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(staging_address + lane * 128 + ((unit ^ (lane & 7)) << 4)),
                       "r"(word.x), "r"(word.y), "r"(word.z), "r"(word.w)
                       : "memory");
        }
      };
      auto finish_with = [&](auto activation_tag) {
        if (residual_tile != nullptr) {
          finish(activation_tag, std::true_type{});
        } else {
          finish(activation_tag, std::false_type{});
        }
      };
      if (activation == TQ_ACT_GELU_TANH) {
        finish_with(std::integral_constant<int, TQ_ACT_GELU_TANH>{});
      } else if (activation == TQ_ACT_GELU_ERF) {
        finish_with(std::integral_constant<int, TQ_ACT_GELU_ERF>{});
      } else {
        finish_with(std::integral_constant<int, TQ_ACT_NONE>{});
      }
      __syncwarp();
      const int unit = lane & 7;
      if (column0 + unit * 8 < columns_left) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + (lane >> 3);
          uint4 word;
          asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                       : "=r"(word.x), "=r"(word.y), "=r"(word.z), "=r"(word.w)
                       : "r"(staging_address + r * 128 + ((unit ^ (r & 7)) << 4))
                       : "memory");
          if (quarter * 32 + r < rows_left) {
            *reinterpret_cast<uint4*>(c_tile + static_cast<long long>(quarter * 32 + r) * ldc + column0 + unit * 8) = word;
          }
        }
      }
      __syncwarp();
    } else if (row < rows_left) {
      T* c_row = c_tile + static_cast<long long>(row) * ldc + column0;
      const T* residual_row = residual_tile == nullptr ? nullptr : residual_tile + static_cast<long long>(row) * ldr + column0;
#pragma unroll
      for (int j = 0; j < 64; ++j) {
        if (column0 + j < columns_left) {
          float value = activate(__uint_as_float(j < 32 ? r0[j] : r1[j - 32]) + bias_tile[column0 + j], activation);
          if (residual_row != nullptr) value += to_compute(residual_row[j]);
          c_row[j] = from_compute<T, float>(value);
        }
      }
    }
  }
}

template <typename T, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bias_act_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  extern __shared__ unsigned char raw_smem[];
  const uint32_t base = (smem_address(raw_smem) + 1023u) & ~1023u;   // swizzled tiles need 1024-byte alignment
  unsigned char* aligned = raw_smem + (base - smem_address(raw_smem));
  float* bias_smem = reinterpret_cast<float*>(aligned + kStages * kStageBytes);        // [2][kTileN]
  const uint32_t barriers = base + kStages * kStageBytes + 2 * kTileN * sizeof(float);
  // barrier slots, 8 bytes each: full[kStages], empty[kStages], tmem_full[2], tmem_empty[2]
  auto full_bar = [&](int s) { return barriers + 8u * s; };
  auto empty_bar = [&](int s) { return barriers + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return barriers + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return barriers + 8u * (2 * kStages + 2 + a); };
  const uint32_t tmem_slot = barriers + 8u * (2 * kStages + 4);
  volatile uint32_t* tmem_slot_pointer =
      reinterpret_cast<volatile uint32_t*>(aligned + kStages * kStageBytes + 2 * kTileN * sizeof(float) + 8 * (2 * kStages + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) p.status.begin();   // this launch's abort word starts clear
    for (int s = 0; s < kStages; ++s) {
      barrier_init(full_bar(s), 1);
      barrier_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      barrier_init(tmem_full_bar(a), 1);
      barrier_init(tmem_empty_bar(a), kEpilogueThreads / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemColumns);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_pointer;

  const int k_blocks = (p.k + kTileK - 1) / kTileK;

  if (warp == 0) {
    // ---- producer --------------------------------------------------------------------------
    if (lane == 0) {
      uint32_t iteration = 0;
      bool alive = true;
      for (long long tile = blockIdx.x; alive && tile < p.num_tiles; tile += gridDim.x) {
        int batch, tile_m, tile_n;
        tile_coordinates(tile, p, batch, tile_m, tile_n);
        for (int kb = 0; kb < k_blocks; ++kb, ++iteration) {
          const int s = iteration % kStages;
          const uint32_t phase = (iteration / kStages) & 1;
          if (!barrier_wait(empty_bar(s), phase ^ 1, p.status, kWaitEmpty)) { alive = false; break; }
          barrier_expect_tx(full_bar(s), kStageBytes);
          const uint32_t smem_a = base + s * kStageBytes;
          const uint32_t smem_b = smem_a + kBytesA;
          const int k0 = kb * kTileK;
          if constexpr (A_MN) {
#pragma unroll
            for (int i = 0; i < kTileM / 64; ++i) tma_load_3d(smem_a + i * kChunkBytes, &map_a, full_bar(s), tile_m * kTileM + i * 64, k0, batch);
          } else {
            tma_load_3d(smem_a, &map_a, full_bar(s), k0, tile_m * kTileM, batch);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int i = 0; i < kTileN / 64; ++i) tma_load_3d(smem_b + i * kChunkBytes, &map_b, full_bar(s), tile_n * kTileN + i * 64, k0, batch);
          } else {
            tma_load_3d(smem_b, &map_b, full_bar(s), k0, tile_n * kTileN, batch);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ------------------------------------------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = instruction_descriptor(std::is_same_v<T, __nv_bfloat16>, A_MN, B_MN);
      // K-major: 8-row groups are 1024 B apart; a step of 16 along K is 32 B inside the swizzle row.
      // MN-major: 64-wide chunks are kChunkBytes apart, groups of 8 K-rows 1024 B; 16 K-rows = 2048 B.
      constexpr uint32_t lead_a = A_MN ? kChunkBytes : 0, lead_b = B_MN ? kChunkBytes : 0;
      constexpr uint32_t step_a16 = (A_MN ? 2048 : 32) >> 4, step_b16 = (B_MN ? 2048 : 32) >> 4;
      // Descriptors as (low, high) words stepped by one add, stage and phase as counters, no
      // tcgen05 fence per k-block: what this lane does between two k-blocks is time the pipe can run dry.
      constexpr uint32_t kHigh = kDescriptorHigh;
      const uint32_t low_a0 = descriptor_low(base, lead_a), low_b0 = descriptor_low(base + kBytesA, lead_b);
      uint32_t s = 0, phase = 0;
      uint32_t local_tile = 0;
      bool alive = true;
      for (long long tile = blockIdx.x; alive && tile < p.num_tiles; tile += gridDim.x, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!barrier_wait(tmem_empty_bar(acc), acc_phase ^ 1, p.status, kWaitTmemEmpty)) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kTileN;
        uint32_t accumulate = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!barrier_wait(full_bar(s), phase, p.status, kWaitFull)) { alive = false; break; }
          const uint32_t low_a = low_a0 + s * (kStageBytes >> 4), low_b = low_b0 + s * (kStageBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < kTileK / kMmaK; ++kk) {
            mma_f16_split(tmem_d, low_a + kk * step_a16, kHigh, low_b + kk * step_b16, kHigh, idesc, accumulate);
            accumulate = 1;
          }
          mma_commit(empty_bar(s));                        // the stage is free once these MMAs have read it
          if (++s == kStages) { s = 0; phase ^= 1; }
        }
        if (alive) mma_commit(tmem_full_bar(acc));         // the tile is complete
      }
    }
  } else {
    // ---- epilogue: warps 2..9; warp w owns tensor-memory lanes 32 (w % 4) .. +31 and the
    // columns of half (w - 2) / 4 ---------------------------------------------------------------
    const int epilogue_thread = threadIdx.x - 64;
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    unsigned char* staging = aligned + kStages * kStageBytes + 2 * kTileN * sizeof(float) + 256 + (warp - 2) * kStoreBytes;
    const bool vector_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) && (p.stride_c % 8 == 0) && (p.n % 8 == 0) &&
                           (p.residual == nullptr || ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0) && (p.stride_r % 8 == 0)));
    uint32_t local_tile = 0;
    for (long long tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++local_tile) {
      int batch, tile_m, tile_n;
      tile_coordinates(tile, p, batch, tile_m, tile_n);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      const int n0 = tile_n * kTileN;
      float* bias_tile = bias_smem + acc * kTileN;
      for (int j = epilogue_thread; j < kTileN; j += kEpilogueThreads) {
        float value = 0.f;
        if (p.bias != nullptr && n0 + j < p.n) value = to_compute(static_cast<const T*>(p.bias)[n0 + j]);
        bias_tile[j] = value;
      }
      // The give-up is decided for the epilogue as a whole: every epilogue thread reaches the named
      // barrier, which also carries the AND of their waits, and all leave together or none does.
      const bool arrived = barrier_wait(tmem_full_bar(acc), acc_phase, p.status, kWaitTmemFull);
      tcgen05_fence_after();
      if (!epilogue_all(arrived)) break;   // also: bias_tile is complete

      T* c_tile = static_cast<T*>(p.c) + static_cast<long long>(batch) * p.stride_c + static_cast<long long>(tile_m) * kTileM * p.ldc + n0;
      const T* residual_tile = p.residual == nullptr ? nullptr : static_cast<const T*>(p.residual) + static_cast<long long>(batch) * p.stride_r +
                                                                  static_cast<long long>(tile_m) * kTileM * p.ldr + n0;
      epilogue_rows<T>(tmem_base + acc * kTileN, quarter, half, lane, bias_tile, c_tile, p.ldc, residual_tile, p.ldr, p.m - tile_m * kTileM,
                       p.n - n0, p.activation, staging, vector_ok);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) barrier_arrive(tmem_empty_bar(acc));   // this warp has read its part of the accumulator
    }
  }

  // ---- teardown: every thread arrives here, also after a wait that gave up -----------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kTmemColumns);
  }
}


// ---------------------------------------------------------------------------------------------
// The CTA-pair variant: two CTAs on neighbouring SMs (a cluster of 2) compute one 256 x 256 tile
// with tcgen05.mma.cta_group::2. Each CTA loads its own 128 rows of A and its own 128 columns of B
// (half the bytes per SM of the single-CTA tile), each CTA's tensor memory holds its 128 rows of the
// accumulator, and each CTA's epilogue warps write those rows. One lane of the even CTA (the
// leader) issues the MMAs for both; the stages' "full" barriers live in the leader and count the
// bytes of both CTAs' TMA loads (the loads name the leader's barrier; they are plain loads, no
// multicast); tcgen05.commit reports to the barriers of both CTAs.

constexpr int kPairStages = 5;
constexpr int kPairTileM = 256;
constexpr uint32_t kPairBytesB = (kTileN / 2) * kTileK * 2;     // 16 KiB: this CTA's half of B
constexpr uint32_t kPairStageBytes = kBytesA + kPairBytesB;      // 32 KiB per CTA per stage
constexpr size_t kPairSmemBytes = 1024 + static_cast<size_t>(kPairStages) * kPairStageBytes + 2 * kTileN * sizeof(float) + 256 +
                                  kEpilogueWarps * kStoreBytes;

__host__ __device__ constexpr uint32_t pair_instruction_descriptor(bool bf16, bool a_mn_major, bool b_mn_major) {
  return (1u << 4) | ((bf16 ? 1u : 0u) << 7) | ((bf16 ? 1u : 0u) << 10) | ((a_mn_major ? 1u : 0u) << 15) |
         ((b_mn_major ? 1u : 0u) << 16) | (static_cast<uint32_t>(kTileN >> 3) << 17) |
         (static_cast<uint32_t>(kPairTileM >> 4) << 24);
}

template <typename T, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bias_act_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const GemmParams p) {
  extern __shared__ unsigned char raw_smem[];
  const uint32_t base = (smem_address(raw_smem) + 1023u) & ~1023u;
  unsigned char* aligned = raw_smem + (base - smem_address(raw_smem));
  float* bias_smem = reinterpret_cast<float*>(aligned + kPairStages * kPairStageBytes);
  const uint32_t barriers = base + kPairStages * kPairStageBytes + 2 * kTileN * sizeof(float);
  auto full_bar = [&](int s) { return barriers + 8u * s; };                       // used in the leader only
  auto empty_bar = [&](int s) { return barriers + 8u * (kPairStages + s); };       // one per CTA
  auto tmem_full_bar = [&](int a) { return barriers + 8u * (2 * kPairStages + a); };      // one per CTA
  auto tmem_empty_bar = [&](int a) { return barriers + 8u * (2 * kPairStages + 2 + a); }; // used in the leader only
  const uint32_t tmem_slot = barriers + 8u * (2 * kPairStages + 4);
  volatile uint32_t* tmem_slot_pointer =
      reinterpret_cast<volatile uint32_t*>(aligned + kPairStages * kPairStageBytes + 2 * kTileN * sizeof(float) + 8 * (2 * kPairStages + 4));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();           // 0: leader, 1: peer
  const long long pair = blockIdx.x >> 1;
  const long long pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    if (blockIdx.x == 0) p.status.begin();   // this launch's abort word starts clear
    for (int s = 0; s < kPairStages; ++s) {
      barrier_init(full_bar(s), 2);                // one arrive.expect_tx from each CTA's producer
      barrier_init(empty_bar(s), 1);               // one commit
    }
    for (int a = 0; a < 2; ++a) {
      barrier_init(tmem_full_bar(a), 1);           // one commit
      barrier_init(tmem_empty_bar(a), 2 * (kEpilogueThreads / 32));   // the epilogue warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, kTmemColumns);
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();                              // the peer's barriers exist before anything signals them
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_pointer;

  const int k_blocks = (p.k + kTileK - 1) / kTileK;

  if (warp == 0) {
    // ---- producer (one lane in each CTA) -----------------------------------------------------
    if (lane == 0) {
      uint32_t iteration = 0;
      bool alive = true;
      for (long long tile = pair; alive && tile < p.num_tiles; tile += pairs) {
        int batch, tile_m, tile_n;
        tile_coordinates(tile, p, batch, tile_m, tile_n);
        const int m0 = tile_m * kPairTileM + static_cast<int>(rank) * kTileM;
        const int n0 = tile_n * kTileN + static_cast<int>(rank) * (kTileN / 2);
        for (int kb = 0; kb < k_blocks; ++kb, ++iteration) {
          const int s = iteration % kPairStages;
          const uint32_t phase = (iteration / kPairStages) & 1;
          if (!barrier_wait(empty_bar(s), phase ^ 1, p.status, kWaitEmpty)) { alive = false; break; }
          const uint32_t leader_full = peer_address(full_bar(s), 0);
          remote_expect_tx(leader_full, kPairStageBytes);
          const uint32_t smem_a = base + s * kPairStageBytes;
          const uint32_t smem_b = smem_a + kBytesA;
          const int k0 = kb * kTileK;
          if constexpr (A_MN) {
#pragma unroll
            for (int i = 0; i < kTileM / 64; ++i) tma_load_3d_pair(smem_a + i * kChunkBytes, &map_a, leader_full, m0 + i * 64, k0, batch);
          } else {
            tma_load_3d_pair(smem_a, &map_a, leader_full, k0, m0, batch);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int i = 0; i < kTileN / 2 / 64; ++i) tma_load_3d_pair(smem_b + i * kChunkBytes, &map_b, leader_full, n0 + i * 64, k0, batch);
          } else {
            tma_load_3d_pair(smem_b, &map_b, leader_full, k0, n0, batch);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer: one lane of the leader CTA, for both ------------------------------------
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc = pair_instruction_descriptor(std::is_same_v<T, __nv_bfloat16>, A_MN, B_MN);
      constexpr uint32_t lead_a = A_MN ? kChunkBytes : 0, lead_b = B_MN ? kChunkBytes : 0;
      constexpr uint32_t step_a = A_MN ? 2048 : 32, step_b = B_MN ? 2048 : 32;
      uint32_t local_tile = 0;
      bool alive = true;
      // The tensor pipe holds only a couple of MMAs ahead of the one it executes, so whatever this
      // lane does between the last MMA of one k-block and the first of the next is time the pipe
      // can run dry: descriptors are (low, high) words stepped by one add, the stage and its
      // phase are counters (no division), and there is no tcgen05 fence per k-block — the
      // operands come from TMA through the full barrier, not from another thread's tcgen05 work.
      constexpr uint32_t kHigh = kDescriptorHigh;
      constexpr uint32_t step_a16 = step_a >> 4, step_b16 = step_b >> 4;
      const uint32_t low_a0 = descriptor_low(base, lead_a), low_b0 = descriptor_low(base + kBytesA, lead_b);
      uint32_t s = 0, phase = 0;
      for (long long tile = pair; alive && tile < p.num_tiles; tile += pairs, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_phase = (local_tile >> 1) & 1;
        if (!barrier_wait(tmem_empty_bar(acc), acc_phase ^ 1, p.status, kWaitTmemEmpty)) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + acc * kTileN;
        uint32_t accumulate = 0;
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!barrier_wait(full_bar(s), phase, p.status, kWaitFull)) { alive = false; break; }
          const uint32_t low_a = low_a0 + s * (kPairStageBytes >> 4), low_b = low_b0 + s * (kPairStageBytes >> 4);
#pragma unroll
          for (int kk = 0; kk < kTileK / kMmaK; ++kk) {
            mma_f16_pair_split(tmem_d, low_a + kk * step_a16, kHigh, low_b + kk * step_b16, kHigh, idesc, accumulate);
            accumulate = 1;
          }
          mma_commit_pair(empty_bar(s));
          if (++s == kPairStages) { s = 0; phase ^= 1; }
        }
        if (alive) mma_commit_pair(tmem_full_bar(acc));
      }
    }
  } else {
    // ---- epilogue: this CTA's 128 rows of the pair's tile, eight warps -------------------------
    const int epilogue_thread = threadIdx.x - 64;
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    unsigned char* staging = aligned + kPairStages * kPairStageBytes + 2 * kTileN * sizeof(float) + 256 + (warp - 2) * kStoreBytes;
    const bool vector_ok = (p.ldc % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15) == 0) && (p.stride_c % 8 == 0) && (p.n % 8 == 0) &&
                           (p.residual == nullptr || ((p.ldr % 8 == 0) && ((reinterpret_cast<uintptr_t>(p.residual) & 15) == 0) && (p.stride_r % 8 == 0)));
    uint32_t local_tile = 0;
    for (long long tile = pair; tile < p.num_tiles; tile += pairs, ++local_tile) {
      int batch, tile_m, tile_n;
      tile_coordinates(tile, p, batch, tile_m, tile_n);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_phase = (local_tile >> 1) & 1;
      const int n0 = tile_n * kTileN;
      float* bias_tile = bias_smem + acc * kTileN;
      for (int j = epilogue_thread; j < kTileN; j += kEpilogueThreads) {
        float value = 0.f;
        if (p.bias != nullptr && n0 + j < p.n) value = to_compute(static_cast<const T*>(p.bias)[n0 + j]);
        bias_tile[j] = value;
      }
      // The give-up is decided for the epilogue as a whole: every epilogue thread reaches the named
      // barrier, which also carries the AND of their waits, and all leave together or none does.
      const bool arrived = barrier_wait(tmem_full_bar(acc), acc_phase, p.status, kWaitTmemFull);
      tcgen05_fence_after();
      if (!epilogue_all(arrived)) break;   // also: bias_tile is complete

      const int row0 = tile_m * kPairTileM + static_cast<int>(rank) * kTileM;
      T* c_tile = static_cast<T*>(p.c) + static_cast<long long>(batch) * p.stride_c + static_cast<long long>(row0) * p.ldc + n0;
      const T* residual_tile = p.residual == nullptr ? nullptr : static_cast<const T*>(p.residual) + static_cast<long long>(batch) * p.stride_r +
                                                                  static_cast<long long>(row0) * p.ldr + n0;
      epilogue_rows<T>(tmem_base + acc * kTileN, quarter, half, lane, bias_tile, c_tile, p.ldc, residual_tile, p.ldr, p.m - row0, p.n - n0,
                       p.activation, staging, vector_ok);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) remote_arrive(peer_address(tmem_empty_bar(acc), 0));   // tell the leader: this part is drained
    }
  }

  // ---- teardown: both CTAs stay until the pair is done (the leader's MMAs read the peer's
  // shared memory and signal its barriers) -----------------------------------------------------
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    tmem_dealloc_pair(tmem_base, kTmemColumns);
  }
}

// ---------------------------------------------------------------------------------------------
// Host

// A three-axis map over one operand: `inner` contiguous elements, `outer` rows `ld` elements apart,
// `batch` matrices `stride` elements apart; box = box_inner x box_outer x 1, 128-byte swizzle.
tq_status make_map(CUtensorMap* map, tq_dtype dtype, const void* pointer, long long inner, long long outer, long long ld,
                   long long batch, long long stride, int box_inner, int box_outer) {
  EncodeTiled encode = encode_tiled();
  TQ_REQUIRE(encode != nullptr, TQ_EXTERNAL, "the CUDA driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(outer), static_cast<cuuint64_t>(batch)};
  // A stride of 0 (one operand shared by the whole batch) is not a legal map stride; such a map
  // gets one matrix and the kernel is launched with batch coordinate 0 for it (see below).
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(stride > 0 ? stride : ld * outer) * 2};
  const cuuint32_t box[3] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_outer), 1};
  const cuuint32_t element_strides[3] = {1, 1, 1};
  const CUresult result = encode(map, dtype == TQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                                 const_cast<void*>(pointer), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TQ_REQUIRE(result == CUDA_SUCCESS, TQ_UNSUPPORTED, "this operand layout cannot be described to TMA (driver code %d)", static_cast<int>(result));
  return TQ_OK;
}

template <typename T>
tq_status launch_pair(bool a_mn, bool b_mn, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p, int32_t device, cudaStream_t stream) {
  auto go = [&](auto kernel) -> tq_status {
    static std::mutex mutex;
    {
      std::lock_guard<std::mutex> lock(mutex);
      TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kPairSmemBytes)));
    }
    long long pairs = sm_count(device) / 2;
    if (p.num_tiles < pairs) pairs = p.num_tiles;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(static_cast<unsigned>(pairs * 2));
    config.blockDim = dim3(kThreads);
    config.dynamicSmemBytes = kPairSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeClusterDimension;
    attribute[0].val.clusterDim.x = 2;
    attribute[0].val.clusterDim.y = 1;
    attribute[0].val.clusterDim.z = 1;
    config.attrs = attribute;
    config.numAttrs = 1;
    TQ_CUDA(cudaLaunchKernelEx(&config, kernel, map_a, map_b, p));
    return check_launch("gemm_bias_act_pair_kernel");
  };
  if (!a_mn && !b_mn) return go(gemm_bias_act_pair_kernel<T, false, false>);
  if (!a_mn && b_mn) return go(gemm_bias_act_pair_kernel<T, false, true>);
  if (a_mn && !b_mn) return go(gemm_bias_act_pair_kernel<T, true, false>);
  return go(gemm_bias_act_pair_kernel<T, true, true>);
}

template <typename T>
tq_status launch(bool a_mn, bool b_mn, const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmParams& p, int32_t device, cudaStream_t stream) {
  auto go = [&](auto kernel) -> tq_status {
    static std::mutex mutex;
    {
      std::lock_guard<std::mutex> lock(mutex);
      TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes)));
    }
    long long ctas = p.num_tiles < sm_count(device) ? p.num_tiles : sm_count(device);
    kernel<<<static_cast<unsigned>(ctas), kThreads, kSmemBytes, stream>>>(map_a, map_b, p);
    return check_launch("gemm_bias_act_kernel");
  };
  if (!a_mn && !b_mn) return go(gemm_bias_act_kernel<T, false, false>);
  if (!a_mn && b_mn) return go(gemm_bias_act_kernel<T, false, true>);
  if (a_mn && !b_mn) return go(gemm_bias_act_kernel<T, true, false>);
  return go(gemm_bias_act_kernel<T, true, true>);
}

}  // namespace
}  // namespace tq

extern "C" tq_status tq_gemm_bias_act_launch(tq_dtype dtype, tq_activation activation, const void* a, int64_t lda,
                                             int32_t trans_a, const void* b, int64_t ldb, int32_t trans_b,
                                             const void* bias, void* c, int64_t ldc, int64_t m, int64_t n, int64_t k,
                                             int64_t batch, int64_t stride_a, int64_t stride_b, int64_t stride_c,
                                             int32_t device, void* stream) {
  return tq_gemm_bias_act_residual_launch(dtype, activation, a, lda, trans_a, b, ldb, trans_b, bias, nullptr, 0, 0, c, ldc, m, n, k,
                                          batch, stride_a, stride_b, stride_c, device, stream);
}

extern "C" tq_status tq_gemm_bias_act_residual_launch(tq_dtype dtype, tq_activation activation, const void* a, int64_t lda,
                                                      int32_t trans_a, const void* b, int64_t ldb, int32_t trans_b,
                                                      const void* bias, const void* residual, int64_t ldr, int64_t stride_r,
                                                      void* c, int64_t ldc, int64_t m, int64_t n, int64_t k, int64_t batch,
                                                      int64_t stride_a, int64_t stride_b, int64_t stride_c, int32_t device,
                                                      void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) {
    return tq_gemm_bias_act_residual_launch(dtype, activation, a, lda, trans_a, b, ldb, trans_b, bias, residual, ldr, stride_r, c, ldc,
                                            m, n, k, batch, stride_a, stride_b, stride_c, d, s);
  });
  TQ_REQUIRE(dtype == TQ_BF16 || dtype == TQ_F16, TQ_UNSUPPORTED,
             "the tensor-core GEMM takes bf16 or f16 operands, not %s", tq::dtype_name(dtype));
  TQ_REQUIRE(activation >= TQ_ACT_NONE && activation <= TQ_ACT_GELU_TANH, TQ_INVALID_ARGUMENT, "unknown activation %d", activation);
  TQ_REQUIRE(m >= 0 && n >= 0 && k >= 0 && batch >= 0, TQ_INVALID_ARGUMENT, "negative extent in m=%lld n=%lld k=%lld batch=%lld",
             (long long)m, (long long)n, (long long)k, (long long)batch);
  if (m == 0 || n == 0 || batch == 0) return TQ_OK;
  TQ_REQUIRE(k > 0, TQ_UNSUPPORTED, "a product over no elements has no kernel");
  TQ_REQUIRE(a != nullptr && b != nullptr && c != nullptr, TQ_INVALID_ARGUMENT, "null operand or result");
  TQ_REQUIRE(m < (1LL << 31) && n < (1LL << 31) && k < (1LL << 31), TQ_UNSUPPORTED, "extents beyond 2^31 have no kernel");
  // TMA's rules: 16-byte-aligned bases, strides that are multiples of 16 bytes.
  const long long a_inner = trans_a ? m : k, a_outer = trans_a ? k : m;
  const long long b_inner = trans_b ? k : n, b_outer = trans_b ? n : k;
  TQ_REQUIRE(lda >= a_inner && ldb >= b_inner && ldc >= n, TQ_INVALID_ARGUMENT, "a leading dimension is smaller than its row");
  TQ_REQUIRE(tq::aligned_to(a, 16) && tq::aligned_to(b, 16) && lda % 8 == 0 && ldb % 8 == 0 &&
                 (batch == 1 || (stride_a % 8 == 0 && stride_b % 8 == 0)),
             TQ_UNSUPPORTED, "operands must be 16-byte aligned with leading dimensions and batch strides that are multiples of 8 elements");
  TQ_REQUIRE(tq::aligned_to(c, 2) && (bias == nullptr || tq::aligned_to(bias, 2)), TQ_INVALID_ARGUMENT, "misaligned result or bias");
  TQ_REQUIRE(residual == nullptr || (tq::aligned_to(residual, 2) && ldr >= n), TQ_INVALID_ARGUMENT,
             "misaligned residual, or its leading dimension is smaller than a row");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  const tq::WaitStatus status = tq::wait_status_for(device);
  TQ_REQUIRE(status.abort != nullptr, TQ_RESOURCE_EXHAUSTED, "no device memory for the status word");

  // Large problems run on CTA pairs (256 x 256 tiles, half the shared-memory operand traffic per
  // SM); problems with at most one row of 128 x 256 tiles keep the single-CTA kernel.
  const bool pair = m > tq::kTileM;
  CUtensorMap map_a, map_b;
  const long long batch_a = stride_a > 0 ? batch : 1, batch_b = stride_b > 0 ? batch : 1;
  const int b_rows = pair ? tq::kTileN / 2 : tq::kTileN;
  if (tq_status s = tq::make_map(&map_a, dtype, a, a_inner, a_outer, lda, batch_a, stride_a, 64, trans_a ? 64 : tq::kTileM)) return s;
  if (tq_status s = tq::make_map(&map_b, dtype, b, b_inner, b_outer, ldb, batch_b, stride_b, 64, trans_b ? b_rows : 64)) return s;
  TQ_REQUIRE(batch == 1 || (stride_a > 0 && stride_b > 0), TQ_UNSUPPORTED,
             "a batch that shares one operand (stride 0) has no kernel; fold the batch into m instead");

  tq::GemmParams p = {};
  p.m = static_cast<int>(m);
  p.n = static_cast<int>(n);
  p.k = static_cast<int>(k);
  p.batch = static_cast<int>(batch);
  const int tile_m = pair ? tq::kPairTileM : tq::kTileM;
  p.tiles_m = static_cast<int>((m + tile_m - 1) / tile_m);
  p.tiles_n = static_cast<int>((n + tq::kTileN - 1) / tq::kTileN);
  p.num_tiles = static_cast<long long>(p.tiles_m) * p.tiles_n * batch;
  p.bias = bias;
  p.residual = residual;
  p.ldr = ldr;
  p.stride_r = stride_r;
  p.c = c;
  p.ldc = ldc;
  p.stride_c = stride_c;
  p.activation = activation;
  p.status = status;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  if (pair) {
    if (dtype == TQ_BF16) return tq::launch_pair<__nv_bfloat16>(trans_a != 0, trans_b == 0, map_a, map_b, p, device, cuda_stream);
    return tq::launch_pair<__half>(trans_a != 0, trans_b == 0, map_a, map_b, p, device, cuda_stream);
  }
  if (dtype == TQ_BF16) return tq::launch<__nv_bfloat16>(trans_a != 0, trans_b == 0, map_a, map_b, p, device, cuda_stream);
  return tq::launch<__half>(trans_a != 0, trans_b == 0, map_a, map_b, p, device, cuda_stream);
}
