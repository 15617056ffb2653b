// Fused attention on the 5th-generation tensor cores (tcgen05), for sm_100a.
//
//   out[b,h,i,:] = sum_j softmax_j(scale * q[b,h,i,:] . k[b,h,j,:]) v[b,h,j,:]     (j <= i when causal)
//
// bf16 or f16 operands with 64-element heads, f32 scores and sums, one rounding of the result. The
// score matrix never leaves the SM: one CTA owns 256 query rows of one head (two tiles of 128) and
// walks the keys 128 at a time with a running row maximum and row sum (the online form of softmax).
//
//   warps 0..3 / 4..7   one softmax group per query tile, one thread per query row: tcgen05.ld of
//                       the f32 scores from tensor memory, row maximum, ex2, row sum; the
//                       probabilities go to shared memory as a K-major swizzled bf16/f16 tile (the
//                       A operand of the second product); the partial result of the previous
//                       step is read from tensor memory and accumulated in registers.
//   warp 8, one lane    producer: TMA loads (128-byte swizzle) of the two query tiles once, then
//                       one 128 x 64 key tile and one value tile per step into two 3-stage rings.
//   warp 9, one lane    issuer: S = Q K^T (128 x 128 x 64, both operands K-major) and
//                       O = P V (128 x 64 x 128, V consumed MN-major exactly as it lies in memory).
//
// While one group runs its softmax the tensor core computes the other group's products. Q, K, V and
// the result are addressed through (batch, head, token) strides, so the three slices of a fused QKV
// projection are read in place and the result is written directly in [batch, token, head, 64] order:
// none of the four packing copies around `bmm -> where -> softmax -> bmm` remains.
//
// Every wait is bounded; a wait that gives up sets the device status word (tq_status_poll) and the
// CTA leaves through the normal teardown, freeing its tensor memory. No load uses multicast.
//
// The reference has no attention kernel: its compiler emits bmm (csrc/tessiq/codegen/gemm.cpp:100-175),
// a host-side mask, the softmax custom op (csrc/custom_ops/softmax/softmax.cu:19-61) and a second bmm
// for the pattern in tests/python/test_models.py:64-67, with the [batch, heads, T, T] scores in memory.
#include <cuda.h>

#include <cmath>
#include <mutex>
#include <type_traits>

#include "common.h"
#include "tcgen05.h"

namespace tq {
namespace {

constexpr int kHeadDim = 64;
constexpr int kRows = 128;            // query rows per softmax group
constexpr int kGroups = 2;            // query tiles per CTA
constexpr int kKeys = 128;            // keys per step
constexpr int kRing = 3;              // stages of the key ring and of the value ring
constexpr int kAttnThreads = 320;     // 8 softmax warps + producer + issuer
constexpr uint32_t kTileBytes = kRows * kHeadDim * 2;       // 16 KiB: a Q, K or V tile
constexpr uint32_t kProbBytes = kRows * kKeys * 2;          // 32 KiB: one group's probabilities
constexpr uint32_t kOffsetQ = 0;
constexpr uint32_t kOffsetK = kOffsetQ + kGroups * kTileBytes;
constexpr uint32_t kOffsetV = kOffsetK + kRing * kTileBytes;
constexpr uint32_t kOffsetP = kOffsetV + kRing * kTileBytes;
constexpr uint32_t kOffsetBarriers = kOffsetP + kGroups * kProbBytes;
constexpr size_t kAttnSmemBytes = 1024 + kOffsetBarriers + 256;
constexpr uint32_t kAttnTmemColumns = 512;   // S0 | S1 | O0 | O1 = 128 + 128 + 64 + 64, rounded to a power of two
constexpr uint32_t kColumnS = 0, kColumnO = 256;

enum AttnWait { kWaitQ = 201, kWaitKeyEmpty = 202, kWaitValueEmpty = 203, kWaitKeyFull = 204, kWaitValueFull = 205,
                kWaitScores = 206, kWaitProbabilities = 207, kWaitPartial = 208 };

struct AttnParams {
  int batch, heads, q_tokens, k_tokens;
  int q_blocks;                    // CTAs per head
  int causal;
  float scale_log2;                // scale * log2(e)
  void* out;
  long long out_batch, out_head, out_token;   // element strides
  int* status;
};

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// f32 accumulator, A and B of type T, M = 128, N = `n`; B MN-major when `b_mn`.
template <typename T>
__host__ __device__ constexpr uint32_t attn_instruction_descriptor(int n, bool b_mn) {
  constexpr uint32_t format = std::is_same_v<T, __nv_bfloat16> ? 1u : 0u;
  return (1u << 4) | (format << 7) | (format << 10) | ((b_mn ? 1u : 0u) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(kRows >> 4) << 24);
}

template <typename T>
__device__ __forceinline__ uint32_t pack_pair(float low, float high) {
  if constexpr (std::is_same_v<T, __nv_bfloat16>) {
    const __nv_bfloat162 pair = __floats2bfloat162_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
  } else {
    const __half2 pair = __floats2half2_rn(low, high);
    return *reinterpret_cast<const uint32_t*>(&pair);
  }
}

__device__ __forceinline__ void store_shared_16(uint32_t address, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(address), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

template <typename T>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  extern __shared__ unsigned char raw_smem[];
  const uint32_t base = (smem_address(raw_smem) + 1023u) & ~1023u;
  unsigned char* aligned = raw_smem + (base - smem_address(raw_smem));
  const uint32_t barriers = base + kOffsetBarriers;
  // barrier slots, 8 bytes each
  const uint32_t q_full = barriers;
  auto k_full = [&](int s) { return barriers + 8u * (1 + s); };
  auto k_empty = [&](int s) { return barriers + 8u * (1 + kRing + s); };
  auto v_full = [&](int s) { return barriers + 8u * (1 + 2 * kRing + s); };
  auto v_empty = [&](int s) { return barriers + 8u * (1 + 3 * kRing + s); };
  auto s_full = [&](int g) { return barriers + 8u * (1 + 4 * kRing + g); };
  auto p_full = [&](int g) { return barriers + 8u * (1 + 4 * kRing + kGroups + g); };
  auto o_full = [&](int g) { return barriers + 8u * (1 + 4 * kRing + 2 * kGroups + g); };
  constexpr int kBarrierCount = 1 + 4 * kRing + 3 * kGroups;
  const uint32_t tmem_slot = barriers + 8u * kBarrierCount;
  volatile uint32_t* tmem_slot_pointer = reinterpret_cast<volatile uint32_t*>(aligned + kOffsetBarriers + 8 * kBarrierCount);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Which rows of which head: heads in launch order, the long (late) query blocks of a head first.
  const int q_block = p.q_blocks - 1 - static_cast<int>(blockIdx.x % p.q_blocks);
  const int head_index = static_cast<int>(blockIdx.x / p.q_blocks);
  const int head = head_index % p.heads, batch = head_index / p.heads;
  const int q0 = q_block * kGroups * kRows;
  const int key_tiles = (p.k_tokens + kKeys - 1) / kKeys;
  // steps of group g: none when its rows lie beyond the queries; under a causal mask only the key
  // tiles that hold a key <= its last row
  int steps[kGroups];
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    const int first = q0 + g * kRows;
    steps[g] = first >= p.q_tokens ? 0 : (p.causal ? min(key_tiles, (min(first + kRows, p.q_tokens) - 1) / kKeys + 1) : key_tiles);
  }
  const int total_steps = max(steps[0], steps[1]);

  if (threadIdx.x == 0) {
    barrier_init(q_full, 1);
    for (int s = 0; s < kRing; ++s) {
      barrier_init(k_full(s), 1);
      barrier_init(k_empty(s), 1);
      barrier_init(v_full(s), 1);
      barrier_init(v_empty(s), 1);
    }
    for (int g = 0; g < kGroups; ++g) {
      barrier_init(s_full(g), 1);
      barrier_init(p_full(g), kRows);
      barrier_init(o_full(g), 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 9) tmem_alloc(tmem_slot, kAttnTmemColumns);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_pointer;

  if (warp == 8) {
    // ---- producer ----------------------------------------------------------------------------
    if (lane == 0) {
      int valid = 0;
      for (int g = 0; g < kGroups; ++g) valid += steps[g] > 0 ? 1 : 0;
      barrier_expect_tx(q_full, valid * kTileBytes);
      for (int g = 0; g < kGroups; ++g) {
        if (steps[g] > 0) tma_load_4d(base + kOffsetQ + g * kTileBytes, &map_q, q_full, 0, q0 + g * kRows, head, batch);
      }
      for (int j = 0; j < total_steps; ++j) {
        const int s = j % kRing;
        const uint32_t phase = (j / kRing) & 1;
        if (!barrier_wait(k_empty(s), phase ^ 1, p.status, kWaitKeyEmpty)) break;
        barrier_expect_tx(k_full(s), kTileBytes);
        tma_load_4d(base + kOffsetK + s * kTileBytes, &map_k, k_full(s), 0, j * kKeys, head, batch);
        if (!barrier_wait(v_empty(s), phase ^ 1, p.status, kWaitValueEmpty)) break;
        barrier_expect_tx(v_full(s), kTileBytes);
        tma_load_4d(base + kOffsetV + s * kTileBytes, &map_v, v_full(s), 0, j * kKeys, head, batch);
      }
    }
  } else if (warp == 9) {
    // ---- issuer ------------------------------------------------------------------------------
    if (lane == 0 && total_steps > 0) {
      constexpr uint32_t idesc_s = attn_instruction_descriptor<T>(kKeys, false);
      constexpr uint32_t idesc_o = attn_instruction_descriptor<T>(kHeadDim, true);
      // S_g = Q_g K^T: both K-major, 8-row groups 1024 B apart, 16 elements of K = 32 B in the swizzle row
      auto scores = [&](int g, int stage) {
        const uint32_t smem_q = base + kOffsetQ + g * kTileBytes, smem_k = base + kOffsetK + stage * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk) {
          mma_f16(tmem_base + kColumnS + g * kKeys, smem_descriptor(smem_q + kk * 32, 0, 1024),
                  smem_descriptor(smem_k + kk * 32, 0, 1024), idesc_s, kk != 0 ? 1u : 0u);
        }
        mma_commit(s_full(g));
      };
      // O_g = P_g V: P K-major in two 64-key halves 16 KiB apart; V MN-major, 16 keys = 2048 B
      auto partial = [&](int g, int stage) {
        const uint32_t smem_p = base + kOffsetP + g * kProbBytes, smem_v = base + kOffsetV + stage * kTileBytes;
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk) {
          mma_f16(tmem_base + kColumnO + g * kHeadDim, smem_descriptor(smem_p + (kk >> 2) * (kProbBytes / 2) + (kk & 3) * 32, 0, 1024),
                  smem_descriptor(smem_v + kk * 2048, kTileBytes, 1024), idesc_o, kk != 0 ? 1u : 0u);
        }
        mma_commit(o_full(g));
      };
      bool alive = barrier_wait(q_full, 0, p.status, kWaitQ) && barrier_wait(k_full(0), 0, p.status, kWaitKeyFull);
      if (alive) {
        tcgen05_fence_after();
        for (int g = 0; g < kGroups; ++g) {
          if (steps[g] > 0) scores(g, 0);
        }
        mma_commit(k_empty(0));
      }
      for (int j = 0; alive && j < total_steps; ++j) {
        const int s = j % kRing, next = (j + 1) % kRing;
        if (!barrier_wait(v_full(s), (j / kRing) & 1, p.status, kWaitValueFull)) break;
        if (j + 1 < total_steps && !barrier_wait(k_full(next), ((j + 1) / kRing) & 1, p.status, kWaitKeyFull)) break;
        for (int g = 0; g < kGroups; ++g) {
          if (j >= steps[g]) continue;
          if (!barrier_wait(p_full(g), j & 1, p.status, kWaitProbabilities)) { alive = false; break; }
          tcgen05_fence_after();
          partial(g, s);
          if (j + 1 < steps[g]) scores(g, next);
        }
        if (!alive) break;
        mma_commit(v_empty(s));
        if (j + 1 < total_steps) mma_commit(k_empty(next));
      }
    }
  } else {
    // ---- softmax groups: warp w of a group owns tensor-memory lanes 32 (w % 4) .. +31 ---------
    const int g = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int query = q0 + g * kRows + row;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tmem_s = tmem_base + kColumnS + g * kKeys + lane_base;
    const uint32_t tmem_o = tmem_base + kColumnO + g * kHeadDim + lane_base;
    const uint32_t smem_p_row = base + kOffsetP + g * kProbBytes + row * 128;
    const uint32_t swizzle = static_cast<uint32_t>(row & 7);
    const int my_steps = steps[g];
    float acc[kHeadDim];
#pragma unroll
    for (int i = 0; i < kHeadDim; ++i) acc[i] = 0.f;
    float row_max = -INFINITY, row_sum = 0.f;
    bool alive = true;
    const int last_allowed = p.causal ? min(query, p.k_tokens - 1) : p.k_tokens - 1;   // the last key this row may see

    auto add_partial = [&]() {
      uint32_t r0[32], r1[32];
      tmem_load_32(tmem_o, r0);
      tmem_load_32(tmem_o + 32, r1);
      tmem_load_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        acc[i] += __uint_as_float(r0[i]);
        acc[32 + i] += __uint_as_float(r1[i]);
      }
    };

    for (int j = 0; j < my_steps; ++j) {
      if (j > 0) {
        if (!barrier_wait(o_full(g), (j - 1) & 1, p.status, kWaitPartial)) { alive = false; break; }
        tcgen05_fence_after();
        add_partial();
      }
      if (!barrier_wait(s_full(g), j & 1, p.status, kWaitScores)) { alive = false; break; }
      tcgen05_fence_after();
      const int key0 = j * kKeys;
      const int limit = last_allowed - key0;                       // columns > limit are masked for this row
      const bool edge = key0 + kKeys - 1 > (p.causal ? min(q0 + g * kRows, p.k_tokens - 1) : p.k_tokens - 1);   // uniform in the group

      // pass 1: the row maximum of this step's scores
      float step_max = -INFINITY;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r0[32], r1[32];
        tmem_load_32(tmem_s + half * 64, r0);
        tmem_load_32(tmem_s + half * 64 + 32, r1);
        tmem_load_wait();
        if (edge) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (half * 64 + i > limit) r0[i] = 0xff800000u;
            if (half * 64 + 32 + i > limit) r1[i] = 0xff800000u;
          }
        }
        float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          m0 = fmaxf(m0, fmaxf(__uint_as_float(r0[i]), __uint_as_float(r0[i + 1])));
          m1 = fmaxf(m1, fmaxf(__uint_as_float(r1[i]), __uint_as_float(r1[i + 1])));
        }
        step_max = fmaxf(step_max, fmaxf(m0, m1));
      }
      const float new_max = fmaxf(row_max, step_max);
      const float alpha = exp2_ftz((row_max - new_max) * p.scale_log2);
      row_max = new_max;
      if (__any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
        for (int i = 0; i < kHeadDim; ++i) acc[i] *= alpha;
      }
      const float shift = -new_max * p.scale_log2;

      // pass 2: probabilities, their sum, and the K-major swizzled tile for the second product
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t r0[32], r1[32];
        tmem_load_32(tmem_s + half * 64, r0);
        tmem_load_32(tmem_s + half * 64 + 32, r1);
        tmem_load_wait();
        if (edge) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (half * 64 + i > limit) r0[i] = 0xff800000u;
            if (half * 64 + 32 + i > limit) r1[i] = 0xff800000u;
          }
        }
        const uint32_t half_base = smem_p_row + half * (kProbBytes / 2);
#pragma unroll
        for (int chunk = 0; chunk < 8; ++chunk) {     // 8 keys = 16 bytes
          uint32_t packed[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = chunk * 8 + e * 2;
            const uint32_t a = i < 32 ? r0[i] : r1[i - 32], b = i < 32 ? r0[i + 1] : r1[i - 31];
            const float pa = exp2_ftz(fmaf(__uint_as_float(a), p.scale_log2, shift));
            const float pb = exp2_ftz(fmaf(__uint_as_float(b), p.scale_log2, shift));
            sum0 += pa;
            sum1 += pb;
            packed[e] = pack_pair<T>(pa, pb);
          }
          store_shared_16(half_base + ((static_cast<uint32_t>(chunk) ^ swizzle) << 4), packed[0], packed[1], packed[2], packed[3]);
        }
      }
      row_sum = row_sum * alpha + (sum0 + sum1);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tile is read by the tensor core's proxy
      tcgen05_fence_before();
      barrier_arrive(p_full(g));
    }

    if (alive && my_steps > 0) {
      if (barrier_wait(o_full(g), (my_steps - 1) & 1, p.status, kWaitPartial)) {
        tcgen05_fence_after();
        add_partial();
        if (query < p.q_tokens) {
          const float inverse = 1.0f / row_sum;
          T* out_row = static_cast<T*>(p.out) + batch * p.out_batch + head * p.out_head + static_cast<long long>(query) * p.out_token;
          const bool vector_ok = (reinterpret_cast<uintptr_t>(out_row) & 15) == 0;
          if (vector_ok) {
#pragma unroll
            for (int v = 0; v < kHeadDim / 8; ++v) {
              uint4 word;
              word.x = pack_pair<T>(acc[v * 8 + 0] * inverse, acc[v * 8 + 1] * inverse);
              word.y = pack_pair<T>(acc[v * 8 + 2] * inverse, acc[v * 8 + 3] * inverse);
              word.z = pack_pair<T>(acc[v * 8 + 4] * inverse, acc[v * 8 + 5] * inverse);
              word.w = pack_pair<T>(acc[v * 8 + 6] * inverse, acc[v * 8 + 7] * inverse);
              *reinterpret_cast<uint4*>(out_row + v * 8) = word;
            }
          } else {
#pragma unroll
            for (int i = 0; i < kHeadDim; ++i) out_row[i] = from_compute<T, float>(acc[i] * inverse);
          }
        }
      }
    }
  }

  // ---- teardown: every thread arrives here, also after a wait that gave up -------------------
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 9) {
    tcgen05_fence_after();
    tmem_dealloc(tmem_base, kAttnTmemColumns);
  }
}

// A four-axis map over one of Q, K, V: 64 contiguous elements, then tokens, heads, batch with the
// caller's element strides; box = 64 x 128 x 1 x 1, 128-byte swizzle, rows beyond the tokens read 0.
tq_status attention_map(CUtensorMap* map, tq_dtype dtype, const void* pointer, long long tokens, long long heads, long long batch,
                        const int64_t* strides) {
  EncodeTiled encode = encode_tiled();
  TQ_REQUIRE(encode != nullptr, TQ_EXTERNAL, "the CUDA driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(kHeadDim), static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(batch)};
  // an axis of extent 1 never moves, so its stride only has to be legal
  const long long token_stride = tokens > 1 ? strides[2] : kHeadDim;
  const long long head_stride = heads > 1 ? strides[1] : kHeadDim;
  const long long batch_stride = batch > 1 ? strides[0] : kHeadDim;
  const cuuint64_t byte_strides[3] = {static_cast<cuuint64_t>(token_stride) * 2, static_cast<cuuint64_t>(head_stride) * 2,
                                      static_cast<cuuint64_t>(batch_stride) * 2};
  const cuuint32_t box[4] = {static_cast<cuuint32_t>(kHeadDim), static_cast<cuuint32_t>(kRows), 1, 1};
  const cuuint32_t element_strides[4] = {1, 1, 1, 1};
  const CUresult result = encode(map, dtype == TQ_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                                 const_cast<void*>(pointer), dims, byte_strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  TQ_REQUIRE(result == CUDA_SUCCESS, TQ_UNSUPPORTED, "this operand layout cannot be described to TMA (driver code %d)", static_cast<int>(result));
  return TQ_OK;
}

bool legal_strides(const void* pointer, const int64_t* strides, long long tokens, long long heads, long long batch) {
  if (!aligned_to(pointer, 16)) return false;
  if (tokens > 1 && (strides[2] < kHeadDim || strides[2] % 8 != 0)) return false;
  if (heads > 1 && (strides[1] <= 0 || strides[1] % 8 != 0)) return false;
  if (batch > 1 && (strides[0] <= 0 || strides[0] % 8 != 0)) return false;
  return true;
}

}  // namespace
}  // namespace tq

extern "C" tq_status tq_attention_launch(tq_dtype dtype, const void* q, const void* k, const void* v, void* out, int64_t batch,
                                         int64_t heads, int64_t q_tokens, int64_t k_tokens, int64_t head_dim,
                                         const int64_t* q_strides, const int64_t* k_strides, const int64_t* v_strides,
                                         const int64_t* out_strides, double scale, int32_t causal, int32_t device, void* stream) {
  TQ_REQUIRE(q_strides != nullptr && k_strides != nullptr && v_strides != nullptr && out_strides != nullptr, TQ_INVALID_ARGUMENT,
             "null strides");
  if (tq::recording()) {
    struct Kept { int64_t q[3], k[3], v[3], out[3]; } kept;
    for (int i = 0; i < 3; ++i) {
      kept.q[i] = q_strides[i];
      kept.k[i] = k_strides[i];
      kept.v[i] = v_strides[i];
      kept.out[i] = out_strides[i];
    }
    return tq::record([=](int32_t d, void* s) {
      return tq_attention_launch(dtype, q, k, v, out, batch, heads, q_tokens, k_tokens, head_dim, kept.q, kept.k, kept.v, kept.out,
                                 scale, causal, d, s);
    });
  }
  TQ_REQUIRE(dtype == TQ_BF16 || dtype == TQ_F16, TQ_UNSUPPORTED, "fused attention takes bf16 or f16 operands, not %s",
             tq::dtype_name(dtype));
  TQ_REQUIRE(batch >= 0 && heads >= 0 && q_tokens >= 0 && k_tokens >= 0, TQ_INVALID_ARGUMENT,
             "negative extent in batch=%lld heads=%lld q_tokens=%lld k_tokens=%lld", (long long)batch, (long long)heads,
             (long long)q_tokens, (long long)k_tokens);
  TQ_REQUIRE(head_dim == tq::kHeadDim, TQ_UNSUPPORTED, "fused attention has a kernel for heads of %d elements, not %lld", tq::kHeadDim,
             (long long)head_dim);
  if (batch == 0 || heads == 0 || q_tokens == 0) return TQ_OK;
  TQ_REQUIRE(k_tokens > 0, TQ_UNSUPPORTED, "a softmax over no keys has no kernel");
  TQ_REQUIRE(std::isfinite(scale) && scale > 0.0, TQ_UNSUPPORTED, "the score scale must be positive and finite, not %g", scale);
  TQ_REQUIRE(q != nullptr && k != nullptr && v != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null operand or result");
  TQ_REQUIRE(q_tokens < (1LL << 30) && k_tokens < (1LL << 30) && heads < 65536 && batch * heads < (1LL << 24), TQ_UNSUPPORTED,
             "extents beyond the kernel's index range");
  TQ_REQUIRE(tq::legal_strides(q, q_strides, q_tokens, heads, batch) && tq::legal_strides(k, k_strides, k_tokens, heads, batch) &&
                 tq::legal_strides(v, v_strides, k_tokens, heads, batch),
             TQ_UNSUPPORTED, "Q, K and V must be 16-byte aligned with positive strides that are multiples of 8 elements (TMA's rules)");
  TQ_REQUIRE(tq::aligned_to(out, 2) && out_strides[0] >= 0 && out_strides[1] >= 0 && out_strides[2] >= 0, TQ_INVALID_ARGUMENT,
             "misaligned result or negative result stride");
  if (tq_status s = tq::use_device(device)) return s;
  int* status = tq::device_status_word(device);
  TQ_REQUIRE(status != nullptr, TQ_RESOURCE_EXHAUSTED, "no device memory for the status word");

  CUtensorMap map_q, map_k, map_v;
  if (tq_status s = tq::attention_map(&map_q, dtype, q, q_tokens, heads, batch, q_strides)) return s;
  if (tq_status s = tq::attention_map(&map_k, dtype, k, k_tokens, heads, batch, k_strides)) return s;
  if (tq_status s = tq::attention_map(&map_v, dtype, v, k_tokens, heads, batch, v_strides)) return s;

  tq::AttnParams p = {};
  p.batch = static_cast<int>(batch);
  p.heads = static_cast<int>(heads);
  p.q_tokens = static_cast<int>(q_tokens);
  p.k_tokens = static_cast<int>(k_tokens);
  p.q_blocks = static_cast<int>((q_tokens + tq::kGroups * tq::kRows - 1) / (tq::kGroups * tq::kRows));
  p.causal = causal != 0;
  p.scale_log2 = static_cast<float>(scale * 1.4426950408889634);
  p.out = out;
  p.out_batch = out_strides[0];
  p.out_head = out_strides[1];
  p.out_token = out_strides[2];
  p.status = status;
  const long long ctas = static_cast<long long>(p.q_blocks) * heads * batch;
  TQ_REQUIRE(ctas < (1LL << 31), TQ_UNSUPPORTED, "too many query blocks for one launch");
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  auto go = [&](auto kernel) -> tq_status {
    static std::mutex mutex;
    {
      std::lock_guard<std::mutex> lock(mutex);
      TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(tq::kAttnSmemBytes)));
    }
    kernel<<<static_cast<unsigned>(ctas), tq::kAttnThreads, tq::kAttnSmemBytes, cuda_stream>>>(map_q, map_k, map_v, p);
    return tq::check_launch("attention_kernel");
  };
  if (dtype == TQ_BF16) return go(tq::attention_kernel<__nv_bfloat16>);
  return go(tq::attention_kernel<__half>);
}
