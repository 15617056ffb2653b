// Fused attention on the 5th-generation tensor cores (tcgen05), for sm_100a.
//
//   out[b,h,i,:] = sum_j softmax_j(scale * q[b,h,i,:] . k[b,h,j,:]) v[b,h,j,:]     (j <= i when causal)
//
// bf16 or f16 operands with 64-element heads, f32 scores and sums, one rounding of the result. The
// score matrix never leaves the SM: one CTA owns 256 query rows of one head (two tiles of 128) and
// walks the keys 128 at a time with a running row maximum and row sum (the online form of softmax).
//
//   warps 0..3 / 4..7   one softmax group per query tile, one thread per query row: tcgen05.ld of
//                       the row's 128 f32 scores (held in registers for both the maximum and the
//                       exponentials), ex2, row sum; the probabilities go back into tensor memory
//                       with tcgen05.st as packed bf16/f16 pairs — the A operand of the second
//                       product — and the partial result of the previous step is read from tensor
//                       memory and folded into the row's 64 accumulators with one FMA each.
//   warp 8, one lane    producer: TMA loads (128-byte swizzle) of the two query tiles once, then one
//                       128 x 64 key tile and one value tile per step into two 4-stage rings; the
//                       first loads leave before the CTA's set-up barrier.
//   warps 9 and 10,     issuers, one per group: S = Q K^T (128 x 128 x 64, both operands K-major in
//   one lane each       shared memory) and O = P V (128 x 64 x 128, P from tensor memory, V consumed
//                       MN-major exactly as it lies in memory). A tcgen05.mma costs its issuing
//                       thread about a hundred cycles and a step needs twelve, so one thread for
//                       both groups was the bottleneck; with one each, no group waits for the other.
//
// Each group has two 128-column buffers of tensor memory: the scores of step j sit in buffer j % 2;
// once the group holds them in registers it writes the probabilities over columns 64..127, and the
// second product writes the step's partial result over columns 0..63. So the scores of step j + 1
// are computed while the group is still working on step j. The softmax groups run with 224
// registers per thread, the other four warps with 56 (setmaxnreg). Q, K, V and
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
constexpr int kRing = 4;              // stages of the key ring and of the value ring
constexpr int kAttnThreads = 384;     // 8 softmax warps; producer and issuer in a third group of four warps
// setmaxnreg moves registers inside the CTA's own allocation (384 threads x 168 at launch): what the
// third group of four warps gives up is exactly what the eight softmax warps take. An increase
// beyond what was released would wait for ever.
constexpr int kLaunchRegisters = 168, kSoftmaxRegisters = 224, kOtherRegisters = 56;
static_assert(256 * (kSoftmaxRegisters - kLaunchRegisters) <= 128 * (kLaunchRegisters - kOtherRegisters),
              "the softmax warps would wait for registers nobody releases");
static_assert(kLaunchRegisters == (65536 / kAttnThreads) / 8 * 8, "ptxas gives a CTA of this size this many registers per thread");
constexpr uint32_t kTileBytes = kRows * kHeadDim * 2;       // 16 KiB: a Q, K or V tile
constexpr uint32_t kOffsetQ = 0;
constexpr uint32_t kOffsetK = kOffsetQ + kGroups * kTileBytes;
constexpr uint32_t kOffsetV = kOffsetK + kRing * kTileBytes;
constexpr uint32_t kOffsetBarriers = kOffsetV + kRing * kTileBytes;
constexpr size_t kAttnSmemBytes = 1024 + kOffsetBarriers + 256;
constexpr uint32_t kAttnTmemColumns = 512;   // two groups x two buffers x 128 columns
constexpr uint32_t kColumnP = 64;            // in a buffer whose scores are spent: O in columns 0..63, P (packed pairs) in 64..127

enum AttnWait { kWaitQ = 201, kWaitKeyEmpty = 202, kWaitValueEmpty = 203, kWaitKeyFull = 204, kWaitValueFull = 205,
                kWaitScores = 206, kWaitProbabilities = 207, kWaitPartial = 208, kWaitBufferFree = 209 };

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
  auto s_full = [&](int g, int b) { return barriers + 8u * (1 + 4 * kRing + 2 * g + b); };
  auto o_full = [&](int g, int b) { return barriers + 8u * (1 + 4 * kRing + 2 * kGroups + 2 * g + b); };
  auto p_full = [&](int g) { return barriers + 8u * (1 + 4 * kRing + 4 * kGroups + g); };
  auto buffer_free = [&](int g) { return barriers + 8u * (1 + 4 * kRing + 5 * kGroups + g); };
  constexpr int kBarrierCount = 1 + 4 * kRing + 6 * kGroups;
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

  // The producer lane sets the barriers up and sends the first loads (both query tiles, the first
  // key and value tiles) on their way before the CTA meets: their latency runs under the
  // tensor-memory allocation and the barrier.
  const bool producer = threadIdx.x == 8 * 32;
  if (producer) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_q) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_k) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_v) : "memory");
    barrier_init(q_full, 1);
    for (int s = 0; s < kRing; ++s) {
      barrier_init(k_full(s), 1);
      barrier_init(k_empty(s), kGroups);      // each group hands a tile back once its product has read it
      barrier_init(v_full(s), 1);
      barrier_init(v_empty(s), kGroups);
    }
    for (int g = 0; g < kGroups; ++g) {
      for (int b = 0; b < 2; ++b) {
        barrier_init(s_full(g, b), 1);
        barrier_init(o_full(g, b), 1);
      }
      barrier_init(p_full(g), kRows / 32);          // one arrival per warp of the group
      barrier_init(buffer_free(g), kRows / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (total_steps > 0) {
      int valid = 0;
      for (int g = 0; g < kGroups; ++g) valid += steps[g] > 0 ? 1 : 0;
      barrier_expect_tx(q_full, valid * kTileBytes);
      for (int g = 0; g < kGroups; ++g) {
        if (steps[g] > 0) tma_load_4d(base + kOffsetQ + g * kTileBytes, &map_q, q_full, 0, q0 + g * kRows, head, batch);
      }
      barrier_expect_tx(k_full(0), kTileBytes);
      tma_load_4d(base + kOffsetK, &map_k, k_full(0), 0, 0, head, batch);
      barrier_expect_tx(v_full(0), kTileBytes);
      tma_load_4d(base + kOffsetV, &map_v, v_full(0), 0, 0, head, batch);
    }
  }
  if (warp == 9) tmem_alloc(tmem_slot, kAttnTmemColumns);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_pointer;

  if (warp >= 8) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegisters));
  if (warp == 8) {
    // ---- producer: the tiles of step 1 onwards (step 0's went out before the CTA met) ------------
    if (lane == 0) {
      for (int j = 1; j < total_steps; ++j) {
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
  } else if (warp == 9 || warp == 10) {
    // ---- issuers: warp 9 for group 0, warp 10 for group 1 -------------------------------------
    // A tcgen05.mma costs its issuing thread on the order of a hundred cycles here, and a step is
    // 12 of them plus two commits: one thread for both groups was the kernel's bottleneck. Each
    // group's issuer follows its own group only, so neither group waits for the other.
    const int g = warp - 9;
    if (lane == 0 && steps[g] > 0) {
      constexpr uint32_t idesc_s = attn_instruction_descriptor<T>(kKeys, false);
      constexpr uint32_t idesc_o = attn_instruction_descriptor<T>(kHeadDim, true);
      // Descriptors as (low, high) words: one constant high word, low words stepped by adds.
      constexpr uint32_t kHighWord = kDescriptorHigh;
      const uint32_t low_q = descriptor_low(base + kOffsetQ + g * kTileBytes, 0), low_k = descriptor_low(base + kOffsetK, 0);
      const uint32_t low_v = descriptor_low(base + kOffsetV, kTileBytes);
      const uint32_t buffers = tmem_base + static_cast<uint32_t>(2 * g * kKeys);     // buffer b at + 128 b
      // S(i) = Q K_i^T into buffer i % 2: both operands K-major, 16 elements of K = 32 B in the swizzle row
      auto scores = [&](int i) {
        const uint32_t k = low_k + (i % kRing) * (kTileBytes >> 4), d = buffers + (i & 1) * kKeys;
#pragma unroll
        for (int kk = 0; kk < kHeadDim / 16; ++kk) mma_f16_split(d, low_q + kk * 2, kHighWord, k + kk * 2, kHighWord, idesc_s, kk != 0 ? 1u : 0u);
        mma_commit(s_full(g, i & 1));
      };
      // O(i) = P_i V_i over columns 0..63 of buffer i % 2: P from tensor memory (columns 64..127, 16
      // keys = 8 columns), V MN-major from shared memory (16 keys = 2048 B)
      auto partial = [&](int i) {
        const uint32_t v = low_v + (i % kRing) * (kTileBytes >> 4), d = buffers + (i & 1) * kKeys;
#pragma unroll
        for (int kk = 0; kk < kKeys / 16; ++kk) mma_f16_tmem_a(d, d + kColumnP + kk * 8, v + kk * (2048 >> 4), kHighWord, idesc_o, kk != 0 ? 1u : 0u);
        mma_commit(o_full(g, i & 1));
      };
      bool alive = barrier_wait(q_full, 0, p.status, kWaitQ) && barrier_wait(k_full(0), 0, p.status, kWaitKeyFull);
      if (alive) {
        tcgen05_fence_after();
        scores(0);
      }
      for (int i = 0; alive && i < steps[g]; ++i) {
        // the scores of step i + 1, once the group has taken O(i-1) out of that buffer (its i-th arrival)
        if (i + 1 < steps[g]) {
          if (!barrier_wait(k_full((i + 1) % kRing), ((i + 1) / kRing) & 1, p.status, kWaitKeyFull)) break;
          if (!barrier_wait(buffer_free(g), i & 1, p.status, kWaitBufferFree)) break;
          tcgen05_fence_after();
          scores(i + 1);
        }
        // the partial result of step i, once the group's probabilities are in tensor memory
        if (!barrier_wait(v_full(i % kRing), (i / kRing) & 1, p.status, kWaitValueFull)) break;
        if (!barrier_wait(p_full(g), i & 1, p.status, kWaitProbabilities)) break;
        tcgen05_fence_after();
        partial(i);
      }
    }
  } else if (warp < 8) {
    // ---- softmax groups: warp w of a group owns tensor-memory lanes 32 (w % 4) .. +31 ---------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegisters));
    const int g = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int query = q0 + g * kRows + row;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const uint32_t tmem_group = tmem_base + static_cast<uint32_t>(2 * g * kKeys) + lane_base;   // buffer b at + 128 b
    const int my_steps = steps[g];
    float acc[kHeadDim];
#pragma unroll
    for (int i = 0; i < kHeadDim; ++i) acc[i] = 0.f;
    float row_max = -INFINITY, row_sum = 0.f;
    bool alive = true;
    const int last_allowed = p.causal ? min(query, p.k_tokens - 1) : p.k_tokens - 1;   // the last key this row may see

    // acc <- acc * scale + (the partial result in buffer b): one FMA per element
    auto add_partial = [&](int b, float scale) {
      uint32_t r0[32], r1[32];
      tmem_load_32(tmem_group + b * kKeys, r0);
      tmem_load_32(tmem_group + b * kKeys + 32, r1);
      tmem_load_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        acc[i] = fmaf(acc[i], scale, __uint_as_float(r0[i]));
        acc[32 + i] = fmaf(acc[32 + i], scale, __uint_as_float(r1[i]));
      }
    };
    // one row of scores: 128 columns, one wait
    auto load_row = [&](uint32_t address, uint32_t (&r)[kKeys], bool edge, int limit) {
#pragma unroll
      for (int c = 0; c < kKeys / 32; ++c) tmem_load_32(address + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
      tmem_load_wait();
      if (edge) {
#pragma unroll
        for (int i = 0; i < kKeys; ++i) {
          if (i > limit) r[i] = 0xff800000u;   // -inf
        }
      }
    };

    // With m_j the running maximum after step j and alpha_j = exp2((m_{j-1} - m_j) scale), the result
    // obeys A_j = A_{j-1} alpha_j + O_j. O_j leaves the tensor core one step late, so the group
    // keeps alpha_j and applies it when it takes O_j out of tensor memory (step j + 1, or the end).
    float alpha_previous = 0.f;
    for (int j = 0; j < my_steps; ++j) {
      const uint32_t tmem_s = tmem_group + (j & 1) * kKeys;
      if (!barrier_wait(s_full(g, j & 1), (j >> 1) & 1, p.status, kWaitScores)) { alive = false; break; }
      tcgen05_fence_after();
      if (threadIdx.x == g * kRows) {      // the first product has read key tile j: hand it back (for the other group too, if it has no step j)
        barrier_arrive(k_empty(j % kRing));
        if (j >= steps[1 - g]) barrier_arrive(k_empty(j % kRing));
      }
      // the partial result of step j - 1 (A_{j-1} = A_{j-2} alpha_{j-1} + O_{j-1}); after it that
      // buffer is free for step j + 1's scores
      if (j > 0) {
        if (!barrier_wait(o_full(g, (j - 1) & 1), ((j - 1) >> 1) & 1, p.status, kWaitPartial)) { alive = false; break; }
        tcgen05_fence_after();
        if (threadIdx.x == g * kRows) {    // the second product has read value tile j - 1
          barrier_arrive(v_empty((j - 1) % kRing));
          if (j - 1 >= steps[1 - g]) barrier_arrive(v_empty((j - 1) % kRing));
        }
        add_partial((j - 1) & 1, alpha_previous);
      }
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) barrier_arrive(buffer_free(g));

      // this step's scores: one row per thread, held in registers for both the maximum and the exponentials
      const int key0 = j * kKeys;
      const int limit = last_allowed - key0;                       // columns > limit are masked for this row
      const bool edge = key0 + kKeys - 1 > (p.causal ? min(q0 + g * kRows, p.k_tokens - 1) : p.k_tokens - 1);   // uniform in the group
      uint32_t r[kKeys];
      load_row(tmem_s, r, edge, limit);
      float m0 = row_max, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kKeys; i += 8) {
        m0 = fmaxf(fmaxf(m0, __uint_as_float(r[i])), __uint_as_float(r[i + 1]));
        m1 = fmaxf(fmaxf(m1, __uint_as_float(r[i + 2])), __uint_as_float(r[i + 3]));
        m2 = fmaxf(fmaxf(m2, __uint_as_float(r[i + 4])), __uint_as_float(r[i + 5]));
        m3 = fmaxf(fmaxf(m3, __uint_as_float(r[i + 6])), __uint_as_float(r[i + 7]));
      }
      const float new_max = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      const float alpha = exp2_ftz((row_max - new_max) * p.scale_log2);
      row_max = new_max;
      alpha_previous = alpha;
      const float shift = -new_max * p.scale_log2;

      // probabilities and their sum; the probabilities go back into tensor memory as the A operand of
      // the second product (16-bit pairs over columns 64..127 of this step's buffer)
      float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
      {
        uint32_t packed[kKeys / 2];
#pragma unroll
        for (int chunk = 0; chunk < kKeys / 8; ++chunk) {
          const float p0 = exp2_ftz(fmaf(__uint_as_float(r[chunk * 8 + 0]), p.scale_log2, shift));
          const float p1 = exp2_ftz(fmaf(__uint_as_float(r[chunk * 8 + 1]), p.scale_log2, shift));
          const float p2 = exp2_ftz(fmaf(__uint_as_float(r[chunk * 8 + 2]), p.scale_log2, shift));
          const float p3 = exp2_ftz(fmaf(__uint_as_float(r[chunk * 8 + 3]), p.scale_log2, shift));
          const float p4 = exp2_ftz(fmaf(__uint_as_float(r[chunk * 8 + 4]), p.scale_log2, shift));
          const float p5 = exp2_ftz(fmaf(__uint_as_float(r[chunk * 8 + 5]), p.scale_log2, shift));
          const float p6 = exp2_ftz(fmaf(__uint_as_float(r[chunk * 8 + 6]), p.scale_log2, shift));
          const float p7 = exp2_ftz(fmaf(__uint_as_float(r[chunk * 8 + 7]), p.scale_log2, shift));
          sum0 += p0 + p4;
          sum1 += p1 + p5;
          sum2 += p2 + p6;
          sum3 += p3 + p7;
          packed[chunk * 4 + 0] = pack_pair<T>(p0, p1);
          packed[chunk * 4 + 1] = pack_pair<T>(p2, p3);
          packed[chunk * 4 + 2] = pack_pair<T>(p4, p5);
          packed[chunk * 4 + 3] = pack_pair<T>(p6, p7);
        }
        tmem_store_32(tmem_s + kColumnP, *reinterpret_cast<const uint32_t(*)[32]>(&packed[0]));
        tmem_store_32(tmem_s + kColumnP + 32, *reinterpret_cast<const uint32_t(*)[32]>(&packed[32]));
        tmem_store_wait();
      }
      row_sum = row_sum * alpha + ((sum0 + sum1) + (sum2 + sum3));
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) barrier_arrive(p_full(g));
    }

    if (alive && my_steps > 0) {
      if (barrier_wait(o_full(g, (my_steps - 1) & 1), ((my_steps - 1) >> 1) & 1, p.status, kWaitPartial)) {
        tcgen05_fence_after();
        add_partial((my_steps - 1) & 1, alpha_previous);
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
