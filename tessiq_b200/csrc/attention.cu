// Fused attention on the 5th-generation tensor cores (tcgen05), for sm_100a.
//
//   out[b,h,i,:] = sum_j softmax_j(scale * q[b,h,i,:] . k[b,h,j,:]) v[b,h,j,:]     (j <= i when causal)
//
// bf16 or f16 operands with 64-element heads, f32 scores and sums, one rounding of the result. The
// score matrix never leaves the SM: one CTA owns 256 query rows of one head (two tiles of 128) and
// walks the keys 128 at a time with a row reference point and row sum (the online form of softmax).
//
//   warps 0..3 / 4..7   one softmax group per query tile, one thread per query row: tcgen05.ld of
//                       the row's 128 f32 scores (held in registers for both the maximum and the
//                       exponentials), ex2, row sum; the probabilities go back into tensor memory
//                       with tcgen05.st as packed bf16/f16 pairs — the A operand of the second
//                       product. The result accumulates in tensor memory across the steps and is
//                       read once, at the end.
//   warp 8, one lane    producer: TMA loads (128-byte swizzle) of the two query tiles once, then one
//                       128 x 64 key tile and one value tile per step into two 4-stage rings; the
//                       first loads leave before the CTA's set-up barrier.
//   warps 9 and 10,     issuers, one per group: S = Q K^T (128 x 128 x 64, both operands K-major in
//   one lane each       shared memory) and O = P V (128 x 64 x 128, P from tensor memory, V consumed
//                       MN-major exactly as it lies in memory). A tcgen05.mma costs its issuing
//                       thread about a hundred cycles and a step needs twelve, so one thread for
//                       both groups was the bottleneck; with one each, no group waits for the other.
//
// softmax is exp(s - m) / sum exp(s - m) for ANY m, so a row keeps the maximum of its first key tile
// as its reference point and moves it only when a later tile rises more than 2^8 above it — then,
// and only then, the row's sum and its 64 accumulators in tensor memory are rescaled (a warp-wide
// slow path, rare on real data). Without that, nothing is read back per step: the second product
// accumulates O += P V in place. Probabilities are at most 2^8, well inside bf16 and f16.
//
// Each group has 256 columns of tensor memory: the scores (0..127), the probabilities as packed
// pairs (128..191) and the result (192..255). A group takes its scores into registers at the start
// of a step and hands the columns back at once, so the scores of step j + 1 are computed while the
// group is still working on step j. The softmax groups run with 224
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
constexpr uint32_t kSubTileBytes = kRows * kHeadDim * 2;     // 16 KiB: 128 rows of 64 elements, one TMA box, one swizzled operand tile
// Shared memory for heads of D elements (D = 64, or 128 = two sub-tiles side by side per tile): the
// query tiles (two groups of 64-wide heads, or the one group of 128-wide heads: 32 KiB either way),
// the key ring, the value ring, the barriers. Heads of 128 get three stages per ring: four would not fit.
template <int D>
struct AttnLayout {
  static constexpr int kSubTiles = D / kHeadDim;
  static constexpr uint32_t kTileBytes = kSubTiles * kSubTileBytes;
  static constexpr int kActiveGroups = D == kHeadDim ? kGroups : 1;
  static constexpr int kRingStages = D == kHeadDim ? kRing : 3;
  static constexpr uint32_t kOffsetQ = 0;
  static constexpr uint32_t kOffsetK = kOffsetQ + kActiveGroups * kTileBytes;
  static constexpr uint32_t kOffsetV = kOffsetK + kRingStages * kTileBytes;
  static constexpr uint32_t kOffsetBarriers = kOffsetV + kRingStages * kTileBytes;
  static constexpr size_t kSmemBytes = 1024 + kOffsetBarriers + 256;
};
static_assert(AttnLayout<128>::kSmemBytes <= 227 * 1024, "the wide-head staging has to fit one CTA's shared memory");
constexpr uint32_t kAttnTmemColumns = 512;   // two groups x 256 columns
constexpr uint32_t kGroupColumns = 256;      // of a group: scores 0..127, probabilities (packed pairs) 128..191, result 192..255 (192..319 for the one group of 128-wide heads)
constexpr uint32_t kColumnP = 128, kColumnO = 192;
constexpr float kSlack = 8.f;                // a row's reference point moves when a tile's maximum is more than 2^kSlack above it

enum AttnWait { kWaitQ = 201, kWaitKeyEmpty = 202, kWaitValueEmpty = 203, kWaitKeyFull = 204, kWaitValueFull = 205,
                kWaitScores = 206, kWaitProbabilities = 207, kWaitPartial = 208, kWaitBufferFree = 209 };

struct AttnParams {
  int batch, heads, q_tokens, k_tokens;
  int head_dim;                    // 8, 16, ... 64: narrower heads ride in 64-wide tiles whose other columns TMA fills with zeros
  int q_blocks;                    // CTAs per head
  int causal;
  float scale_log2;                // scale * log2(e)
  void* out;
  long long out_batch, out_head, out_token;   // element strides
  WaitStatus status;
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

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
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

template <typename T, int D>
__global__ void __launch_bounds__(kAttnThreads, 1)
attention_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                 const __grid_constant__ CUtensorMap map_v, const AttnParams p) {
  using L = AttnLayout<D>;
  constexpr int kRing = L::kRingStages;                 // (hides the namespace's value: heads of 128 have three stages)
  constexpr uint32_t kTileBytes = L::kTileBytes, kOffsetQ = L::kOffsetQ, kOffsetK = L::kOffsetK, kOffsetV = L::kOffsetV;
  constexpr uint32_t kOffsetBarriers = L::kOffsetBarriers;
  constexpr int kSubTiles = L::kSubTiles;
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
  auto s_full = [&](int g) { return barriers + 8u * (1 + 4 * kRing + g); };                   // the scores of a step are in tensor memory
  auto s_free = [&](int g) { return barriers + 8u * (1 + 4 * kRing + kGroups + g); };          // ... and in the group's registers
  auto p_full = [&](int g) { return barriers + 8u * (1 + 4 * kRing + 2 * kGroups + g); };      // the probabilities of a step are in tensor memory
  auto pv_done = [&](int g) { return barriers + 8u * (1 + 4 * kRing + 3 * kGroups + g); };     // ... and the second product has consumed them
  constexpr int kBarrierCount = 1 + 4 * kRing + 4 * kGroups;
  const uint32_t tmem_slot = barriers + 8u * kBarrierCount;
  volatile uint32_t* tmem_slot_pointer = reinterpret_cast<volatile uint32_t*>(aligned + kOffsetBarriers + 8 * kBarrierCount);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // Which rows of which head: heads in launch order, the long (late) query blocks of a head first.
  const int q_block = p.q_blocks - 1 - static_cast<int>(blockIdx.x % p.q_blocks);
  const int head_index = static_cast<int>(blockIdx.x / p.q_blocks);
  const int head = head_index % p.heads, batch = head_index / p.heads;
  const int q0 = q_block * L::kActiveGroups * kRows;
  const int key_tiles = (p.k_tokens + kKeys - 1) / kKeys;
  // steps of group g: none when its rows lie beyond the queries; under a causal mask only the key
  // tiles that hold a key <= its last row
  int steps[kGroups];
#pragma unroll
  for (int g = 0; g < kGroups; ++g) {
    const int first = q0 + g * kRows;
    steps[g] = (g >= L::kActiveGroups || first >= p.q_tokens)
                   ? 0 : (p.causal ? min(key_tiles, (min(first + kRows, p.q_tokens) - 1) / kKeys + 1) : key_tiles);
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
    if (blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) p.status.begin();   // this launch's abort word starts clear
    barrier_init(q_full, 1);
    for (int s = 0; s < kRing; ++s) {
      barrier_init(k_full(s), 1);
      barrier_init(k_empty(s), kGroups);      // each group hands a tile back once its product has read it
      barrier_init(v_full(s), 1);
      barrier_init(v_empty(s), kGroups);
    }
    for (int g = 0; g < kGroups; ++g) {
      barrier_init(s_full(g), 1);
      barrier_init(pv_done(g), 1);
      barrier_init(p_full(g), kRows / 32);          // one arrival per warp of the group
      barrier_init(s_free(g), kRows / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (total_steps > 0) {
      int valid = 0;
      for (int g = 0; g < kGroups; ++g) valid += steps[g] > 0 ? 1 : 0;
      barrier_expect_tx(q_full, valid * kTileBytes);
      for (int g = 0; g < kGroups; ++g) {
        if (steps[g] > 0) {
          for (int h = 0; h < kSubTiles; ++h)
            tma_load_4d(base + kOffsetQ + g * kTileBytes + h * kSubTileBytes, &map_q, q_full, h * kHeadDim, q0 + g * kRows, head, batch);
        }
      }
      barrier_expect_tx(k_full(0), kTileBytes);
      for (int h = 0; h < kSubTiles; ++h) tma_load_4d(base + kOffsetK + h * kSubTileBytes, &map_k, k_full(0), h * kHeadDim, 0, head, batch);
      barrier_expect_tx(v_full(0), kTileBytes);
      for (int h = 0; h < kSubTiles; ++h) tma_load_4d(base + kOffsetV + h * kSubTileBytes, &map_v, v_full(0), h * kHeadDim, 0, head, batch);
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
        for (int h = 0; h < kSubTiles; ++h)
          tma_load_4d(base + kOffsetK + s * kTileBytes + h * kSubTileBytes, &map_k, k_full(s), h * kHeadDim, j * kKeys, head, batch);
        if (!barrier_wait(v_empty(s), phase ^ 1, p.status, kWaitValueEmpty)) break;
        barrier_expect_tx(v_full(s), kTileBytes);
        for (int h = 0; h < kSubTiles; ++h)
          tma_load_4d(base + kOffsetV + s * kTileBytes + h * kSubTileBytes, &map_v, v_full(s), h * kHeadDim, j * kKeys, head, batch);
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
      const uint32_t low_v = descriptor_low(base + kOffsetV, kSubTileBytes);
      const uint32_t columns = tmem_base + static_cast<uint32_t>(g) * kGroupColumns;
      // S(i) = Q K_i^T: both operands K-major, 16 elements of K = 32 B in the swizzle row
      auto scores = [&](int i) {
        const uint32_t k = low_k + (i % kRing) * (kTileBytes >> 4);
        // (a 128-wide head is two 64-wide sub-tiles side by side: the same steps in the second one)
#pragma unroll
        for (int h = 0; h < kSubTiles; ++h) {
#pragma unroll
          for (int kk = 0; kk < kHeadDim / 16; ++kk)
            mma_f16_split(columns, low_q + h * (kSubTileBytes >> 4) + kk * 2, kHighWord, k + h * (kSubTileBytes >> 4) + kk * 2, kHighWord, idesc_s,
                          (h != 0 || kk != 0) ? 1u : 0u);
        }
        mma_commit(s_full(g));
      };
      // O += P_i V_i (O = for the first step): P from tensor memory (16 keys = 8 columns), V MN-major
      // from shared memory (16 keys = 2048 B)
      auto partial = [&](int i) {
        const uint32_t v = low_v + (i % kRing) * (kTileBytes >> 4);
        // (a 128-wide head: the second sub-tile of V gives result columns 64..127)
#pragma unroll
        for (int h = 0; h < kSubTiles; ++h) {
#pragma unroll
          for (int kk = 0; kk < kKeys / 16; ++kk)
            mma_f16_tmem_a(columns + kColumnO + h * kHeadDim, columns + kColumnP + kk * 8, v + h * (kSubTileBytes >> 4) + kk * (2048 >> 4), kHighWord,
                           idesc_o, (i != 0 || kk != 0) ? 1u : 0u);
        }
        mma_commit(pv_done(g));
      };
      bool alive = barrier_wait(q_full, 0, p.status, kWaitQ) && barrier_wait(k_full(0), 0, p.status, kWaitKeyFull);
      if (alive) {
        tcgen05_fence_after();
        scores(0);
      }
      for (int i = 0; alive && i < steps[g]; ++i) {
        // the scores of step i + 1, once the group holds those of step i in registers
        if (i + 1 < steps[g]) {
          if (!barrier_wait(k_full((i + 1) % kRing), ((i + 1) / kRing) & 1, p.status, kWaitKeyFull)) break;
          if (!barrier_wait(s_free(g), i & 1, p.status, kWaitBufferFree)) break;
          tcgen05_fence_after();
          scores(i + 1);
        }
        // the second product of step i, once the group's probabilities are in tensor memory
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
    const uint32_t tmem_group = tmem_base + static_cast<uint32_t>(g) * kGroupColumns + lane_base;
    const int my_steps = steps[g];
    float reference = -INFINITY, row_sum = 0.f;     // -inf: the row has seen no finite score yet
    bool alive = true;
    const int last_allowed = p.causal ? min(query, p.k_tokens - 1) : p.k_tokens - 1;   // the last key this row may see

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
    // the second product of step j has finished: its probabilities and its value tile are spent
    auto wait_product = [&](int j) {
      if (!barrier_wait(pv_done(g), j & 1, p.status, kWaitPartial)) return false;
      tcgen05_fence_after();
      if (threadIdx.x == g * kRows) {
        barrier_arrive(v_empty(j % kRing));
        if (j >= steps[1 - g]) barrier_arrive(v_empty(j % kRing));     // for the other group too, if it has no step j
      }
      return true;
    };

    for (int j = 0; j < my_steps; ++j) {
      if (!barrier_wait(s_full(g), j & 1, p.status, kWaitScores)) { alive = false; break; }
      tcgen05_fence_after();
      if (threadIdx.x == g * kRows) {      // the first product has read key tile j: hand it back (for the other group too, if it has no step j)
        barrier_arrive(k_empty(j % kRing));
        if (j >= steps[1 - g]) barrier_arrive(k_empty(j % kRing));
      }
      // this step's scores: one row per thread, held in registers for both the maximum and the
      // exponentials; the columns go back to the issuer at once
      const int key0 = j * kKeys;
      const int limit = last_allowed - key0;                       // columns > limit are masked for this row
      const bool edge = key0 + kKeys - 1 > (p.causal ? min(q0 + g * kRows, p.k_tokens - 1) : p.k_tokens - 1);   // uniform in the group
      uint32_t r[kKeys];
      load_row(tmem_group, r, edge, limit);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) barrier_arrive(s_free(g));

      // (three-input maximum, and below two-element FMA and add: the step is bound by the number of
      // instructions its eight softmax warps issue, so every element costs half an instruction for
      // the maximum, half for the scaling, one ex2, half for the sum and half for the rounding)
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < kKeys; i += 8) {
        m0 = max3(m0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
        m1 = max3(m1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
        m2 = max3(m2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
        m3 = max3(m3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
      }
      const float tile_max = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
      // The reference point: the first tile's maximum, moved only when a tile rises more than
      // 2^kSlack above it (from -inf, any finite maximum does). `factor` rescales what the row has
      // gathered so far; it is 1 for a row that stays.
      float factor = 1.f;
      const bool moves = j == 0 || (tile_max - reference) * p.scale_log2 > kSlack;       // false for NaN
      if (moves) {
        if (j != 0) factor = exp2_ftz((reference - tile_max) * p.scale_log2);             // from -inf: 0, and nothing was gathered
        reference = tile_max;
      }
      const bool rescale = j != 0 && __any_sync(0xffffffffu, moves);
      const float shift = reference == -INFINITY ? 0.f : -reference * p.scale_log2;       // all scores -inf so far: every probability is 0

      // probabilities and their sum; the probabilities go back into tensor memory as the A operand of
      // the second product (16-bit pairs)
      float2 sum0 = make_float2(0.f, 0.f), sum1 = sum0, sum2 = sum0, sum3 = sum0;
      uint32_t packed[kKeys / 2];
      const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(shift, shift);
#pragma unroll
      for (int chunk = 0; chunk < kKeys / 8; ++chunk) {
        const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(r[chunk * 8 + 0]), __uint_as_float(r[chunk * 8 + 1])), scale2, shift2);
        const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(r[chunk * 8 + 2]), __uint_as_float(r[chunk * 8 + 3])), scale2, shift2);
        const float2 t2 = __ffma2_rn(make_float2(__uint_as_float(r[chunk * 8 + 4]), __uint_as_float(r[chunk * 8 + 5])), scale2, shift2);
        const float2 t3 = __ffma2_rn(make_float2(__uint_as_float(r[chunk * 8 + 6]), __uint_as_float(r[chunk * 8 + 7])), scale2, shift2);
        const float2 e0 = make_float2(exp2_ftz(t0.x), exp2_ftz(t0.y));
        const float2 e1 = make_float2(exp2_ftz(t1.x), exp2_ftz(t1.y));
        const float2 e2 = make_float2(exp2_ftz(t2.x), exp2_ftz(t2.y));
        const float2 e3 = make_float2(exp2_ftz(t3.x), exp2_ftz(t3.y));
        sum0 = __fadd2_rn(sum0, e0);
        sum1 = __fadd2_rn(sum1, e1);
        sum2 = __fadd2_rn(sum2, e2);
        sum3 = __fadd2_rn(sum3, e3);
        packed[chunk * 4 + 0] = pack_pair<T>(e0.x, e0.y);
        packed[chunk * 4 + 1] = pack_pair<T>(e1.x, e1.y);
        packed[chunk * 4 + 2] = pack_pair<T>(e2.x, e2.y);
        packed[chunk * 4 + 3] = pack_pair<T>(e3.x, e3.y);
      }
      const float2 sum01 = __fadd2_rn(sum0, sum1), sum23 = __fadd2_rn(sum2, sum3);
      const float tile_sum = (sum01.x + sum01.y) + (sum23.x + sum23.y);
      row_sum = row_sum * factor + tile_sum;

      // The previous step's product still reads the probability columns and adds into the result:
      // wait for it (it had this step's loads and exponentials to finish), then write.
      if (j > 0) {
        if (!wait_product(j - 1)) { alive = false; break; }
        if (rescale) {       // rare: some row of this warp moved its reference point
          if constexpr (D == kHeadDim) {
            uint32_t o0[32], o1[32];
            tmem_load_32(tmem_group + kColumnO, o0);
            tmem_load_32(tmem_group + kColumnO + 32, o1);
            tmem_load_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              o0[i] = __float_as_uint(__uint_as_float(o0[i]) * factor);
              o1[i] = __float_as_uint(__uint_as_float(o1[i]) * factor);
            }
            tmem_store_32(tmem_group + kColumnO, o0);
            tmem_store_32(tmem_group + kColumnO + 32, o1);
          } else {             // 128 result columns, 32 at a time: the probabilities are still in registers
#pragma unroll 1
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_load_32(tmem_group + kColumnO + c * 32, o);
              tmem_load_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
              tmem_store_32(tmem_group + kColumnO + c * 32, o);
            }
          }
        }
      }
      tmem_store_32(tmem_group + kColumnP, *reinterpret_cast<const uint32_t(*)[32]>(&packed[0]));
      tmem_store_32(tmem_group + kColumnP + 32, *reinterpret_cast<const uint32_t(*)[32]>(&packed[32]));
      tmem_store_wait();
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) barrier_arrive(p_full(g));
    }

    if constexpr (D != kHeadDim) {
      // the one group of wide heads: the result row leaves tensor memory 32 columns at a time
      if (alive && my_steps > 0 && wait_product(my_steps - 1)) {
        // (the tensor-memory loads are warp-wide: every lane takes part, rows beyond the queries only skip the stores)
        const bool stores = query < p.q_tokens;
        const float inverse = 1.0f / row_sum;
        T* out_row = static_cast<T*>(p.out) + batch * p.out_batch + head * p.out_head + static_cast<long long>(query) * p.out_token;
        const bool vector_ok = (reinterpret_cast<uintptr_t>(out_row) & 15) == 0;
        const int width = p.head_dim;
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          if (c * 32 >= width) break;
          uint32_t o[32];
          tmem_load_32(tmem_group + kColumnO + c * 32, o);
          tmem_load_wait();
          if (!stores) continue;
          if (vector_ok) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              if (c * 32 + v * 8 < width) {
                uint4 word;
                word.x = pack_pair<T>(__uint_as_float(o[v * 8 + 0]) * inverse, __uint_as_float(o[v * 8 + 1]) * inverse);
                word.y = pack_pair<T>(__uint_as_float(o[v * 8 + 2]) * inverse, __uint_as_float(o[v * 8 + 3]) * inverse);
                word.z = pack_pair<T>(__uint_as_float(o[v * 8 + 4]) * inverse, __uint_as_float(o[v * 8 + 5]) * inverse);
                word.w = pack_pair<T>(__uint_as_float(o[v * 8 + 6]) * inverse, __uint_as_float(o[v * 8 + 7]) * inverse);
                *reinterpret_cast<uint4*>(out_row + c * 32 + v * 8) = word;
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              if (c * 32 + i < width) out_row[c * 32 + i] = from_compute<T, float>(__uint_as_float(o[i]) * inverse);
            }
          }
        }
      }
    } else
    if (alive && my_steps > 0 && wait_product(my_steps - 1)) {
      uint32_t o0[32], o1[32];
      tmem_load_32(tmem_group + kColumnO, o0);
      tmem_load_32(tmem_group + kColumnO + 32, o1);
      tmem_load_wait();
      if (query < p.q_tokens) {
        const float inverse = 1.0f / row_sum;
        T* out_row = static_cast<T*>(p.out) + batch * p.out_batch + head * p.out_head + static_cast<long long>(query) * p.out_token;
        const bool vector_ok = (reinterpret_cast<uintptr_t>(out_row) & 15) == 0;
        const int width = p.head_dim;       // a multiple of 8: whole 16-byte vectors
        if (vector_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint4 word;
            if (v * 8 < width) {
              word.x = pack_pair<T>(__uint_as_float(o0[v * 8 + 0]) * inverse, __uint_as_float(o0[v * 8 + 1]) * inverse);
              word.y = pack_pair<T>(__uint_as_float(o0[v * 8 + 2]) * inverse, __uint_as_float(o0[v * 8 + 3]) * inverse);
              word.z = pack_pair<T>(__uint_as_float(o0[v * 8 + 4]) * inverse, __uint_as_float(o0[v * 8 + 5]) * inverse);
              word.w = pack_pair<T>(__uint_as_float(o0[v * 8 + 6]) * inverse, __uint_as_float(o0[v * 8 + 7]) * inverse);
              *reinterpret_cast<uint4*>(out_row + v * 8) = word;
            }
            if (32 + v * 8 < width) {
              word.x = pack_pair<T>(__uint_as_float(o1[v * 8 + 0]) * inverse, __uint_as_float(o1[v * 8 + 1]) * inverse);
              word.y = pack_pair<T>(__uint_as_float(o1[v * 8 + 2]) * inverse, __uint_as_float(o1[v * 8 + 3]) * inverse);
              word.z = pack_pair<T>(__uint_as_float(o1[v * 8 + 4]) * inverse, __uint_as_float(o1[v * 8 + 5]) * inverse);
              word.w = pack_pair<T>(__uint_as_float(o1[v * 8 + 6]) * inverse, __uint_as_float(o1[v * 8 + 7]) * inverse);
              *reinterpret_cast<uint4*>(out_row + 32 + v * 8) = word;
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (i < width) out_row[i] = from_compute<T, float>(__uint_as_float(o0[i]) * inverse);
            if (32 + i < width) out_row[32 + i] = from_compute<T, float>(__uint_as_float(o1[i]) * inverse);
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

// A four-axis map over one of Q, K, V: `head_dim` contiguous elements, then tokens, heads, batch with
// the caller's element strides; box = 64 x 128 x 1 x 1, 128-byte swizzle. Rows beyond the tokens read
// 0, and so do the columns beyond a head narrower than 64: zeros add nothing to q . k and give
// result columns nobody stores, so a narrow head runs through the same 64-wide tiles.
tq_status attention_map(CUtensorMap* map, tq_dtype dtype, const void* pointer, long long head_dim, long long tokens, long long heads,
                        long long batch, const int64_t* strides) {
  EncodeTiled encode = encode_tiled();
  TQ_REQUIRE(encode != nullptr, TQ_EXTERNAL, "the CUDA driver does not provide cuTensorMapEncodeTiled");
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(head_dim), static_cast<cuuint64_t>(tokens), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(batch)};
  // an axis of extent 1 never moves, so its stride only has to be legal
  const long long token_stride = tokens > 1 ? strides[2] : head_dim;
  const long long head_stride = heads > 1 ? strides[1] : head_dim;
  const long long batch_stride = batch > 1 ? strides[0] : head_dim;
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

bool legal_strides(const void* pointer, const int64_t* strides, long long head_dim, long long tokens, long long heads, long long batch) {
  if (!aligned_to(pointer, 16)) return false;
  if (tokens > 1 && (strides[2] < head_dim || strides[2] % 8 != 0)) return false;
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
  TQ_REQUIRE(head_dim >= 8 && head_dim <= 2 * tq::kHeadDim && head_dim % 8 == 0, TQ_UNSUPPORTED,
             "fused attention has a kernel for heads of 8, 16, ... %d elements, not %lld", 2 * tq::kHeadDim, (long long)head_dim);
  if (batch == 0 || heads == 0 || q_tokens == 0) return TQ_OK;
  TQ_REQUIRE(k_tokens > 0, TQ_UNSUPPORTED, "a softmax over no keys has no kernel");
  TQ_REQUIRE(std::isfinite(scale) && scale > 0.0, TQ_UNSUPPORTED, "the score scale must be positive and finite, not %g", scale);
  TQ_REQUIRE(q != nullptr && k != nullptr && v != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null operand or result");
  TQ_REQUIRE(q_tokens < (1LL << 30) && k_tokens < (1LL << 30) && heads < 65536 && batch * heads < (1LL << 24), TQ_UNSUPPORTED,
             "extents beyond the kernel's index range");
  TQ_REQUIRE(tq::legal_strides(q, q_strides, head_dim, q_tokens, heads, batch) && tq::legal_strides(k, k_strides, head_dim, k_tokens, heads, batch) &&
                 tq::legal_strides(v, v_strides, head_dim, k_tokens, heads, batch),
             TQ_UNSUPPORTED, "Q, K and V must be 16-byte aligned with positive strides that are multiples of 8 elements (TMA's rules)");
  TQ_REQUIRE(tq::aligned_to(out, 2) && out_strides[0] >= 0 && out_strides[1] >= 0 && out_strides[2] >= 0, TQ_INVALID_ARGUMENT,
             "misaligned result or negative result stride");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  const tq::WaitStatus status = tq::wait_status_for(device);
  TQ_REQUIRE(status.abort != nullptr, TQ_RESOURCE_EXHAUSTED, "no device memory for the status word");

  CUtensorMap map_q, map_k, map_v;
  if (tq_status s = tq::attention_map(&map_q, dtype, q, head_dim, q_tokens, heads, batch, q_strides)) return s;
  if (tq_status s = tq::attention_map(&map_k, dtype, k, head_dim, k_tokens, heads, batch, k_strides)) return s;
  if (tq_status s = tq::attention_map(&map_v, dtype, v, head_dim, k_tokens, heads, batch, v_strides)) return s;

  tq::AttnParams p = {};
  p.batch = static_cast<int>(batch);
  p.heads = static_cast<int>(heads);
  p.q_tokens = static_cast<int>(q_tokens);
  p.k_tokens = static_cast<int>(k_tokens);
  p.head_dim = static_cast<int>(head_dim);
  const bool wide = head_dim > tq::kHeadDim;             // two sub-tiles side by side, one group of 128 rows per CTA
  const long long cta_rows = (wide ? 1 : tq::kGroups) * tq::kRows;
  p.q_blocks = static_cast<int>((q_tokens + cta_rows - 1) / cta_rows);
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
  auto go = [&](auto kernel, size_t smem) -> tq_status {
    static std::mutex mutex;
    {
      std::lock_guard<std::mutex> lock(mutex);
      TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    }
    kernel<<<static_cast<unsigned>(ctas), tq::kAttnThreads, smem, cuda_stream>>>(map_q, map_k, map_v, p);
    return tq::check_launch("attention_kernel");
  };
  if (wide) {
    constexpr size_t smem = tq::AttnLayout<2 * tq::kHeadDim>::kSmemBytes;
    if (dtype == TQ_BF16) return go(tq::attention_kernel<__nv_bfloat16, 2 * tq::kHeadDim>, smem);
    return go(tq::attention_kernel<__half, 2 * tq::kHeadDim>, smem);
  }
  constexpr size_t smem = tq::AttnLayout<tq::kHeadDim>::kSmemBytes;
  if (dtype == TQ_BF16) return go(tq::attention_kernel<__nv_bfloat16, tq::kHeadDim>, smem);
  return go(tq::attention_kernel<__half, tq::kHeadDim>, smem);
}
