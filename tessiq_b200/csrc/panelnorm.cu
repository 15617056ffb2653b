// softmax / LayerNorm over the last axis of a TRANSPOSED view of a tensor too large for the chip,
// with every element read from HBM once and written once.
//
//   in  packed [batch, rows, cols];  out packed [batch, cols, rows]
//   out[b][c][:] = softmax(in[b][:, c])    or    LayerNorm(in[b][:, c]) * weight[:] + bias[:]
//
// A column's statistics need every row, so the data is visited twice: statistics, then a
// transposing normalise. The tensor is walked in PANELS of columns — 512 bytes of every row, all the
// rows: 16 MiB at 32768 rows — small enough that a panel is still in L2 when its second visit comes.
// One persistent kernel, one CTA per SM, does both visits, as two pipelines that run side by side
// and meet only through flags in global memory:
//
//   first visit   S(p, k): statistics of panel p over the k-th chunk of rows. One partial per column
//                 goes to scratch. The CTA that completes a group of chunks (a ticket) folds the
//                 group's partials into one row, the CTA that completes the panel's last group folds
//                 the group rows into the panel's statistics and raises the panel's flag — fixed-order
//                 merges, so the result does not depend on which CTA folds;
//   second visit  N(p, k): the same piece again (an L2 hit), once panel p's flag is up: normalise,
//                 transpose V x V blocks in registers, write runs of `out`.
//
// Each pipeline has its own queue of items in global memory (panel-major order), its own producer
// warp, its own ring of shared-memory stages (a stage = 64 rows x 512 bytes, filled by one TMA tile
// load) and its own group of eight consumer warps. The S producer only ever waits for ring space and
// for the N pipeline not to fall more than `lead` panels behind (that bounds what L2 has to hold);
// the N producer waits for the panel's flag, copies the panel's statistics into shared memory and
// then streams the item's stages. Two publisher warps turn the S consumers' accumulators of a
// finished item into the chunk's partial row and do the ticketed folds, off the consumers' path.
//
// Nothing an S item needs ever waits for an N item, and the flag an N item waits for depends only on
// S items that were drawn before it could be, so every wait ends. Every wait is bounded all the same:
// one that gives up writes the device status word (and where it was) and the CTA leaves after its
// copies in flight have landed. A stage carries its running number, which the consumers check.
// Loads of the first visit carry an L2 evict-last policy, loads of the second visit and the stores
// evict-first, so the output stream does not push a panel out between its visits.
//
// The reference reaches this operation as pack (csrc/tessiq/codegen/pack.cpp:41-94) followed by its
// softmax (csrc/custom_ops/softmax/softmax.cu:19-61) or LayerNorm (csrc/tessiq/codegen/norm.cpp:22-135)
// kernel: four passes over HBM.
#include <algorithm>

#include "common.h"
#include "reducers.h"
#include "tcgen05.h"

namespace tq {
namespace {

constexpr int kGroupWarps = 8;                    // consumer warps of one pipeline
constexpr int kConsumerWarps = 2 * kGroupWarps;   // warps 0-7: first visit, warps 8-15: second visit
constexpr int kProducerWarpS = kConsumerWarps;
constexpr int kProducerWarpN = kConsumerWarps + 1;
constexpr int kPublisherWarp0 = kConsumerWarps + 2;
constexpr int kPublisherWarps = 2;                // each takes every other finished item
constexpr int kPanelThreads = (kConsumerWarps + 2 + kPublisherWarps) * 32;
constexpr int kPieceBytes = 512;                  // bytes of one row inside a panel
constexpr int kStageRows = 64;
constexpr int kStageBytes = kStageRows * kPieceBytes;
constexpr int kMaxStages = 6;                     // per ring
constexpr int kFoldGroup = 8;                     // chunks folded together at the first level
constexpr int kMinRows = 256;                     // shorter columns are not worth a panel walk
constexpr int kRowMultiple = kStageRows;
constexpr unsigned kFlagPolls = 1u << 22;
constexpr int kStatusPanelFlag = 0x504e4c31;         // "PNL1": a panel's flag never went up
constexpr int kStatusPanelData = 0x504e4c32;         // "PNL2": a stage's data never arrived
constexpr int kStatusPanelRing = 0x504e4c33;         // "PNL3": a stage was never handed back
constexpr int kStatusPanelPublish = 0x504e4c34;      // "PNL4": the publishers' next item never came
constexpr int kStatusPanelScratch = 0x504e4c35;      // "PNL5": the publishers never handed the accumulators back
constexpr int kStatusPanelStatsBuffer = 0x504e4c36;  // "PNL6": a statistics buffer was never handed back
constexpr int kStatusPanelStats = 0x504e4c37;        // "PNL7": a panel's statistics never reached shared memory
constexpr int kStatusPanelLead = 0x504e4c38;         // "PNL8": the second visit never caught up
constexpr int kStatusPanelOrder = 0x504e4c39;        // "PNL9": a stage arrived out of order

constexpr uint32_t kItemFirst = 2u, kItemLast = 4u, kItemExit = 8u;

struct PanelArgs {
  void* out;
  const void* weight;
  const void* bias;
  long long rows, cols;
  int panels_per_matrix;    // cols / columns per panel
  int panels;               // batch * panels_per_matrix
  int chunk_rows;           // rows per work item, a multiple of two stages
  int chunks;               // ceil(rows / chunk_rows)
  int lead;                 // panels the first visit may run ahead of the second
  int abreast;              // neighbouring panels walked together
  int policy;               // bit 0: first visit evict-last; bit 1: second visit evict-first; bit 2: stores evict-first
  int stages_s, stages_n;
  float eps;
  float2* partials;         // [panels][chunks][columns per panel]
  float2* group_partials;   // [panels][groups of chunks][columns per panel]
  float2* stats;            // [panels][columns per panel]
  unsigned* group_counters; // [panels][groups] S items finished
  unsigned* counters;       // [panels] groups folded
  unsigned* ready;          // [panels] statistics final
  unsigned* queue_s;        // next first-visit item
  unsigned* queue_n;        // next second-visit item
  unsigned* begun_n;        // second-visit items whose flag was seen up (what the first visit's lead is measured against)
  WaitStatus status;
};

__device__ __forceinline__ uint64_t l2_policy(int kind) {   // 0 normal, 1 evict-last, 2 evict-first
  uint64_t policy;
  if (kind == 1) {
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  } else if (kind == 2) {
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  } else {
    asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(policy));
  }
  return policy;
}

__device__ __forceinline__ void tma_load_2d_hinted(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}

template <typename T, int V>
__device__ __forceinline__ void store_hinted(T* pointer, const Vec<T, V>& value, uint64_t policy) {
  static_assert(sizeof(T) * V == 16, "panel stores are 16 bytes");
  const uint4 raw = *reinterpret_cast<const uint4*>(&value);
  asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;" ::"l"(pointer), "r"(raw.x), "r"(raw.y), "r"(raw.z),
               "r"(raw.w), "l"(policy)
               : "memory");
}

__device__ __forceinline__ unsigned load_acquire(const unsigned* pointer) {
  unsigned value;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(value) : "l"(pointer) : "memory");
  return value;
}

__device__ __forceinline__ void store_release(unsigned* pointer, unsigned value) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(pointer), "r"(value) : "memory");
}

// A bounded mbarrier wait that leaves a trace: the first wait of the device to give up writes its code
// to the status word and, behind it, where it was (CTA, thread, and three values of the caller).
constexpr uint32_t kPanelSpinLimit = 1u << 18;
__device__ __forceinline__ void panel_give_up(const WaitStatus& status, int code, int d0 = 0, int d1 = 0, int d2 = 0, int d3 = 0) {
  int* sticky = status.sticky();
  if (atomicCAS(sticky, 0, code) == 0) {
    sticky[1] = static_cast<int>(blockIdx.x);
    sticky[2] = static_cast<int>(threadIdx.x);
    sticky[3] = d0;
    sticky[4] = d1;
    sticky[5] = d2;
    sticky[6] = d3;
  }
  status.set_abort();
}

__device__ __forceinline__ bool panel_wait(uint32_t bar, uint32_t parity, const WaitStatus& status, int code, int d0, int d1, int d2,
                                           uint32_t limit = kPanelSpinLimit) {
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (barrier_try_wait(bar, parity)) return true;
    if ((spin & 0x3ff) == 0x3ff && status.aborted()) return false;
  }
  panel_give_up(status, code, d0, d1, d2, static_cast<int>(parity));
  return false;
}

// The per-column partial a chunk leaves behind and how partials merge. KIND 0: (reference point,
// sum of exp(x - reference)); KIND 1: (mean, sum of squared deviations) of `count` rows, merged with
// the pairwise update of Chan et al. (the weights through a fast reciprocal: they are ratios of
// small whole numbers).
template <typename T, int KIND> struct PanelStat;

template <typename T>
struct PanelStat<T, 0> {
  using R = SoftmaxStatReducer<T>;
  using Acc = typename R::Acc;
  __device__ static float2 pack(const Acc& a) { return make_float2(a.m, a.s); }
  __device__ static Acc unpack(float2 p, float) { return Acc{p.x, p.y}; }
  __device__ static Acc identity() { return R::identity(); }
  __device__ static Acc combine(const Acc& a, const Acc& b) { return R::combine(a, b); }
  __device__ static float2 finish(const Acc& a, long long rows) {
    const typename R::Out o = R::finish(a, rows, false);
    return make_float2(o.m, o.s);
  }
};

template <typename T>
struct PanelStat<T, 1> {
  using R = MomentsReducer<T>;
  using Acc = typename R::Acc;
  __device__ static float2 pack(const Acc& a) { return make_float2(a.mean, a.m2); }
  __device__ static Acc unpack(float2 p, float count) { return Acc{count, p.x, p.y, 0.f}; }
  __device__ static Acc identity() { return R::identity(); }
  __device__ static Acc combine(const Acc& a, const Acc& b) {
    if (a.n == 0.f) return b;
    const float n = a.n + b.n;
    const float share = __fdividef(b.n, n);
    const float delta = b.mean - a.mean;
    return Acc{n, fmaf(delta, share, a.mean), a.m2 + b.m2 + delta * delta * (a.n * share), 0.f};
  }
  __device__ static float2 finish(const Acc& a, long long rows) {
    const typename R::Out o = R::finish(a, rows, false);
    return make_float2(o.mean, o.variance);
  }
};

// The first visit's per-thread state for two neighbouring columns, with the arithmetic on both at
// once (the .f32x2 forms of add, mul and fma: the consumer warps are bound by the instructions they
// issue, not by memory). The values and their order are those of the scalar reducers.
template <typename T, int KIND> struct PairState;

// Online softmax statistics around a lazy reference point (see SoftmaxStatReducer): the reference is
// kept negated, and both columns take the rare slow path when either needs it.
template <typename T>
struct PairState<T, 0> {
  float2 negated_reference, sum;
  __device__ void reset() {
    negated_reference = make_float2(INFINITY, INFINITY);   // reference -inf: the first element takes the slow path
    sum = make_float2(0.f, 0.f);
  }
  __device__ void seed(T, T) {}
  __device__ static void slow(float x, float t, float& negated, float& total) {
    if (x == -INFINITY) {
      t = x;                                  // contributes nothing, the reference stays
    } else {
      total *= stat_exp2(-t);                 // 0 for the first element; NaN for a NaN or a second +inf
      negated = -x;
      t = 0.f;
    }
    total += stat_exp2(t);
  }
  __device__ void step(T a, T b) {
    constexpr float kLog2e = 1.4426950408889634f;
    const float2 x = make_float2(to_compute(a), to_compute(b));
    const float2 t = __fmul2_rn(__fadd2_rn(x, negated_reference), make_float2(kLog2e, kLog2e));
    const float worst = ExtremeReducer<float, true>::combine(t.x, t.y);
    if (!(worst <= SoftmaxStatReducer<T>::kSlack)) {   // far above the reference, the first element, or a NaN
      slow(x.x, t.x, negated_reference.x, sum.x);
      slow(x.y, t.y, negated_reference.y, sum.y);
      return;
    }
    sum = __fadd2_rn(sum, make_float2(stat_exp2(t.x), stat_exp2(t.y)));
  }
  // One row of a thread's P pairs behind a single test, so that the common path is P independent
  // scale / ex2 / add chains with no branch between them; the rare path is `step`, pair by pair.
  template <int P>
  __device__ static void step_row(PairState (&pairs)[P], const Vec<T, 2 * P>& x) {
    constexpr float kLog2e = 1.4426950408889634f;
    float2 t[P];
    float worst = -INFINITY;
#pragma unroll
    for (int e = 0; e < P; ++e) {
      t[e] = __fmul2_rn(__fadd2_rn(make_float2(to_compute(x.v[2 * e]), to_compute(x.v[2 * e + 1])), pairs[e].negated_reference),
                        make_float2(kLog2e, kLog2e));
      worst = ExtremeReducer<float, true>::combine(worst, ExtremeReducer<float, true>::combine(t[e].x, t[e].y));
    }
    if (!(worst <= SoftmaxStatReducer<T>::kSlack)) {
#pragma unroll
      for (int e = 0; e < P; ++e) pairs[e].step(x.v[2 * e], x.v[2 * e + 1]);
      return;
    }
#pragma unroll
    for (int e = 0; e < P; ++e) pairs[e].sum = __fadd2_rn(pairs[e].sum, make_float2(stat_exp2(t[e].x), stat_exp2(t[e].y)));
  }
  __device__ float4 packed(int) const { return make_float4(-negated_reference.x, sum.x, -negated_reference.y, sum.y); }
};

// Shifted moments (see MomentsReducer): sums of (x - pivot) and (x - pivot)^2, the pivot kept negated.
template <typename T>
struct PairState<T, 1> {
  float2 negated_pivot, s1, s2;
  __device__ void reset() {
    negated_pivot = make_float2(0.f, 0.f);
    s1 = make_float2(0.f, 0.f);
    s2 = make_float2(0.f, 0.f);
  }
  __device__ void seed(T a, T b) { negated_pivot = make_float2(-to_compute(a), -to_compute(b)); }
  __device__ void step(T a, T b) {
    const float2 d = __fadd2_rn(make_float2(to_compute(a), to_compute(b)), negated_pivot);
    s1 = __fadd2_rn(s1, d);
    s2 = __ffma2_rn(d, d, s2);
  }
  template <int P>
  __device__ static void step_row(PairState (&pairs)[P], const Vec<T, 2 * P>& x) {
#pragma unroll
    for (int e = 0; e < P; ++e) pairs[e].step(x.v[2 * e], x.v[2 * e + 1]);
  }
  __device__ float4 packed(int count) const {
    using R = MomentsReducer<T>;
    const typename R::Acc a = R::template to_acc<1>(typename R::template Local<1>{-negated_pivot.x, s1.x, s2.x, static_cast<float>(count)});
    const typename R::Acc b = R::template to_acc<1>(typename R::template Local<1>{-negated_pivot.y, s1.y, s2.y, static_cast<float>(count)});
    return make_float4(a.mean, a.m2, b.mean, b.m2);
  }
};

__device__ __forceinline__ unsigned ticket_acq_rel(unsigned* counter) {
  unsigned ticket;
  asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(ticket) : "l"(counter) : "memory");
  return ticket;
}

// A publisher warp's fold of `n` partial rows ([n][columns] float2; row i covers `unit` data rows,
// the last one what is left of `rows_left`) into one row at `out`, in row order. Lane l owns columns
// [l * C, l * C + C), C = columns / 32, read two at a time. FINAL writes the finished statistics
// instead of a mergeable partial.
template <typename T, int KIND, bool FINAL>
__device__ __forceinline__ void fold_rows(const float2* rows, int n, int unit, long long rows_left, float2* out, long long total_rows) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  constexpr int kColumns = 32 * V;
  constexpr int kMine = kColumns / 32;     // columns per lane: 4 or 8
  constexpr int kBatch = 16 / kMine;       // rows in flight: 8 float4 loads per lane
  using S = PanelStat<T, KIND>;
  using Acc = typename S::Acc;
  const int lane = threadIdx.x & 31;
  const float4* mine = reinterpret_cast<const float4*>(rows + lane * kMine);
  const long long tail = rows_left - static_cast<long long>(n - 1) * unit;
  const float last_count = static_cast<float>(tail < unit ? tail : unit);
  Acc total[kMine];
#pragma unroll
  for (int e = 0; e < kMine; ++e) total[e] = S::identity();
  for (int i = 0; i < n; i += kBatch) {
    float4 batch[kBatch][kMine / 2];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (i + u < n) {
#pragma unroll
        for (int h = 0; h < kMine / 2; ++h) batch[u][h] = __ldcg(mine + static_cast<long long>(i + u) * (kColumns / 2) + h);
      }
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      if (i + u < n) {
        const float count = i + u == n - 1 ? last_count : static_cast<float>(unit);
#pragma unroll
        for (int h = 0; h < kMine / 2; ++h) {
          total[2 * h] = S::combine(total[2 * h], S::unpack(make_float2(batch[u][h].x, batch[u][h].y), count));
          total[2 * h + 1] = S::combine(total[2 * h + 1], S::unpack(make_float2(batch[u][h].z, batch[u][h].w), count));
        }
      }
    }
  }
#pragma unroll
  for (int h = 0; h < kMine / 2; ++h) {
    const float2 a = FINAL ? S::finish(total[2 * h], total_rows) : S::pack(total[2 * h]);
    const float2 b = FINAL ? S::finish(total[2 * h + 1], total_rows) : S::pack(total[2 * h + 1]);
    reinterpret_cast<float4*>(out + lane * kMine)[h] = make_float4(a.x, a.y, b.x, b.y);
  }
}

// A publisher warp: what a finished S item leaves behind. The consumer warps' packed accumulators
// (`scratch`, [8 warps][columns], `warp_rows` data rows behind each) become this chunk's partial row;
// then two levels of "last one in folds": the warp whose chunk completes a group of kFoldGroup chunks
// folds the group's rows into one, and the warp whose group completes the panel folds the group rows
// into the panel's statistics and raises its flag. `scratch` is handed back as soon as it is read.
// Ordering: a warp's stores, a warp barrier, then lane 0's acquire-release ticket — so whoever draws
// the last ticket sees every earlier partial, and its own lanes read them after a second barrier.
template <typename T, int KIND>
__device__ __forceinline__ void publish_partial(const PanelArgs& args, int panel, int chunk, float warp_rows, const float2* scratch,
                                                uint32_t scratch_empty) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  constexpr int kColumns = 32 * V;
  constexpr int kMine = kColumns / 32;
  using S = PanelStat<T, KIND>;
  using Acc = typename S::Acc;
  const int lane = threadIdx.x & 31;
  float2 row[kMine];
#pragma unroll
  for (int h = 0; h < kMine / 2; ++h) {
    const float4 first = reinterpret_cast<const float4*>(scratch + lane * kMine)[h];
    Acc left = S::unpack(make_float2(first.x, first.y), warp_rows), right = S::unpack(make_float2(first.z, first.w), warp_rows);
#pragma unroll
    for (int w = 1; w < kGroupWarps; ++w) {
      const float4 next = reinterpret_cast<const float4*>(scratch + w * kColumns + lane * kMine)[h];
      left = S::combine(left, S::unpack(make_float2(next.x, next.y), warp_rows));
      right = S::combine(right, S::unpack(make_float2(next.z, next.w), warp_rows));
    }
    row[2 * h] = S::pack(left);
    row[2 * h + 1] = S::pack(right);
  }
  __syncwarp();
  if (lane == 0) barrier_arrive(scratch_empty);
  float4* partial = reinterpret_cast<float4*>(args.partials + (static_cast<long long>(panel) * args.chunks + chunk) * kColumns + lane * kMine);
#pragma unroll
  for (int h = 0; h < kMine / 2; ++h) partial[h] = make_float4(row[2 * h].x, row[2 * h].y, row[2 * h + 1].x, row[2 * h + 1].y);

  const int group = chunk / kFoldGroup;
  const int groups = (args.chunks + kFoldGroup - 1) / kFoldGroup;
  const int members = args.chunks - group * kFoldGroup < kFoldGroup ? args.chunks - group * kFoldGroup : kFoldGroup;
  __syncwarp();
  unsigned ticket = 0;
  if (lane == 0) ticket = ticket_acq_rel(args.group_counters + static_cast<long long>(panel) * groups + group);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  if (ticket != static_cast<unsigned>(members - 1)) return;
  __syncwarp();
  const long long rows_left = args.rows - static_cast<long long>(group) * kFoldGroup * args.chunk_rows;   // from this group's first row on
  fold_rows<T, KIND, false>(args.partials + (static_cast<long long>(panel) * args.chunks + group * kFoldGroup) * kColumns, members,
                            args.chunk_rows, rows_left, args.group_partials + (static_cast<long long>(panel) * groups + group) * kColumns,
                            args.rows);
  __syncwarp();
  if (lane == 0) ticket = ticket_acq_rel(args.counters + panel);
  ticket = __shfl_sync(0xffffffffu, ticket, 0);
  if (ticket != static_cast<unsigned>(groups - 1)) return;
  __syncwarp();
  fold_rows<T, KIND, true>(args.group_partials + static_cast<long long>(panel) * groups * kColumns, groups,
                           kFoldGroup * args.chunk_rows, args.rows, args.stats + static_cast<long long>(panel) * kColumns, args.rows);
  __syncwarp();
  if (lane == 0) store_release(args.ready + panel, 1u);
}

// Shared memory: S ring [stages_s][32 KiB] | N ring [stages_n][32 KiB] | scratch [2][8 warps][columns]
// float2 | statistics [2][columns] float2 | stage notes S[kMaxStages], N[kMaxStages] | publish notes [2] |
// mbarriers: S full/empty [kMaxStages] each, N full/empty [kMaxStages] each, scratch_full[2],
// scratch_empty[2], stats_full[2], stats_empty[2].
// A stage note is (flags | running number << 4, panel, chunk, stage index within the item | stages
// of the item << 16).
template <typename T, int KIND>
__global__ void __launch_bounds__(kPanelThreads, 1) panel_normalize_kernel(const __grid_constant__ CUtensorMap map, const PanelArgs args) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  constexpr int kColumns = 32 * V;
  constexpr int kRowBlocks = kStageRows / V;                      // V x V blocks along the rows of a stage: 16 or 8
  constexpr int kBlocksPerThread = kRowBlocks * 32 / (kGroupWarps * 32);   // 2 or 1
  constexpr int kRowsPerWarp = kStageRows / kGroupWarps;          // first visit: rows of a stage per warp
  constexpr float kLog2e = 1.4426950408889634f;
  using S = PanelStat<T, KIND>;
  using R = typename S::R;
  extern __shared__ __align__(128) unsigned char panel_smem[];
  __shared__ int give_up;

  unsigned char* data_s = panel_smem;
  unsigned char* data_n = data_s + static_cast<size_t>(args.stages_s) * kStageBytes;
  float2* scratch = reinterpret_cast<float2*>(data_n + static_cast<size_t>(args.stages_n) * kStageBytes);   // [2][8 warps][columns]
  float2* stats_smem = scratch + 2 * kGroupWarps * kColumns;                                                 // [2][columns]
  uint4* notes_s = reinterpret_cast<uint4*>(stats_smem + 2 * kColumns);
  uint4* notes_n = notes_s + kMaxStages;
  uint4* publish_note = notes_n + kMaxStages;
  uint64_t* barriers = reinterpret_cast<uint64_t*>(publish_note + 2);
  const uint32_t full_s0 = smem_address(barriers), empty_s0 = full_s0 + 8 * kMaxStages;
  const uint32_t full_n0 = empty_s0 + 8 * kMaxStages, empty_n0 = full_n0 + 8 * kMaxStages;
  const uint32_t scratch_full0 = empty_n0 + 8 * kMaxStages, scratch_empty0 = scratch_full0 + 16;
  const uint32_t stats_full0 = scratch_empty0 + 16, stats_empty0 = stats_full0 + 16;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      barrier_init(full_s0 + 8 * s, 1);
      barrier_init(empty_s0 + 8 * s, kGroupWarps);
      barrier_init(full_n0 + 8 * s, 1);
      barrier_init(empty_n0 + 8 * s, kGroupWarps);
    }
    for (int b = 0; b < 2; ++b) {
      barrier_init(scratch_full0 + 8 * b, kGroupWarps);
      barrier_init(scratch_empty0 + 8 * b, 1);
      barrier_init(stats_full0 + 8 * b, 1);
      barrier_init(stats_empty0 + 8 * b, kGroupWarps);
    }
    give_up = 0;
    if (blockIdx.x == 0) args.status.begin();
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const unsigned per_panel = static_cast<unsigned>(args.chunks);
  const unsigned total = static_cast<unsigned>(args.panels) * per_panel;   // items of each pipeline
  int producer_stage = 0;          // a producer's ring position, kept for the teardown
  uint32_t producer_phase = 0;

  if (warp == kProducerWarpS || warp == kProducerWarpN) {
    // ---- producers: lane 0 draws items of its pipeline and streams their stages in ---------------
    const bool second = warp == kProducerWarpN;
    const uint64_t policy = second ? l2_policy((args.policy & 2) ? 2 : 0) : l2_policy((args.policy & 1) ? 1 : 0);
    unsigned* queue = second ? args.queue_n : args.queue_s;
    const uint32_t full0 = second ? full_n0 : full_s0, empty0 = second ? empty_n0 : empty_s0;
    const uint32_t data0 = smem_address(second ? data_n : data_s);
    uint4* notes = second ? notes_n : notes_s;
    const int stages = second ? args.stages_n : args.stages_s;
    unsigned prepared = 0;   // N items prepared so far
    unsigned issued = 0;     // stages issued so far
    unsigned seen_n = 0;     // S producer: second-visit items begun, when last looked at
    unsigned drawn = 0;
    if (lane == 0) drawn = atomicAdd(queue, 1u);
    bool running = true;
    while (running) {
      const unsigned item = __shfl_sync(0xffffffffu, drawn, 0);
      if (lane == 0 && item < total) drawn = atomicAdd(queue, 1u);   // the next draw lands while this item is issued
      const bool exit_item = item >= total;
      // items walk `abreast` neighbouring panels together, chunk by chunk: the pieces of one row that
      // neighbouring panels hold are then fetched at about the same time, which HBM likes
      const unsigned abreast = static_cast<unsigned>(args.abreast);
      const unsigned within = exit_item ? 0u : item % (abreast * per_panel);
      const int panel = exit_item ? 0 : static_cast<int>(item / (abreast * per_panel) * abreast + within % abreast);
      const int chunk = exit_item ? 0 : static_cast<int>(within / abreast);
      int subs = 1;
      long long row = 0;
      int column = 0;
      if (!exit_item) {
        const long long row0 = static_cast<long long>(chunk) * args.chunk_rows;
        const long long count = args.rows - row0 < args.chunk_rows ? args.rows - row0 : args.chunk_rows;
        subs = static_cast<int>(count / kStageRows);
        row = static_cast<long long>(panel / args.panels_per_matrix) * args.rows + row0;
        column = (panel % args.panels_per_matrix) * kColumns;
      }
      int ok = 1;
      if (!second && !exit_item) {
        // the first visit may not run more than `lead` panels ahead of the second
        if (lane == 0 && item >= seen_n + static_cast<unsigned>(args.lead) * per_panel) {
          ok = 0;
          for (unsigned spin = 0; spin < kFlagPolls; ++spin) {
            seen_n = load_acquire(args.begun_n);
            if (item < seen_n + static_cast<unsigned>(args.lead) * per_panel) {
              ok = 1;
              break;
            }
            __nanosleep(100);
          }
          if (!ok) panel_give_up(args.status, kStatusPanelLead, static_cast<int>(item), static_cast<int>(seen_n));
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
      }
      if (second && !exit_item) {
        // the panel's statistics: wait for the flag, then copy them into the buffer this item uses
        const int buffer = prepared & 1;
        if (lane == 0) {
          ok = panel_wait(stats_empty0 + 8 * buffer, ((prepared >> 1) & 1) ^ 1, args.status, kStatusPanelStatsBuffer,
                          static_cast<int>(prepared), panel, chunk) ? 1 : 0;
          if (ok) {
            unsigned seen = 0;
            for (unsigned spin = 0; spin < kFlagPolls; ++spin) {
              seen = load_acquire(args.ready + panel);
              if (seen != 0) break;
              __nanosleep(40);
            }
            if (seen == 0) {
              panel_give_up(args.status, kStatusPanelFlag, panel, chunk);
              ok = 0;
            }
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
          const float4* source = reinterpret_cast<const float4*>(args.stats + static_cast<long long>(panel) * kColumns);
          float4* target = reinterpret_cast<float4*>(stats_smem + buffer * kColumns);
#pragma unroll
          for (int h = 0; h < kColumns / 64; ++h) target[h * 32 + lane] = __ldcg(source + h * 32 + lane);
          __syncwarp();
          if (lane == 0) {
            barrier_arrive(stats_full0 + 8 * buffer);
            atomicAdd(args.begun_n, 1u);
          }
          ++prepared;
        }
      }
      if (!ok) {
        *reinterpret_cast<volatile int*>(&give_up) = 1;
        break;
      }
      if (lane == 0) {
        for (int s = 0; s < subs; ++s) {
          if (*reinterpret_cast<volatile int*>(&give_up) != 0 ||
              !panel_wait(empty0 + 8 * producer_stage, producer_phase ^ 1, args.status, kStatusPanelRing, producer_stage,
                          static_cast<int>(item), s)) {
            *reinterpret_cast<volatile int*>(&give_up) = 1;
            running = false;
            break;
          }
          uint32_t kind = exit_item ? kItemExit : 0u;
          if (s == 0) kind |= kItemFirst;
          if (s == subs - 1) kind |= kItemLast;
          kind |= issued << 4;
          ++issued;
          notes[producer_stage] = make_uint4(kind, static_cast<uint32_t>(panel), static_cast<uint32_t>(chunk),
                                             static_cast<uint32_t>(s) | (static_cast<uint32_t>(subs) << 16));
          if (exit_item) {
            barrier_arrive(full0 + 8 * producer_stage);
          } else {
            barrier_expect_tx(full0 + 8 * producer_stage, kStageBytes);
            tma_load_2d_hinted(data0 + producer_stage * kStageBytes, &map, full0 + 8 * producer_stage, column,
                               static_cast<int>(row + s * kStageRows), policy);
          }
          if (++producer_stage == stages) {
            producer_stage = 0;
            producer_phase ^= 1;
          }
        }
        if (exit_item) running = false;
      }
      running = __shfl_sync(0xffffffffu, running ? 1 : 0, 0) != 0;
    }
  } else if (warp >= kPublisherWarp0) {
    // ---- publisher warps: turn finished S items into partial rows, fold, raise flags. Warp w takes
    // the CTA's items w, w + 2, ... through scratch buffer w ------------------------------------------
    const int buffer = warp - kPublisherWarp0;
    unsigned published = 0;
    while (true) {
      // a wait that may last the whole kernel: the CTA's next first-visit item, or the end
      int ok = 1;
      if (lane == 0) {
        ok = panel_wait(scratch_full0 + 8 * buffer, published & 1, args.status, kStatusPanelPublish, static_cast<int>(published), buffer, 0,
                        64 * kPanelSpinLimit) ? 1 : 0;
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) {
        *reinterpret_cast<volatile int*>(&give_up) = 1;
        break;
      }
      const uint4 note = publish_note[buffer];
      if (note.x & kItemExit) break;
      publish_partial<T, KIND>(args, static_cast<int>(note.y), static_cast<int>(note.z), __uint_as_float(note.w),
                               scratch + buffer * kGroupWarps * kColumns, scratch_empty0 + 8 * buffer);
      ++published;
    }
  } else if (warp < kGroupWarps) {
    // ---- first-visit consumers ----------------------------------------------------------------------
    const int stages = args.stages_s;
    PairState<T, KIND> local[V / 2];
    int stage = 0;
    uint32_t phase = 0;
    unsigned handed = 0;      // items handed to the publishers
    unsigned expected = 0;    // running number of the next stage
    bool alive = true;
    while (true) {
      if (!panel_wait(full_s0 + 8 * stage, phase, args.status, kStatusPanelData, stage, static_cast<int>(handed), 0)) {
        alive = false;
        break;
      }
      const uint4 note = notes_s[stage];
      if ((note.x >> 4) != expected) {
        panel_give_up(args.status, kStatusPanelOrder, static_cast<int>(note.x), static_cast<int>(expected), stage);
        alive = false;
        break;
      }
      ++expected;
      if (note.x & kItemExit) break;
      const int sub = static_cast<int>(note.w & 0xffffu);
      // rows warp, warp + 8, ... of the stage; the warp reads one whole 512-byte row at a time
      const Vec<T, V>* mine = reinterpret_cast<const Vec<T, V>*>(data_s + static_cast<size_t>(stage) * kStageBytes +
                                                                 static_cast<size_t>(warp) * kPieceBytes) + lane;
      if (note.x & kItemFirst) {
        const Vec<T, V> x = mine[0];
#pragma unroll
        for (int e = 0; e < V / 2; ++e) {
          local[e].reset();
          local[e].seed(x.v[2 * e], x.v[2 * e + 1]);
        }
      }
#pragma unroll
      for (int i = 0; i < kRowsPerWarp; ++i) {
        const Vec<T, V> x = mine[i * kGroupWarps * (kPieceBytes / 16)];
        PairState<T, KIND>::template step_row<V / 2>(local, x);
      }
      __syncwarp();
      if (lane == 0) barrier_arrive(empty_s0 + 8 * stage);
      if (note.x & kItemLast) {
        const int seen = (sub + 1) * kRowsPerWarp;   // data rows behind this thread's accumulators
        const int buffer = handed & 1;
        if (!panel_wait(scratch_empty0 + 8 * buffer, ((handed >> 1) & 1) ^ 1, args.status, kStatusPanelScratch, static_cast<int>(handed),
                        static_cast<int>(note.y), static_cast<int>(note.z))) {
          alive = false;
          break;
        }
        float2* slot = scratch + (buffer * kGroupWarps + warp) * kColumns + lane * V;
#pragma unroll
        for (int e = 0; e < V / 2; ++e) reinterpret_cast<float4*>(slot)[e] = local[e].packed(seen);
        if (threadIdx.x == 0) publish_note[buffer] = make_uint4(0u, note.y, note.z, __float_as_uint(static_cast<float>(seen)));
        __syncwarp();
        if (lane == 0) barrier_arrive(scratch_full0 + 8 * buffer);
        ++handed;
      }
      if (++stage == stages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (!alive) {
      *reinterpret_cast<volatile int*>(&give_up) = 1;
    } else {
      // tell both publisher warps that no more items come
      for (int last = 0; last < 2 && alive; ++last, ++handed) {
        const int buffer = handed & 1;
        if (panel_wait(scratch_empty0 + 8 * buffer, ((handed >> 1) & 1) ^ 1, args.status, kStatusPanelScratch, static_cast<int>(handed), -1, -1)) {
          if (threadIdx.x == 0) publish_note[buffer] = make_uint4(kItemExit, 0u, 0u, 0u);
          __syncwarp();
          if (lane == 0) barrier_arrive(scratch_full0 + 8 * buffer);
        } else {
          alive = false;
          *reinterpret_cast<volatile int*>(&give_up) = 1;
        }
      }
    }
  } else {
    // ---- second-visit consumers --------------------------------------------------------------------
    const int stages = args.stages_n;
    const int gwarp = warp - kGroupWarps;
    const uint64_t store_policy = l2_policy((args.policy & 4) ? 2 : 0);
    const T* weight = static_cast<const T*>(args.weight);
    const T* bias = static_cast<const T*>(args.bias);
    // 8 consecutive lanes take 8 consecutive 16-byte column blocks (conflict-free shared-memory
    // reads); a warp is 8 column blocks x 4 row blocks, the group 32 x 8 per step.
    const int column_block = (lane & 7) + 8 * (gwarp & 3);
    const int row_block = (lane >> 3) + 4 * (gwarp >> 2);
    float2 negated_first[V], second[V];   // per column, each value twice: the operands of the paired arithmetic
    T* item_target = nullptr;
    const T* item_weight = nullptr;
    const T* item_bias = nullptr;
    int stage = 0;
    uint32_t phase = 0;
    unsigned normalized = 0;  // items begun
    unsigned expected = 0;
    bool alive = true;
    while (true) {
      if (!panel_wait(full_n0 + 8 * stage, phase, args.status, kStatusPanelData, stage, static_cast<int>(normalized), 1)) {
        alive = false;
        break;
      }
      const uint4 note = notes_n[stage];
      if ((note.x >> 4) != expected) {
        panel_give_up(args.status, kStatusPanelOrder, static_cast<int>(note.x), static_cast<int>(expected), stage);
        alive = false;
        break;
      }
      ++expected;
      if (note.x & kItemExit) break;
      const int panel = static_cast<int>(note.y), chunk = static_cast<int>(note.z), sub = static_cast<int>(note.w & 0xffffu);
      const unsigned char* tile = data_n + static_cast<size_t>(stage) * kStageBytes;
      if (note.x & kItemFirst) {
        const int buffer = normalized & 1;
        if (!panel_wait(stats_full0 + 8 * buffer, (normalized >> 1) & 1, args.status, kStatusPanelStats, static_cast<int>(normalized), panel,
                        chunk)) {
          alive = false;
          break;
        }
        const float2* stats = stats_smem + buffer * kColumns + column_block * V;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          const float2 st = stats[j];
          const float scale = KIND == 0 ? st.y : rsqrtf(st.y + args.eps);
          negated_first[j] = make_float2(-st.x, -st.x);
          second[j] = make_float2(scale, scale);
        }
        __syncwarp();
        if (lane == 0) barrier_arrive(stats_empty0 + 8 * buffer);
        ++normalized;
        const long long matrix = panel / args.panels_per_matrix;
        const long long c = static_cast<long long>(panel % args.panels_per_matrix) * kColumns + column_block * V;
        const long long r = static_cast<long long>(chunk) * args.chunk_rows + row_block * V;
        item_target = static_cast<T*>(args.out) + matrix * args.rows * args.cols + c * args.rows + r;
        item_weight = weight != nullptr ? weight + r : nullptr;
        item_bias = bias != nullptr ? bias + r : nullptr;
      }
      Vec<T, V> block[kBlocksPerThread][V];
#pragma unroll
      for (int q = 0; q < kBlocksPerThread; ++q) {
#pragma unroll
        for (int i = 0; i < V; ++i) {
          block[q][i] = *reinterpret_cast<const Vec<T, V>*>(tile + static_cast<size_t>((row_block + 8 * q) * V + i) * kPieceBytes +
                                                             column_block * 16);
        }
      }
#pragma unroll
      for (int q = 0; q < kBlocksPerThread; ++q) {
        const int r = sub * kStageRows + 8 * q * V;   // this block's first row, from the thread's first row of the item
        float2 scale[V / 2], shift[V / 2];            // LayerNorm: weight and bias of rows r + 2 h, r + 2 h + 1
        if constexpr (KIND == 1) {
          Vec<T, V> weights, biases;
          if (item_weight != nullptr) weights = *reinterpret_cast<const Vec<T, V>*>(item_weight + r);
          if (item_bias != nullptr) biases = *reinterpret_cast<const Vec<T, V>*>(item_bias + r);
#pragma unroll
          for (int h = 0; h < V / 2; ++h) {
            scale[h] = item_weight != nullptr ? make_float2(to_compute(weights.v[2 * h]), to_compute(weights.v[2 * h + 1])) : make_float2(1.f, 1.f);
            shift[h] = item_bias != nullptr ? make_float2(to_compute(biases.v[2 * h]), to_compute(biases.v[2 * h + 1])) : make_float2(0.f, 0.f);
          }
        }
        T* line_target = item_target + r;
#pragma unroll
        for (int j = 0; j < V; ++j) {
          Vec<T, V> line;
#pragma unroll
          for (int h = 0; h < V / 2; ++h) {
            const float2 x = make_float2(to_compute(block[q][2 * h].v[j]), to_compute(block[q][2 * h + 1].v[j]));
            const float2 d = __fadd2_rn(x, negated_first[j]);
            float2 y;
            if constexpr (KIND == 0) {
              const float2 t = __fmul2_rn(d, make_float2(kLog2e, kLog2e));
              y = __fmul2_rn(make_float2(stat_exp2(t.x), stat_exp2(t.y)), second[j]);
            } else {
              y = __ffma2_rn(__fmul2_rn(d, second[j]), scale[h], shift[h]);
            }
            line.v[2 * h] = from_compute<T, float>(y.x);
            line.v[2 * h + 1] = from_compute<T, float>(y.y);
          }
          store_hinted<T, V>(line_target, line, store_policy);
          line_target += args.rows;
        }
      }
      // the stage goes back only after every value read from it has been used (handing it back right
      // after the shared-memory loads were issued can let the next tile land under the last of them)
      __syncwarp();
      if (lane == 0) barrier_arrive(empty_n0 + 8 * stage);
      if (++stage == stages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (!alive) *reinterpret_cast<volatile int*>(&give_up) = 1;
  }

  // Teardown. After a give-up the CTA must not leave while a tile load may still land in its shared
  // memory: each producer lane waits (bounded) for the last arming of every stage of its ring.
  // Stages before its ring position were last armed in its current phase, the others one phase back
  // (a never-armed stage answers at once).
  __syncthreads();
  if (give_up != 0 && lane == 0 && (warp == kProducerWarpS || warp == kProducerWarpN)) {
    const bool second = warp == kProducerWarpN;
    const uint32_t full0 = second ? full_n0 : full_s0;
    const int stages = second ? args.stages_n : args.stages_s;
    for (int s = 0; s < stages; ++s) {
      const uint32_t parity = s < producer_stage ? producer_phase : producer_phase ^ 1;
      for (uint32_t spin = 0; spin < kPanelSpinLimit; ++spin) {
        if (barrier_try_wait(full0 + 8 * s, parity)) break;
      }
    }
  }
}

// The settings, all measured on B200 at [32768, 4096] (see the table in the file's last comment).
constexpr int kLeadPanels = 8;       // panels the first visit may run ahead of the second
constexpr int kAbreast = 1;          // neighbouring panels walked together
constexpr int kChunkRows = 512;      // rows per work item
constexpr int kStagesS = 3, kStagesN = 3;
constexpr int kPolicy = 7;           // first visit evict-last, second visit and stores evict-first
constexpr long long kMinBytes = 256ll << 20;

struct PanelLayout {
  int columns;          // per panel
  int panels_per_matrix, panels, chunk_rows, chunks, groups;
  size_t partial_bytes, group_bytes, stats_bytes, flag_bytes;   // flags: group counters, panel counters, ready, queue
  size_t total() const { return partial_bytes + group_bytes + stats_bytes + flag_bytes; }
};

PanelLayout panel_layout(tq_dtype dtype, long long batch, long long rows, long long cols) {
  PanelLayout l = {};
  l.columns = kPieceBytes / dtype_size(dtype);
  l.panels_per_matrix = static_cast<int>(cols / l.columns);
  l.panels = static_cast<int>(batch * l.panels_per_matrix);
  l.chunk_rows = kChunkRows;
  l.chunks = static_cast<int>((rows + l.chunk_rows - 1) / l.chunk_rows);
  l.groups = (l.chunks + kFoldGroup - 1) / kFoldGroup;
  auto round_up = [](size_t v) { return (v + 255) / 256 * 256; };
  l.partial_bytes = round_up(static_cast<size_t>(l.panels) * l.chunks * l.columns * sizeof(float2));
  l.group_bytes = round_up(static_cast<size_t>(l.panels) * l.groups * l.columns * sizeof(float2));
  l.stats_bytes = round_up(static_cast<size_t>(l.panels) * l.columns * sizeof(float2));
  l.flag_bytes = round_up((static_cast<size_t>(l.panels) * (l.groups + 2) + 3) * sizeof(unsigned));
  return l;
}

template <typename T, int KIND>
tq_status run_panels(const CUtensorMap& map, PanelArgs args, int32_t device, cudaStream_t stream) {
  constexpr int V = 16 / static_cast<int>(sizeof(T));
  constexpr int kColumns = 32 * V;
  args.stages_s = kStagesS;
  args.stages_n = std::min(kStagesN, static_cast<int>((220 * 1024 - (2 * kGroupWarps + 2) * kColumns * sizeof(float2)) / kStageBytes) - args.stages_s);
  const size_t smem = static_cast<size_t>(args.stages_s + args.stages_n) * kStageBytes + (2 * kGroupWarps + 2) * kColumns * sizeof(float2) +
                      (2 * kMaxStages + 2) * 16 + (4 * kMaxStages + 8) * 8;
  auto kernel = panel_normalize_kernel<T, KIND>;
  TQ_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
  const long long items = static_cast<long long>(args.panels) * args.chunks;
  long long grid = sm_count(device);
  if (grid > items) grid = items;
  kernel<<<static_cast<unsigned>(grid), kPanelThreads, smem, stream>>>(map, args);
  return check_launch("panel_normalize_kernel");
}

}  // namespace

bool panel_takes(tq_dtype dtype, long long batch, long long rows, long long cols) {
  if (dtype != TQ_F32) return false;   // the kernel is written for the 2-byte types as well, but measured behind the other forms for them
  const int size = dtype_size(dtype);
  const int columns = kPieceBytes / size;
  if (batch < 1 || rows < kMinRows || rows % kRowMultiple != 0 || cols % columns != 0) return false;
  const long long panel_bytes = rows * kPieceBytes;
  const long long panels = batch * (cols / columns);
  const long long chunks = (rows + kChunkRows - 1) / kChunkRows;
  if (panel_bytes > (32ll << 20)) return false;                       // a panel has to stay in L2 between its visits
  if (batch * rows * cols * size < kMinBytes) return false;   // smaller tensors stay in L2 whole: the three-pass form has its second read there too
  if (panels < 4 || panels * chunks >= (1ll << 30) || panels > (1 << 24)) return false;
  if (batch * rows >= (1ll << 31) || cols >= (1ll << 31)) return false;   // TMA coordinates are 32 bits
  return true;
}

size_t panel_workspace_bytes(tq_dtype dtype, long long batch, long long rows, long long cols) {
  return panel_takes(dtype, batch, rows, cols) ? panel_layout(dtype, batch, rows, cols).total() : 0;
}

tq_status panel_normalize_launch(int kind, tq_dtype dtype, const void* in, void* out, const void* weight, const void* bias,
                                 long long batch, long long rows, long long cols, float eps, void* workspace, size_t workspace_bytes,
                                 int32_t device, cudaStream_t stream, bool* handled) {
  *handled = false;
  if (!panel_takes(dtype, batch, rows, cols)) return TQ_OK;
  if (!aligned_to(in, 16) || !aligned_to(out, 16) || (weight != nullptr && !aligned_to(weight, 16)) ||
      (bias != nullptr && !aligned_to(bias, 16))) {
    return TQ_OK;
  }
  const PanelLayout l = panel_layout(dtype, batch, rows, cols);
  TQ_REQUIRE(workspace != nullptr && workspace_bytes >= l.total() && aligned_to(workspace, 16), TQ_INVALID_ARGUMENT,
             "the panel normalisation needs %zu bytes of 16-byte-aligned scratch and was given %zu", l.total(), workspace_bytes);
  const WaitStatus status = wait_status_for(device);
  TQ_REQUIRE(status.abort != nullptr, TQ_RESOURCE_EXHAUSTED, "no device memory for the status word");

  // in[batch * rows, cols] as a two-axis map; a tile is one stage: 512 bytes of 64 consecutive rows.
  EncodeTiled encode = encode_tiled();
  TQ_REQUIRE(encode != nullptr, TQ_EXTERNAL, "the CUDA driver does not provide cuTensorMapEncodeTiled");
  const int size = dtype_size(dtype);
  CUtensorMap map;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(batch * rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * size};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(l.columns), static_cast<cuuint32_t>(kStageRows)};
  const cuuint32_t element_strides[2] = {1, 1};
  const CUtensorMapDataType type = dtype == TQ_F32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                   : dtype == TQ_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult encoded = encode(&map, type, 2, const_cast<void*>(in), dims, strides, box, element_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                  CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (encoded != CUDA_SUCCESS) return TQ_OK;   // not describable to TMA: the three-pass form takes it

  unsigned char* base = static_cast<unsigned char*>(workspace);
  PanelArgs args = {};
  args.out = out;
  args.weight = weight;
  args.bias = bias;
  args.rows = rows;
  args.cols = cols;
  args.panels_per_matrix = l.panels_per_matrix;
  args.panels = l.panels;
  args.chunk_rows = l.chunk_rows;
  args.chunks = l.chunks;
  args.lead = kLeadPanels;
  args.abreast = l.panels % kAbreast == 0 ? kAbreast : 1;
  args.policy = kPolicy;
  args.eps = eps;
  args.partials = reinterpret_cast<float2*>(base);
  args.group_partials = reinterpret_cast<float2*>(base + l.partial_bytes);
  args.stats = reinterpret_cast<float2*>(base + l.partial_bytes + l.group_bytes);
  args.group_counters = reinterpret_cast<unsigned*>(base + l.partial_bytes + l.group_bytes + l.stats_bytes);
  args.counters = args.group_counters + static_cast<size_t>(l.panels) * l.groups;
  args.ready = args.counters + l.panels;
  args.queue_s = args.ready + l.panels;
  args.queue_n = args.queue_s + 1;
  args.begun_n = args.queue_s + 2;
  args.status = status;
  TQ_CUDA(cudaMemsetAsync(args.group_counters, 0, l.flag_bytes, stream));
#define TQ_PANEL(T) (kind == 0 ? run_panels<T, 0>(map, args, device, stream) : run_panels<T, 1>(map, args, device, stream))
  tq_status s = TQ_OK;
  switch (dtype) {
    case TQ_F32: s = TQ_PANEL(float); break;
    case TQ_F16: s = TQ_PANEL(__half); break;
    default: s = TQ_PANEL(__nv_bfloat16); break;
  }
#undef TQ_PANEL
  if (s == TQ_OK) *handled = true;
  return s;
}

}  // namespace tq
