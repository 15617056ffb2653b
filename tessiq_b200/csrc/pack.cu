// Pack: gathers a strided / expanded / permuted view into a packed buffer, bit for bit.
//
// The host first drops extents of 1 and merges axes that are contiguous with one another, so the
// kernels see the smallest rank that describes the view. Then one of three kernels runs:
//   copy       the collapsed view is one contiguous run: a device-to-device copy on the stream;
//   transpose  the destination's fastest axis is strided in the source while another axis has
//              source stride 1 (a transposed or permuted view). Aligned shapes take the
//              register-block kernel (128-bit loads and stores, no shared memory); others go
//              through TILE x TILE tiles in padded shared memory. Either way both the HBM reads
//              and the HBM writes are whole sectors, and the remaining axes are unravelled once
//              per tile, not per element;
//   gather     anything else (slices, expanded axes, odd permutations): one thread per element,
//              32-bit index arithmetic when the element count allows it.
// The result is what pack_source's kernel writes (csrc/tessiq/codegen/pack.cpp:41-94): element i
// of the packed buffer is the view's element at the unravelled coordinates of i.
#include <vector>

#include "common.h"

namespace tq {
namespace {

constexpr int kMaxRank = 8;

struct View {
  int rank;
  long long sizes[kMaxRank];
  long long strides[kMaxRank];
};

template <int BYTES> struct Word;
template <> struct Word<1> { using type = uint8_t; };
template <> struct Word<2> { using type = uint16_t; };
template <> struct Word<4> { using type = uint32_t; };
template <> struct Word<8> { using type = uint2; };
template <> struct Word<16> { using type = uint4; };

template <typename W, typename Index>
__global__ void __launch_bounds__(256)
pack_gather_kernel(const W* __restrict__ src, W* __restrict__ dst, Index total, View view) {
  const Index i = static_cast<Index>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total) return;
  Index rest = i;
  long long offset = 0;
#pragma unroll
  for (int d = kMaxRank - 1; d >= 0; --d) {
    if (d < view.rank) {
      const Index extent = static_cast<Index>(view.sizes[d]);
      const Index coordinate = rest % extent;
      rest /= extent;
      offset += static_cast<long long>(coordinate) * view.strides[d];
    }
  }
  dst[i] = src[offset];
}

// Tiled transpose. The view, after collapsing, has its last axis (`cols`, destination-fastest)
// strided by `col_stride` in the source and axis `row_axis` (`rows`) with source stride 1. A tile
// covers TILE rows x TILE cols. Threads are 32 x 8; PER = TILE / 32 elements per thread per line.
template <typename W, int TILE>
__global__ void __launch_bounds__(256)
pack_transpose_kernel(const W* __restrict__ src, W* __restrict__ dst, View view, int row_axis,
                      long long row_tiles, long long col_tiles) {
  __shared__ W tile[TILE][TILE + (sizeof(W) >= 4 ? 1 : 4 / sizeof(W))];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int last = view.rank - 1;
  const long long rows = view.sizes[row_axis], cols = view.sizes[last];
  const long long col_stride = view.strides[last];

  // the grid holds fewer than 2^31 tiles: 32-bit divisions, a quarter of the instructions of 64-bit ones
  unsigned tile_id = blockIdx.x;
  const long long col_tile = tile_id % static_cast<unsigned>(col_tiles);
  tile_id /= static_cast<unsigned>(col_tiles);
  const long long row_tile = tile_id % static_cast<unsigned>(row_tiles);
  long long batch = tile_id / static_cast<unsigned>(row_tiles);

  // Unravel the batch index over the remaining axes; `dst_stride` is the packed stride.
  long long src_base = 0, dst_base = 0, dst_stride = cols, row_dst_stride = 0;
  for (int d = last - 1; d >= 0; --d) {
    if (d == row_axis) {
      row_dst_stride = dst_stride;
    } else {
      const long long coordinate = batch % view.sizes[d];
      batch /= view.sizes[d];
      src_base += coordinate * view.strides[d];
      dst_base += coordinate * dst_stride;
    }
    dst_stride *= view.sizes[d];
  }

  const long long row0 = row_tile * TILE, col0 = col_tile * TILE;
  // Read: consecutive threads walk the source-contiguous axis (rows).
  for (int c = ty; c < TILE; c += 8) {
    const long long col = col0 + c;
    if (col < cols) {
#pragma unroll
      for (int r = tx; r < TILE; r += 32) {
        const long long row = row0 + r;
        if (row < rows) tile[c][r] = src[src_base + row + col * col_stride];
      }
    }
  }
  __syncthreads();
  // Write: consecutive threads walk the destination-contiguous axis (cols).
  for (int r = ty; r < TILE; r += 8) {
    const long long row = row0 + r;
    if (row < rows) {
#pragma unroll
      for (int c = tx; c < TILE; c += 32) {
        const long long col = col0 + c;
        if (col < cols) dst[dst_base + row * row_dst_stride + col] = tile[c][r];
      }
    }
  }
}

// Register-block transpose, no shared memory. Each thread loads V vectors of V elements along the
// source-contiguous axis (a V x V block), transposes the block in registers, and stores V vectors
// along the destination-contiguous axis. A warp is 8 row-blocks x 4 column-blocks, so every load
// instruction of a warp reads 4 runs of 8 x 16 bytes and every store writes 8 runs of 4 x 16 bytes:
// whole 32-byte sectors in both directions. A CTA of 256 threads covers 16V x 16V elements.
// Needs rows, cols and every stride involved to be multiples of V and 16-byte-aligned bases.
template <typename W, int V>
__global__ void __launch_bounds__(256)
pack_transpose_blocks(const W* __restrict__ src, W* __restrict__ dst, View view, int row_axis,
                      long long row_tiles, long long col_tiles) {
  constexpr int kTile = 16 * V;
  const int last = view.rank - 1;
  const long long rows = view.sizes[row_axis], cols = view.sizes[last];
  const long long col_stride = view.strides[last];

  // the grid holds fewer than 2^31 tiles: 32-bit divisions, a quarter of the instructions of 64-bit ones
  unsigned tile_id = blockIdx.x;
  const long long col_tile = tile_id % static_cast<unsigned>(col_tiles);
  tile_id /= static_cast<unsigned>(col_tiles);
  const long long row_tile = tile_id % static_cast<unsigned>(row_tiles);
  long long batch = tile_id / static_cast<unsigned>(row_tiles);
  long long src_base = 0, dst_base = 0, dst_stride = cols, row_dst_stride = 0;
  for (int d = last - 1; d >= 0; --d) {
    if (d == row_axis) {
      row_dst_stride = dst_stride;
    } else {
      const long long coordinate = batch % view.sizes[d];
      batch /= view.sizes[d];
      src_base += coordinate * view.strides[d];
      dst_base += coordinate * dst_stride;
    }
    dst_stride *= view.sizes[d];
  }

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int tr = (lane & 7) + 8 * (warp & 1);
  const int tc = (lane >> 3) + 4 * (warp >> 1);
  const long long r0 = row_tile * kTile + tr * V, c0 = col_tile * kTile + tc * V;
  if (r0 >= rows || c0 >= cols) return;
  Vec<W, V> block[V];
#pragma unroll
  for (int i = 0; i < V; ++i) block[i] = load_stream<W, V>(src + src_base + r0 + (c0 + i) * col_stride);
#pragma unroll
  for (int j = 0; j < V; ++j) {
    Vec<W, V> line;
#pragma unroll
    for (int i = 0; i < V; ++i) line.v[i] = block[i].v[j];
    store_stream<W, V>(dst + dst_base + (r0 + j) * row_dst_stride + c0, line);
  }
}

View collapse(int rank, const int64_t* sizes, const int64_t* strides) {
  View v = {};
  for (int d = 0; d < rank; ++d) {
    if (sizes[d] == 1) continue;
    if (v.rank > 0 && v.strides[v.rank - 1] == strides[d] * sizes[d]) {
      v.sizes[v.rank - 1] *= sizes[d];
      v.strides[v.rank - 1] = strides[d];
    } else {
      v.sizes[v.rank] = sizes[d];
      v.strides[v.rank] = strides[d];
      ++v.rank;
    }
  }
  if (v.rank == 0) {
    v.rank = 1;
    v.sizes[0] = 1;
    v.strides[0] = 1;
  }
  return v;
}

template <int BYTES>
tq_status run_pack(const View& view, long long total, const void* src, void* dst, cudaStream_t stream) {
  using W = typename Word<BYTES>::type;
  const W* source = static_cast<const W*>(src);
  W* target = static_cast<W*>(dst);
  const int last = view.rank - 1;

  if (view.rank == 1 && view.strides[0] == 1) {
    const long long bytes = total * BYTES;
    if (aligned_to(src, 16) && aligned_to(dst, 16) && bytes % 16 == 0) {
      TQ_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, stream));
      return TQ_OK;
    }
  }

  if (view.strides[last] != 1 && view.strides[last] != 0) {
    int row_axis = -1;
    for (int d = last - 1; d >= 0; --d) {
      if (view.strides[d] == 1 && view.sizes[d] >= 16) {
        row_axis = d;
        break;
      }
    }
    if (row_axis >= 0 && view.sizes[last] >= 16) {
      constexpr int kV = BYTES == 1 ? 8 : 16 / BYTES;
      bool blocks_ok = aligned_to(src, 16) && aligned_to(dst, 16) && view.sizes[last] % kV == 0 &&
                       view.sizes[row_axis] % kV == 0;
      for (int d = 0; d <= last && blocks_ok; ++d) {
        if (d != row_axis && view.strides[d] % kV != 0) blocks_ok = false;
      }
      if (blocks_ok) {
        constexpr int kBlockTile = 16 * kV;
        const long long row_tiles = (view.sizes[row_axis] + kBlockTile - 1) / kBlockTile;
        const long long col_tiles = (view.sizes[last] + kBlockTile - 1) / kBlockTile;
        long long batches = 1;
        for (int d = 0; d < last; ++d) {
          if (d != row_axis) batches *= view.sizes[d];
        }
        const long long blocks = batches * row_tiles * col_tiles;
        if (blocks <= 0x7fffffffLL) {
          pack_transpose_blocks<W, kV><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
              source, target, view, row_axis, row_tiles, col_tiles);
          return check_launch("pack_transpose_blocks");
        }
      }
      constexpr int kTile = BYTES >= 4 ? 32 : (BYTES == 2 ? 64 : 128);
      const long long row_tiles = (view.sizes[row_axis] + kTile - 1) / kTile;
      const long long col_tiles = (view.sizes[last] + kTile - 1) / kTile;
      long long batches = 1;
      for (int d = 0; d < last; ++d) {
        if (d != row_axis) batches *= view.sizes[d];
      }
      const long long blocks = batches * row_tiles * col_tiles;
      if (blocks <= 0x7fffffffLL) {
        pack_transpose_kernel<W, kTile><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            source, target, view, row_axis, row_tiles, col_tiles);
        return check_launch("pack_transpose_kernel");
      }
    }
  }

  const long long blocks = (total + 255) / 256;
  TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld elements are more than the pack kernel's grid holds", total);
  if (total < 0x7fffffffLL) {
    pack_gather_kernel<W, unsigned><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        source, target, static_cast<unsigned>(total), view);
  } else {
    pack_gather_kernel<W, long long><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        source, target, total, view);
  }
  return check_launch("pack_gather_kernel");
}

// Element j of a 16-byte vector of 2-byte floats as a float: bf16 is the upper half of an f32, so an
// element is one shift or one mask of the 32-bit word that holds it.
template <int V>
__device__ __forceinline__ float half_element(const Vec<__nv_bfloat16, V>& v, int j) {
  const uint32_t word = reinterpret_cast<const uint32_t*>(&v)[j >> 1];
  return __uint_as_float((j & 1) ? (word & 0xffff0000u) : (word << 16));
}
template <int V>
__device__ __forceinline__ float half_element(const Vec<__half, V>& v, int j) { return __half2float(v.v[j]); }
template <typename T, int V>
__device__ __forceinline__ float half_element(const Vec<T, V>& v, int j) { return to_compute(v.v[j]); }

// The register-block transpose with a normalisation applied on the way: out[b][c][r] =
// f(in[b][r][c]). KIND 0: softmax over r with per-column statistics (max, 1/sum); KIND 1:
// LayerNorm over r with per-column (mean, variance) and weight/bias indexed by r. A thread loads
// RB vectors of V consecutive c (rows r0 .. r0+RB-1), and stores V vectors of RB consecutive r.
// A warp is kLanesR lanes along r by kLanesC along c, chosen so that its stores are 64-byte runs
// (kLanesR * RB elements) and its loads at least that; a CTA is 4 warps along r by 2 along c.
// RB is 4 for every type: with 8 x 8 blocks of 2-byte elements a thread held 32 registers of data
// and 16 of statistics, 63 in all, and four CTAs per SM were too few to keep the memory busy (the
// same kernel with the statistics replaced by constants, 48 registers, five CTAs: 100 us against
// 127 at [32768, 4096] bf16, and it is not the statistics' loads that cost, see below).
template <typename T, int V, int RB, int KIND>
__global__ void __launch_bounds__(256)
transpose_normalize_kernel(const T* __restrict__ in, T* __restrict__ out, const float2* __restrict__ stats,
                           const T* __restrict__ weight, const T* __restrict__ bias, long long rows, long long cols,
                           long long row_tiles, long long col_tiles, float eps) {
  constexpr int kLanesR = 64 / (RB * static_cast<int>(sizeof(T)));   // 4 (f32) or 8 (2-byte types)
  constexpr int kLanesC = 32 / kLanesR;
  constexpr int kTileRows = 4 * kLanesR * RB, kTileCols = 2 * kLanesC * V;
  static_assert(kLanesC * V == 32, "a warp's columns are one statistic per lane");
  unsigned tile_id = blockIdx.x;   // fewer than 2^31 tiles: 32-bit divisions
  const long long row_tile = tile_id % static_cast<unsigned>(row_tiles);
  tile_id /= static_cast<unsigned>(row_tiles);
  const long long col_tile = tile_id % static_cast<unsigned>(col_tiles);
  const long long batch = tile_id / static_cast<unsigned>(col_tiles);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lane_c = lane % kLanesC, lane_r = lane / kLanesC;
  const long long warp_c0 = col_tile * kTileCols + (warp & 1) * 32;
  const long long c0 = warp_c0 + lane_c * V, r0 = row_tile * kTileRows + ((warp >> 1) * kLanesR + lane_r) * RB;
  const bool active = r0 < rows && c0 < cols;
  const T* source = in + batch * rows * cols;
  T* target = out + batch * rows * cols;

  Vec<T, V> block[RB];
#pragma unroll
  for (int i = 0; i < RB; ++i) {
    if (active) {
      block[i] = load_stream<T, V>(source + (r0 + i) * cols + c0);
    } else {
#pragma unroll
      for (int e = 0; e < V; ++e) block[i].v[e] = T();
    }
  }
  // The statistics of the warp's 32 columns: one coalesced request (lane l fetches column l) and two
  // shuffles per column, instead of V requests per thread whose lanes touch separate sectors.
  float2 held = make_float2(0.f, 0.f);
  if (warp_c0 + lane < cols) held = __ldg(stats + batch * cols + warp_c0 + lane);
  if (KIND == 1) held.y = rsqrtf(held.y + eps);
  float scale[RB], shift[RB];    // per row r0 + i (LayerNorm only); r0 is a multiple of RB: one vector each
  Vec<T, RB> weights, biases;
  if (KIND == 1 && weight != nullptr && active) weights = *reinterpret_cast<const Vec<T, RB>*>(weight + r0);
  if (KIND == 1 && bias != nullptr && active) biases = *reinterpret_cast<const Vec<T, RB>*>(bias + r0);
#pragma unroll
  for (int i = 0; i < RB; ++i) {
    scale[i] = (KIND == 1 && weight != nullptr && active) ? to_compute(weights.v[i]) : 1.0f;
    shift[i] = (KIND == 1 && bias != nullptr && active) ? to_compute(biases.v[i]) : 0.0f;
  }
#pragma unroll
  for (int j = 0; j < V; ++j) {
    // column c0 + j's statistics, from the lane that fetched them (every lane takes part in the shuffles)
    const float first = __shfl_sync(0xffffffffu, held.x, lane_c * V + j);
    const float second = __shfl_sync(0xffffffffu, held.y, lane_c * V + j);
    Vec<T, RB> line;
    if constexpr (sizeof(T) == 2) {
      // Two rows at a time: with four rows per thread the kernel issues twice the instructions per
      // element it did with eight (the per-thread part is shared by half as many), and at 70 % of the
      // issue slots that showed. The two-element forms of add / mul / fma and one conversion per pair
      // of results halve the arithmetic; the values are those of the scalar expressions below.
#pragma unroll
      for (int i = 0; i < RB; i += 2) {
        const float2 x = make_float2(half_element(block[i], j), half_element(block[i + 1], j));
        const float2 centred = __fadd2_rn(x, make_float2(-first, -first));
        float2 y;
        if constexpr (KIND == 0) {
          const float2 t = __fmul2_rn(centred, make_float2(1.4426950408889634f, 1.4426950408889634f));
          float2 e;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.x) : "f"(t.x));
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e.y) : "f"(t.y));
          y = __fmul2_rn(e, make_float2(second, second));
        } else {
          y = __ffma2_rn(__fmul2_rn(centred, make_float2(second, second)), make_float2(scale[i], scale[i + 1]),
                         make_float2(shift[i], shift[i + 1]));
        }
        store_pair(&line.v[i], y);
      }
    } else {
#pragma unroll
      for (int i = 0; i < RB; ++i) {
        const float x = to_compute(block[i].v[j]);
        float y;
        if constexpr (KIND == 0) {
          float e;
          const float t = (x - first) * 1.4426950408889634f;
          asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
          y = e * second;
        } else {
          y = (x - first) * second * scale[i] + shift[i];
        }
        line.v[i] = from_compute<T, float>(y);
      }
    }
    if (active) store_stream<T, RB>(target + (c0 + j) * rows + r0, line);
  }
}

template <typename T, int KIND>
tq_status run_transpose_normalize(const void* in, void* out, const void* stats, const void* weight, const void* bias,
                                  long long batch, long long rows, long long cols, float eps, cudaStream_t stream) {
  constexpr int kV = 16 / sizeof(T);
  constexpr int kRB = 4;
  constexpr int kLanesR = 64 / (kRB * static_cast<int>(sizeof(T)));
  constexpr int kTileRows = 4 * kLanesR * kRB, kTileCols = 2 * (32 / kLanesR) * kV;
  TQ_REQUIRE(rows % kV == 0 && cols % kV == 0 && aligned_to(in, 16) && aligned_to(out, 16) && aligned_to(stats, 8) &&
                 (weight == nullptr || aligned_to(weight, 16)) && (bias == nullptr || aligned_to(bias, 16)),
             TQ_UNSUPPORTED, "the transposing normalisation needs extents that are multiples of %d and 16-byte-aligned tensors", kV);
  const long long row_tiles = (rows + kTileRows - 1) / kTileRows, col_tiles = (cols + kTileCols - 1) / kTileCols;
  const long long blocks = batch * row_tiles * col_tiles;
  TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld tiles are more than a grid holds", blocks);
  transpose_normalize_kernel<T, kV, kRB, KIND><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
      static_cast<const T*>(in), static_cast<T*>(out), static_cast<const float2*>(stats), static_cast<const T*>(weight),
      static_cast<const T*>(bias), rows, cols, row_tiles, col_tiles, eps);
  return check_launch("transpose_normalize_kernel");
}

}  // namespace

tq_status transpose_normalize_launch(int kind, tq_dtype dtype, const void* in, void* out, const void* stats, const void* weight,
                                     const void* bias, long long batch, long long rows, long long cols, float eps, cudaStream_t stream) {
#define TQ_TN(T)                                                                                                    \
  return kind == 0 ? run_transpose_normalize<T, 0>(in, out, stats, weight, bias, batch, rows, cols, eps, stream)      \
                   : run_transpose_normalize<T, 1>(in, out, stats, weight, bias, batch, rows, cols, eps, stream)
  switch (dtype) {
    case TQ_F32: TQ_TN(float);
    case TQ_F16: TQ_TN(__half);
    case TQ_BF16: TQ_TN(__nv_bfloat16);
    default: return fail(TQ_UNSUPPORTED, "the transposing normalisation has no kernel for element type %s", dtype_name(dtype));
  }
#undef TQ_TN
}

}  // namespace tq

extern "C" tq_status tq_pack_launch(int32_t element_bytes, int32_t rank, const int64_t* sizes,
                                    const int64_t* strides, const void* src, void* dst,
                                    int32_t device, void* stream) {
  if (tq::recording()) {
    TQ_REQUIRE(rank >= 0 && rank <= tq::kMaxRank && (rank == 0 || (sizes != nullptr && strides != nullptr)), TQ_INVALID_ARGUMENT,
               "a pack of rank %d cannot be recorded", rank);
    std::vector<int64_t> kept_sizes(sizes, sizes + rank), kept_strides(strides, strides + rank);
    return tq::record([=](int32_t d, void* s) {
      return tq_pack_launch(element_bytes, rank, kept_sizes.data(), kept_strides.data(), src, dst, d, s);
    });
  }
  TQ_REQUIRE(rank >= 0, TQ_INVALID_ARGUMENT, "negative rank %d", rank);
  TQ_REQUIRE(rank <= tq::kMaxRank, TQ_UNSUPPORTED, "the pack kernel takes up to %d axes, not %d", tq::kMaxRank, rank);
  TQ_REQUIRE(rank == 0 || (sizes != nullptr && strides != nullptr), TQ_INVALID_ARGUMENT, "null sizes or strides");
  long long total = 1;
  for (int d = 0; d < rank; ++d) {
    TQ_REQUIRE(sizes[d] >= 0, TQ_INVALID_ARGUMENT, "negative extent %lld on axis %d", (long long)sizes[d], d);
    TQ_REQUIRE(strides[d] >= 0, TQ_UNSUPPORTED, "negative stride %lld on axis %d has no kernel", (long long)strides[d], d);
    total *= sizes[d];
  }
  if (total == 0) return TQ_OK;
  TQ_REQUIRE(src != nullptr && dst != nullptr, TQ_INVALID_ARGUMENT, "null source or destination");
  TQ_REQUIRE(element_bytes == 1 || element_bytes == 2 || element_bytes == 4 || element_bytes == 8 || element_bytes == 16,
             TQ_UNSUPPORTED, "elements of %d bytes have no pack kernel", element_bytes);
  TQ_REQUIRE(tq::aligned_to(src, element_bytes) && tq::aligned_to(dst, element_bytes), TQ_INVALID_ARGUMENT,
             "pointers must be aligned to the element width");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  const tq::View view = tq::collapse(rank, sizes, strides);
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
  switch (element_bytes) {
    case 1: return tq::run_pack<1>(view, total, src, dst, cuda_stream);
    case 2: return tq::run_pack<2>(view, total, src, dst, cuda_stream);
    case 4: return tq::run_pack<4>(view, total, src, dst, cuda_stream);
    case 8: return tq::run_pack<8>(view, total, src, dst, cuda_stream);
    default: return tq::run_pack<16>(view, total, src, dst, cuda_stream);
  }
}
