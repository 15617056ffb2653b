// Eval-mode BatchNorm over a packed [n, c, inner] tensor: y = x * alpha + beta with
// alpha = weight / sqrt(var + eps) and beta = bias - mean * alpha per channel
// (csrc/tessiq/codegen/norm.cpp:137-199). Two kernels, as in the reference
// (csrc/tessiq/torch/eager_norm.cpp:136-199): by plane when a plane is long enough to give a CTA
// work (no index division at all), by element otherwise.
#include "common.h"

namespace tq {
namespace {

template <typename T, typename P>
__device__ __forceinline__ void channel_terms(const P* weight, const P* bias, const P* mean,
                                              const P* var, long long channel, float eps,
                                              typename Compute<T>::type& alpha,
                                              typename Compute<T>::type& beta) {
  using C = typename Compute<T>::type;
  const C w = weight ? static_cast<C>(to_compute(weight[channel])) : C(1);
  const C b = bias ? static_cast<C>(to_compute(bias[channel])) : C(0);
  const C m = static_cast<C>(to_compute(mean[channel]));
  const C v = static_cast<C>(to_compute(var[channel]));
  alpha = w / sqrt(v + static_cast<C>(eps));
  beta = b - m * alpha;
}

// grid = (chunks, planes); a plane is `inner` contiguous elements of one (n, c).
template <typename T, typename P, int VEC>
__global__ void __launch_bounds__(256)
batch_norm_by_plane(const T* __restrict__ in, T* __restrict__ out, const P* __restrict__ weight,
                    const P* __restrict__ bias, const P* __restrict__ mean,
                    const P* __restrict__ var, long long channels, long long inner, float eps) {
  using C = typename Compute<T>::type;
  const long long plane = blockIdx.y;
  C alpha, beta;
  channel_terms<T, P>(weight, bias, mean, var, plane % channels, eps, alpha, beta);
  const T* source = in + plane * inner;
  T* target = out + plane * inner;
  const long long vectors = inner / VEC;
  for (long long v = static_cast<long long>(blockIdx.x) * 256 + threadIdx.x; v < vectors;
       v += static_cast<long long>(gridDim.x) * 256) {
    Vec<T, VEC> x = load_stream<T, VEC>(source + v * VEC);
    Vec<T, VEC> y;
#pragma unroll
    for (int e = 0; e < VEC; ++e) y.v[e] = from_compute<T, C>(to_compute(x.v[e]) * alpha + beta);
    store_stream<T, VEC>(target + v * VEC, y);
  }
}

template <typename T, typename P, typename Index>
__global__ void __launch_bounds__(256)
batch_norm_by_element(const T* __restrict__ in, T* __restrict__ out, const P* __restrict__ weight,
                      const P* __restrict__ bias, const P* __restrict__ mean,
                      const P* __restrict__ var, Index total, Index channels, Index inner, float eps) {
  using C = typename Compute<T>::type;
  const Index i = static_cast<Index>(blockIdx.x) * 256 + threadIdx.x;
  if (i >= total) return;
  C alpha, beta;
  channel_terms<T, P>(weight, bias, mean, var, (i / inner) % channels, eps, alpha, beta);
  out[i] = from_compute<T, C>(to_compute(in[i]) * alpha + beta);
}

template <typename T, typename P>
tq_status run(const void* in, const void* weight, const void* bias, const void* mean, const void* var,
              void* out, long long n, long long c, long long inner, double eps, cudaStream_t stream) {
  const T* source = static_cast<const T*>(in);
  T* target = static_cast<T*>(out);
  const P* w = static_cast<const P*>(weight);
  const P* b = static_cast<const P*>(bias);
  const P* m = static_cast<const P*>(mean);
  const P* v = static_cast<const P*>(var);
  const long long planes = n * c, total = planes * inner;
  constexpr int kVec = 16 / sizeof(T);
  if (inner >= 1024 && planes <= 65535 && inner % kVec == 0 && aligned_to(in, 16) && aligned_to(out, 16)) {
    long long chunks = (inner / kVec + 255) / 256;
    if (chunks > 64) chunks = 64;
    dim3 grid(static_cast<unsigned>(chunks), static_cast<unsigned>(planes));
    batch_norm_by_plane<T, P, kVec><<<grid, 256, 0, stream>>>(source, target, w, b, m, v, c, inner,
                                                                static_cast<float>(eps));
    return check_launch("batch_norm_by_plane");
  }
  const long long blocks = (total + 255) / 256;
  TQ_REQUIRE(blocks <= 0x7fffffffLL, TQ_UNSUPPORTED, "%lld elements are more than a grid holds", total);
  if (total < 0x7fffffffLL) {
    batch_norm_by_element<T, P, unsigned><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        source, target, w, b, m, v, static_cast<unsigned>(total), static_cast<unsigned>(c),
        static_cast<unsigned>(inner), static_cast<float>(eps));
  } else {
    batch_norm_by_element<T, P, long long><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
        source, target, w, b, m, v, total, c, inner, static_cast<float>(eps));
  }
  return check_launch("batch_norm_by_element");
}

}  // namespace
}  // namespace tq

extern "C" tq_status tq_batch_norm_eval_launch(tq_dtype dtype, tq_dtype param_dtype, const void* in,
                                               const void* weight, const void* bias,
                                               const void* running_mean, const void* running_var,
                                               void* out, int64_t n, int64_t c, int64_t inner,
                                               double eps, int32_t device, void* stream) {
  TQ_RECORD_OR_RUN([=](int32_t d, void* s) {
    return tq_batch_norm_eval_launch(dtype, param_dtype, in, weight, bias, running_mean, running_var, out, n, c, inner, eps, d, s);
  });
  TQ_REQUIRE(n >= 0 && c >= 0 && inner >= 0, TQ_INVALID_ARGUMENT, "negative extent in [%lld, %lld, %lld]",
             (long long)n, (long long)c, (long long)inner);
  if (n == 0 || c == 0 || inner == 0) return TQ_OK;
  TQ_REQUIRE(in != nullptr && out != nullptr, TQ_INVALID_ARGUMENT, "null input or output");
  TQ_REQUIRE(running_mean != nullptr && running_var != nullptr, TQ_UNSUPPORTED,
             "eval BatchNorm without running statistics has no kernel");
  tq::DeviceScope device_scope(device);
  if (tq_status s = device_scope.status()) return s;
  cudaStream_t cuda_stream = static_cast<cudaStream_t>(stream);
#define TQ_BN(T, P) return tq::run<T, P>(in, weight, bias, running_mean, running_var, out, n, c, inner, eps, cuda_stream)
  if (dtype == TQ_F32 && param_dtype == TQ_F32) TQ_BN(float, float);
  if (dtype == TQ_F64 && param_dtype == TQ_F64) TQ_BN(double, double);
  if (dtype == TQ_BF16 && param_dtype == TQ_BF16) TQ_BN(__nv_bfloat16, __nv_bfloat16);
  if (dtype == TQ_BF16 && param_dtype == TQ_F32) TQ_BN(__nv_bfloat16, float);
  if (dtype == TQ_F16 && param_dtype == TQ_F16) TQ_BN(__half, __half);
  if (dtype == TQ_F16 && param_dtype == TQ_F32) TQ_BN(__half, float);
#undef TQ_BN
  return tq::fail(TQ_UNSUPPORTED, "eval BatchNorm has no kernel for %s data with %s parameters",
                  tq::dtype_name(dtype), tq::dtype_name(param_dtype));
}
