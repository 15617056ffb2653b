/* TEST INFRASTRUCTURE — a plain-C restatement of the arithmetic on tessiq's GPU hot path.
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs may load this file's
 * library. Nothing under tessiq_b200/ links, loads or calls it.
 *
 * Each function restates, as a sequential host loop, what one of the reference's kernels computes,
 * from the reference's own kernel sources (cited per function). It is checked against PyTorch's CPU
 * kernels — which is what the reference's CPU device tessiq:0 runs (see oracle/tessiq0.py) — and
 * against the golden vectors under tests/golden/. Sums are accumulated in double so that the
 * restatement can serve as the "float64 ground truth" the reference's own reduction tests compare
 * against (tests/python/test_eager.py:517-537).
 *
 * Build: make -C oracle      (gcc -O2 -shared -fPIC -o liboracle.so restate.c -lm)
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TQ_EXPORT __attribute__((visibility("default")))

/* ---- bf16 storage ----------------------------------------------------------------------- */

static float bf16_to_float(uint16_t bits) {
  uint32_t word = (uint32_t)bits << 16;
  float value;
  memcpy(&value, &word, sizeof(value));
  return value;
}

/* Round to nearest even, NaN kept quiet: what c10::BFloat16(float) does. */
static uint16_t float_to_bf16(float value) {
  uint32_t word;
  memcpy(&word, &value, sizeof(word));
  if (value != value) return 0x7fc0;
  word += 0x7fffu + ((word >> 16) & 1u);
  return (uint16_t)(word >> 16);
}

TQ_EXPORT void tq_oracle_bf16_to_f32(const uint16_t* in, float* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = bf16_to_float(in[i]);
}
TQ_EXPORT void tq_oracle_f32_to_bf16(const float* in, uint16_t* out, int64_t n) {
  for (int64_t i = 0; i < n; ++i) out[i] = float_to_bf16(in[i]);
}

/* ---- elementwise expressions (ops.toml) --------------------------------------------------- */

/* ops.toml's `expression` rows with scalar_t = float; gelu_tanh is torch's
 * 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))) (aten gelu, approximate="tanh"). */
static float unary_f32(int op, float x) {
  switch (op) {
    case 0: return fabsf(x);
    case 1: return -x;
    case 2: return x < 0.0f ? 0.0f : x;                       /* relu: keeps NaN and -0.0 */
    case 3: return 1.0f / (1.0f + expf(-x));                  /* sigmoid */
    case 4: return sqrtf(x);
    case 5: return tanhf(x);
    case 6: return expf(x);
    case 7: return expm1f(x);
    case 8: return logf(x);
    case 9: return log1pf(x);
    case 10: return log2f(x);
    case 11: return log10f(x);
    case 12: return 1.0f / sqrtf(x);                          /* rsqrt */
    case 13: return 1.0f / x;                                 /* reciprocal */
    case 14: return sinf(x);
    case 15: return cosf(x);
    case 16: return tanf(x);
    case 17: return asinf(x);
    case 18: return acosf(x);
    case 19: return atanf(x);
    case 20: return sinhf(x);
    case 21: return coshf(x);
    case 22: return floorf(x);
    case 23: return ceilf(x);
    case 24: return truncf(x);
    case 25: return rintf(x);                                 /* round: half to even */
    case 26: return erff(x);
    case 27: return erfcf(x);
    case 28: return 0.5f * x * (1.0f + erff(x * 0.70710678118654752440f)); /* gelu */
    case 29: {                                                /* gelu_tanh */
      const float inner = 0.7978845608028654f * (x + 0.044715f * x * x * x);
      return 0.5f * x * (1.0f + tanhf(inner));
    }
    case 30: return x / (1.0f + expf(-x));                    /* silu */
    case 31: return x * (1.0f / (1.0f + expf(-1.702f * x)));  /* fast_gelu.cpp:23 */
    default: return NAN;
  }
}

/* Index = position in this list; oracle/restate.py holds the same order. */
TQ_EXPORT int tq_oracle_unary_f32(int op, const float* x, float* y, int64_t n) {
  if (op < 0 || op > 31) return 1;
  for (int64_t i = 0; i < n; ++i) y[i] = unary_f32(op, x[i]);
  return 0;
}

/* benchmark config 1, one element at a time, in float: gelu_tanh(x + b) * sigmoid(x) - 0.5 x with
 * b read as i % cols (the cycled read of csrc/tessiq/codegen/kernel.cpp:168-206). */
TQ_EXPORT void tq_oracle_chain_gelu_sigmoid_f32(const float* x, const float* b, float* y,
                                                int64_t n, int64_t cols) {
  for (int64_t i = 0; i < n; ++i) {
    const float t0 = x[i] + b[i % cols];
    const float t1 = unary_f32(29, t0);
    const float t2 = unary_f32(3, x[i]);
    y[i] = t1 * t2 - x[i] * 0.5f;
  }
}

/* benchmark config 5: t = tanh(exp(a + b) * b); y = a > 0 ? t : a, in float (the caller rounds). */
TQ_EXPORT void tq_oracle_chain_six_ops_f32(const float* a, const float* b, float* y, int64_t n) {
  for (int64_t i = 0; i < n; ++i) {
    const float t = tanhf(expf(a[i] + b[i]) * b[i]);
    y[i] = a[i] > 0.0f ? t : a[i];
  }
}

/* ---- reductions over [outer, reduce, inner] (cuda_emitter.cpp:159-210) ------------------ */

/* op: 0 sum, 1 mean, 2 amax, 3 amin. The sum is carried in double. amax/amin propagate NaN
 * (cuda_emitter.cpp:52-65) and start from the slice's first element (:44-46). */
TQ_EXPORT void tq_oracle_reduce_f32(int op, const float* in, double* out, int64_t outer,
                                    int64_t reduce, int64_t inner) {
  for (int64_t o = 0; o < outer; ++o) {
    for (int64_t i = 0; i < inner; ++i) {
      const float* base = in + o * reduce * inner + i;
      double acc = base[0];
      for (int64_t r = 1; r < reduce; ++r) {
        const double v = base[r * inner];
        if (op <= 1) {
          acc += v;
        } else if (acc != acc) {
          /* stays NaN */
        } else if (v != v) {
          acc = v;
        } else if (op == 2 ? v > acc : v < acc) {
          acc = v;
        }
      }
      if (op == 1) acc /= (double)reduce;
      out[o * inner + i] = acc;
    }
  }
}

/* argmax: first index of the maximum, NaN counts as the maximum (aten.argmax on tessiq:0). */
TQ_EXPORT void tq_oracle_argmax_f32(const float* in, int64_t* out, int64_t outer, int64_t reduce,
                                    int64_t inner) {
  for (int64_t o = 0; o < outer; ++o) {
    for (int64_t i = 0; i < inner; ++i) {
      const float* base = in + o * reduce * inner + i;
      int64_t best = 0;
      float best_value = base[0];
      for (int64_t r = 1; r < reduce; ++r) {
        const float v = base[r * inner];
        if (best_value != best_value) break; /* the first NaN wins */
        if (v != v || v > best_value) {
          best = r;
          best_value = v;
        }
      }
      out[o * inner + i] = best;
    }
  }
}

/* Exact integer reductions (tests/python/test_eager.py:543-560): op 0 sum (wraps), 2 amax, 3 amin. */
TQ_EXPORT void tq_oracle_reduce_i64(int op, const int64_t* in, int64_t* out, int64_t outer,
                                    int64_t reduce, int64_t inner) {
  for (int64_t o = 0; o < outer; ++o) {
    for (int64_t i = 0; i < inner; ++i) {
      const int64_t* base = in + o * reduce * inner + i;
      uint64_t sum = (uint64_t)base[0];
      int64_t extreme = base[0];
      for (int64_t r = 1; r < reduce; ++r) {
        const int64_t v = base[r * inner];
        sum += (uint64_t)v;
        if (op == 2 ? v > extreme : v < extreme) extreme = v;
      }
      out[o * inner + i] = op == 0 ? (int64_t)sum : extreme;
    }
  }
}

/* ---- softmax over [outer, extent, inner] (csrc/custom_ops/softmax/softmax.cu:19-61) ------ */
/* Three passes: maximum, sum of exp(x - max), scale. The maximum here propagates NaN, as
 * aten::_softmax does on tessiq:0 (the reference's own kernel uses fmaxf and drops it). */
TQ_EXPORT void tq_oracle_softmax_f32(const float* in, float* out, int64_t outer, int64_t extent,
                                     int64_t inner) {
  for (int64_t o = 0; o < outer; ++o) {
    for (int64_t i = 0; i < inner; ++i) {
      const float* base = in + o * extent * inner + i;
      float* target = out + o * extent * inner + i;
      float maximum = base[0];
      for (int64_t r = 1; r < extent; ++r) {
        const float v = base[r * inner];
        if (maximum != maximum) break;
        if (v != v || v > maximum) maximum = v;
      }
      double sum = 0.0;
      for (int64_t r = 0; r < extent; ++r) sum += (double)expf(base[r * inner] - maximum);
      for (int64_t r = 0; r < extent; ++r) {
        target[r * inner] = (float)((double)expf(base[r * inner] - maximum) / sum);
      }
    }
  }
}

/* ---- LayerNorm (csrc/tessiq/codegen/norm.cpp:54-63,97-135) ------------------------------- */
/* Two passes: mean, then the centred sum of squares; rstd = 1/sqrt(var + eps);
 * y = (x - mean) * rstd * w + b; null weight/bias are skipped. Statistics in double. */
TQ_EXPORT void tq_oracle_layer_norm_f32(const float* in, const float* weight, const float* bias,
                                        float* out, float* mean_out, float* rstd_out, int64_t rows,
                                        int64_t width, double eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* x = in + r * width;
    double sum = 0.0;
    for (int64_t i = 0; i < width; ++i) sum += x[i];
    const double mean = sum / (double)width;
    double squares = 0.0;
    for (int64_t i = 0; i < width; ++i) squares += (x[i] - mean) * (x[i] - mean);
    const double rstd = 1.0 / sqrt(squares / (double)width + eps);
    if (mean_out) mean_out[r] = (float)mean;
    if (rstd_out) rstd_out[r] = (float)rstd;
    for (int64_t i = 0; i < width; ++i) {
      double y = (x[i] - mean) * rstd;
      if (weight) y *= weight[i];
      if (bias) y += bias[i];
      out[r * width + i] = (float)y;
    }
  }
}

/* RMSNorm (csrc/custom_ops/rms_norm/rms_norm.cu:15-42). */
TQ_EXPORT void tq_oracle_rms_norm_f32(const float* in, const float* weight, float* out,
                                      int64_t rows, int64_t width, double eps) {
  for (int64_t r = 0; r < rows; ++r) {
    const float* x = in + r * width;
    double squares = 0.0;
    for (int64_t i = 0; i < width; ++i) squares += (double)x[i] * x[i];
    const double scale = 1.0 / sqrt(squares / (double)width + eps);
    for (int64_t i = 0; i < width; ++i) out[r * width + i] = (float)(x[i] * scale * (weight ? weight[i] : 1.0f));
  }
}

/* Eval BatchNorm over [n, c, inner] (csrc/tessiq/codegen/norm.cpp:141-155):
 * alpha = w / sqrt(var + eps), beta = b - mean * alpha, y = x * alpha + beta, in float. */
TQ_EXPORT void tq_oracle_batch_norm_eval_f32(const float* in, const float* weight,
                                             const float* bias, const float* mean,
                                             const float* var, float* out, int64_t n, int64_t c,
                                             int64_t inner, double eps) {
  for (int64_t plane = 0; plane < n * c; ++plane) {
    const int64_t channel = plane % c;
    const float alpha = (weight ? weight[channel] : 1.0f) / sqrtf(var[channel] + (float)eps);
    const float beta = (bias ? bias[channel] : 0.0f) - mean[channel] * alpha;
    for (int64_t i = 0; i < inner; ++i) out[plane * inner + i] = in[plane * inner + i] * alpha + beta;
  }
}

/* ---- pack (csrc/tessiq/codegen/pack.cpp:41-94) ------------------------------------------- */
/* Element i of the packed result is the view's element at the coordinates i unravels to. */
TQ_EXPORT int tq_oracle_pack(int element_bytes, int rank, const int64_t* sizes,
                             const int64_t* strides, const void* src, void* dst) {
  if (rank < 0 || rank > 8) return 1;
  int64_t total = 1;
  for (int d = 0; d < rank; ++d) total *= sizes[d];
  for (int64_t i = 0; i < total; ++i) {
    int64_t rest = i, offset = 0;
    for (int d = rank - 1; d >= 0; --d) {
      offset += (rest % sizes[d]) * strides[d];
      rest /= sizes[d];
    }
    memcpy((char*)dst + i * element_bytes, (const char*)src + offset * element_bytes,
           (size_t)element_bytes);
  }
  return 0;
}

/* ---- GEMM + bias + GELU -------------------------------------------------------------------- */
/* act(A[m,k] @ B + bias[n]) in double; B is [k,n] (trans_b = 0) or [n,k] (trans_b = 1, the
 * nn.Linear layout of csrc/custom_ops/gemm_bias_gelu_tanh/gemm_bias_gelu_tanh.cpp:20-23).
 * act: 0 none, 1 gelu (erf), 2 gelu (tanh). The float64 ground truth of
 * tests/python/test_gemm_bias_gelu_tanh.py:61-67. */
TQ_EXPORT void tq_oracle_gemm_bias_act_f64(const double* a, const double* b, const double* bias,
                                           double* c, int64_t m, int64_t n, int64_t k, int trans_b,
                                           int act) {
  for (int64_t i = 0; i < m; ++i) {
    for (int64_t j = 0; j < n; ++j) {
      double acc = 0.0;
      for (int64_t p = 0; p < k; ++p) acc += a[i * k + p] * (trans_b ? b[j * k + p] : b[p * n + j]);
      if (bias) acc += bias[j];
      if (act == 1) {
        acc = 0.5 * acc * (1.0 + erf(acc * 0.70710678118654752440));
      } else if (act == 2) {
        const double inner = 0.7978845608028654 * (acc + 0.044715 * acc * acc * acc);
        acc = 0.5 * acc * (1.0 + tanh(inner));
      }
      c[i * n + j] = acc;
    }
  }
}

/* ---- attention ------------------------------------------------------------------------------ */
/* out[i,:] = sum_j softmax_j(scale * q[i,:] . k[j,:]) v[j,:] for ONE head in double, keys j <= i
 * only when causal. This is the mathematical value of the node sequence the reference runs for
 * tests/python/test_models.py:64-67 — bmm (csrc/tessiq/codegen/gemm.cpp:100-175), the scaling,
 * an optional lower-triangular mask, softmax over the last axis with the row maximum subtracted
 * (csrc/custom_ops/softmax/softmax.cu:19-61), bmm — without the roundings between the nodes. */
TQ_EXPORT void tq_oracle_attention_f64(const double* q, const double* k, const double* v, double* out,
                                       int64_t q_tokens, int64_t k_tokens, int64_t width, double scale,
                                       int causal) {
  double* scores = (double*)malloc(sizeof(double) * (size_t)(k_tokens > 0 ? k_tokens : 1));
  for (int64_t i = 0; i < q_tokens; ++i) {
    const int64_t keys = causal ? (i + 1 < k_tokens ? i + 1 : k_tokens) : k_tokens;
    double top = -INFINITY;
    for (int64_t j = 0; j < keys; ++j) {
      double dot = 0.0;
      for (int64_t d = 0; d < width; ++d) dot += q[i * width + d] * k[j * width + d];
      scores[j] = dot * scale;
      if (scores[j] > top) top = scores[j];
    }
    double total = 0.0;
    for (int64_t j = 0; j < keys; ++j) {
      scores[j] = exp(scores[j] - top);
      total += scores[j];
    }
    for (int64_t d = 0; d < width; ++d) {
      double acc = 0.0;
      for (int64_t j = 0; j < keys; ++j) acc += scores[j] * v[j * width + d];
      out[i * width + d] = acc / total;
    }
  }
  free(scores);
}
