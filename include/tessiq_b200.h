/* tessiq_b200 — C ABI of the B200 (sm_100a) kernel layer for tessiq's data-parallel hot path.
 *
 * Every entry point is `extern "C"`, takes plain pointers and sizes, returns a `tq_status`, and
 * leaves a human-readable reason in a thread-local slot read with `tq_last_error()`. Nothing here
 * names a torch type. Unless an entry point says otherwise:
 *
 *   - every data pointer is DEVICE memory on CUDA device `device` (the CUDA ordinal, i.e. the
 *     reference's `tessiq:k` is ordinal k-1);
 *   - `stream` is a raw `cudaStream_t` (0 = the legacy default stream); launches are asynchronous
 *     and the caller orders readers of the result through that stream, exactly like
 *     `Kernel::launch(tensors, out, stream)` in the reference (csrc/tessiq/torch/kernel.h:59-66);
 *   - a zero-element problem launches nothing and returns TQ_OK
 *     (csrc/tessiq/torch/fused.cpp:157-160, csrc/tessiq/torch/pack.cpp:93-96);
 *   - TQ_UNSUPPORTED means "decline": the arguments are well formed but there is no kernel for
 *     them; the reference's caller then runs its own fallback (csrc/tessiq/support/error.h:17-18).
 *     This library never computes anything on the host.
 *
 * Status codes map one to one onto the reference's `ErrorCode` (csrc/tessiq/support/error.h:14-27)
 * so a binding keeps the reference's exception mapping (csrc/bindings/module.cpp:75-92).
 */
#ifndef TESSIQ_B200_H_
#define TESSIQ_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t tq_status;
enum {
  TQ_OK = 0,
  TQ_INVALID_ARGUMENT = 1,   /* ErrorCode::kInvalidArgument   -> ValueError   */
  TQ_UNSUPPORTED = 2,        /* ErrorCode::kUnsupported       -> TypeError (decline) */
  TQ_NOT_FOUND = 3,          /* ErrorCode::kNotFound          -> KeyError     */
  TQ_RESOURCE_EXHAUSTED = 4, /* ErrorCode::kResourceExhausted -> MemoryError  */
  TQ_EXTERNAL = 5,           /* ErrorCode::kExternal          -> RuntimeError */
  TQ_INTERNAL = 6            /* ErrorCode::kInternal          -> RuntimeError */
};

/* Element types. The numbering is this library's own; the reference's are ir::DType
 * (csrc/tessiq/ir/types.h:18-26) and codegen::ElementType (csrc/tessiq/codegen/precompiled.h:36-47). */
typedef int32_t tq_dtype;
enum {
  TQ_F32 = 0,
  TQ_F64 = 1,
  TQ_F16 = 2,
  TQ_BF16 = 3,
  TQ_I32 = 4,
  TQ_I64 = 5,
  TQ_BOOL = 6 /* one byte, 0 or 1 */
};

/* ------------------------------------------------------------------------------------------ */
/* Library                                                                                      */

/* ABI version of this header: major*1000 + minor. */
int32_t tq_abi_version(void);

/* The reason for the calling thread's most recent non-OK status. Never null; valid until the
 * thread's next failing call. Replaces Error::message() (csrc/tessiq/support/error.h:37). */
const char* tq_last_error(void);

/* Bytes per element of `dtype`, or 0 for an unknown code. */
int32_t tq_dtype_size(tq_dtype dtype);

/* Number of CUDA devices visible (0 without a driver; never an error).
 * Replaces the CUDA half of registry device discovery (csrc/tessiq/runtime/registry.cpp:25-67). */
int32_t tq_device_count(void);

/* ------------------------------------------------------------------------------------------ */
/* Runtime: per-GPU streams and a per-GPU arena                                                 */
/* Replaces CudaDevice's single blocking copy stream and legacy-stream launches                 */
/* (csrc/tessiq/runtime/cuda_device.cpp:34-147) and the stubbed getStream/recordStream          */
/* (csrc/tessiq/torch/backend.cpp:165-168,357-363).                                             */

/* Creates a non-blocking stream on `device`. */
tq_status tq_stream_create(int32_t device, void** stream);
tq_status tq_stream_destroy(int32_t device, void* stream);
tq_status tq_stream_synchronize(int32_t device, void* stream);

/* A bump arena: one cudaMalloc of `bytes` on `device`, carved by offset. This is the device side
 * of the reference's arena memory plan (csrc/tessiq/ir/recipe.cpp:56, which the reference's
 * executor never used). `tq_arena_at` returns base+offset after a bounds check. */
typedef struct tq_arena tq_arena;
tq_status tq_arena_create(int32_t device, size_t bytes, tq_arena** arena);
tq_status tq_arena_destroy(tq_arena* arena);
tq_status tq_arena_at(const tq_arena* arena, size_t offset, size_t bytes, void** pointer);
size_t tq_arena_bytes(const tq_arena* arena);

/* ------------------------------------------------------------------------------------------ */
/* Fused elementwise chains                                                                     */
/* Replaces CudaEmitter::emit(FusedKernel) + compile_cached + load_program                      */
/* (csrc/tessiq/codegen/cuda_emitter.cpp:212-255, csrc/tessiq/torch/fused.cpp:470-527) and      */
/* FusedKernel::launch (csrc/tessiq/torch/fused.cpp:127-194); also the eager one-op kernels of  */
/* run_elementwise (csrc/tessiq/torch/eager.cpp:461-493,546-624).                                */

/* One compiled fusion group. `program` is a text description, one statement per line:
 *
 *     math fast|precise                      optional; default fast (see tq_fused_create)
 *     in <name> <dtype> same|repeated|cycled|strided
 *     scalar <name> <dtype>                  a by-value argument, given at launch as a double
 *     <name> = <op> <arg> [<arg> [<arg>]]    arg: a value name or a numeric literal
 *     <name> = cast <arg> <dtype>
 *     out <name> <dtype>
 *
 * dtypes: f32 f64 f16 bf16 i32 i64 bool. `same` reads element i, `repeated` reads i / d (one
 * operand element per run of d outputs, e.g. an [N,1] column), `cycled` reads i % d (e.g. a bias
 * row), `strided` maps i through sizes/strides given at launch — the four kinds of
 * OperandRead (csrc/tessiq/codegen/kernel.h:33-66, csrc/tessiq/codegen/kernel.cpp:210-244).
 * Ops are the reference's ops.toml elementwise names (abs add div mul neg relu sigmoid sqrt sub
 * tanh exp expm1 log log1p log2 log10 pow rsqrt reciprocal sin cos tan asin acos atan sinh cosh
 * floor ceil trunc round erf erfc gelu) plus gelu_tanh silu fast_gelu swiglu maximum minimum
 * gt ge lt le eq ne logical_and logical_or logical_not bitwise_not where cast.
 * f16/bf16 values are computed in f32 registers and rounded once, at the store or at a cast.
 *
 * `math fast` selects hardware-approximation sequences whose relative error is bounded by 4e-6
 * for f32; `math precise` selects the CUDA math library's functions, as the reference's NVRTC
 * kernels do. f64 is always precise.
 *
 * Errors: TQ_INVALID_ARGUMENT for a malformed program, TQ_UNSUPPORTED for an op/dtype pair with no
 * kernel (ints outside add sub mul neg relu abs maximum minimum compare where cast,
 * csrc/tessiq/torch/eager.cpp:66-69), TQ_EXTERNAL if NVRTC fails. */
typedef struct tq_fused tq_fused;
tq_status tq_fused_create(const char* program, tq_fused** kernel);
tq_status tq_fused_destroy(tq_fused* kernel);

/* Compiled kernels are kept on disk between processes, keyed by FNV-1a of (source, sm_100a, NVRTC
 * version), under $TESSIQ_CACHE_DIR (default ~/.cache/tessiq_b200; empty string disables) — the
 * reference's cubin cache (csrc/tessiq/codegen/cubin_cache.cpp:43-64,127-168). A cache that cannot
 * be read or written is ignored. Counters since the library was loaded; any pointer may be null. */
tq_status tq_cubin_cache_stats(int64_t* hits, int64_t* misses, int64_t* stores);

/* The CUDA source the selector instantiated (for tests and reports). Copies at most `capacity`
 * bytes including the terminator; returns the full length in `*length` when non-null. */
tq_status tq_fused_source(const tq_fused* kernel, char* buffer, size_t capacity, size_t* length);

/* Layout of one strided operand: rank <= 8, sizes of the OUTPUT, strides of the operand in
 * elements (0 for a broadcast axis). Negative strides are refused (kernel.cpp:84-88). */
typedef struct tq_layout {
  int32_t rank;
  int64_t sizes[8];
  int64_t strides[8];
} tq_layout;

/* Runs the group over `elements` outputs.
 *   inputs[k]    device pointer of the k-th `in`, in program order
 *   divisors[j]  the divisor of the j-th repeated/cycled `in`, in program order
 *   layouts[j]   the layout of the j-th strided `in`, in program order (may be null if none)
 *   scalars[j]   the j-th `scalar`, as a double (converted the way torch converts scalars,
 *                csrc/tessiq/torch/eager.cpp:533-544)
 * Pointers may have any alignment that suits their element type: 16-byte-aligned operands take
 * the 128-bit path, others a narrower one. */
tq_status tq_fused_launch(const tq_fused* kernel,
                          const void* const* inputs,
                          void* out,
                          int64_t elements,
                          const int64_t* divisors,
                          const tq_layout* layouts,
                          const double* scalars,
                          int32_t device,
                          void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Reductions                                                                                   */
/* Replaces CudaEmitter::emit(ReductionKernel) (csrc/tessiq/codegen/cuda_emitter.cpp:159-210),   */
/* ReductionKernel::launch (csrc/tessiq/torch/fused.cpp:212-285) and the eager two-pass          */
/* reduce() (csrc/tessiq/torch/eager_reduction.cpp:163-255).                                     */

typedef int32_t tq_reduce_op;
enum {
  TQ_SUM = 0,
  TQ_MEAN = 1, /* sum / (T)reduce after the sum (cuda_emitter.cpp:166) */
  TQ_AMAX = 2, /* NaN-propagating (cuda_emitter.cpp:52-65) */
  TQ_AMIN = 3,
  TQ_ARGMAX = 4 /* first index of the maximum, NaN counts as the maximum; result is int64.
                   No counterpart kernel in the reference: aten.argmax runs on its host. */
};

/* Scratch bytes `tq_reduce_launch` needs for these extents (0 when it needs none). The scratch
 * holds per-CTA partials of slices that are split over several CTAs and a ticket counter. */
tq_status tq_reduce_workspace_bytes(tq_reduce_op op,
                                    tq_dtype dtype,
                                    int64_t outer,
                                    int64_t reduce,
                                    int64_t inner,
                                    int32_t device,
                                    size_t* bytes);

/* Reduces `in`, viewed as a packed [outer, reduce, inner], to a packed [outer, inner] `out`
 * (csrc/tessiq/codegen/reduction.h:69-117). Output type: the input's, except TQ_ARGMAX -> int64
 * and TQ_SUM of int32 -> int64 (torch's promotion, eager_reduction.cpp:77-89). f16/bf16 are
 * accumulated in f32. `workspace` must hold `tq_reduce_workspace_bytes` bytes of device memory
 * that no other launch in flight uses; it may be null when that size is 0. reduce == 0, or a
 * mean over an integer type, is TQ_UNSUPPORTED (reduction.cpp:110-113,148-152). */
tq_status tq_reduce_launch(tq_reduce_op op,
                           tq_dtype dtype,
                           const void* in,
                           void* out,
                           int64_t outer,
                           int64_t reduce,
                           int64_t inner,
                           void* workspace,
                           size_t workspace_bytes,
                           int32_t device,
                           void* stream);

/* The same reduction for callers that cannot allocate device memory and have nowhere to get
 * scratch from: code that runs where cudaMalloc is off limits (a host callback on a stream, a
 * latency-critical loop that must not take the allocator's lock or risk an implicit device
 * synchronisation, a plugin whose host hands it tensors but no allocator), or that must keep its
 * device-memory footprint fixed after start-up. This entry point has no counterpart in the
 * reference, whose reductions always take their temporary from its caching allocator.
 *
 * It behaves like tq_reduce_launch with the scratch taken from a fixed array of
 * TQ_STATIC_SCRATCH_BYTES bytes that is part of the library's device image: every GPU that loads
 * the library holds that array until the process exits, whether or not this function is called.
 * It never calls cudaMalloc, cudaFree or any allocating library routine.
 *
 *   - Extents whose scratch need (tq_reduce_workspace_bytes) exceeds TQ_STATIC_SCRATCH_BYTES are
 *     refused with TQ_RESOURCE_EXHAUSTED and a message naming both sizes; nothing is launched.
 *     Reductions that need no scratch at all are never refused for size.
 *   - The first call on each device looks up the array's device address (one host-side runtime
 *     query, no device work). Make that first call outside of any stream capture.
 *   - All calls on a device share the one array. A call clears the words it needs cleared itself,
 *     on `stream`, so the previous call's leftovers are harmless; but two calls whose kernels can
 *     overlap on the GPU (different streams without an ordering between them, or two host
 *     threads on different streams) race on the array and give wrong results. Order such calls
 *     with events, or use tq_reduce_launch with separate scratch. */
#define TQ_STATIC_SCRATCH_BYTES 131072
tq_status tq_reduce_launch_static(tq_reduce_op op,
                                  tq_dtype dtype,
                                  const void* in,
                                  void* out,
                                  int64_t outer,
                                  int64_t reduce,
                                  int64_t inner,
                                  int32_t device,
                                  void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Pack: strided / expanded / permuted view -> packed copy                                      */
/* Replaces pack_source + pack_on_device (csrc/tessiq/codegen/pack.cpp:41-94,                    */
/* csrc/tessiq/torch/pack.cpp:80-122). Bit-exact byte copy.                                      */

/* element_bytes in {1,2,4,8,16}; rank <= 8 (rank 9 declines, tests/python/test_pack.py:117-128);
 * sizes are the view's extents, strides the view's strides in elements (>= 0). */
tq_status tq_pack_launch(int32_t element_bytes,
                         int32_t rank,
                         const int64_t* sizes,
                         const int64_t* strides,
                         const void* src,
                         void* dst,
                         int32_t device,
                         void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Row kernels: softmax, LayerNorm, RMSNorm, eval BatchNorm                                     */

/* softmax over the middle extent of a packed [outer, extent, inner] tensor
 * (csrc/custom_ops/softmax/softmax.cu:19-61, softmax.cpp:30-61). dtype f32/f16/bf16/f64;
 * statistics in f32 (f64 for f64). `out_dtype` is `dtype`, or TQ_F32 for a half input
 * (aten::_softmax's half_to_float). NaN in a row makes the whole row NaN, as torch does. */
tq_status tq_softmax_launch(tq_dtype dtype,
                            tq_dtype out_dtype,
                            const void* in,
                            void* out,
                            int64_t outer,
                            int64_t extent,
                            int64_t inner,
                            int32_t device,
                            void* stream);

/* LayerNorm forward over the last `width` elements of each of `rows` packed rows
 * (csrc/tessiq/codegen/norm.cpp:22-135, csrc/tessiq/torch/eager_norm.cpp:226-271; the custom op
 * csrc/custom_ops/layer_norm/layer_norm.nvcc.cu:43-120). Two passes over registers: the mean,
 * then the centred sum of squares; rstd = 1/sqrt(var + eps); y = (x-mean)*rstd*weight + bias.
 * weight, bias, mean, rstd may each be null (skipped). `stat_dtype` is the type of mean/rstd
 * (torch returns them in the input's type for f16/bf16 inputs). */
tq_status tq_layer_norm_launch(tq_dtype dtype,
                               const void* in,
                               const void* weight,
                               const void* bias,
                               void* out,
                               void* mean,
                               void* rstd,
                               tq_dtype stat_dtype,
                               int64_t rows,
                               int64_t width,
                               double eps,
                               int32_t device,
                               void* stream);

/* softmax and LayerNorm over the last axis of a TRANSPOSED view, without packing the view first.
 * `in` is a packed [batch, rows, cols] tensor; the operation runs over `rows` for every (batch,
 * column) and the result is written packed as [batch, cols, rows] — i.e. op(in.transpose(-1, -2), -1).
 * This is what the reference reaches as pack_on_device followed by the row kernel
 * (python/tessiq/executor.py:201 then csrc/custom_ops/softmax/softmax.cu:19-61 or
 * csrc/tessiq/codegen/norm.cpp:22-135): four passes over the data; here it is three — per-column
 * statistics read in place, then one transposing pass that normalises. LayerNorm's weight and bias
 * (either may be null) have `rows` elements. dtype f32/f16/bf16; rows and cols must be multiples
 * of 16 / sizeof(element) and the tensors 16-byte aligned, else TQ_UNSUPPORTED (pack, then use the
 * row entry points). `workspace` must hold tq_transposed_workspace_bytes bytes.
 * Long columns of a small tensor (8192 to 51200 rows, at most 32 MiB, rows a multiple of 8 vectors and
 * cols of 2) take TWO passes instead: a cluster of 8 CTAs keeps a slab of columns by all the rows in
 * its shared memory and reads HBM once. tq_transposed_passes reports which form a shape takes (2 or
 * 3), so that a caller can choose between this entry and pack + row kernels before it launches (the
 * reference decides only after the fact, when a kernel declines: csrc/tessiq/torch/custom.cpp:563-598). */
tq_status tq_transposed_workspace_bytes(int32_t layer_norm, tq_dtype dtype, int64_t batch, int64_t rows,
                                        int64_t cols, int32_t device, size_t* bytes);
tq_status tq_transposed_passes(int32_t layer_norm, tq_dtype dtype, int64_t batch, int64_t rows, int64_t cols,
                               int32_t device, int32_t* passes);
/* Which kernel tq_*_transposed_launch runs for a shape (the pointers' alignment can still send a
 * call to the three-pass form): statistics read in place + a transposing normalise (two launches);
 * the column slab kept in a cluster's shared memory; or the persistent kernel that walks panels of
 * columns with TMA (one launch, statistics and normalise side by side; f32 tensors of 256 MiB and
 * more whose rows are a multiple of 64 and whose columns a multiple of 128). */
enum { TQ_TRANSPOSED_THREE_PASS = 0, TQ_TRANSPOSED_SLAB = 1, TQ_TRANSPOSED_PANELS = 2 };
tq_status tq_transposed_form(int32_t layer_norm, tq_dtype dtype, int64_t batch, int64_t rows, int64_t cols,
                             int32_t device, int32_t* form);
tq_status tq_softmax_transposed_launch(tq_dtype dtype, const void* in, void* out, int64_t batch, int64_t rows,
                                       int64_t cols, void* workspace, size_t workspace_bytes, int32_t device,
                                       void* stream);
tq_status tq_layer_norm_transposed_launch(tq_dtype dtype, const void* in, const void* weight, const void* bias,
                                          void* out, int64_t batch, int64_t rows, int64_t cols, double eps,
                                          void* workspace, size_t workspace_bytes, int32_t device, void* stream);

/* RMSNorm: y = x * rsqrt(mean(x^2) + eps) * weight (csrc/custom_ops/rms_norm/rms_norm.cu:15-42). */
tq_status tq_rms_norm_launch(tq_dtype dtype,
                             const void* in,
                             const void* weight,
                             void* out,
                             int64_t rows,
                             int64_t width,
                             double eps,
                             int32_t device,
                             void* stream);

/* Eval-mode BatchNorm over a packed [n, c, inner] tensor: alpha = w/sqrt(var+eps),
 * beta = b - mean*alpha, y = x*alpha + beta (csrc/tessiq/codegen/norm.cpp:137-199,
 * csrc/tessiq/torch/eager_norm.cpp:136-199). weight/bias may be null (1 and 0). The four
 * per-channel vectors have `param_dtype` (f32 for half inputs in torch's mixed mode, else dtype). */
tq_status tq_batch_norm_eval_launch(tq_dtype dtype,
                                    tq_dtype param_dtype,
                                    const void* in,
                                    const void* weight,
                                    const void* bias,
                                    const void* running_mean,
                                    const void* running_var,
                                    void* out,
                                    int64_t n,
                                    int64_t c,
                                    int64_t inner,
                                    double eps,
                                    int32_t device,
                                    void* stream);

/* ------------------------------------------------------------------------------------------ */
/* GEMM (+ bias + activation)                                                                    */
/* Replaces launch_gemm (csrc/tessiq/codegen/blas.cpp:92-193) with its bias pre-fill kernel      */
/* (csrc/tessiq/codegen/gemm.cpp:186-199), and the custom ops gemm_bias_gelu_tanh                */
/* (csrc/custom_ops/gemm_bias_gelu_tanh/gemm_bias_gelu_tanh.nvcc.cu:219-288) and gemm_bias_gelu  */
/* (csrc/custom_ops/gemm_bias_gelu/gemm_bias_gelu.nvcc.cu:90-158).                               */

typedef int32_t tq_activation;
enum { TQ_ACT_NONE = 0, TQ_ACT_GELU_ERF = 1, TQ_ACT_GELU_TANH = 2 };

/* C[b] = act(op(A[b]) @ op(B[b]) + bias), row-major, bf16 or f16 operands, f32 accumulation in
 * tensor memory, one rounding to the output type after bias and activation.
 *   op(A) is [m,k]: trans_a == 0 -> A is row-major [m,k] with leading dimension lda (elements);
 *                   trans_a != 0 -> A is stored as [k,m] with leading dimension lda.
 *   op(B) is [k,n]: trans_b == 0 -> B is row-major [k,n] (the `A @ B` form);
 *                   trans_b != 0 -> B is stored as [n,k] (the nn.Linear weight form).
 * Transposed operands are consumed in place, never copied (csrc/tessiq/codegen/gemm.cpp:28-53).
 * bias is one value per output column ([n], same dtype as C) or null.
 * batch >= 1 with element strides stride_a/b/c between problems (0 = shared operand).
 * Requirements (else TQ_UNSUPPORTED, the caller's decline): 16-byte-aligned base pointers and
 * leading dimensions/strides that are multiples of 8 elements (TMA's rules). */
tq_status tq_gemm_bias_act_launch(tq_dtype dtype,
                                  tq_activation activation,
                                  const void* a,
                                  int64_t lda,
                                  int32_t trans_a,
                                  const void* b,
                                  int64_t ldb,
                                  int32_t trans_b,
                                  const void* bias,
                                  void* c,
                                  int64_t ldc,
                                  int64_t m,
                                  int64_t n,
                                  int64_t k,
                                  int64_t batch,
                                  int64_t stride_a,
                                  int64_t stride_b,
                                  int64_t stride_c,
                                  int32_t device,
                                  void* stream);

/* The same with a residual added after the activation and before the one rounding:
 *   C[b] = act(op(A[b]) @ op(B[b]) + bias) + R[b]
 * R is row-major [m,n] with leading dimension ldr and batch stride stride_r (elements), of C's type,
 * or null (then this is tq_gemm_bias_act_launch). It replaces the elementwise `add` kernel the
 * reference launches after a projection for `x + linear(y)` (a fused group of
 * csrc/tessiq/codegen/cuda_emitter.cpp:212-255 reading the GEMM's result back from memory). */
tq_status tq_gemm_bias_act_residual_launch(tq_dtype dtype,
                                           tq_activation activation,
                                           const void* a,
                                           int64_t lda,
                                           int32_t trans_a,
                                           const void* b,
                                           int64_t ldb,
                                           int32_t trans_b,
                                           const void* bias,
                                           const void* residual,
                                           int64_t ldr,
                                           int64_t stride_r,
                                           void* c,
                                           int64_t ldc,
                                           int64_t m,
                                           int64_t n,
                                           int64_t k,
                                           int64_t batch,
                                           int64_t stride_a,
                                           int64_t stride_b,
                                           int64_t stride_c,
                                           int32_t device,
                                           void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Fused attention                                                                              */
/* The reference has no attention kernel. This entry point replaces the sequence its compiler   */
/* emits for `softmax(q @ k.T * scale [masked]) @ v` (the pattern of                            */
/* tests/python/test_models.py:64-67): a bmm through launch_gemm                                */
/* (csrc/tessiq/codegen/gemm.cpp:100-175), host-side mask operators, the softmax custom op      */
/* (csrc/custom_ops/softmax/softmax.cu:19-61), a second bmm, and the pack kernels around them    */
/* (csrc/tessiq/codegen/pack.cpp:41-94), with the [batch, heads, T, T] scores in device memory. */

/* out[b,h,i,:] = sum_j softmax_j(scale * q[b,h,i,:] . k[b,h,j,:]) * v[b,h,j,:], over j <= i when
 * causal != 0 (a lower-triangular mask aligned at the first query and the first key), else over
 * every key. bf16 or f16; scores, maxima and sums in f32; one rounding of the result.
 *   q is [batch, heads, q_tokens, head_dim], k and v are [batch, heads, k_tokens, head_dim], out is
 *   [batch, heads, q_tokens, head_dim]; each is addressed through three ELEMENT strides
 *   {batch, head, token} and its head_dim elements are contiguous — so the slices of a fused QKV
 *   projection are read where they lie and the result can be written in [batch, token, head, dim]
 *   order.
 * head_dim is 8, 16, ... 128: the kernel works on 64-wide tiles, one per head up to 64 elements and two
 * side by side beyond (then one group of 128 query rows per CTA instead of two); the columns a head
 * does not have are filled with zeros by TMA. Declines (TQ_UNSUPPORTED): any other head_dim, a scale that is not positive and finite, q/k/v that
 * are not 16-byte aligned or whose strides are not positive multiples of 8 elements (TMA's rules).
 * Bounded waits report through tq_status_poll like the GEMM's. */
tq_status tq_attention_launch(tq_dtype dtype,
                              const void* q,
                              const void* k,
                              const void* v,
                              void* out,
                              int64_t batch,
                              int64_t heads,
                              int64_t q_tokens,
                              int64_t k_tokens,
                              int64_t head_dim,
                              const int64_t* q_strides,
                              const int64_t* k_strides,
                              const int64_t* v_strides,
                              const int64_t* out_strides,
                              double scale,
                              int32_t causal,
                              int32_t device,
                              void* stream);

/* ------------------------------------------------------------------------------------------ */
/* Recipes: a compiled graph's launches, replayed by native code                                */
/* Replaces the per-call Python interpreter loop of RecipeExecutor                              */
/* (python/tessiq/executor.py:146-239), to which the reference attributes 42 % + 34 % of a call   */
/* (README.md:333-337).                                                                         */

/* Between tq_recipe_begin_recording and tq_recipe_end_recording every tq_*_launch call made by the
 * calling thread is appended to the recipe instead of being launched: scalar arguments and the
 * small argument arrays (sizes, strides, divisors, layouts, scalars, input pointer lists) are
 * copied; data pointers, scratch pointers and tq_fused handles are kept as given, so those buffers
 * and handles must outlive the recipe and stay where they are (plan them in a tq_arena). The
 * (device, stream) given while recording are ignored. tq_recipe_run launches the recorded steps in
 * order on its own (device, stream), stopping at the first step that fails; it makes no Python
 * call and may itself be captured into a CUDA graph. One thread records into one recipe at a
 * time; a recipe may be run from any thread once recording has ended. */
typedef struct tq_recipe tq_recipe;
tq_status tq_recipe_create(tq_recipe** recipe);
tq_status tq_recipe_destroy(tq_recipe* recipe);
tq_status tq_recipe_begin_recording(tq_recipe* recipe);
tq_status tq_recipe_end_recording(tq_recipe* recipe);
int64_t tq_recipe_steps(const tq_recipe* recipe);
tq_status tq_recipe_run(const tq_recipe* recipe, int32_t device, void* stream);

/* Reads and clears the device-side status word of `device`: 0 when every bounded wait inside
 * this library's kernels completed, otherwise a code naming the wait that gave up. Synchronises
 * `stream` first. */
tq_status tq_status_poll(int32_t device, void* stream, int32_t* device_status);

/* ---- One runtime over several GPUs of one process ------------------------------------------------
 * Replaces the reference's device layer for this path (csrc/tessiq/runtime/cuda_device.cpp:34-147: one
 * blocking copy stream per device, everything else on the legacy stream; allocator.cpp:56-108;
 * registry.cpp:50-54: tessiq:k is CUDA ordinal k-1). tq_runtime_create checks the list the way the
 * reference checks its `device` option (python/tessiq/backend.py:95-104: unknown entries are an
 * invalid-argument error, not a fallback) and gives every listed GPU a non-blocking stream, a slice
 * of arena memory (a bump pointer: tq_runtime_alloc hands out 256-byte-aligned ranges until
 * tq_runtime_release rewinds the slice) and an event. A sharded executor enqueues the same kernels on
 * every GPU's stream; tq_runtime_fork orders the other streams after one GPU's (inputs scattered),
 * tq_runtime_join orders one GPU's stream after all the others (results gathered). */
typedef struct tq_runtime tq_runtime;
tq_status tq_runtime_create(const int32_t* devices, int32_t count, size_t arena_bytes_per_device, tq_runtime** runtime);
tq_status tq_runtime_destroy(tq_runtime* runtime);
int32_t tq_runtime_device_count(const tq_runtime* runtime);
tq_status tq_runtime_device(const tq_runtime* runtime, int32_t index, int32_t* device);
tq_status tq_runtime_stream(const tq_runtime* runtime, int32_t index, void** stream);
tq_status tq_runtime_alloc(tq_runtime* runtime, int32_t index, size_t bytes, void** pointer);
tq_status tq_runtime_release(tq_runtime* runtime, int32_t index);
size_t tq_runtime_arena_used(const tq_runtime* runtime, int32_t index);
tq_status tq_runtime_fork(tq_runtime* runtime, int32_t from);
tq_status tq_runtime_join(tq_runtime* runtime, int32_t onto);
tq_status tq_runtime_synchronize(tq_runtime* runtime);

/* ---- Global reductions over the GPUs of one box ------------------------------------------------
 * The reference has no multi-GPU execution (one target device per recipe,
 * python/tessiq/recipe.py:117-161); these entry points are what its recipes shard under: a reduction
 * over every element of a tensor whose elements are split over several GPUs is, per GPU and on one
 * stream, tq_reduce_partial_launch -> tq_allreduce_scalar -> tq_reduce_finish_launch.
 *
 * tq_comm: an NCCL communicator (NCCL is opened at run time; TQ_NOT_FOUND when libnccl.so.2 is not
 * available). One process per GPU: one rank calls tq_comm_unique_id, hands the 128 bytes to the
 * others by its own means, and every rank calls tq_comm_create with its GPU current-able. One process
 * that drives several GPUs: tq_comm_create_all fills one communicator per listed device. */
typedef struct tq_comm tq_comm;
tq_status tq_comm_unique_id(void* id, size_t bytes);
tq_status tq_comm_create(const void* id, size_t bytes, int32_t rank, int32_t world, int32_t device, tq_comm** comm);
tq_status tq_comm_create_all(const int32_t* devices, int32_t count, tq_comm** comms);
tq_status tq_comm_destroy(tq_comm* comm);
int32_t tq_comm_rank(const tq_comm* comm);
int32_t tq_comm_world(const tq_comm* comm);

/* In-place all-reduce of `count` elements of `buffer` (device memory of the communicator's GPU) over
 * the communicator's ranks, on `stream`: TQ_SUM, TQ_AMAX (maximum) or TQ_AMIN (minimum). */
tq_status tq_allreduce_scalar(tq_comm* comm, void* buffer, int64_t count, tq_dtype dtype, tq_reduce_op op,
                              int32_t device, void* stream);

/* The local part: `count` packed elements of `in` (f32, f16 or bf16) reduced to a two-float partial
 * at `partial` (8-byte aligned device memory): TQ_SUM / TQ_MEAN give {sum in f32, 0}; TQ_AMAX gives
 * {maximum with a NaN replaced by -inf, 1 if a NaN was seen}, to be all-reduced with TQ_AMAX; TQ_AMIN
 * gives {minimum with a NaN replaced by +inf, -1 if a NaN was seen}, to be all-reduced with TQ_AMIN.
 * Scratch as for tq_reduce_launch over [1, count, 1] (tq_reduce_workspace_bytes). */
tq_status tq_reduce_partial_launch(tq_reduce_op op, tq_dtype dtype, const void* in, void* partial, int64_t count,
                                   void* workspace, size_t workspace_bytes, int32_t device, void* stream);

/* The finish: the combined two-float partial becomes one element of `dtype` at `out`: the sum, the
 * sum divided by `total_count` (TQ_MEAN), or the extreme — NaN when the flag word is not zero. */
tq_status tq_reduce_finish_launch(tq_reduce_op op, tq_dtype dtype, const void* partial, void* out, int64_t total_count,
                                  int32_t device, void* stream);

/* A self-test of the give-up path: launches one warp that waits, for at most `polls` looks, on a
 * barrier that cannot complete, and returns by itself. Afterwards tq_status_poll reports 0x53454c46
 * ("SELF"). looks[0] = the looks the wait took (= polls); looks[1] = how long, in units of 1024
 * clock cycles, one of the library's own bounded waits in the same launch then took to leave
 * (it leaves at its first look at the launch's abort word, which it takes every 1024 polls), or -1 if
 * it completed. Kernels
 * launched afterwards are not affected: the abort word belongs to the launch. Synchronises `stream`.
 * No counterpart in the reference. */
tq_status tq_selftest_bounded_wait(int32_t device, void* stream, int32_t polls, int32_t* looks);

/* The first `count` (<= 64) 32-bit words of the device's status block, without clearing it: word 0 is
 * what tq_status_poll returns, the words behind it say where the wait that gave up was (CTA, thread
 * and up to four values of the kernel's own choosing). Call it before tq_status_poll. Synchronises
 * `stream`. No counterpart in the reference. */
tq_status tq_status_detail(int32_t device, void* stream, int32_t* words, int32_t count);

#ifdef __cplusplus
}
#endif

#endif /* TESSIQ_B200_H_ */
