/* C ABI of the sm_100a kernel library (libttb200.so): the lowest boundary of the backend.
 *
 * In tt-mlir every per-op executor under runtime/lib/ttnn/operations/ ends in one call into
 * the tt-metal TTNN library (`::ttnn::matmul`, `::ttnn::quantize`, ...).  Each launcher below
 * replaces one of those library calls with a hand-written CUDA kernel; the citation beside a
 * declaration names the reference call site it stands in for.  The C++ runtime target in
 * tt-mlir_b200/runtime/ is the only intended caller, but nothing here depends on it: plain
 * pointers, sizes and enums only, no C++ or torch types.
 *
 * Conventions
 *  - every function returns TTB_OK (0) or a TTB_ERR_* code; ttb_last_error() gives the text
 *    of the calling thread's most recent failure.  Nothing throws, aborts or exits.
 *  - `stream` is a cudaStream_t passed as void*; launches are asynchronous on it.
 *  - pointers are device pointers on the current device unless a name says `host`.
 *  - `dtype` arguments use the numeric values of tt::target::DataType
 *    (include/ttmlir/Target/Common/types.fbs:19-42).
 *  - tensors are dense row-major unless strides are passed explicitly.
 */
#ifndef TTB_KERNELS_H
#define TTB_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TTB_API __attribute__((visibility("default")))

enum {
  TTB_OK = 0,
  TTB_ERR_CUDA = 1,        /* a CUDA runtime / driver call failed */
  TTB_ERR_INVALID = 2,     /* bad argument (shape, alignment, null pointer) */
  TTB_ERR_UNSUPPORTED = 3, /* valid request this build has no kernel for */
  TTB_ERR_NCCL = 4,        /* NCCL call failed or NCCL could not be loaded */
  TTB_ERR_DEVICE = 5       /* a kernel reported a failure through its status word */
};

enum {
  TTB_DTYPE_FLOAT32 = 0,
  TTB_DTYPE_FLOAT16 = 1,
  TTB_DTYPE_BFLOAT16 = 2,
  TTB_DTYPE_UINT32 = 9,
  TTB_DTYPE_UINT16 = 10,
  TTB_DTYPE_UINT8 = 11,
  TTB_DTYPE_INT32 = 12,
  TTB_DTYPE_INT8 = 17
};

TTB_API const char *ttb_last_error(void);
TTB_API size_t ttb_dtype_size(int dtype);

/* ---- device, streams, memory, events ------------------------------------------------------
 * Stand in for what MeshDevice / command queues / buffers provide to runtime/lib/ttnn
 * (openMeshDevice runtime/lib/ttnn/runtime.cpp:582-624, toLayout/toHost :861-933). */
TTB_API int ttb_device_count(int *count);
TTB_API int ttb_set_device(int device);
TTB_API int ttb_device_info(int device, int *sm_count, size_t *total_mem, int *cc_major, int *cc_minor);
TTB_API int ttb_stream_create(void **stream);
TTB_API int ttb_stream_destroy(void *stream);
TTB_API int ttb_stream_sync(void *stream);
TTB_API int ttb_device_sync(void);
/* Stream-ordered allocation from the device's default memory pool (kept warm, never trimmed). */
TTB_API int ttb_malloc(void **ptr, size_t bytes, void *stream);
TTB_API int ttb_free(void *ptr, void *stream);
/* What the current device's default memory pool holds: bytes reserved from the driver, bytes handed
 * out right now, and the high-water mark of the latter since it was last reset (reset_high != 0
 * resets it to the current use after reading).  A call sequence that must not allocate leaves the
 * high-water mark where a reset put it.  Any of the outputs may be null. */
TTB_API int ttb_mempool_stats(uint64_t *reserved, uint64_t *used, uint64_t *used_high, int reset_high);
TTB_API int ttb_host_alloc_pinned(void **ptr, size_t bytes);
TTB_API int ttb_host_free_pinned(void *ptr);
/* *pinned = 1 when `ptr` is page-locked host memory (a copy from it is a true asynchronous DMA). */
TTB_API int ttb_host_is_pinned(const void *ptr, int *pinned);
TTB_API int ttb_memcpy_h2d(void *dst, const void *host_src, size_t bytes, void *stream);
TTB_API int ttb_memcpy_d2h(void *host_dst, const void *src, size_t bytes, void *stream);
TTB_API int ttb_memcpy_d2d(void *dst, const void *src, size_t bytes, void *stream);
TTB_API int ttb_memset(void *dst, int byte, size_t bytes, void *stream);
TTB_API int ttb_event_create(void **event);
TTB_API int ttb_event_destroy(void *event);
TTB_API int ttb_event_record(void *event, void *stream);
TTB_API int ttb_event_sync(void *event);
TTB_API int ttb_stream_wait_event(void *stream, void *event);
TTB_API int ttb_event_elapsed_ms(void *start, void *stop, float *ms);
/* Traces: what BeginTraceCaptureOp / EndTraceCaptureOp / ExecuteTraceOp do on the device
 * (runtime/lib/ttnn/operations/trace/{begin_trace_capture,end_trace_capture,execute_trace}.cpp call
 * ::ttnn::operations::trace::begin_trace_capture / end_trace_capture / execute_trace).  Everything
 * enqueued on `stream` between begin and end (kernels, stream-ordered allocations and frees) is
 * recorded instead of run; end turns the recording into an executable CUDA graph; launch replays
 * it.  abort ends a recording that failed half way and leaves the stream usable. */
TTB_API int ttb_trace_begin(void *stream);
TTB_API int ttb_trace_end(void *stream, void **trace);
TTB_API int ttb_trace_abort(void *stream);
TTB_API int ttb_trace_launch(void *trace, void *stream);
TTB_API int ttb_trace_destroy(void *trace);
TTB_API int ttb_stream_is_recording(void *stream, int *recording);
/* Number of kernels this library has launched in the calling process (all threads). */
TTB_API uint64_t ttb_launch_count(void);
/* Per-launch profiling (the CUDA-event counterpart of the reference's Tracy zones around each op,
 * runtime/lib/ttnn/program_executor.cpp:223-237).  While enabled every launcher brackets its
 * kernel with an event pair on the launching stream and notes the launch's algorithmic FLOPs and
 * bytes.  ttb_prof_summary waits for the recorded events and writes a JSON array of
 * {"tag", "launches", "ms", "flops", "bytes"} aggregated per kernel family.  Enabling clears
 * earlier records.  Meant for measurement runs, not for production submits. */
TTB_API int ttb_prof_enable(int on);
TTB_API int ttb_prof_summary(char *json_out, size_t cap);

/* ---- quantization: ::ttnn::quantize / dequantize / requantize
 * (runtime/lib/ttnn/operations/eltwise/quantization/quantization.cpp:173-187).
 * Arithmetic follows the torch goldens tools/golden/mapping.py:2534-2582:
 *   quantize   q = clamp(rne(x * (1/scale)) + zp, qmin, qmax)      (f32, 1/scale rounded once)
 *   dequantize x = float(q - zp) * scale
 *   requantize q' = quantize(dequantize(q))
 * qmin/qmax come from the output dtype: INT8 [-128,127], UINT8 [0,255], INT32 full range unless
 * `clamp_i8` is set, in which case an INT32 container holds values clamped to [-128,127]
 * (how tt-mlir stores quantized tensors, lib/Dialect/TTNN/Pipelines/TTNNPipelines.cpp:349-351).
 * Per-axis variants take one scale / zero point per index of `axis`; the tensor is viewed as
 * [outer, axis_len, inner]. */
TTB_API int ttb_quantize(const void *in, int in_dtype, void *out, int out_dtype, size_t n,
                         float scale, int32_t zero_point, int clamp_i8, void *stream);
TTB_API int ttb_dequantize(const void *in, int in_dtype, void *out, int out_dtype, size_t n,
                           float scale, int32_t zero_point, void *stream);
TTB_API int ttb_requantize(const void *in, int in_dtype, void *out, int out_dtype, size_t n,
                           float in_scale, int32_t in_zp, float out_scale, int32_t out_zp,
                           int clamp_i8, void *stream);
TTB_API int ttb_quantize_per_axis(const void *in, int in_dtype, void *out, int out_dtype,
                                  size_t outer, size_t axis_len, size_t inner,
                                  const float *scales, const int32_t *zero_points, int clamp_i8,
                                  void *stream);
TTB_API int ttb_dequantize_per_axis(const void *in, int in_dtype, void *out, int out_dtype,
                                    size_t outer, size_t axis_len, size_t inner,
                                    const float *scales, const int32_t *zero_points, void *stream);
TTB_API int ttb_requantize_per_axis(const void *in, int in_dtype, void *out, int out_dtype,
                                    size_t outer, size_t axis_len, size_t inner,
                                    const float *in_scales, const int32_t *in_zps,
                                    const float *out_scales, const int32_t *out_zps, int clamp_i8,
                                    void *stream);
/* quantize -> requantize -> dequantize in one pass over the data (per-tensor parameters).
 * `q1` / `q2` may be null; when given, the intermediate integer tensors are written too. */
TTB_API int ttb_quant_chain(const void *in, int in_dtype, void *q1, int q1_dtype, void *q2,
                            int q2_dtype, void *out, int out_dtype, size_t n, float scale1,
                            int32_t zp1, float scale2, int32_t zp2, int clamp_i8, void *stream);

/* ---- elementwise: ::ttnn::relu/.../add/... (runtime/lib/ttnn/operations/eltwise/unary/unary.cpp:133-273,
 * binary/binary.cpp:37-127, binary/binary_composite.cpp, ternary/where.cpp).
 * `op` uses the flatbuffer enum values (EltwiseUnaryOpType / EltwiseBinaryOpType,
 * include/ttmlir/Target/TTNN/operations/eltwise.fbs:11-26,133-166); composite binary ops
 * are offset by TTB_BINARY_COMPOSITE_BASE.  Math is done in f32 (i32 for integer inputs of
 * integer ops) and rounded once to the output dtype. */
#define TTB_BINARY_COMPOSITE_BASE 100
TTB_API int ttb_eltwise_unary(int op, const void *in, int in_dtype, void *out, int out_dtype,
                              size_t n, float param, void *stream);
/* Broadcasting binary op over a rank-`rank` output (rank <= 8).  Strides are in elements,
 * 0 on broadcast dimensions. */
TTB_API int ttb_eltwise_binary(int op, const void *a, int a_dtype, const void *b, int b_dtype,
                               void *out, int out_dtype, int rank, const int64_t *out_shape,
                               const int64_t *a_strides, const int64_t *b_strides, void *stream);
TTB_API int ttb_where(const void *cond, int cond_dtype, const void *a, const void *b, int dtype,
                      void *out, int rank, const int64_t *out_shape, const int64_t *c_strides,
                      const int64_t *a_strides, const int64_t *b_strides, void *stream);
TTB_API int ttb_clamp(const void *in, int dtype, void *out, size_t n, float lo, float hi,
                      void *stream);
/* ::ttnn::typecast (runtime/lib/ttnn/operations/layout/typecast.cpp:26-27). */
TTB_API int ttb_typecast(const void *in, int in_dtype, void *out, int out_dtype, size_t n,
                         void *stream);
/* ::ttnn::full / zeros / ones / arange (runtime/lib/ttnn/operations/creation/). */
TTB_API int ttb_fill(void *out, int dtype, size_t n, double value, void *stream);
TTB_API int ttb_arange(void *out, int dtype, size_t n, double start, double step, void *stream);
/* silu(gate) * up with both roundings of the unfused chain kept (SwiGLU gating). */
TTB_API int ttb_silu_mul(const void *gate, const void *up, void *out, int dtype, size_t n,
                         void *stream);

/* ---- normalisation / reductions
 * ::ttnn::softmax (operations/normalization/softmax.cpp:32-33), ::ttnn::rms_norm
 * (operations/normalization/rms_norm.cpp:40-47), ::ttnn::sum/mean/max/min
 * (operations/reduction/reduction.cpp:40-58).  Tensor viewed as [outer, len, inner]. */
TTB_API int ttb_softmax(const void *in, void *out, int dtype, size_t outer, size_t len,
                        size_t inner, void *stream);
TTB_API int ttb_rms_norm(const void *in, const void *weight, const void *bias, void *out,
                         int dtype, size_t rows, size_t cols, float eps, void *stream);
/* out = rms_norm(a + b); `sum_out` (nullable) receives a + b rounded to dtype. */
TTB_API int ttb_add_rms_norm(const void *a, const void *b, const void *weight, void *sum_out,
                             void *out, int dtype, size_t rows, size_t cols, float eps,
                             void *stream);
/* Split normalisations (hidden dimension sharded over the mesh).  ttb_norm_row_stats reduces each row of x (+ residual)
 * into the reference's tile-layout statistics: mode 0 (::ttnn::rms_norm_pre_all_gather,
 * operations/normalization/rms_norm_pre_all_gather.cpp) writes [rows, 32] with mean(x^2) in column 0; mode 1
 * (::ttnn::layer_norm_pre_all_gather) writes [rows, 64] with sum(x^2) in column 0 and sum(x) in column 32; mode 2 writes
 * the plain f32 sum of squares per row (the exchange buffer of distributed_rms_norm).  Other columns are zero. */
TTB_API int ttb_norm_row_stats(const void *x, const void *residual, void *stats, int dtype, int stats_dtype, size_t rows,
                               size_t cols, int mode, void *stream);
/* y = act(rms_norm(x + residual) * weight + bias) over the last dimension (::ttnn::experimental::dit_rms_norm_unary_fused,
 * operations/normalization/dit_rms_norm_unary_fused.cpp), and the local half of ::ttnn::fused_rms_minimal
 * (distributed_rms_norm.cpp) when `row_sumsq` gives each row's sum of squares over all `total_cols` columns of the
 * distributed row.  residual, weight, bias, row_sumsq nullable.  act: 0 none, 1 relu, 2 relu6, 3 silu, 4 mish,
 * 5 sigmoid, 6 hardsigmoid, 7 tanh, 8 log, 9 softplus, 10 gelu, 11 sqrt. */
TTB_API int ttb_rms_norm_apply(const void *x, const void *residual, const void *weight, const void *bias, const float *row_sumsq,
                               void *y, int dtype, size_t rows, size_t cols, size_t total_cols, float eps, int act, void *stream);
/* ::ttnn::layer_norm_post_all_gather (operations/normalization/layer_norm_post_all_gather.cpp): `stats` is
 * [rows, 64 * blocks], one mode-1 block per device; mean and variance of the whole row of cols * blocks elements
 * normalise the local `cols` columns. */
TTB_API int ttb_layer_norm_post_all_gather(const void *x, const void *stats, const void *weight, const void *bias, void *y,
                                           int dtype, int stats_dtype, size_t rows, size_t cols, size_t blocks, float eps,
                                           void *stream);
/* op: 0 sum, 1 mean, 2 max, 3 min (ReductionOpType, operations/reduction.fbs:6-11). */
TTB_API int ttb_reduce(int op, const void *in, void *out, int dtype, size_t outer, size_t len,
                       size_t inner, void *stream);

/* ::ttnn::layer_norm (runtime/lib/ttnn/operations/normalization/layer_norm.cpp): each of `rows`
 * rows of `cols` elements is normalised with its own mean and biased variance, in f32, then
 * scaled / shifted by `weight` / `bias` (nullable, `cols` elements). */
TTB_API int ttb_layer_norm(const void *in, const void *weight, const void *bias, void *out, int dtype,
                           size_t rows, size_t cols, float eps, void *stream);
/* ::ttnn::argmax (operations/reduction/argmax.cpp): index (Int32) of the first maximum along the
 * middle dimension of [outer, len, inner]; a NaN counts as the maximum. */
TTB_API int ttb_argmax(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner,
                       void *stream);
/* ::ttnn::cumprod (operations/cumprod/cumprod.cpp): running product along the middle dimension of
 * [outer, len, inner]; the running product is one step wider than the elements (f32 for 16-bit types, f64 for f32,
 * as torch's CPU scan keeps it) and every prefix is rounded to the element type. */
TTB_API int ttb_cumprod(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner, void *stream);
/* ::ttnn::prod (operations/reduction/prod.cpp): product over the middle dimension of [outer, len, inner] in f32
 * (Int32: 64-bit product truncated), result [outer, inner]. */
TTB_API int ttb_prod(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner, void *stream);
/* ::ttnn::batch_norm with training = false (operations/normalization/batch_norm.cpp): over [outer, channels, inner],
 * y = (x - mean[c]) / sqrt(var[c] + eps) * weight[c] + bias[c] in f32; weight / bias nullable. */
TTB_API int ttb_batch_norm_inference(const void *x, const void *mean, const void *var, const void *weight, const void *bias,
                                     void *y, int dtype, size_t outer, size_t channels, size_t inner, float eps,
                                     void *stream);
/* ::ttnn::upsample (operations/pool/upsample.cpp): NHWC [n, h, w, c] -> [n, h * scale_h, w * scale_w, c], nearest
 * (bilinear = 0) or bilinear with align_corners = false. */
TTB_API int ttb_upsample2d(const void *in, void *out, int dtype, size_t n, size_t h, size_t w, size_t c, int scale_h,
                           int scale_w, int bilinear, void *stream);
/* ::ttnn::group_norm (operations/normalization/group_norm.cpp) on channels-last [images, 1, pixels, channels]: a
 * group is channels / groups consecutive channels; mean and biased variance over a group's pixels of one image in
 * f32, then scale / shift per channel (weight / bias nullable, `channels` entries). */
TTB_API int ttb_group_norm(const void *x, const void *weight, const void *bias, void *y, int dtype, size_t images,
                           size_t pixels, size_t channels, size_t groups, float eps, void *stream);
/* ::ttnn::conv_transpose2d (operations/conv/conv_transpose2d.cpp): NHWC input [n, h, w, c], weights
 * [c, o / groups, kh, kw], bias [o] (nullable), NHWC output with
 * ho = (h - 1) * stride_h - 2 * pad_top + dil_h * (kh - 1) + out_pad_h + 1 (likewise wo); f32 accumulation, one
 * rounding.  A CUDA-core kernel. */
TTB_API int ttb_conv_transpose2d(const void *x, const void *weight, const void *bias, void *out, int dtype, int64_t n,
                                 int64_t h, int64_t w, int64_t c, int64_t o, int kh, int kw, int stride_h, int stride_w,
                                 int pad_top, int pad_left, int out_pad_h, int out_pad_w, int dil_h, int dil_w, int groups,
                                 void *stream);
/* ::ttnn::batch_norm with training = true (operations/normalization/batch_norm.cpp:45-72) on [outer, channels, inner]:
 * normalises with the batch mean and the biased batch variance of each channel and moves `running_mean` /
 * `running_var` in place: running = momentum * batch + (1 - momentum) * running.  weight / bias nullable. */
TTB_API int ttb_batch_norm_training(const void *x, void *running_mean, void *running_var, const void *weight, const void *bias,
                                    void *y, int dtype, size_t outer, size_t channels, size_t inner, float eps, float momentum,
                                    void *stream);
/* ::ttnn::max_pool2d with return_indices (operations/pool/pool2d.cpp, MaxPool2dWithIndicesOp): NHWC, symmetric
 * padding [pad_top, pad_left]; `indices` (Int32, UInt32 or UInt16) holds iy * w + ix of each maximum inside its
 * image's plane; the first maximum wins. */
TTB_API int ttb_max_pool2d_with_indices(const void *in, void *out, void *indices, int dtype, int index_dtype, int n, int h, int w,
                                        int c, int ho, int wo, int kh, int kw, int stride_h, int stride_w, int pad_top,
                                        int pad_left, int dil_h, int dil_w, void *stream);
/* ::ttnn::experimental::rotary_embedding_llama (operations/transformer/rotary_embedding_llama.cpp):
 * y = x * cos + (x @ T) * sin with the 32 x 32 matrix `trans_mat` applied to every 32-wide piece of the head
 * dimension.  x is [rows, head_dim]; row r reads cache row (r / cos_div) % cos_mod. */
TTB_API int ttb_rotary_embedding_llama(const void *x, const void *cos_cache, const void *sin_cache, const void *trans_mat, void *y,
                                       int dtype, size_t rows, size_t head_dim, size_t cos_mod, size_t cos_div, void *stream);
/* ::ttnn::experimental::dropout (operations/eltwise/unary/dropout.cpp): zero with probability `prob`, else x * scale.
 * Counter-based generator: the result depends only on (seed, stream_id, element index). */
TTB_API int ttb_dropout(const void *x, void *y, int dtype, size_t n, float prob, float scale, uint32_t seed, uint32_t stream_id,
                        void *stream);
/* ::ttnn::rand (operations/rand/rand.cpp): uniform values in [low, high). */
TTB_API int ttb_rand_uniform(void *y, int dtype, size_t n, float low, float high, uint32_t seed, uint32_t stream_id, void *stream);
/* ::ttnn::experimental::conv3d (operations/conv/conv3d.cpp): NDHWC input [n, d, h, w, c], NDHWC output, symmetric
 * padding (zeros, or the edge value when `replicate`), no dilation.  `weight_strides5` are the weight's element strides
 * over (out channel, in channel within the group, kd, kh, kw): [O, C/g, kD, kH, kW] tensors and TTNN's prepared
 * [kD*kH*kW*C/g, O] matrices are both read in place.  bias [o], nullable.  A CUDA-core kernel. */
TTB_API int ttb_conv3d(const void *x, const void *weight, const void *bias, void *y, int dtype, int n, int d, int h, int w, int c,
                       int o, int kd, int kh, int kw, int sd, int sh, int sw, int pd, int ph, int pw, int groups, int replicate,
                       const int64_t *weight_strides5, void *stream);
/* ::ttnn::experimental::gelu_bw (operations/eltwise/binary/experimental_binary_backward.cpp): grad * gelu'(x). */
TTB_API int ttb_gelu_backward(const void *grad, const void *x, void *y, int dtype, size_t n, int tanh_approx, void *stream);
/* ::ttnn::embedding_bw (operations/embedding/embedding_backward.cpp): out[v, :] = sum of grad rows whose index is v
 * ([vocab, dim]; f32 accumulation in `workspace`, one rounding). */
TTB_API size_t ttb_embedding_backward_workspace_bytes(size_t vocab, size_t dim);
TTB_API int ttb_embedding_backward(const void *indices, const void *grad, void *out, int index_dtype, int dtype, size_t rows,
                                   size_t vocab, size_t dim, void *workspace, void *stream);
/* ttml::metal::adamw (operations/ttml/adamw.cpp), in place on param, exp_avg, exp_avg_sq and (amsgrad, nullable)
 * max_exp_avg_sq.  beta*_pow are beta^step.  Stochastic rounding applies to bf16 parameters. */
TTB_API int ttb_adamw(void *param, const void *grad, void *exp_avg, void *exp_avg_sq, void *max_exp_avg_sq, int param_dtype,
                      int grad_dtype, int moment_dtype, size_t n, float lr, float beta1, float beta2, float beta1_pow, float beta2_pow,
                      float eps, float weight_decay, int stochastic_rounding, uint32_t seed, void *stream);
/* ::ttnn::cumsum (operations/cumsum/cumsum.cpp): running sum along the middle dimension. */
TTB_API int ttb_cumsum(const void *in, void *out, int dtype, size_t outer, size_t len, size_t inner,
                       void *stream);

/* ---- pooling: ::ttnn::max_pool2d / avg_pool2d (runtime/lib/ttnn/operations/pool/pool2d.cpp:20-139)
 * over an NHWC activation [n, h, w, c] -> [n, ho, wo, c].  Paddings are top, left, bottom, right;
 * `padding_has_four` says whether the op carried four paddings (applied as data before pooling,
 * which changes the ceil-mode rule) or two.  ttb_pool2d_out_shape gives ho, wo. */
TTB_API int ttb_pool2d_out_shape(int is_max, int h, int w, int kh, int kw, int sh, int sw, int pt, int pl,
                                 int pb, int pr, int dh, int dw, int ceil_mode, int padding_has_four,
                                 int *ho, int *wo);
TTB_API int ttb_pool2d(const void *in, void *out, int dtype, int is_max, int n, int h, int w, int c, int kh,
                       int kw, int sh, int sw, int pt, int pl, int pb, int pr, int dh, int dw,
                       int ceil_mode, int count_include_pad, int padding_has_four, void *stream);

/* ::ttnn::embedding (operations/embedding/embedding.cpp): out[r, :] = table[indices[r], :].
 * Indices are Int32 / UInt32 / UInt16 or a float type holding integers.  An index outside
 * [0, vocab) reads row 0 and sets a flag that ttb_embedding_status returns and clears (after
 * synchronising the device). */
TTB_API int ttb_embedding(const void *indices, const void *table, void *out, int index_dtype, int dtype,
                          size_t rows, size_t vocab, size_t dim, void *stream);
TTB_API int ttb_embedding_status(int *bad_index_seen);
/* ::ttnn::pad (operations/data_movement/pad.cpp): `low[i]` / `high[i]` elements of `value` in front
 * of / behind dimension i. */
TTB_API int ttb_pad(const void *in, void *out, int dtype, int rank, const int64_t *in_shape,
                    const int64_t *low, const int64_t *high, double value, void *stream);

/* ---- KV cache and decode attention (runtime/lib/ttnn/operations/kv_cache/{fill_cache,update_cache}.cpp,
 * operations/transformer/scaled_dot_product_attention_decode.cpp; goldens tools/golden/mapping.py:
 * 3582-3670, 2417-2482).  Caches are [cache_users, heads, max_seq, head_dim].
 *  fill_cache    cache[batch_offset + b, h, :seq] = input[b, h]  (input [users, heads, seq, head_dim]); the
 *                rows up to the next multiple of 32 are zeroed when the cache has them
 *  update_cache  cache[batch_offset + b, h, index] = input[0, h, b]  (input [1, heads, users, head_dim]),
 *                `index` = element 0 of a device tensor, read by the kernel.  An index outside the cache
 *                writes nothing and sets a flag (ttb_update_cache_status synchronises, returns and clears it)
 *  sdpa_decode   q [1, batch, heads, head_dim] against k, v [batch, kv_heads, seq, head_dim]; keys after
 *                cur_pos[b] (Int32, nullable) are masked when is_causal; `mask` (nullable, the tensors'
 *                dtype) is [mask_users, 1, mask_heads, seq] with extents 1 or full; scores are
 *                (q.k + mask) * scale.  bf16 / f16, head_dim 64 / 128 / 256, heads / kv_heads in {1,2,4,8}.
 *                `workspace`: ttb_sdpa_decode_workspace_bytes(...) bytes of device memory. */
TTB_API int ttb_fill_cache(void *cache, const void *input, int dtype, size_t users, size_t heads, size_t seq,
                           size_t max_seq, size_t head_dim, size_t batch_offset, size_t cache_users, void *stream);
TTB_API int ttb_update_cache(void *cache, const void *input, const void *index, int dtype, int index_dtype,
                             size_t users, size_t heads, size_t max_seq, size_t head_dim, size_t batch_offset,
                             size_t cache_users, void *stream);
TTB_API int ttb_update_cache_status(int *bad_index_seen);
TTB_API size_t ttb_sdpa_decode_workspace_bytes(int batch, int heads, int seq, int head_dim);
TTB_API int ttb_sdpa_decode(const void *q, const void *k, const void *v, const void *cur_pos, const void *mask,
                            void *out, int dtype, int batch, int heads, int kv_heads, int seq, int head_dim,
                            int mask_users, int mask_heads, float scale, int is_causal, void *workspace,
                            size_t workspace_bytes, void *stream);

/* Paged KV cache (runtime/lib/ttnn/operations/kv_cache/paged_{update,fill}_cache.cpp, operations/transformer/
 * paged_scaled_dot_product_attention_decode.cpp; goldens tools/golden/mapping.py:8745-8844, 8926-9007).  The
 * cache is [blocks, heads, block_size, head_dim]; `page_table` [users, pages] gives the physical block of every
 * logical block of a user (entries clamped into range, as the goldens clamp them).
 *   ttb_paged_update_cache  input [users, seq, heads, head_dim]: token s of user b -> position update_index[b] + s
 *                           (page_table may be null: logical = physical block)
 *   ttb_paged_fill_cache    input [users, heads, seq, head_dim]: position s of user b, whose page-table row is
 *                           batch_idx[b] (b when batch_idx is null) -> position s
 *   ttb_sdpa_decode_paged   ttb_sdpa_decode with k / v read through the page table (Int32); the sequence length is
 *                           pages_per_user * block_size; workspace as ttb_sdpa_decode_workspace_bytes for that length */
TTB_API int ttb_paged_update_cache(void *cache, const void *input, const void *update_index, const void *page_table,
                                   int dtype, int index_dtype, int table_dtype, size_t users, size_t seq, size_t heads,
                                   size_t blocks, size_t block_size, size_t pages, size_t head_dim, void *stream);
TTB_API int ttb_paged_fill_cache(void *cache, const void *input, const void *page_table, const void *batch_idx, int dtype,
                                 int table_dtype, int batch_idx_dtype, size_t users, size_t heads, size_t seq,
                                 size_t blocks, size_t block_size, size_t table_rows, size_t pages, size_t head_dim,
                                 void *stream);
TTB_API int ttb_sdpa_decode_paged(const void *q, const void *k, const void *v, const void *page_table, const void *cur_pos,
                                  const void *mask, void *out, int dtype, int batch, int heads, int kv_heads, int blocks,
                                  int block_size, int pages_per_user, int head_dim, int mask_users, int mask_heads,
                                  float scale, int is_causal, void *workspace, size_t workspace_bytes, void *stream);

/* ---- indexing: ::ttnn::gather / scatter / sort / topk / sampling (runtime/lib/ttnn/operations/data_movement/
 * {gather,scatter,sort}.cpp, operations/reduction/{topk,sampling}.cpp; goldens tools/golden/mapping.py:5384-5437,
 * 5624-5640, 5927-5958, 5994-6019).
 *   ttb_gather   out[i] = x[..., index[i], ...] along `dim`; out has the index tensor's shape (torch.gather)
 *   ttb_scatter  out = x, then out[..., index[i], ...] (op)= src[i] along `dim`; reduce_type is the flatbuffer's
 *                ScatterReduceType: 7 plain scatter, 0 sum, 2 max, 3 min, 6 prod (the input's own value takes part).
 *                Duplicates are applied in increasing position along `dim`, the order of torch's CPU loop, so the
 *                result is the same on every run.  Sums and products of 16-bit tensors are accumulated in f32 and
 *                rounded once, as torch does; that takes a workspace of ttb_scatter_workspace_bytes.
 *   An index outside its dimension is skipped (gather: reads as 0) and reported by ttb_index_status (cleared on read).
 *   ttb_sort     every row of [rows, n] sorted (stable; NaN last ascending / first descending, as torch.sort);
 *                the first `take` values and / or positions of each row are written (take = n: a full sort;
 *                take = k with `descending` = largest: top-k).  Workspace: ttb_sort_workspace_bytes(rows, n).
 *   ttb_sampling one draw per row among `candidates` pre-selected logits: softmax(values / temp), the k most probable
 *                kept (k = 0 or >= candidates: all), of those the shortest prefix whose mass reaches p (p outside (0, 1):
 *                all), then inverse-CDF sampling with a counter-based generator of (seed, row); the result is the chosen
 *                candidate's entry of `indices`.  values / p / temp share `dtype`; k is UInt32.  At most 4096 candidates. */
TTB_API int ttb_gather(const void *x, const void *index, void *out, int dtype, int index_dtype, int rank,
                       const int64_t *x_shape, const int64_t *index_shape, int dim, void *stream);
TTB_API size_t ttb_scatter_workspace_bytes(int dtype, int reduce_type, size_t elements);
TTB_API int ttb_scatter(const void *x, const void *index, const void *src, void *out, int dtype, int index_dtype, int rank,
                        const int64_t *x_shape, const int64_t *index_shape, const int64_t *src_shape, int dim,
                        int reduce_type, void *workspace, size_t workspace_bytes, void *stream);
TTB_API int ttb_index_status(int *bad_index_seen);
TTB_API size_t ttb_sort_workspace_bytes(size_t rows, size_t n);
TTB_API int ttb_sort(const void *x, void *values, void *indices, int dtype, int index_dtype, size_t rows, size_t n,
                     size_t take, int descending, void *workspace, size_t workspace_bytes, void *stream);
TTB_API int ttb_sampling(const void *values, const void *indices, const void *k, const void *p, const void *temp, void *out,
                         int dtype, int index_dtype, int out_dtype, int rows, int candidates, uint64_t seed, void *stream);

/* ---- data movement: ::ttnn::permute / slice / concat / repeat / transpose
 * (runtime/lib/ttnn/operations/data_movement/). One gather kernel covers them: out is dense
 * row-major of `out_shape`; element (i0..ik) is read from in + in_offset + sum(i_d * in_strides[d]). */
TTB_API int ttb_strided_copy(const void *in, void *out, int elem_size, int rank,
                             const int64_t *out_shape, const int64_t *in_strides,
                             int64_t in_offset, void *stream);
/* Writes a dense `in` of `in_shape` into a window of a larger dense tensor (concat pieces). */
TTB_API int ttb_strided_scatter(const void *in, void *out, int elem_size, int rank,
                                const int64_t *in_shape, const int64_t *out_strides,
                                int64_t out_offset, void *stream);
/* ::ttnn::experimental::rotary_embedding (operations/transformer/rotary_embedding.cpp:28-29):
 * out = x*cos + rotate_half(x)*sin over [batch*heads, seq, head_dim]; cos/sin are
 * [seq, head_dim] (lib/Dialect/TTNN/Transforms/Fusing/RoPEFusingPattern.cpp:49-51). */
TTB_API int ttb_rotary_embedding(const void *x, const void *cos, const void *sin, void *out,
                                 int dtype, size_t batch_heads, size_t seq, size_t head_dim,
                                 void *stream);
/* The same with x read as [batch, heads, seq, head_dim] through element strides
 * {batch, head, seq} (head_dim contiguous, strides multiples of 16 bytes): a head split that is a
 * pure permutation of [batch, seq, heads, head_dim] needs no pass of its own.  out is dense. */
TTB_API int ttb_rotary_embedding_strided(const void *x, const void *cos, const void *sin, void *out,
                                         int dtype, size_t batch, size_t heads, size_t seq,
                                         size_t head_dim, const int64_t *x_strides3, void *stream);

/* ---- contractions: ::ttnn::matmul / ::ttnn::linear (operations/matmul/matmul.cpp:75-80,117-122).
 * C[b] = act(A[b]^(ta) * B[b]^(tb) + bias), f32 accumulation, one rounding to `c_dtype`.
 * A is [M,K] (or [K,M] when trans_a), B is [K,N] (or [N,K] when trans_b), both dense with the
 * given batch strides in elements (0 = broadcast).  `bias` (nullable) has N elements of
 * `bias_dtype`.  `act`: TTB_ACT_*.  `round_steps` is a bit mask that keeps a fused launch equal
 * to the op chain it replaces: bit 0 rounds to c_dtype after the product (a separate matmul op
 * would have stored it), bit 1 rounds again after the bias add (a separate add op).
 * bf16/f16 inputs whose shapes fit run on the tcgen05 tensor-core kernel; everything else
 * (f32, odd shapes) runs on the SIMT kernel. */
enum { TTB_ACT_NONE = 0, TTB_ACT_RELU = 1, TTB_ACT_SILU = 2, TTB_ACT_GELU = 3, TTB_ACT_SIGMOID = 4 };
TTB_API int ttb_gemm(const void *a, const void *b, const void *bias, void *c, int ab_dtype,
                     int bias_dtype, int c_dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                     int trans_a, int trans_b, int64_t a_batch_stride, int64_t b_batch_stride,
                     int act, int round_steps, void *stream);
/* Up to three products C_i[m, n_i] = A[m, k] * B_i[n_i, k]^T that share A (the q / k / v projections of
 * one activation) in one launch: their tiles form one list, so narrow problems fill the SMs a wide
 * one leaves idle.  Row-major, 16-bit A and B_i, no bias / activation.  Equivalent to `count` calls
 * of ttb_gemm with trans_b = 1 (which is what runs when the tensor-core kernel declines).
 * No reference counterpart (three ::ttnn::linear calls). */
TTB_API int ttb_gemm_grouped(const void *a, const void *const *b, void *const *c, const int64_t *n, int count,
                             int ab_dtype, int c_dtype, int64_t m, int64_t k, void *stream);

/* ttb_gemm_grouped with the rotary embedding of the results in `rope_mask` (bit i = problem i) applied in the
 * epilogue: the columns of C_i are heads of `head_dim` values, row r has position r mod seq, cos / sin are
 * [seq, head_dim] tables in `dtype`; each head becomes x cos + rotate_half(x) sin computed from the product rounded
 * to `dtype` (bit-equal to ttb_gemm_grouped followed by ttb_rotary_embedding_strided, but stored in the product's
 * own [m, n_i] layout).  TTB_ERR_UNSUPPORTED when the tensor-core kernel does not take the problem (head_dim other
 * than 128, n_i not whole heads, 32-bit types): run the two steps separately then.
 * No reference counterpart (::ttnn::linear followed by ::ttnn::experimental::rotary_embedding,
 * runtime/lib/ttnn/operations/transformer/rotary_embedding.cpp:11-37). */
TTB_API int ttb_gemm_grouped_rope(const void *a, const void *const *b, void *const *c, const int64_t *n, int count,
                                  int dtype, int64_t m, int64_t k, const void *cos, const void *sin, int rope_mask,
                                  int64_t seq, int64_t head_dim, void *stream);

/* out[m, n] = act(round(a1 * b1^T + bias1) + round(a2 * b2^T + bias2)), act = TTB_ACT_NONE or TTB_ACT_RELU: two
 * products that share their shape [m, n] (a1 [m, k1], b1 [n, k1]; a2 [m, k2], b2 [n, k2]; 16-bit, row-major; biases
 * [n] in `bias_dtype`, nullable), each rounded to `dtype` with its bias as its own op rounds it, then added, rounded
 * and activated -- a pointwise convolution plus the pointwise projection of its residual branch as one launch.
 * Bit-equal to ttb_gemm(a2, b2, bias2) followed by ttb_gemm_fused(a1, b1, bias1, extra = that, TTB_EXTRA_ADD[_RELU]).
 * TTB_ERR_UNSUPPORTED when the tensor-core kernel does not take the problem: run the ops one by one then.
 * No reference counterpart (two ::ttnn::conv2d calls, ::ttnn::add, ::ttnn::relu; operations/conv/conv2d.cpp:16-94). */
TTB_API int ttb_gemm_dual_add(const void *a1, const void *b1, const void *bias1, const void *a2, const void *b2,
                              const void *bias2, void *out, int dtype, int bias_dtype, int64_t m, int64_t n, int64_t k1,
                              int64_t k2, int act, void *stream);

/* ttb_gemm with a second, full-size epilogue operand `extra` ([batch, m, n], dense, in
 * `c_dtype`), combined with the result of the bias / activation chain the way separate ops
 * would (the chain's result is rounded to `c_dtype` first):
 *   TTB_EXTRA_ADD       c = round(result + extra)                  linear followed by ::ttnn::add (a residual)
 *   TTB_EXTRA_ADD_RELU  c = relu(round(result + extra))            ... followed by ::ttnn::relu
 *   TTB_EXTRA_SILU_MUL  c = round(round(silu(extra)) * result)     ::ttnn::silu + ::ttnn::multiply (SwiGLU gating)
 * On the tensor-core kernel this is one launch; elsewhere the elementwise kernels finish the job.
 * No reference counterpart: the reference runs these as separate ttnn ops. */
enum { TTB_EXTRA_NONE = 0, TTB_EXTRA_ADD = 1, TTB_EXTRA_SILU_MUL = 2, TTB_EXTRA_ADD_RELU = 3 };
TTB_API int ttb_gemm_fused(const void *a, const void *b, const void *bias, void *c, int ab_dtype,
                           int bias_dtype, int c_dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                           int trans_a, int trans_b, int64_t a_batch_stride, int64_t b_batch_stride,
                           int act, int round_steps, const void *extra, int extra_op, void *stream);
/* Quantized contraction: the ::ttnn::matmul / ::ttnn::linear call of runtime/lib/ttnn/operations/
 * matmul/matmul.cpp:75-80 when its operands are quantized (8-bit integers; the compiler moves the
 * dequantize below the op, lib/Dialect/TTIR/Transforms/QuantDequantConversion.cpp).  c = a b with exact
 * 32-bit integer accumulation; operands Int8 or UInt8, layouts as ttb_gemm.  c_dtype Int32 stores the
 * accumulators.  A float c_dtype stores round(float(acc) * scale) -- the dequantize op that follows,
 * fused: scale = deq_scale[column] (per output channel, f32) or deq_scalar when deq_scale is null.
 * The weight layout (trans_b, no trans_a, batch 1, k a multiple of 16) runs on the tensor cores
 * (tcgen05.mma kind::i8); everything else on a CUDA-core kernel.  Results are exact integers, so the two
 * agree bit for bit.  ttb_gemm_i8_simt forces the CUDA-core kernel (cross-check). */
TTB_API int ttb_gemm_i8(const void *a, const void *b, void *c, int a_dtype, int b_dtype, int c_dtype,
                        int64_t batch, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                        int64_t a_batch_stride, int64_t b_batch_stride, const float *deq_scale,
                        float deq_scalar, void *stream);
/* ttb_gemm_i8 with a float result, followed by + bias[n] (bias in a float type): a quantized linear layer
 * (::ttnn::matmul on the 8-bit values, ::ttnn::dequantize, ::ttnn::add) in one call; the dequantized
 * value is rounded to c_dtype before the bias is added, as the separate ops round. */
TTB_API int ttb_gemm_i8_bias(const void *a, const void *b, void *c, int a_dtype, int b_dtype, int c_dtype,
                             int64_t batch, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                             int64_t a_batch_stride, int64_t b_batch_stride, const float *deq_scale,
                             float deq_scalar, const void *bias, int bias_dtype, void *stream);
TTB_API int ttb_gemm_i8_simt(const void *a, const void *b, void *c, int a_dtype, int b_dtype, int c_dtype,
                             int64_t batch, int64_t m, int64_t n, int64_t k, int trans_a, int trans_b,
                             int64_t a_batch_stride, int64_t b_batch_stride, const float *deq_scale,
                             float deq_scalar, void *stream);
/* Health of the tensor-core kernel: every wait inside it is bounded, and a wait that gives up
 * records where.  *status == 0 means no launch of this process has timed out.  Synchronises. */
TTB_API int ttb_gemm_tcgen05_status(int *status);
/* Same contract, forced onto the SIMT kernel (reference implementation for the fast path). */
TTB_API int ttb_gemm_simt(const void *a, const void *b, const void *bias, void *c, int ab_dtype,
                          int bias_dtype, int c_dtype, int64_t batch, int64_t m, int64_t n,
                          int64_t k, int trans_a, int trans_b, int64_t a_batch_stride,
                          int64_t b_batch_stride, int act, int round_steps, void *stream);

/* ::ttnn::conv2d (runtime/lib/ttnn/operations/conv/conv2d.cpp:83-87; semantics
 * include/ttmlir/Dialect/TTIR/IR/TTIROps.td:3959-4033): NHWC activations [N,H,W,C], weights
 * [O, C/groups, kH, kW], bias with O elements (nullable), f32 accumulation, one rounding.
 * padding = {top, left, bottom, right}.  Implemented as a gather into GEMM operand layout
 * followed by the contraction kernel; 1x1 stride-1 convolutions go straight to the GEMM.
 * `workspace` must hold ttb_conv2d_workspace_bytes(...) bytes (0 bytes needed -> may be null). */
TTB_API size_t ttb_conv2d_workspace_bytes(int dtype, int64_t n, int64_t h, int64_t w, int64_t c,
                                          int64_t o, int kh, int kw, int stride_h, int stride_w,
                                          const int *padding4, int dil_h, int dil_w, int groups);
TTB_API int ttb_conv2d(const void *x, const void *weight, const void *bias, void *out, int dtype,
                       int bias_dtype, int64_t n, int64_t h, int64_t w, int64_t c, int64_t o,
                       int kh, int kw, int stride_h, int stride_w, const int *padding4, int dil_h,
                       int dil_w, int groups, int act, void *workspace, void *stream);
/* ttb_conv2d with the second epilogue operand of ttb_gemm_fused: `extra` is an NHWC tensor of the
 * output's shape and type (a residual branch), `extra_op` one of TTB_EXTRA_*. */
TTB_API int ttb_conv2d_fused(const void *x, const void *weight, const void *bias, void *out, int dtype,
                             int bias_dtype, int64_t n, int64_t h, int64_t w, int64_t c, int64_t o, int kh,
                             int kw, int stride_h, int stride_w, const int *padding4, int dil_h, int dil_w,
                             int groups, int act, const void *extra, int extra_op, void *workspace,
                             void *stream);

/* Convolution on quantized operands: the ::ttnn::conv2d call of runtime/lib/ttnn/operations/conv/
 * conv2d.cpp:16-94 when input and weight are quantized (8-bit integers; the compiler gives the op an i32
 * accumulator result type, lib/Dialect/TTIR/IR/TTIROps.cpp:1516-1577).  Layouts as ttb_conv2d; exact
 * 32-bit integer accumulation.  out_dtype Int32 stores the accumulators; a float out_dtype stores
 * round(float(acc) * scale), scale = deq_scale[output channel] or deq_scalar (the dequantize that follows,
 * fused).  `workspace`: ttb_conv2d_workspace_bytes with the input's dtype (0 for pointwise). */
TTB_API int ttb_conv2d_i8(const void *x, const void *weight, void *out, int x_dtype, int w_dtype, int out_dtype,
                          int64_t n, int64_t h, int64_t w, int64_t c, int64_t o, int kh, int kw, int stride_h,
                          int stride_w, const int *padding4, int dil_h, int dil_w, int groups,
                          const float *deq_scale, float deq_scalar, void *workspace, void *stream);

/* conv2d for callers that must not allocate.  No counterpart in the reference: tt-mlir's
 * runtime always lets the device library allocate its own intermediates.
 *
 * Some hosts of this library cannot call cudaMalloc at the point where they run a convolution:
 * code inside a latency-critical serving loop whose memory was handed out up front by an
 * arena it does not own, or a plugin whose embedding application forbids device allocation
 * after start-up.  ttb_conv2d needs a workspace for the gathered receptive fields and the
 * re-ordered weights; this variant takes that workspace from a fixed buffer of
 * TTB_CONV2D_STATIC_SCRATCH_BYTES that is part of the library's device image (each GPU that
 * loads the library carries it until the process ends) and otherwise behaves exactly like
 * ttb_conv2d -- same kernels, same results.  It calls no cudaMalloc / cudaFree and no
 * allocating library routine; the caller still supplies input, weight, bias and output.
 *
 *  - The buffer has two parts: the convolution's workspace in front and, at its end,
 *    TTB_CONV2D_STATIC_GEMM_BYTES for the partial sums that the CUDA-core contraction keeps when
 *    it splits a long reduction over several thread blocks (f32 convolutions and shapes too small
 *    or too ragged for the tensor-core kernel take that path; elsewhere that scratch comes from
 *    the memory pool).  A convolution whose workspace (ttb_conv2d_workspace_bytes) exceeds
 *    TTB_CONV2D_STATIC_SCRATCH_BYTES - TTB_CONV2D_STATIC_GEMM_BYTES is refused with
 *    TTB_ERR_INVALID and a message naming both sizes; so are extents that are not positive or
 *    whose byte count overflows.
 *  - The first call on each device looks up the buffer's device address; make that first
 *    call during start-up, before any stream capture begins.  The address is kept for the life
 *    of the process: do not use the library across a cudaDeviceReset of that device.
 *  - All calls share the one buffer and it keeps whatever the previous call left there.
 *    The split-reduction counters are the only part that must start at zero, and every call
 *    clears them on its stream before its kernels run; every other byte a launch reads was
 *    written by the same launch sequence before.  Two calls whose kernels overlap on the GPU
 *    (different streams) would overwrite each other's scratch; issue them on one stream or order
 *    them yourself. */
#define TTB_CONV2D_STATIC_SCRATCH_BYTES (32u << 20)
#define TTB_CONV2D_STATIC_GEMM_BYTES (4u << 20)
TTB_API int ttb_conv2d_static(const void *x, const void *weight, const void *bias, void *out,
                              int dtype, int bias_dtype, int64_t n, int64_t h, int64_t w, int64_t c,
                              int64_t o, int kh, int kw, int stride_h, int stride_w,
                              const int *padding4, int dil_h, int dil_w, int groups, int act,
                              void *stream);

/* ::ttnn::transformer::scaled_dot_product_attention
 * (runtime/lib/ttnn/operations/transformer/scaled_dot_product_attention.cpp:41-45; golden
 * tools/golden/mapping.py:8398-8500): out = softmax(q k^T * scale + mask) v with f32 softmax.
 * q [B,Hq,Sq,D], k/v [B,Hkv,Skv,D] (Hq a multiple of Hkv: grouped-query attention), out like q.
 * `mask` (nullable) is additive, [B or 1, Hq or 1, Sq, Skv] in `dtype`; `is_causal` masks j > i. */
TTB_API int ttb_sdpa(const void *q, const void *k, const void *v, const void *mask, void *out,
                     int dtype, int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q,
                     int64_t seq_kv, int64_t head_dim, int64_t mask_batch, int64_t mask_heads,
                     int is_causal, float scale, void *stream);
/* ::ttnn::transformer::flash_mla_prefill (operations/transformer/flash_mla_prefill.cpp; golden
 * tools/golden/mapping.py:8662-8692): q [B, Hq, Sq, Dqk], k [B, Hkv, Skv, Dqk], v [B, Hkv, Skv, Dv] or null (then the first
 * Dv columns of k), optional additive mask [B or 1, Hq or 1, Sq, Skv], out [B, Hq, Sq, Dv].  A CUDA-core kernel. */
TTB_API int ttb_flash_mla_prefill(const void *q, const void *k, const void *v, const void *mask, void *out, int dtype,
                                  int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv,
                                  int64_t head_dim_qk, int64_t head_dim_v, int64_t mask_batch, int64_t mask_heads,
                                  int is_causal, float scale, void *stream);
/* mask[u, 0, 0, j] = 0 for j <= cur_pos[u], -inf beyond: the additive mask of one decode step per user
 * (::ttnn::transformer::paged_flash_multi_latent_attention_decode builds the same from its cur_pos tensor). */
TTB_API int ttb_cur_pos_mask(void *mask, const int32_t *cur_pos, int dtype, int64_t users, int64_t seq_kv, void *stream);
/* ::ttnn::experimental::indexer_score_dsa (operations/transformer/indexer_score_dsa.cpp; golden
 * tools/golden/mapping.py:8695-8742): out[b, 0, s, t] = sum_h relu(q[b, h, s, :] . k[b, 0, t, :]) * weights[b, h, s, 0]
 * for keys t <= offset + s, -inf for later ones.  q [batch, heads, seq_q, head_dim], k [batch, 1, seq_kv, head_dim],
 * weights [batch, heads, seq_q, 1], out [batch, 1, seq_q, seq_kv]; bf16 or f16, f32 accumulation, one rounding.
 * `offset` is chunk_start_idx plus, on a mesh, the sequence positions held by the devices before this one. */
TTB_API int ttb_indexer_score_dsa(const void *q, const void *k, const void *weights, void *out, int dtype, int64_t batch,
                                  int64_t heads, int64_t seq_q, int64_t seq_kv, int64_t head_dim, int64_t offset, void *stream);
/* Causal attention of a prefill chunk that starts at position `offset`: query row r sees keys 0 .. r + offset
 * (::ttnn::transformer::chunked_scaled_dot_product_attention once its paged keys and values are gathered,
 * operations/transformer/chunked_scaled_dot_product_attention.cpp; golden tools/golden/mapping.py:8847-8912).  The
 * tensor-core kernel applies the offset itself; other problems build an additive mask in `workspace`
 * (ttb_sdpa_causal_offset_workspace_bytes) and take the general path. */
TTB_API size_t ttb_sdpa_causal_offset_workspace_bytes(int dtype, int64_t seq_q, int64_t seq_kv);
TTB_API int ttb_sdpa_causal_offset(const void *q, const void *k, const void *v, void *out, int dtype, int64_t batch,
                                   int64_t heads_q, int64_t heads_kv, int64_t seq_q, int64_t seq_kv, int64_t head_dim,
                                   int64_t offset, float scale, void *workspace, void *stream);
/* out[u, h, t, :] = cache[page_table[u, t / block_size], h, t % block_size, :]: the paged cache
 * [num_blocks, heads, block_size, head_dim] of every user as one sequence of max_blocks * block_size positions. */
TTB_API int ttb_paged_gather(const void *cache, const void *page_table, void *out, int dtype, int table_dtype, int64_t users,
                             int64_t heads, int64_t block_size, int64_t max_blocks, int64_t head_dim, int64_t num_blocks,
                             void *stream);
/* ttb_sdpa without a mask tensor, with every operand addressed as [batch, heads, seq, head_dim]
 * through element strides {batch, head, seq} (head_dim contiguous, strides multiples of 16 bytes).
 * Lets the caller skip the head split of q/k/v and the head merge of the output
 * (::ttnn::permute / ::ttnn::transformer::concatenate_heads around the attention op).
 * Returns TTB_ERR_UNSUPPORTED when no kernel takes the problem with these strides (the
 * tensor-core kernel needs head_dim 128 and a 16-bit type); dense strides always work. */
TTB_API int ttb_sdpa_strided(const void *q, const void *k, const void *v, void *out, int dtype,
                             int64_t batch, int64_t heads_q, int64_t heads_kv, int64_t seq_q,
                             int64_t seq_kv, int64_t head_dim, const int64_t *q_strides3,
                             const int64_t *k_strides3, const int64_t *v_strides3,
                             const int64_t *out_strides3, int is_causal, float scale, void *stream);

/* Status word of the tcgen05 attention kernel: 0, or (site << 8) | 1 of the first bounded wait
 * that ran out (the launch then produced no valid output).  No reference counterpart. */
TTB_API int ttb_sdpa_tcgen05_status(int *status);
/* Both tensor-core kernels (GEMM / convolution and attention) in one call, for the current device and
 * without a device-wide synchronise: the status words as above; clear != 0 resets a word that was
 * set, so that one timeout is reported once.  ttb_tcgen05_set_status writes the words the way a
 * timed-out launch would (zeros clear them): it lets the error path above the kernels be tested
 * without making a GPU wait run out.  ttb_tcgen05_set_wait_limit sets the limit of every bounded
 * wait in these kernels in SM clock cycles (<= 0: the default, 2e9 = about a second).
 * No reference counterpart (the reference's device timeouts live in tt-metal). */
TTB_API int ttb_tcgen05_status(int *gemm_status, int *sdpa_status, int clear);
TTB_API int ttb_tcgen05_set_status(int gemm_status, int sdpa_status);
TTB_API int ttb_tcgen05_set_wait_limit(long long cycles);

/* ---- collectives on a 1xN mesh: ::ttnn::all_reduce / all_gather / reduce_scatter
 * (runtime/lib/ttnn/operations/ccl/all_reduce.cpp:36-37, all_gather.cpp:38-41,
 * reduce_scatter.cpp:60-67).  Thin, status-returning wrappers over NCCL, which is loaded with
 * dlopen at first use.  `comm` is an ncclComm_t as void*; `id128` is a 128-byte ncclUniqueId.
 * `reduce_type` is the serialised ttcore::ReduceType: 0 sum, 1 mean, 2 max, 3 min. */
TTB_API int ttb_nccl_version(int *version);
TTB_API int ttb_nccl_unique_id(char *id128);
TTB_API int ttb_comm_init_rank(void **comm, int nranks, const char *id128, int rank);
TTB_API int ttb_comm_init_all(void **comms, int ndev, const int *devices);
TTB_API int ttb_comm_destroy(void *comm);
TTB_API int ttb_group_start(void);
TTB_API int ttb_group_end(void);
TTB_API int ttb_all_reduce(void *comm, const void *in, void *out, size_t count, int dtype,
                           int reduce_type, void *stream);
/* Concatenates each rank's `send_count` elements in rank order (gather along dimension 0). */
TTB_API int ttb_all_gather(void *comm, const void *in, void *out, size_t send_count, int dtype,
                           void *stream);
TTB_API int ttb_reduce_scatter(void *comm, const void *in, void *out, size_t recv_count, int dtype,
                               int reduce_type, void *stream);
TTB_API int ttb_broadcast(void *comm, const void *in, void *out, size_t count, int dtype, int root,
                          void *stream);
/* ---- mixture of experts (operations/ccl/all_to_all_dispatch.cpp, all_to_all_combine.cpp, moe_expert_token_remap.cpp;
 * operations/matmul/matmul.cpp ::ttnn::sparse_matmul).  `mapping` is the [experts, devices] one-hot ownership table as
 * Int32; a device numbers its own experts in ascending global order.
 * ttb_moe_local_index: local_idx[e] = this device's number for expert e, or -1.
 * ttb_moe_dispatch_mask: clears the rows of the gathered [rows, hidden] token buffer none of whose k experts
 *   (indices [rows, k], Int32) lives on this device -- the local half of ::ttnn::all_to_all_dispatch.
 * ttb_moe_combine_partial: partial[p, slot, b, s, :] = expert_out[local expert, token(p, b, s), :] when the expert in
 *   metadata[token, slot] lives here, else 0; summing the partials of all devices (one owner per expert) gives
 *   destination p's ::ttnn::all_to_all_combine result [k, batch, seq, hidden].  Tokens of destination p are its
 *   batch rows (seq_sharded = 0) or its sequence positions (seq_sharded = 1) of the global token grid.
 * ttb_moe_expert_token_remap: mapping[t, le] = topk[t, e] for the selected experts that live here (0 elsewhere),
 *   reduced[block, le] = 1 when a token of the block of `reduction` tokens selected local expert le.
 * ttb_sparse_matmul: c[i] = a[a_per_entry ? i : i / experts] (m x k) * b[i % experts] (k x n) for the `entries`
 *   whose sparsity[i] is non-zero; the others are cleared.  bf16 / f16, f32 accumulation, one rounding. */
TTB_API int ttb_moe_local_index(const int32_t *mapping, int32_t *local_idx, int experts, int devices, int device, void *stream);
/* ... from a table of owners instead (owner[e] = mesh coordinate of expert e; ::ttnn::all_to_all_dispatch_metadata). */
TTB_API int ttb_moe_local_index_owner(const int32_t *owner, int32_t *local_idx, int experts, int device, void *stream);
TTB_API int ttb_moe_dispatch_mask(void *tokens, const int32_t *indices, const int32_t *local_idx, int dtype, size_t rows,
                                  size_t hidden, int k, int experts, void *stream);
TTB_API int ttb_moe_combine_partial(const void *expert_out, const int32_t *metadata, const int32_t *local_idx, void *partial,
                                    int dtype, int devices, int k, int batch, int seq, size_t hidden, int experts,
                                    int local_experts, int seq_sharded, void *stream);
TTB_API int ttb_moe_expert_token_remap(const void *topk, const int32_t *metadata, const int32_t *local_idx, void *mapping,
                                       void *reduced, int dtype, int reduced_dtype, size_t tokens, int k, int experts,
                                       int local_experts, int reduction, void *stream);
TTB_API int ttb_sparse_matmul(const void *a, const void *b, const void *sparsity, void *c, int dtype, int sparsity_dtype,
                              int64_t entries, int64_t experts, int a_per_entry, int64_t m, int64_t n, int64_t k, void *stream);
/* ::ttnn::point_to_point (operations/ccl/point_to_point.cpp): the sender's half and the receiver's half of one copy. */
TTB_API int ttb_send(void *comm, const void *in, size_t count, int dtype, int peer, void *stream);
TTB_API int ttb_recv(void *comm, void *out, size_t count, int dtype, int peer, void *stream);

/* ---- all-reduce over peer memory (NVLink loads/stores, no NCCL in the data path).
 * A "symm" object is one rank's view of a set of workspaces, one per rank of a 1xN mesh, each
 * mapped by every other rank: CUDA IPC when ranks are processes (create_rank: collective, the
 * NCCL communicator only carries the 64-byte handles), peer access when one process drives all
 * devices (create_all).  `max_bytes` bounds the operand of one all-reduce; a workspace takes
 * 4 x max_bytes + 32 KiB.
 * ttb_symm_all_reduce: out = sum over ranks of in (f32 accumulation in rank order, so every rank
 * gets the same bits), or with `residual` (replicated, same shape) out = round(round(sum) +
 * residual), which is ::ttnn::all_reduce followed by ::ttnn::add.  Collective: every rank calls
 * it in the same order with the same count.  Returns TTB_ERR_UNSUPPORTED for operands it does
 * not take (type other than bf16/f16/f32, more than max_bytes, not 16-byte multiples).
 * Waits on peers are bounded; ttb_symm_status reports a wait that ran out ((phase << 8) | peer + 1).
 * Replaces, for sums, ::ttnn::all_reduce (runtime/lib/ttnn/operations/ccl/all_reduce.cpp:36-37). */
TTB_API int ttb_symm_create_rank(void **symm, void *comm, int rank, int nranks, size_t max_bytes,
                                 void *stream);
TTB_API int ttb_symm_create_all(void **symms, int ndev, const int *devices, size_t max_bytes);
TTB_API int ttb_symm_destroy(void *symm);
TTB_API size_t ttb_symm_max_bytes(void *symm);
/* Where the NEXT ttb_symm_all_reduce of this rank stages its operand.  A producer (the GEMM
 * before the all-reduce) that writes its result there and passes the same pointer as `in` saves
 * the all-reduce its staging copy.  The memory is only valid as that operand: it is reused two
 * all-reduces later. */
TTB_API int ttb_symm_input_buffer(void *symm, size_t bytes, void **ptr);
TTB_API int ttb_symm_status(void *symm, int *status);
/* The all-reduce numbers its launches, and its flags and staging regions follow that number: every
 * rank must be at the same count when a collective starts.  After a collective that some rank never
 * joined (a timeout), the ranks compare their counts on the host and all adopt the largest before the
 * next one.  Only between collectives, with none in flight. */
TTB_API int ttb_symm_launch_count(void *symm, uint32_t *launches);
TTB_API int ttb_symm_set_launch_count(void *symm, uint32_t launches);
/* Resets the status word after a reported timeout, so that later collectives are judged on their own. */
TTB_API int ttb_symm_clear_status(void *symm);
/* How long a barrier of this rank's all-reduce kernels may wait for a peer's flag, in SM clock cycles
 * (<= 0: the default, 2e9 = about a second).  A rank whose peers never launch returns after this long
 * with the status word set instead of hanging the GPU. */
TTB_API int ttb_symm_set_wait_limit(void *symm, long long cycles);
TTB_API int ttb_symm_all_reduce(void *symm, const void *in, const void *residual, void *out,
                                size_t count, int dtype, void *stream);
/* The fused producer path: the GEMM in front of an all-reduce stores each row block of its
 * partial result straight into the workspace of the rank that will reduce it (TMA stores over
 * NVLink from the GEMM's epilogue), so the reduce-scatter half of the exchange overlaps the GEMM.
 *   ttb_symm_push_targets(symm, bytes, targets, &rank, &n)  where this rank's partial of row block
 *       o goes (one pointer per rank; valid for the next all-reduce of `symm` only);
 *   ttb_gemm_push(a, b, targets, n, dtype, m, n_cols, k, stream)  C = A B^T scattered to the targets
 *       (needs m / n rows per block to be a multiple of 128; TTB_ERR_UNSUPPORTED otherwise);
 *   ttb_symm_all_reduce_pushed(symm, residual, out, count, dtype, stream)  sums the n partials of
 *       the own block locally, adds `residual` (nullable), shares the result with every rank. */
/* SwiGLU gating as one contraction: out[M, N] = silu(A Wg^T) * (A Wu^T) with Wg, Wu [N, K] (the
 * "transpose_b" layout), bf16 / f16.  Fuses linear(x, Wg), linear(x, Wu), silu, multiply of
 * runtime/lib/ttnn/operations/{matmul/matmul.cpp:86-125, eltwise/unary, eltwise/binary} and rounds
 * where those ops round. */
TTB_API int ttb_gemm_swiglu(const void *a, const void *w_gate, const void *w_up, void *out, int dtype,
                            int64_t m, int64_t n, int64_t k, void *stream);
TTB_API int ttb_symm_push_targets(void *symm, size_t bytes, void **targets, int *rank, int *nranks);
TTB_API int ttb_gemm_push(const void *a, const void *b, void *const *targets, int nranks, int ab_dtype,
                          int64_t m, int64_t n, int64_t k, void *stream);
TTB_API int ttb_symm_all_reduce_pushed(void *symm, const void *residual, void *out, size_t count,
                                       int dtype, void *stream);
/* The reduce-scatter half alone, for an all_reduce whose result is only read through a mesh_partition along the
 * same mesh axis (runtime/lib/ttnn/operations/ccl/{all_reduce.cpp:13-39, mesh_partition.cpp:13-29} back to back):
 * `out` receives this rank's slice of the sum only -- count / nranks elements, block `rank` of the flattened
 * operand -- plus the matching part of `residual` ([count], nullable).  Nothing is pushed to the peers; the second
 * barrier and the final copy of ttb_symm_all_reduce fall away.  `count` must split into 16-byte aligned slices. */
TTB_API int ttb_symm_reduce_scatter(void *symm, const void *in, const void *residual, void *out, size_t count, int dtype,
                                    void *stream);
TTB_API int ttb_symm_reduce_scatter_pushed(void *symm, const void *residual, void *out, size_t count, int dtype,
                                           void *stream);

#ifdef __cplusplus
}
#endif

#endif /* TTB_KERNELS_H */
