/*
 * ovk_cuda.h - C ABI of the B200 (sm_100a) quantized matrix-product library.
 *
 * This is the CUDA sibling of the reference's kernel-launch layer
 * (crates/vk-compute) narrowed to the four quantized operators of
 * crates/onnx-vulkan-core/src/interp.rs: MatMulNBits, DynamicQuantizeLinear,
 * MatMulInteger (+ fused scale/bias epilogue) and QLinearConv / ConvInteger.
 * Every entry point names the reference interface it replaces.
 *
 * Conventions
 *  - plain pointers and sizes only; device pointers are ordinary CUDA device
 *    addresses (they survive the pointer arithmetic ONNX Runtime performs on
 *    allocations, so no handle table like crates/vulkan-ep/src/device_mem.rs
 *    :100-176 is needed);
 *  - every call returns an ovk_status; the message is read with
 *    ovk_last_error(); nothing throws across the boundary;
 *  - operator calls only ENQUEUE on the context's stream (as
 *    vk-compute stream_dispatch, crates/vk-compute/src/stream.rs:370-398);
 *    only ovk_flush and ovk_download wait (flush :702, stream_download :773);
 *  - dtype codes are the reference's ElementType values
 *    (crates/onnx-vulkan-core/src/graph.rs:13-41);
 *  - there is no CPU fallback: a form the kernels do not cover returns
 *    OVK_UNSUPPORTED before anything is launched (the reference's fail-loud
 *    rule, README.md:328-336).
 */
#ifndef OVK_CUDA_H
#define OVK_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define OVK_API
#else
#define OVK_API __attribute__((visibility("default")))
#endif

typedef enum ovk_status {
    OVK_OK = 0,
    OVK_INVALID_ARGUMENT = 1, /* bad shape / pointer / alignment (anyhow ensure! failures) */
    OVK_UNSUPPORTED = 2,      /* a form refused at load time by the reference too */
    OVK_BACKEND = 3,          /* a CUDA call failed (core::Error::Backend, src/error.rs:6-14) */
    OVK_TIMEOUT = 4           /* a bounded device-side wait gave up; the context stays usable */
} ovk_status;

typedef enum ovk_dtype {
    OVK_FLOAT = 1,
    OVK_UINT8 = 2,
    OVK_INT8 = 3,
    OVK_INT32 = 6,
    OVK_INT64 = 7,
    OVK_FLOAT16 = 10
} ovk_dtype;

typedef struct ovk_ctx ovk_ctx;
typedef struct ovk_nbits_weight ovk_nbits_weight;
typedef struct ovk_mmi_weight ovk_mmi_weight;
typedef struct ovk_qconv_weight ovk_qconv_weight;

/* ------------------------------------------------------------------ context
 * Replaces VkContext::new (crates/vk-compute/src/context.rs:360): one device,
 * one in-order stream.  `stream` may be an existing cudaStream_t (e.g. the
 * stream ONNX Runtime or torch is using) or NULL to create one. */
OVK_API int32_t ovk_ctx_create(int32_t device, void *stream, ovk_ctx **out);
OVK_API void ovk_ctx_destroy(ovk_ctx *ctx);
/* Message of the last failed call on this context (or on context creation when ctx is NULL). */
OVK_API const char *ovk_last_error(const ovk_ctx *ctx);
/* Name of the kernel variant the last operator call selected (the role of
 * KernelCache::pipeline_keys in the reference's routing tests,
 * crates/onnx-vulkan-core/tests/conv_integer_im2col.rs:163-178). */
OVK_API const char *ovk_last_kernel(const ovk_ctx *ctx);
/* Number of kernels this context has launched since it was created. */
OVK_API uint64_t ovk_launch_count(const ovk_ctx *ctx);
/* The cudaStream_t operator calls are enqueued on. */
OVK_API void *ovk_stream(const ovk_ctx *ctx);
/* Bytes of the context's grow-on-demand device workspace (row sums, the padded
 * channels-last image of a convolution, split-K partial sums); 0 until an
 * operator needed one.  A diagnostic without a counterpart in the reference,
 * whose buffers come from a recycling pool (crates/vk-compute/src/buffer.rs:303). */
OVK_API size_t ovk_workspace_bytes(const ovk_ctx *ctx);

/* flush (stream.rs:702): wait for everything enqueued; also reports a
 * device-side wait that timed out (OVK_TIMEOUT). */
OVK_API int32_t ovk_flush(ovk_ctx *ctx);
/* Exercises the failure report without a failure: enqueues a one-thread kernel
 * that waits, with a limit of 1000 polls, on a barrier nothing arrives at, and
 * records that the wait ran out.  The next ovk_flush returns OVK_TIMEOUT with
 * a message naming the self-test; the context stays usable.  (The reference
 * has no device-side waits; its failure report is the Result of flush,
 * crates/vk-compute/src/stream.rs:702.) */
OVK_API int32_t ovk_selftest_device_timeout(ovk_ctx *ctx);
/* Measures what the tensor core delivers: multiply-accumulates per clock per SM
 * of back-to-back 128 x 256 tcgen05.mma over operands resident in shared
 * memory, for dtype OVK_INT8 (kind::i8) or OVK_FLOAT16 (kind::f16).  Waits for
 * the result.  Times SMs times the SM clock it is the dense peak the int8
 * kernels are measured against.  (The reference measures its own ceiling the
 * same way in crates/onnx-vulkan-core/examples/conv_integer_coop.rs; its library has no counterpart.) */
OVK_API int32_t ovk_probe_mma_rate(ovk_ctx *ctx, int32_t dtype, double *mac_per_clk_per_sm);
/* create_storage_buffer (buffer.rs:239) / recycle_storage_buffer (:303) */
OVK_API int32_t ovk_alloc(ovk_ctx *ctx, size_t bytes, void **dptr);
OVK_API int32_t ovk_free(ovk_ctx *ctx, void *dptr);
/* stream_upload_at (stream.rs:310-367), stream_download_into (:918, waits),
 * stream_fill (:481; bytes and offset multiples of 4) */
OVK_API int32_t ovk_upload(ovk_ctx *ctx, void *dst, size_t offset, const void *src, size_t bytes);
OVK_API int32_t ovk_download(ovk_ctx *ctx, const void *src, size_t offset, void *dst, size_t bytes);
OVK_API int32_t ovk_fill(ovk_ctx *ctx, void *dst, size_t offset, size_t bytes, uint32_t value);
/* measure_dispatch_gpu (pipeline.rs:246): device time between the two calls, in ms. */
OVK_API int32_t ovk_timer_start(ovk_ctx *ctx);
OVK_API int32_t ovk_timer_stop(ovk_ctx *ctx, float *ms);

/* -------------------------------------------------------------- MatMulNBits
 * interp::matmul_nbits (crates/onnx-vulkan-core/src/interp.rs:6429-6561) and
 * its predicate (:452-464).
 *
 * B is [N, n_blocks, block_size/2] u8 with element 2i in the low nibble,
 * scales [N*n_blocks] f32 or f16, zero_points [N, ceil(n_blocks/2)] u8 nibble
 * packed (NULL = implicit 8), all device pointers in the operator's own
 * layout.  prepack plays the role packed_b (:2712) plays for MatMulInteger: it
 * is called once per weight and may build a decode-friendly copy.  The
 * original three buffers must stay alive as long as the weight object.
 * bits must be 4, block_size a positive multiple of 8. */
#define OVK_NBITS_DEFAULT 0u
#define OVK_NBITS_NO_DECODE_COPY 1u /* keep only the operator layout (generic kernels) */
OVK_API int32_t ovk_nbits_prepack(ovk_ctx *ctx, const void *b, const void *scales,
                                  int32_t scales_dtype, const void *zero_points, int64_t n,
                                  int64_t k, int64_t bits, int64_t block_size, uint32_t flags,
                                  ovk_nbits_weight **out);
OVK_API void ovk_nbits_weight_destroy(ovk_ctx *ctx, ovk_nbits_weight *w);
/* Y[M,N] = A[M,K] x dequant(B).  a_dtype / y_dtype: OVK_FLOAT or OVK_FLOAT16.
 * Routes M = 1 (decode, matrix-vector) and M > 1 (prefill) internally, as
 * shaders::matmul_nbits::route (shaders/matmul_nbits.rs:430-436) does. */
OVK_API int32_t ovk_matmul_nbits(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a,
                                 int32_t a_dtype, int64_t m, void *y, int32_t y_dtype);

/* The same product for up to four weights that read the SAME activations (the
 * q, k and v projections of a decoder layer, gate and up): Y_j = A x dequant(B_j).
 * Results are those of one ovk_matmul_nbits call per weight.  When the decode
 * kernel applies (M <= 8) and the weights share K, block size and tile shape,
 * all of them run in ONE launch, which in a decode step saves a dependent
 * launch per extra weight; otherwise the calls are made one by one.  This entry
 * point has no counterpart in the reference, whose interpreter dispatches
 * MatMulNBits nodes one at a time (interp.rs:1071). */
OVK_API int32_t ovk_matmul_nbits_group(ovk_ctx *ctx, int32_t count,
                                       const ovk_nbits_weight *const *weights, const void *a,
                                       int32_t a_dtype, int64_t m, void *const *ys, int32_t y_dtype);

/* ------------------------------------- several GPUs of one box (no counterpart)
 * The reference drives one device per process (crates/vk-compute/src/context.rs
 * :685-711) and has no exchange step; these verbs are what the column-split
 * MatMulNBits prefill needs from a host that runs one process per GPU.
 *
 * Buffers that other ranks write into - every rank's copy of Y, and one flag
 * block per rank - come from ovk_comm_alloc (cudaMalloc, zero filled).
 * ovk_comm_export turns one into a 64-byte handle the host hands to the other
 * processes over any channel it has (the role an ncclUniqueId plays);
 * ovk_comm_import maps a peer's buffer here and ovk_comm_release unmaps it.
 * ovk_comm_init then makes the context rank `rank` of `world` (at most 8):
 * flag_blocks[r] is rank r's flag block (ovk_comm_flag_bytes() bytes, 256-byte
 * aligned, zero), flag_blocks[rank] this context's own.  Collective calls
 * (ovk_matmul_nbits_nsplit, ovk_allgather_cols, ovk_comm_barrier) must be made in
 * the same order by every rank; each is enqueued like any operator call and
 * ends with a wait, on the device, for the peers' stores - bounded by the
 * time-out (about a second unless set), after which the stream goes on and the
 * next ovk_flush returns OVK_TIMEOUT.  Peer memory is only ever touched by plain
 * loads and stores of this library's own kernels. */
#define OVK_COMM_HANDLE_BYTES 64
#define OVK_COMM_MAX_RANKS 8
OVK_API size_t ovk_comm_flag_bytes(void);
OVK_API int32_t ovk_comm_alloc(ovk_ctx *ctx, size_t bytes, void **dptr);
OVK_API int32_t ovk_comm_export(ovk_ctx *ctx, void *dptr, void *handle_out);
OVK_API int32_t ovk_comm_import(ovk_ctx *ctx, const void *handle, void **peer_ptr);
OVK_API int32_t ovk_comm_release(ovk_ctx *ctx, void *peer_ptr);
OVK_API int32_t ovk_comm_init(ovk_ctx *ctx, int32_t rank, int32_t world, void *const *flag_blocks);
OVK_API int32_t ovk_comm_set_timeout_ms(ovk_ctx *ctx, int32_t ms);
/* Every rank's earlier work on its stream is complete when the barrier has passed. */
OVK_API int32_t ovk_comm_barrier(ovk_ctx *ctx);
/* The exchange step of a column split: this rank's block y_shard [m, n_shard]
 * (contiguous; NULL = it already sits in columns [col0, col0 + n_shard) of this
 * rank's own matrix) is stored into those columns of EVERY rank's matrix
 * y_peers[r] ([m, n_total], row major), and the stream then waits until every
 * peer has done the same here.  dtype: OVK_FLOAT16, OVK_FLOAT or OVK_INT32. */
OVK_API int32_t ovk_allgather_cols(ovk_ctx *ctx, const void *y_shard, int32_t dtype, int64_t m,
                                   int64_t n_shard, int64_t col0, int64_t n_total,
                                   void *const *y_peers);
/* The same exchange with one store per 16 bytes instead of one per rank:
 * y_multicast is a multicast mapping of the ranks' matrices (NVLink SHARP: an
 * address the NVSwitch resolves to the same offset of every rank's buffer, set
 * up by the host with the driver's multicast objects, or taken from a runtime
 * that has - torch's symmetric memory gives one).  A block leaves this GPU's
 * links once and the switch delivers it to every rank, this one included.
 * y_peers is still needed (the flags and the ragged-edge stores use plain peer
 * mappings); NULL for y_multicast is ovk_allgather_cols. */
OVK_API int32_t ovk_allgather_cols_multicast(ovk_ctx *ctx, const void *y_shard, int32_t dtype,
                                             int64_t m, int64_t n_shard, int64_t col0,
                                             int64_t n_total, void *const *y_peers,
                                             void *y_multicast);
/* MatMulNBits split over weight columns: w holds columns [col0, col0 + N_w) of
 * the operator's weight (a plain slice of its three tensors), A is the whole
 * [m, K] activation matrix on every rank, and the call leaves the whole
 * Y [m, n_total] in every rank's y_peers[r].  For fp16 results of the prefill
 * kernel with per-block scaling (block sizes 128 and 256, or f32 scales) the
 * kernel's own store warp writes each finished tile into every rank's matrix,
 * so the exchange overlaps the product (up to four ranks: with more peers per
 * store warp the two steps measured faster one after the other); other forms
 * compute the block and then run the exchange of ovk_allgather_cols.  Results are those of ovk_matmul_nbits
 * on the unsplit weight (the same kernel on the same columns). */
OVK_API int32_t ovk_matmul_nbits_nsplit(ovk_ctx *ctx, const ovk_nbits_weight *w, const void *a,
                                        int32_t a_dtype, int64_t m, int64_t col0, int64_t n_total,
                                        void *const *y_peers, int32_t y_dtype);
/* The same with the tiles stored through a multicast mapping of the ranks'
 * matrices (see ovk_allgather_cols_multicast): one store per 16 bytes from the
 * kernel's store warp, whatever the number of ranks. */
OVK_API int32_t ovk_matmul_nbits_nsplit_multicast(ovk_ctx *ctx, const ovk_nbits_weight *w,
                                                  const void *a, int32_t a_dtype, int64_t m,
                                                  int64_t col0, int64_t n_total,
                                                  void *const *y_peers, void *y_multicast,
                                                  int32_t y_dtype);

/* ------------------------------------------------- DynamicQuantizeLinear
 * interp::dynamic_quantize / quantize_on_device (interp.rs:1945-2085) with the
 * PARTIAL and QUANTIZE passes of shaders/dynamic_quantize.rs:106-222.  x, y,
 * y_scale (1 f32) and y_zero_point (1 u8) are device pointers; the results
 * stay on the device.  n = 0 writes scale 1, zero point 0 (:1949-1966). */
OVK_API int32_t ovk_dynamic_quantize(ovk_ctx *ctx, const float *x, int64_t n, uint8_t *y,
                                     float *y_scale, uint8_t *y_zero_point);
/* The same when the kernel that produced x has already folded its range into
 * `range` (OVK_EPILOGUE_RANGE of the fused MatMulInteger / ConvInteger nodes):
 * the range pass is skipped, as quantize_on_device skips it for a tensor with a
 * computed range (interp.rs:1979-1983, ExecutionEnv::set_range execution.rs:107).
 * `range` is a slot of four u32 (16 bytes) on the device, zero before the
 * producer runs; this call leaves it zero again, ready for the next producer -
 * so a folded range serves ONE quantization. */
OVK_API int32_t ovk_dynamic_quantize_folded(ovk_ctx *ctx, const float *x, int64_t n, uint32_t *range,
                                            uint8_t *y, float *y_scale, uint8_t *y_zero_point);
/* interp::decomposed_gelu (interp.rs:9060-9084, shader shaders/elementwise.rs:71-118):
 * the exact GELU as the graph spells it, Div -> Erf -> Add -> Mul -> Mul, in one
 * pass with every step rounded on its own: e = erf(x / divisor) + offset;
 * out = factor_first ? x * (e * factor) : (x * e) * factor, erf by the five-term
 * rational approximation the reference uses. */
OVK_API int32_t ovk_decomposed_gelu(ovk_ctx *ctx, const float *x, int64_t n, float divisor,
                                    float offset, float factor, int32_t factor_first, float *out);
/* interp::decomposed_gelu_quantize (interp.rs:9125-9150; rewrite.rs:699-735;
 * shaders/dynamic_quantize.rs:224-247): DynamicQuantizeLinear(DecomposedGelu(x))
 * as one node.  Both passes compute the GELU from x again, with the function
 * ovk_decomposed_gelu applies, so the f32 GELU - the largest tensor of a
 * transformer MLP - is never stored and every byte equals the two nodes'. */
OVK_API int32_t ovk_decomposed_gelu_quantize(ovk_ctx *ctx, const float *x, int64_t n, float divisor,
                                             float offset, float factor, int32_t factor_first,
                                             uint8_t *y, float *y_scale, uint8_t *y_zero_point);

/* ----------------------------------------------------------- MatMulInteger
 * packed_b (interp.rs:2712-2768, shader PACK_B shaders/matmul_integer.rs
 * :135-158): B [K,N] u8/i8 constant -> tensor-core layout, once per weight. */
OVK_API int32_t ovk_mmi_prepack(ovk_ctx *ctx, const void *b, int32_t b_signed, int64_t k,
                                int64_t n, ovk_mmi_weight **out);
OVK_API void ovk_mmi_weight_destroy(ovk_ctx *ctx, ovk_mmi_weight *w);
/* interp::matmul_integer (interp.rs:2090-2183): out[M,N] i32 = sum_k (a - a_zp)(b - b_zp).
 * a_zp / b_zp point to ONE byte each on the device (per-tensor, read by the
 * kernel without a read-back); NULL means 0. */
OVK_API int32_t ovk_matmul_integer(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a,
                                   int32_t a_signed, int64_t m, const void *a_zp,
                                   const void *b_zp, int32_t *out);
/* The same product for callers that must not allocate device memory (this
 * entry point has no counterpart in the reference).  ovk_matmul_integer keeps
 * the row sums it needs for a non-zero weight zero point in the context's
 * workspace, which grows with cudaMallocAsync on demand; hosts that hand out
 * every device byte from their own arena, or that cannot take an allocation
 * (and the synchronisation it may bring) inside a request, call this instead.
 * The row sums then live in a fixed array of 65536 int32 (256 KB) that is part
 * of the library image on every GPU that loads it.  It calls no cudaMalloc,
 * cudaFree or allocating library routine.
 *  - m above 65536 rows is refused with OVK_INVALID_ARGUMENT;
 *  - the first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress); make that first call before any stream capture;
 *  - all calls share the one array: calls whose kernels may overlap on the GPU
 *    (different streams or contexts) race on it - serialise them.  The array
 *    keeps the previous call's row sums; they are rewritten before they are
 *    read, so nothing has to be cleared;
 *  - two host threads making the first call on a device at the same time both
 *    look the address up and store the same value: harmless;
 *  - it always runs the 128-row tiles, never the 256 x 256 tiles
 *    ovk_matmul_integer picks for long K and many tiles, so on such shapes it
 *    is slower.
 * Results are identical to ovk_matmul_integer. */
OVK_API int32_t ovk_matmul_integer_static_scratch(ovk_ctx *ctx, const ovk_mmi_weight *w,
                                                  const void *a, int32_t a_signed, int64_t m,
                                                  const void *a_zp, const void *b_zp, int32_t *out);
/* interp::matmul_integer_scale_bias (interp.rs:2405-2572): the fused
 * MatMulInteger -> Cast -> Mul -> Add [-> Relu] node,
 *   out = fl(fl(float(acc) * s) + bias),  s = scale or fl(scale * product),
 * bit-identical to the unfused graph.  A step is 0 (one value) or 1 (one per
 * column), as interp::column_step (:2600-2610); other broadcasts are refused
 * (the reference runs them unfused).  range (may be NULL) is a zero-initialised
 * slot of four u32 whose first two receive the bits of max(-min,0) and
 * max(max,0) of the stored values by atomic max, for the
 * ovk_dynamic_quantize_folded that follows. */
#define OVK_EPILOGUE_RELU 1u
#define OVK_EPILOGUE_RANGE 2u
OVK_API int32_t ovk_matmul_integer_scale_bias(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a,
                                              int32_t a_signed, int64_t m, const void *a_zp,
                                              const void *b_zp, const float *scale,
                                              int32_t scale_step, const float *product,
                                              int32_t product_step, const float *bias,
                                              int32_t bias_step, uint32_t flags, uint32_t *range,
                                              float *out);
/* interp::integer_scale_bias_unfused (interp.rs:2630-2665): what the reference
 * runs when a scale, product or bias broadcasts over rows and the fused node
 * does not apply - Cast, Mul, Add [, Relu] over the int32 result of
 * ovk_matmul_integer / ovk_conv_integer, here as one pass:
 *   out[r][c] = fl(fl(float(acc[r][c]) * s) + bias),  s = scale or fl(scale * product),
 * every operand addressed by (row stride, column stride) in elements: {0, 0} one
 * value, {0, 1} one per column, {1, 0} one per row, {cols, 1} a full matrix.
 * Same bits as the separate nodes.  No range is folded (flags: OVK_EPILOGUE_RELU only). */
OVK_API int32_t ovk_integer_scale_bias_unfused(ovk_ctx *ctx, const int32_t *acc, int64_t rows,
                                               int64_t cols, const float *scale,
                                               int64_t scale_row_stride, int64_t scale_col_stride,
                                               const float *product, int64_t product_row_stride,
                                               int64_t product_col_stride, const float *bias,
                                               int64_t bias_row_stride, int64_t bias_col_stride,
                                               uint32_t flags, float *out);
/* The same products for up to four weights that read the SAME A - the q, k and
 * v projections over one DynamicQuantizeLinear result: out_j = A x B_j with the
 * members' own column constants.  One launch when every member takes the
 * 128-row tensor-core tiles (then a member's tiles are just more tiles of the
 * same grid, which also fills the SMs better than three narrow products), one
 * call per member otherwise; results are those of separate calls.  scale_step
 * and bias_step apply to every member; product is one value (NULL: none); no
 * range is folded.  No counterpart in the reference, whose interpreter
 * dispatches MatMulInteger nodes one at a time (interp.rs:1071). */
OVK_API int32_t ovk_matmul_integer_group(ovk_ctx *ctx, int32_t count,
                                         const ovk_mmi_weight *const *weights, const void *a,
                                         int32_t a_signed, int64_t m, const void *a_zp,
                                         const void *b_zp, int32_t *const *outs);
OVK_API int32_t ovk_matmul_integer_scale_bias_group(ovk_ctx *ctx, int32_t count,
                                                    const ovk_mmi_weight *const *weights,
                                                    const void *a, int32_t a_signed, int64_t m,
                                                    const void *a_zp, const void *b_zp,
                                                    const float *const *scales, int32_t scale_step,
                                                    const float *product, int32_t product_step,
                                                    const float *const *biases, int32_t bias_step,
                                                    uint32_t flags, float *const *outs);
/* interp::qlinear_matmul (interp.rs:4845-4875): MatMulInteger then
 * requantize(inner = 1, axis_len = ratio_len); ratio is a device array of
 * ratio_len (1 or N) floats computed by the caller as (a_scale*b_scale)/y_scale. */
OVK_API int32_t ovk_qlinear_matmul(ovk_ctx *ctx, const ovk_mmi_weight *w, const void *a,
                                   int32_t a_signed, int64_t m, const void *a_zp,
                                   const void *b_zp, const float *ratio, int64_t ratio_len,
                                   int32_t y_zp, int32_t y_signed, void *out);

/* ------------------------------------------------ ConvInteger / QLinearConv
 * Geometry follows interp::conv_geometry (interp.rs:3439-3536): x is NCHW
 * (a 1-D convolution is passed with W = 1, KW = 1), w is
 * [C_out, C_in/group, KH, KW]; pads = {h_begin, w_begin, h_end, w_end}
 * already resolved from auto_pad by the caller. */
typedef struct ovk_conv_params {
    int64_t n, c_in, h, w;
    int64_t pads[4];
    int64_t strides[2];
    int64_t dilations[2];
} ovk_conv_params;
OVK_API int32_t ovk_qconv_prepack(ovk_ctx *ctx, const void *w, int32_t w_signed, int64_t c_out,
                                  int64_t c_in_per_group, int64_t kh, int64_t kw, int64_t group,
                                  ovk_qconv_weight **out);
OVK_API void ovk_qconv_weight_destroy(ovk_ctx *ctx, ovk_qconv_weight *w);
/* Output spatial size for these parameters; OVK_INVALID_ARGUMENT when degenerate. */
OVK_API int32_t ovk_conv_output_shape(const ovk_qconv_weight *w, const ovk_conv_params *p,
                                      int64_t *h_out, int64_t *w_out);
/* interp::conv_integer_with (interp.rs:4421-4651): i32 accumulators, NCHW. */
OVK_API int32_t ovk_conv_integer(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x,
                                 int32_t x_signed, const ovk_conv_params *p, int32_t x_zp,
                                 int32_t w_zp, int32_t *out);
/* interp::conv_integer_scale_bias (interp.rs:4359-4420): the fused
 * ConvInteger -> Cast -> Mul -> Add [-> Relu] node,
 *   out[n,c,h,w] = fl(fl(float(acc) * s[c]) + bias[c]),  s = scale or fl(scale * product),
 * bit-identical to the unfused graph.  A step is 0 (one value) or 1 (one per
 * output channel), the two broadcasts interp::channel_step (:4404-4417) takes;
 * others are refused (the reference runs them unfused).  flags and range as in
 * ovk_matmul_integer_scale_bias. */
OVK_API int32_t ovk_conv_integer_scale_bias(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x,
                                            int32_t x_signed, const ovk_conv_params *p, int32_t x_zp,
                                            int32_t w_zp, const float *scale, int32_t scale_step,
                                            const float *product, int32_t product_step,
                                            const float *bias, int32_t bias_step, uint32_t flags,
                                            uint32_t *range, float *out);
/* interp::qlinear_conv (interp.rs:4796-4837) = ConvInteger + requantize
 * (interp.rs:4714-4788, shaders/qlinear.rs:28-63):
 *   y = sat(rne(f32(acc + bias[c]) * ratio[c]) + y_zp).
 * ratio is a HOST array of C_out floats, (x_scale*w_scale[c])/y_scale computed
 * in f32 left to right as interp::requantize_ratio (:4682-4694) does; bias is
 * a device array of C_out int32 or NULL. */
OVK_API int32_t ovk_qlinear_conv(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x,
                                 int32_t x_signed, const ovk_conv_params *p, int32_t x_zp,
                                 int32_t w_zp, const float *ratio_host, const int32_t *bias,
                                 int32_t y_zp, int32_t y_signed, void *y);
/* QLinearConv over channels-last tensors.  The reference keeps activations
 * channels-last between the layers of its tensor path (to_hwc once, then HWC
 * from layer to layer: shaders/conv_integer.rs:485-527, interp.rs:5719-5748);
 * here the layout is "padded NHWC": [n][h + top + bottom][w + left + right][c]
 * with the frame holding the tensor's zero point - exactly what the
 * tensor-core kernel computes from, so a layer that receives it skips the
 * layout pass, and a layer that produces it writes 16 channels per store
 * straight into the interior of the next layer's input (whose frame the caller
 * filled once with that layer's x_zero_point = this layer's y_zero_point).
 *  - x_layout OVK_LAYOUT_PADDED_NHWC: x is padded NHWC whose frame is p->pads;
 *  - y_layout OVK_LAYOUT_PADDED_NHWC: y is padded NHWC with frame y_pads
 *    {top, left, bottom, right}; only its interior is written; C_out must be a
 *    multiple of 16.
 * Either layout may be OVK_LAYOUT_NCHW (then this is ovk_qlinear_conv).  Taken
 * by the group-1, symmetric-weight tensor-core kernel (strides up to 4);
 * other geometries are refused with OVK_UNSUPPORTED in a channels-last layout.  Same bytes as
 * ovk_qlinear_conv. */
#define OVK_LAYOUT_NCHW 0
#define OVK_LAYOUT_PADDED_NHWC 1
OVK_API int32_t ovk_qlinear_conv_layout(ovk_ctx *ctx, const ovk_qconv_weight *w, const void *x,
                                        int32_t x_signed, int32_t x_layout, const ovk_conv_params *p,
                                        int32_t x_zp, int32_t w_zp, const float *ratio_host,
                                        const int32_t *bias, int32_t y_zp, int32_t y_signed, void *y,
                                        int32_t y_layout, const int64_t *y_pads);
/* The two ends of a channels-last chain (to_hwc, shaders/conv_integer.rs:485-527):
 * NCHW u8/i8 [n, c, h, w] -> padded NHWC with the frame set to the byte `fill`,
 * and back (the frame is dropped).  c a multiple of 4; out 16-byte aligned. */
OVK_API int32_t ovk_nchw_to_padded_nhwc(ovk_ctx *ctx, const void *x, int64_t n, int64_t c, int64_t h,
                                        int64_t w, const int64_t *pads, int32_t fill, void *out);
OVK_API int32_t ovk_padded_nhwc_to_nchw(ovk_ctx *ctx, const void *x, int64_t n, int64_t c, int64_t h,
                                        int64_t w, const int64_t *pads, void *out);
/* The REQUANTIZE pass on its own (shaders/qlinear.rs:28-63): c = (i / inner) % axis_len. */
OVK_API int32_t ovk_requantize(ovk_ctx *ctx, const int32_t *acc, int64_t count, int64_t inner,
                               int64_t axis_len, const int32_t *bias, const float *ratio,
                               int32_t y_zp, int32_t y_signed, void *out);

/* ------------------------------------- neighbours of the lm_head product
 * interp::gather_block_quantized (interp.rs:2874-2990, kernel
 * shaders/gather_block_quantized.rs:26-57): out[j, c] = (unpack(table[idx[j], c])
 * - zp) * scale for a [rows, cols/2] u8 table of 4-bit elements (element 2i in
 * the low nibble), scales [rows, cols/block_size] f32 or f16, zero points
 * [rows, ceil(n_blocks/2)] u8 nibble packed (NULL = implicit 8).  Negative
 * indices count from the end.  out is [count, cols] f32 or f16.
 * indices are int32 or int64 (indices_dtype).  With indices_on_host = 1 they
 * are a HOST array: an index outside the table is refused before anything is
 * enqueued, as the reference does.  With 0 they are read on the device (the
 * token a previous ovk_argmax produced, no round trip): an index outside the
 * table writes a row of zeros and makes the next ovk_flush return
 * OVK_INVALID_ARGUMENT. */
OVK_API int32_t ovk_gather_block_quantized(ovk_ctx *ctx, const void *table, const void *scales,
                                           int32_t scales_dtype, const void *zero_points,
                                           int64_t rows, int64_t cols, int64_t bits,
                                           int64_t block_size, const void *indices,
                                           int32_t indices_dtype, int32_t indices_on_host,
                                           int64_t count, void *out, int32_t out_dtype);
/* ArgMax over one axis, first occurrence (interp::arg_extreme_axis, interp.rs
 * :8552-8690; Outputs::argmax executor.rs:379; kernels shaders/reduction.rs
 * :76-190): x is [outer, c, inner] f32 or f16 on the device, out [outer*inner]
 * int64 on the device.  As in the reference's kernels a value is a candidate
 * only if it is greater than -FLT_MAX (NaN and -inf never are) and a row
 * without candidates answers 0. */
OVK_API int32_t ovk_argmax(ovk_ctx *ctx, const void *x, int32_t x_dtype, int64_t outer, int64_t c,
                           int64_t inner, int64_t *out);

/* ------------------------- the rest of the QOperator chain around QLinearConv
 * interp::qlinear_add (interp.rs:4878-4962, kernel shaders/qlinear.rs:69-143):
 * C = saturate(rne(fma(A, ra, fma(B, rb, fixed)))) with ra = A_scale/C_scale,
 * rb = B_scale/C_scale, fixed = c_zp - fma(ra, a_zp, rb*b_zp) in f32 - MLAS's
 * kernel operation for operation, including ORT's exchange of the operands when
 * A is constant along the innermost broadcast span.  General ONNX broadcasting up
 * to rank 8; shapes, scales and zero points are host values.  a, b, out are
 * device pointers to u8 (is_signed = 0) or i8 codes; out_shape (8 entries) and
 * out_rank receive the broadcast shape (may be NULL). */
OVK_API int32_t ovk_qlinear_add(ovk_ctx *ctx, const void *a, const int64_t *a_shape, int32_t a_rank,
                                float a_scale, int32_t a_zp, const void *b, const int64_t *b_shape,
                                int32_t b_rank, float b_scale, int32_t b_zp, float c_scale,
                                int32_t c_zp, int32_t is_signed, void *out, int64_t *out_shape,
                                int32_t *out_rank);
/* MaxPool on quantized codes (shaders/qlinear.rs:145-211): x is [n, c, h, w]
 * u8 / i8; kernel, strides, dilations have 2 entries, pads 4 (h_begin, w_begin,
 * h_end, w_end); floor mode; padding taps are skipped.  h_out / w_out receive
 * the output size. */
OVK_API int32_t ovk_maxpool_q(ovk_ctx *ctx, const void *x, int32_t is_signed, int64_t n, int64_t c,
                              int64_t h, int64_t w, const int64_t *kernel, const int64_t *strides,
                              const int64_t *pads, const int64_t *dilations, void *out,
                              int64_t *h_out, int64_t *w_out);
/* QuantizeLinear / DequantizeLinear (interp.rs:5055-5177, shaders/quantize_linear.rs):
 * channel of element i is (i / inner) % axis_len (per-tensor: inner = axis_len = 1);
 * scale is a device array of axis_len floats, zero_point a device array of
 * axis_len codes of the quantized type (int32 for int32 input) or NULL. */
OVK_API int32_t ovk_quantize_linear(ovk_ctx *ctx, const float *x, int64_t n, int64_t inner,
                                    int64_t axis_len, const float *scale, const void *zero_point,
                                    int32_t is_signed, void *out);
OVK_API int32_t ovk_dequantize_linear(ovk_ctx *ctx, const void *x, int32_t x_dtype, int64_t n,
                                      int64_t inner, int64_t axis_len, const float *scale,
                                      const void *zero_point, float *out);
/* interp::qlinear_global_average_pool (interp.rs:4975-5000): dequantize, average
 * over the hw elements of each of the n*c planes (a sequential f32 sum, as the
 * reference's pooling kernel forms it, shaders/pooling.rs:38-54), quantize. */
OVK_API int32_t ovk_qlinear_global_average_pool(ovk_ctx *ctx, const void *x, int32_t is_signed,
                                                int64_t n, int64_t c, int64_t hw, float x_scale,
                                                int32_t x_zp, float y_scale, int32_t y_zp, void *out);

#ifdef __cplusplus
}
#endif
#endif /* OVK_CUDA_H */
