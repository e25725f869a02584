/*
 * simnets_b200.h -- C ABI of the B200 (sm_100a) Similarity / MEX operator library.
 *
 * Every entry point is plain C: pointers, sizes, POD descriptors.  Device entry
 * points enqueue work on the caller's CUDA stream (passed as void* so that this
 * header needs no CUDA include), never synchronise, never allocate and never
 * free: the caller owns all buffers, including the scratch workspace whose size
 * the *_workspace_bytes queries return.  (One entry point is the exception on
 * scratch: simnets_mex_forward_static_scratch keeps its scratch in a fixed
 * device array inside the library; it still allocates nothing.)  Return value: 0 on success, a negative
 * SIMNETS_E_* code for a rejected call, a positive cudaError_t for a launch
 * failure.  simnets_status_string() renders either.
 *
 * Tensors are dense row-major NCHW, float32 (dtype 0) or float64 (dtype 1).
 *
 * Each declaration cites the interface of the reference implementation
 * (HUJI-Deep/simnets-tf, paths relative to that project) that it stands in for.
 */
#ifndef SIMNETS_B200_H
#define SIMNETS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SIMNETS_API __attribute__((visibility("default")))

/* ---- status codes ------------------------------------------------------ */
enum {
    SIMNETS_OK = 0,
    SIMNETS_E_NULL = -1,          /* a required pointer is NULL                   */
    SIMNETS_E_DESC = -2,          /* descriptor fails the reference's validation  */
    SIMNETS_E_DTYPE = -3,         /* dtype is neither float32 (0) nor float64 (1) */
    SIMNETS_E_WORKSPACE = -4,     /* workspace missing or too small               */
    SIMNETS_E_UNSUPPORTED = -5,   /* valid, but outside what this build handles   */
    SIMNETS_E_TOO_LARGE = -6      /* exceeds a fixed capacity (static scratch)    */
};

enum { SIMNETS_F32 = 0, SIMNETS_F64 = 1 };
enum { SIMNETS_SIM_L1 = 0, SIMNETS_SIM_L2 = 1 };

/* ---- descriptor flags --------------------------------------------------- */
/* Gradient outputs are overwritten by default, as the reference does
 * (src/kernels/similarity_grad_kernel_cpu.cpp:62,176; mex_grad_kernel_cpu.cpp:249).
 * With ACCUMULATE the parameter-gradient entry points add into the destination,
 * so that a data-parallel step can point them straight at its gradient bucket. */
#define SIMNETS_FLAG_ACCUMULATE        (1u << 0)
/* Use the one-thread-per-output kernels for every shape (slow, shape-agnostic). */
#define SIMNETS_FLAG_FORCE_DIRECT      (1u << 1)
/* MEX only: never use the factorised evaluation, always the per-term exp form. */
#define SIMNETS_FLAG_MEX_EXACT         (1u << 2)
/* Similarity, L2 + normalization_term without ignore_nan_input: the reference's
 * fast op adds -0.5*K*log(2*pi) to the whole output tensor inside its batch loop
 * (src/kernels/similarity_kernel_cpu.cpp:118-120), so sample n receives the
 * constant (batch - n) times.  By default this library adds it once per element,
 * which is what the reference's own SimilarityRef op does
 * (src/kernels/similarity_ref_kernel_cpu.cpp:89-93); this flag reproduces the
 * fast op's behaviour instead. */
#define SIMNETS_FLAG_SIM_BATCH_CONST_QUIRK (1u << 3)
/* Similarity, extension without a reference counterpart: L1 with NaN inputs
 * skipped (term contributes 0).  Requires similarity_function == L1. */
#define SIMNETS_FLAG_SIM_L1_SKIP_NAN   (1u << 4)

/* MEX only: keep the factorised GEMM on the CUDA cores (no tcgen05 tensor-core kernels). */
#define SIMNETS_FLAG_MEX_NO_TENSORCORE (1u << 5)

/* MEX only: run the tensor-core kernels that compute one tile per CTA instead of the persistent,
 * warp-specialised ones (same results; kept for comparison measurements). */
#define SIMNETS_FLAG_MEX_TC_ONE_TILE   (1u << 7)

/* MEX only: never pair the tiles of sibling regions (layers whose unshared regions alternate along the width
 * otherwise run on kernels that read and write pixel pairs); same results, kept for comparison measurements. */
#define SIMNETS_FLAG_MEX_NO_PAIR_TILES (1u << 9)

/* Test hook, simnets_mex_forward on a pair-tile shape only: the kernel's MMA role withholds the completion signal of
 * its first accumulator and every bounded wait is shortened to a fraction of a millisecond, so that one wait runs out.
 * Nothing hangs or faults: the roles leave their loops, tensor memory is freed, word 1 of the workspace status is set
 * (simnets_mex_workspace_status) and the exact kernels launched behind the tensor-core kernel redo the work. */
#define SIMNETS_FLAG_MEX_TEST_EXPIRE_WAIT (1u << 10)

/* simnets_similarity_forward only, float32, L2 without ignore_nan_input (other calls ignore the flag): evaluate the
 * squared differences through their expansion  sum s x^2 - 2 sum (s t) x + sum s t^2  as ONE matrix product on the
 * tensor cores (split-TF32 operands, FP32 accumulation) instead of term by term as the reference does
 * (include/utils/similarity_utils.hpp:26-36).  Opt-in because the expansion cancels where the reference's form does
 * not: TOLERANCE |y - y_ref| <= 1e-3 * max|y_ref| (the default kernels hold 1e-5); inputs must be finite.  The
 * gradients always use the term-by-term kernels. */
#define SIMNETS_FLAG_SIM_L2_TENSORCORE (1u << 11)

/* Similarity entry points: `weights` holds raw values and the op works on their absolute value, as the reference's
 * Keras layer feeds K.abs(weights) to the op (python/simnets/keras.py:65); simnets_similarity_params_grad then returns
 * the gradient with respect to the raw values, sign(weights) * dL/d|weights| (0 where a weight is 0).  Saves the
 * separate abs, sign and multiply passes over the weights. */
#define SIMNETS_FLAG_SIM_ABS_WEIGHTS   (1u << 12)

/* simnets_mex_forward / simnets_mex_forward_pool2x2: the per-position extrema are already in the workspace
 * (see simnets_mex_workspace_maxima); ignored by shapes for which that function returns NULL. */
#define SIMNETS_FLAG_MEX_MAXIMA_GIVEN  (1u << 13)

/* MEX entry points that take a workspace, float32: `offsets` holds raw values and the op works on each (region,
 * instance) row minus its log-sum-exp, as the reference's Keras layer does with `normalize_offsets=True` in front of the
 * op (python/simnets/keras.py:155-160); the offsets-gradient entry points then return the gradient with respect to
 * the raw values, d - softmax(row) * sum(d).  Saves the separate normalisation kernels in both directions.  Not accepted
 * (SIMNETS_E_UNSUPPORTED) by calls that run without a workspace: float64, SIMNETS_FLAG_FORCE_DIRECT, SIMNETS_FLAG_MEX_EXACT,
 * simnets_mex_forward_static_scratch. */
#define SIMNETS_FLAG_MEX_NORMALIZED_OFFSETS (1u << 14)

/* MEX gradient entry points only: dy is given at half resolution, dy[batch, M * channels_out, height_out / 2,
 * width_out / 2], each value standing for the 2x2 window of output positions that a 2x2 / stride-2 sum pooling
 * added up (the gradient of such a pooling copies its dy to the four inputs; with this flag the copy is never
 * materialised).  height_out and width_out must be even, else SIMNETS_E_UNSUPPORTED.  No counterpart in the
 * reference, whose graphs run the pooling gradient as a separate TensorFlow op. */
#define SIMNETS_FLAG_MEX_DY_POOLED2    (1u << 6)

/* MEX gradient entry points only: the workspace is the one the last simnets_mex_forward call was given for the
 * same input, offsets, descriptor and flags (SIMNETS_FLAG_MEX_DY_POOLED2 aside) and nothing has written to it
 * since, other gradient calls of that layer excepted.  The per-position maxima and the offsets tables that the
 * forward pass left there are then used as they are instead of being computed again (same values, fewer
 * launches).  Ignored where the forward pass of the shape does not leave them.  The caller owns the promise: a
 * workspace that was reused in between gives wrong gradients, not an error. */
#define SIMNETS_FLAG_MEX_WORKSPACE_PRIMED (1u << 8)

/* ---- Similarity ---------------------------------------------------------- */
/* Mirrors the attrs of the Similarity op family (src/ops/similarity_op.cpp:61-75)
 * and the dimensions SimilarityKernelCommon::CalculateDimensions derives
 * (include/kernels/similarity_kernel_common.hpp:113-164).
 * templates / weights: [num_instances, channels, block_h, block_w]. */
typedef struct simnets_sim_desc {
    int32_t dtype;
    int32_t batch, channels, height, width;
    int32_t num_instances;
    int32_t block_h, block_w;
    int32_t stride_h, stride_w;
    int32_t pad_h, pad_w;
    int32_t similarity_function;        /* SIMNETS_SIM_L1 | SIMNETS_SIM_L2 */
    int32_t normalization_term;
    int32_t ignore_nan_input;
    float   normalization_term_fudge;
    float   out_of_bounds_value;
    uint32_t flags;
} simnets_sim_desc;

/* Output height/width: floor((in + 2*pad - block)/stride) + 1
 * (include/utils/im2col.hpp:101-108 with round_down = true;
 *  shape function SimilarityShape, src/ops/similarity_op.cpp:8-53).
 * Also performs the constructor's attr validation
 * (include/kernels/similarity_kernel_common.hpp:84-110). */
SIMNETS_API int simnets_similarity_output_dims(const simnets_sim_desc* d, int32_t* out_h, int32_t* out_w);

SIMNETS_API size_t simnets_similarity_workspace_bytes(const simnets_sim_desc* d);

/* Similarity forward: y[batch, num_instances, out_h, out_w].
 * Replaces SimilarityKernelGPU<T>::Compute (src/kernels/similarity_kernel_gpu.cu:24-133),
 * oracle SimilarityKernelCPU<T>::Compute (src/kernels/similarity_kernel_cpu.cpp:19-122). */
SIMNETS_API int simnets_similarity_forward(const simnets_sim_desc* d,
                                           const void* x, const void* templates, const void* weights,
                                           void* y, void* workspace, size_t workspace_bytes, void* stream);

/* Similarity forward that also leaves, per sample and output position, the maximum and the minimum of y over the
 * instances: ch_max[batch, out_h, out_w], ch_min likewise (either may be NULL; NaN entries are ignored as by fmax).
 * A MEX layer whose blocks span exactly the channels of one pixel (block [C, 1, 1]) needs that extremum of every
 * patch to stabilise its log-sum-exp, and in a SimNet the Similarity layer always feeds such a MEX layer
 * (README.md:114-131): written straight into the MEX workspace (simnets_mex_workspace_maxima) it saves the MEX forward
 * pass its own pass over the input (SIMNETS_FLAG_MEX_MAXIMA_GIVEN).  The short-patch kernels produce the extrema on the
 * way, the other forward kernels by a small kernel behind them.  float32 only.  No counterpart in the reference. */
SIMNETS_API int simnets_similarity_forward_extrema(const simnets_sim_desc* d,
                                                   const void* x, const void* templates, const void* weights,
                                                   void* y, void* ch_max, void* ch_min,
                                                   void* workspace, size_t workspace_bytes, void* stream);

/* Status words of a Similarity workspace after simnets_similarity_forward used it, copied to host_out[0..1] as
 * simnets_mex_workspace_status does.  host_out[0] is always 0; host_out[1] != 0: the tensor-core kernel of
 * SIMNETS_FLAG_SIM_L2_TENSORCORE gave up on a bounded wait between its roles and the term-by-term kernel launched
 * behind it recomputed the output (valid, only slow).  No counterpart in the reference. */
SIMNETS_API int simnets_similarity_workspace_status(const void* workspace, void* stream, int32_t* host_out);

/* dL/dinput.  Replaces SimilarityInputGradKernelGPU (src/kernels/similarity_grad_kernel_gpu.cu:155-269),
 * oracle SimilarityInputGradKernelCPU (src/kernels/similarity_grad_kernel_cpu.cpp:158-270). */
SIMNETS_API int simnets_similarity_input_grad(const simnets_sim_desc* d,
                                              const void* x, const void* templates, const void* weights,
                                              const void* dy, void* dx,
                                              void* workspace, size_t workspace_bytes, void* stream);

/* dL/dtemplates and dL/dweights, summed over batch and positions.
 * Replaces SimilarityParametersGradKernelGPU (src/kernels/similarity_grad_kernel_gpu.cu:24-143),
 * oracle SimilarityParametersGradKernelCPU (src/kernels/similarity_grad_kernel_cpu.cpp:23-146). */
SIMNETS_API int simnets_similarity_params_grad(const simnets_sim_desc* d,
                                               const void* x, const void* templates, const void* weights,
                                               const void* dy, void* dtemplates, void* dweights,
                                               void* workspace, size_t workspace_bytes, void* stream);

/* ---- MEX ------------------------------------------------------------------ */
/* Mirrors the attrs of the Mex op family (src/ops/mex_op.cpp:58-74).  padding and
 * strides may hold -1 ("whole image dimension", src/kernels/mex_kernel_common.cpp:8-27);
 * the region lists have length 1 ([d] means [-1, d, d]) or 3.
 * offsets: [num_regions, num_instances, block_c, block_h, block_w]. */
typedef struct simnets_mex_desc {
    int32_t dtype;
    int32_t batch, channels, height, width;
    int32_t num_instances;
    int32_t blocks[3];                  /* c, h, w */
    int32_t strides[3];
    int32_t padding[3];
    float   epsilon;                    /* may be +inf / -inf */
    int32_t softmax_mode;
    float   blocks_out_of_bounds_value;
    int32_t blocks_round_down;
    int32_t use_unshared_regions;
    int32_t shared_offset_region[3];
    int32_t n_shared_offset_region;     /* 1 or 3 */
    int32_t unshared_offset_region[3];
    int32_t n_unshared_offset_region;   /* 1 or 3 */
    uint32_t flags;
} simnets_mex_desc;

/* Everything MexDimensionsData::CalculateDimensions computes
 * (src/kernels/mex_kernel_common.cpp:63-158, include/kernels/mex_kernel_common.hpp:11-58). */
typedef struct simnets_mex_geometry {
    int32_t block_c, block_h, block_w;
    int32_t stride_c, stride_h, stride_w;
    int32_t pad_c, pad_h, pad_w;
    int32_t channels_out, height_out, width_out;
    int32_t channels_out_total;         /* channels_out * num_instances */
    int32_t region_c, region_h, region_w;     /* shared_offsets_region_*: extent of one region */
    int32_t offsets_c, offsets_h, offsets_w;  /* number of regions along each axis */
    int32_t num_regions, region_size;
    int32_t M, K, N;
    int32_t is_1x1;
} simnets_mex_geometry;

/* Host only.  Validates like MEXKernelCommon's constructor and
 * CalculateDimensionsWithConext (src/kernels/mex_kernel_common.cpp:29-58,161-170). */
SIMNETS_API int simnets_mex_dims(const simnets_mex_desc* d, simnets_mex_geometry* out);

/* Host only.  Same symbol, argument order and return value (num_regions, or -1) as the
 * reference's helper library libmex_dims_helper.so (src/kernels/mex_dims_helper.cpp:8-44),
 * which python/simnets/ops/mex.py:17-38 calls through ctypes.  A padding / strides list of
 * length 1 is broadcast to three entries (the reference reads past the end of such a list). */
SIMNETS_API int get_mex_offsets_nregions(int n_input_dim, const int* input_dim,
                                         int n_padding, const int* padding,
                                         int n_strides, const int* strides,
                                         int num_instances, int blocks_round_down, int use_unshared_regions,
                                         int n_blocks, const int* blocks,
                                         int n_shared_offset_region, const int* shared_offset_region,
                                         int n_unshared_offset_region, const int* unshared_offset_region);

SIMNETS_API size_t simnets_mex_workspace_bytes(const simnets_mex_desc* d);

/* MEX forward: y[batch, num_instances * channels_out, height_out, width_out].
 * Replaces MEXKernelGPU<T>::Compute (src/kernels/mex_kernel_gpu.cu:60-159),
 * oracle MEXKernelCPU<T>::Compute + mex_forward_cpu (src/kernels/mex_kernel_cpu.cpp:11-38,60-159). */
SIMNETS_API int simnets_mex_forward(const simnets_mex_desc* d,
                                    const void* x, const void* offsets, void* y,
                                    void* workspace, size_t workspace_bytes, void* stream);

/* Where simnets_mex_forward reads the per-position extrema of the patches from (float32 [batch, N], N = positions per
 * sample; the maximum for epsilon > 0, the minimum for epsilon < 0), inside a workspace of this descriptor; NULL for
 * shapes whose forward kernels find the extrema themselves.  A caller that fills it (e.g. with
 * simnets_similarity_forward_extrema of the layer in front, when every patch is exactly the channels of one pixel)
 * passes SIMNETS_FLAG_MEX_MAXIMA_GIVEN to simnets_mex_forward / simnets_mex_forward_pool2x2, which then skip their
 * pass over the input; wrong values there break the numerical safety of the evaluation, not just its speed. */
SIMNETS_API void* simnets_mex_workspace_maxima(const simnets_mex_desc* d, void* workspace);

/* MEX forward plus the 2x2 / stride-2 sum pooling of its output, the pair of layers the reference's example networks
 * repeat (README.md:114-131, there `4 * AveragePooling2D(2)` behind the Mex layer): y as simnets_mex_forward writes it
 * (the gradient entry points need it) and y_pooled[batch, num_instances * channels_out, height_out / 2, width_out / 2].
 * float32 only, height_out and width_out even, else SIMNETS_E_UNSUPPORTED.  On the pair-tile kernels the pooling is
 * done by the forward kernel's epilogue (y is not read again); elsewhere a pooling kernel runs behind the forward
 * kernels.  Each pooled value is (y00 + y01) + (y10 + y11).  No counterpart in the reference, whose graphs use
 * TensorFlow's pooling op. */
SIMNETS_API int simnets_mex_forward_pool2x2(const simnets_mex_desc* d,
                                            const void* x, const void* offsets, void* y, void* y_pooled,
                                            void* workspace, size_t workspace_bytes, void* stream);

/* Status words of a MEX workspace after the calls that used it, copied to host_out[0..1] by one 8-byte asynchronous
 * device-to-host copy on `stream` (synchronise the stream before reading; pinned host memory keeps the copy
 * asynchronous).  No counterpart in the reference, whose kernels have nothing to report.
 *   host_out[0] != 0: the offsets of the call made the factorised evaluation unsafe (a non-finite offset, or
 *                     |epsilon| * (max - min) of a row above 60); the exact per-term kernels computed the results.
 *   host_out[1] != 0: a tensor-core kernel gave up on a bounded wait between its roles (about two seconds) and left
 *                     early; the exact kernels launched behind it recomputed the outputs of that call, so they are
 *                     valid, only slow.  Not expected outside SIMNETS_FLAG_MEX_TEST_EXPIRE_WAIT.
 * The words are cleared by the next call that runs the prepasses on this workspace (every call without
 * SIMNETS_FLAG_MEX_WORKSPACE_PRIMED). */
SIMNETS_API int simnets_mex_workspace_status(const void* workspace, void* stream, int32_t* host_out);

/* MEX forward for callers that have no scratch to give.  No counterpart in the reference: its
 * OpKernels always obtain temporaries from TensorFlow's allocator (context->allocate_temp).
 *
 * Some hosts of this library cannot hand it a workspace: an operator plugin loaded into a serving
 * runtime that has pre-assigned every byte of device memory to its own arena, a callback running
 * inside someone else's executor where calling a device allocator is forbidden, or a partitioned
 * GPU whose share is already fully committed.  For them this entry point computes the function
 * simnets_mex_forward computes (same descriptor, same output tensor), but keeps its scratch (offset
 * exponentials, per-position maxima, the safety flag) in a fixed device array inside the library,
 * SIMNETS_MEX_STATIC_SCRATCH_BYTES large, which each GPU that loads the library holds until the
 * process exits.  It calls no device allocator and no allocating library routine.
 *
 *  - Route and tolerance: the call honours d->flags and adds SIMNETS_FLAG_MEX_NO_TENSORCORE, i.e. it
 *    always runs the CUDA-core kernels (the fixed array has no room for tensor-core operand tiles).
 *    float64 and the float32 shapes that need no scratch give the bits simnets_mex_forward gives; for
 *    the float32 shapes that simnets_mex_forward sends to the tensor cores the two results agree to
 *    the library's float32 bound, |a - b| <= 1e-5 * max(1, |b|), and each is within that bound of the
 *    reference's float64 result.
 *  - Problems whose forward scratch exceeds the array are rejected with SIMNETS_E_TOO_LARGE before
 *    anything is launched (scratch need = 4 bytes * (batch*N + 2*num_regions*M*K) plus a few hundred
 *    bytes of padding; use simnets_mex_forward with a caller workspace for those).
 *  - The first call on each device looks up the array's device address; make that first call outside
 *    any stream capture.
 *  - All calls share the one array and it keeps whatever the previous call left; the call itself
 *    clears the part that must start at zero.  Two calls that overlap on the same GPU (different
 *    streams or threads) race on it: serialise them.
 */
#define SIMNETS_MEX_STATIC_SCRATCH_BYTES (8u << 20)
SIMNETS_API int simnets_mex_forward_static_scratch(const simnets_mex_desc* d,
                                                   const void* x, const void* offsets, void* y, void* stream);

/* dL/dinput.  Replaces MEXGradInputKernelGPU (src/kernels/mex_grad_kernel_gpu.cu:23-205),
 * oracle MEXGradInputKernelCPU (src/kernels/mex_grad_kernel_cpu.cpp:23-209). */
SIMNETS_API int simnets_mex_input_grad(const simnets_mex_desc* d,
                                       const void* x, const void* offsets, const void* y, const void* dy,
                                       void* dx, void* workspace, size_t workspace_bytes, void* stream);

/* dL/doffsets, summed over batch and region positions.
 * Replaces MEXGradOffsetsKernelGPU (src/kernels/mex_grad_kernel_gpu.cu:207-374),
 * oracle MEXGradOffsetsKernelCPU (src/kernels/mex_grad_kernel_cpu.cpp:211-370). */
SIMNETS_API int simnets_mex_offsets_grad(const simnets_mex_desc* d,
                                         const void* x, const void* offsets, const void* y, const void* dy,
                                         void* doffsets, void* workspace, size_t workspace_bytes, void* stream);

/* Both MEX gradients in one call (same results as the two calls above; the work they share -- offset
 * exponentials, per-position maxima -- is done once).  Stands in for running MexInputGrad and MexOffsetsGrad
 * back to back, which is what the reference's gradient function always does (python/simnets/ops/mex.py:47-81). */
SIMNETS_API int simnets_mex_backward(const simnets_mex_desc* d,
                                     const void* x, const void* offsets, const void* y, const void* dy,
                                     void* dx, void* doffsets, void* workspace, size_t workspace_bytes, void* stream);

/* ---- measurement probe ---------------------------------------------------- */
/* Launches a register-only kernel of independent FP32 fused multiply-adds on every SM (packed != 0: the packed
 * two-lane instruction) and returns the number of fused multiply-adds it executes, or a negative value on error.
 * Time it with events on `stream`: FMAs / seconds is the FP32-pipe peak that "fraction of FP32 peak" figures of
 * the Similarity kernels are quoted against.  `scratch`: at least 4 bytes of device memory (never written).
 * No counterpart in the reference. */
SIMNETS_API int64_t simnets_fp32_fma_probe(int32_t packed, int32_t iters, void* scratch, void* stream);

/* ---- sum pooling ----------------------------------------------------------- */
/* y[p, h, w] = x[p, 2h, 2w] + x[p, 2h, 2w+1] + x[p, 2h+1, 2w] + x[p, 2h+1, 2w+1] over a dense float32 tensor
 * [planes, height, width] (planes = batch * channels); height and width even, else SIMNETS_E_UNSUPPORTED.
 * The 2x2 sum pooling the reference's example networks put behind every MEX layer (README.md:114-131, there
 * `4 * AveragePooling2D(2)`).  No counterpart in the reference's own sources: its graphs use TensorFlow's pooling
 * op.  Its gradient is not an entry point: the MEX gradient entry points take the pooled dy directly
 * (SIMNETS_FLAG_MEX_DY_POOLED2). */
SIMNETS_API int simnets_sum_pool2x2_forward(int64_t planes, int32_t height, int32_t width,
                                            const void* x, void* y, void* stream);

/* ---- softmax cross-entropy -------------------------------------------------- */
/* The loss of the reference's example networks (README.md:108-111: softmax + categorical cross-entropy, in TensorFlow
 * a chain of softmax / log / multiply / reduce kernels and their gradients) and its gradient in one launch:
 *   loss[0]             = scale * sum_b (logsumexp(logits[b, :]) - logits[b, labels[b]])
 *   dlogits[b, c]       = scale * (softmax(logits[b, :])[c] - (c == labels[b]))         (dlogits may be NULL)
 * logits, dlogits: float32 [batch, classes] on the device; labels: int64 [batch] on the device (a label outside
 * [0, classes) contributes neither loss nor gradient); loss: one float32 on the device.  scale = 1 / global batch
 * gives the mean over a data-parallel job's whole batch.  The sum over the batch is taken in a fixed order.
 * No counterpart in the reference's own sources. */
SIMNETS_API size_t simnets_softmax_cross_entropy_workspace_bytes(int32_t batch);
SIMNETS_API int simnets_softmax_cross_entropy(int32_t batch, int32_t classes, float scale,
                                              const float* logits, const int64_t* labels, float* loss, float* dlogits,
                                              void* workspace, size_t workspace_bytes, void* stream);

/* ---- normalize_offsets ------------------------------------------------------ */
/* The `normalize_offsets` option of the reference's Keras Mex layer (python/simnets/keras.py:155-160): each of the
 * `rows` = num_regions * num_instances rows of `k` = block_c * block_h * block_w float32 offsets minus its log-sum-exp;
 * and the gradient of that map, doffsets = dout - softmax(offsets) * sum(dout) per row.  In the reference this is a
 * chain of TensorFlow ops around the Mex op, so there is no counterpart in its C++ sources. */
SIMNETS_API int simnets_normalize_offsets_forward(int64_t rows, int32_t k, const void* offsets, void* out, void* stream);
SIMNETS_API int simnets_normalize_offsets_backward(int64_t rows, int32_t k, const void* offsets, const void* dout,
                                                   void* doffsets, void* stream);

/* ---- misc ----------------------------------------------------------------- */
SIMNETS_API const char* simnets_status_string(int status);
/* Number of kernels this library has launched in this process (all devices). */
SIMNETS_API uint64_t simnets_launch_count(void);
/* ABI version of this header. */
SIMNETS_API int simnets_abi_version(void);

#ifdef __cplusplus
}
#endif
#endif /* SIMNETS_B200_H */
