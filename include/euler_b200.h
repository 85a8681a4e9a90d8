/*
 * euler_b200.h -- C ABI of the B200 (sm_100a) convolution library.
 *
 * This is the boundary a host-language binding (C++, ctypes, cgo, JNI ...) talks to.  It carries
 * the same information as the reference's C++ descriptor `euler::eld_conv_t` and the same two-step
 * protocol (describe + set up once, then execute many times), but with plain C types only: no
 * std::string, no C++ classes, no torch types.  The C++ host library (host/euler_host.cpp, built
 * against the reference's own include/euler.hpp) implements the reference's C++ surface
 * (eld_conv_t::setup / elx_conv / reorder<>) on top of these functions.
 *
 * Each entry point names the reference interface it replaces (file:line in the reference project).
 *
 * Pointers passed to elb_conv_execute may be host or device memory (detected per call); pointers
 * passed to elb_conv_enqueue must be device memory of the plan's device.  Tensor layouts are the
 * reference's blocked layouts: nChw16c activations, OIhw16i16o weights (goihw for depthwise),
 * fp32 bias of ALIGNUP(oc,16) elements.
 *
 * Environment variables the library reads:
 *   EULER_VERBOSE=1     one "euler-perf, ..." line per executed convolution on stdout, in the
 *                       reference's format (src/elx_conv.cpp:190-211, src/el_init.cpp:18-22)
 *   EULER_LOG_LEVEL=n   lowest severity printed (1 trace .. 5 error; default 3 = info), as
 *                       src/el_init.cpp:24-27; messages go to stderr
 *   EULER_GPUS=G        elb_conv_multi_create without a device list: split over GPUs 0..G-1
 *   ELB_HOST_CHUNKS=k   elb_conv_execute with host tensors: cut the batch into k chunks
 *   ELB_I8_CTA2=1, ELB_WINO_CTA2=1   run the tcgen05 kernels on pairs of CTAs (cta_group::2); measured
 *                       not faster than single CTAs, kept as a tested option
 *   ELB_FORCE_SIMT=1, ELB_F32_NO_FLAT=1   select the CUDA-core int8 kernel / the three-kernel fp32
 *                       direct path where the tcgen05 single-kernel path would run (used by the tests
 *                       to cover both)
 * Nothing else in the environment changes which kernel runs.
 */
#ifndef EULER_B200_H_
#define EULER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ELB_API __attribute__((visibility("default")))

/* Return codes: numerically equal to ELD_OK/ELD_UNIMPLEMENTED/ELD_GENERAL_ERROR and
 * ELX_OK/ELX_UNIMPLEMENTED/ELX_GENERAL_ERROR (include/euler.hpp:45-56). */
enum { ELB_OK = 0, ELB_UNIMPLEMENTED = 1, ELB_GENERAL_ERROR = 2 };

/* Algorithms (include/euler.hpp:35-42). */
enum {
  ELB_CONV_AUTO = 0, ELB_CONV_DIRECT_1X1 = 1, ELB_CONV_DIRECT = 2, ELB_CONV_DIRECT_VMG = 3,
  ELB_CONV_WINOGRAD = 4, ELB_DECONV_DIRECT = 5
};
/* Element types (include/euler.hpp:66-73). */
enum { ELB_DT_UNDEF = 0, ELB_F32 = 1, ELB_F16 = 2, ELB_U8 = 3, ELB_S8 = 4, ELB_S32 = 5 };
/* Tensor formats (include/euler.hpp:75-89). */
enum {
  ELB_FMT_UNDEF = 0, ELB_NCHW, ELB_NHWC, ELB_NCHW16C, ELB_NCHW8C, ELB_OIHW, ELB_HWIO, ELB_OIHW16I16O,
  ELB_OIHW8I8O, ELB_GOIHW, ELB_GHWIO, ELB_GOIHW16I16O, ELB_GOIHW8I8O
};
/* Propagation kinds (include/euler.hpp:92-97); only forward_inference is implemented. */
enum { ELB_FORWARD_TRAINING = 0, ELB_FORWARD_INFERENCE = 1, ELB_BACKWARD_DATA = 2, ELB_BACKWARD_WEIGHTS = 3 };
/* Quantisation sampling kinds (include/euler.hpp:99-103). */
enum { ELB_FINE = 0, ELB_COARSE = 1, ELB_CALIBRATED = 2 };

/* Plain-C mirror of euler::eld_conv_t (include/euler.hpp:110-187).  Tuning knobs of the CPU
 * implementation (blocking / partition / nthreads / streaming_hint, flatting.o) have no meaning on
 * the GPU and are not part of this struct; execution_mode is carried only to be validated.
 * flatting.t is carried because the reference's int8 depthwise kernel rounds a u8 output pixel
 * differently depending on its position inside a chunk of flatting.t pixels. */
typedef struct elb_conv_desc {
  int32_t n, g, ic, oc, ih, iw, oh, ow, kh, kw;        /* dims                      :113-115 */
  int32_t pad_l, pad_r, pad_t, pad_b;                  /* pads                      :116     */
  int32_t stride_h, stride_w;                          /* strides                   :117     */
  int32_t dilation_h, dilation_w;                      /* dilations                 :118     */
  int32_t dt_input, dt_weights, dt_output, dt_bias;    /* data_type                 :121-126 */
  int32_t fmt_input, fmt_weights, fmt_output;          /* formats                   :131     */
  int32_t prop_kind;                                   /*                           :134     */
  int32_t algorithm, tile_size;                        /*                           :137-138 */
  int32_t with_relu, with_bias, with_ip_sum, with_op_sum, with_argmax;   /*         :140-144 */
  int32_t f16c_opt, disable_autoparam;                 /*                           :145,148 */
  float relu_lower, relu_upper;                        /* relu_bound                :150     */
  int32_t execution_mode;                              /*                           :156     */
  float input_scale, input_z;                          /* input_quant               :168     */
  float tinput_scale, tinput_z;                        /* wino_tinput_quant         :168     */
  float output_scale, output_z;                        /* output_quant              :168     */
  float sum_scale, sum_z;                              /* sum_quant                 :168     */
  int32_t sampling_kind;                               /*                           :169     */
  int32_t flatting_t;                                  /* flatting.t (depthwise)    :158     */
  int32_t device;                                      /* CUDA device ordinal; -1 = current device */
} elb_conv_desc_t;

/* What setup() computes (include/euler.hpp:181-183 byte_sizes / sizes) plus what it chose. */
typedef struct elb_conv_info {
  int32_t algorithm;          /* resolved from ELB_CONV_AUTO                    src/eld_conv.cpp:148-159 */
  int32_t tile_size;          /* resolved Winograd tile (6 = F(4x4,3x3))        src/eld_conv.cpp:231-236 */
  int32_t kernel;             /* ELB_KERNEL_* below                                                   */
  int32_t device;
  uint64_t size_input, size_weights, size_output, size_bias;           /* elements, src/eld_conv.cpp:99-112 */
  uint64_t bytes_input, bytes_weights, bytes_output, bytes_bias;       /* bytes,    src/eld_conv.cpp:123-126 */
  uint64_t workspace_bytes;   /* device memory the plan holds (packed weights, constants, t-buffers) */
  int32_t launches_per_call;  /* kernels one steady-state execute launches */
  int32_t reserved;
} elb_conv_info_t;

enum {
  ELB_KERNEL_NONE = 0,
  ELB_KERNEL_I8_GEMM_UMMA = 1,      /* int8 1x1: tcgen05 kind::i8, TMEM s32 accumulators            */
  ELB_KERNEL_I8_CONV_UMMA = 2,      /* int8 KxK implicit GEMM: TMA-tiled operand fetch + tcgen05     */
  ELB_KERNEL_I8_SIMT = 3,           /* int8 any shape: dp4a CUDA-core kernel (small / odd shapes)    */
  ELB_KERNEL_WINO_F32_UMMA = 4,     /* fp32 F(4x4,3x3): transforms + 3xTF32 tcgen05 batched GEMM     */
  ELB_KERNEL_WINO_I8_UMMA = 5,      /* int8 F(4x4,3x3): quantising transforms + tcgen05 kind::i8     */
  ELB_KERNEL_I8_DEPTHWISE = 6,      /* int8 depthwise 3x3: bandwidth-bound dp4a kernel               */
  ELB_KERNEL_F32_DIRECT_UMMA = 7,   /* fp32 1x1 / KxK direct: implicit GEMM on the 3xTF32 tcgen05 kernel */
  ELB_KERNEL_F32_SMALL_IC = 8       /* fp32 3x3 s1 p1 Winograd request with <= 4 input channels: direct kernel (tcgen05
                                       implicit GEMM for an nchw image into 64 channels, CUDA cores otherwise) */
};

typedef struct elb_conv elb_conv_t;      /* the plan; replaces `elx_conv_t *xc` (include/euler.hpp:186) */

/* Sizes and algorithm choice only -- replaces eld_conv_t::setup(false) (src/eld_conv.cpp:59-163). */
ELB_API int elb_conv_sizes(const elb_conv_desc_t *desc, elb_conv_info_t *info);

/* Validate, choose the kernel and build the plan -- replaces eld_conv_t::setup(true)
 * (src/eld_conv.cpp:59-316) and the elx_*_t constructors it calls.  Unsupported descriptors return
 * ELB_UNIMPLEMENTED (there is no CPU fallback); the reference would abort() through el_error. */
ELB_API int elb_conv_create(const elb_conv_desc_t *desc, elb_conv_t **plan);

ELB_API int elb_conv_info(const elb_conv_t *plan, elb_conv_info_t *info);

/* Run the convolution and wait for it -- replaces elx_conv(desc, output, input, weights, bias)
 * (include/euler.hpp:190, src/elx_conv.cpp:213-240) with eager_mode = true.  As in the reference,
 * weights and bias are read on the FIRST call only (quantised / transformed / packed into the
 * plan's workspace); later calls ignore them.  `output` is also read when with_ip_sum is set.
 * Host pointers are staged through the plan's device buffers inside this call. */
ELB_API int elb_conv_execute(elb_conv_t *plan, void *output, const void *input, const void *weights,
                             const void *bias);

/* Same work, device pointers only, enqueued on `cuda_stream` (a cudaStream_t; NULL = default
 * stream) without waiting -- the eager_mode = false path (src/elx_conv.cpp:228-236,
 * src/elx_stream.cpp:54-62).  The first-call weight preparation is still done synchronously. */
ELB_API int elb_conv_enqueue(elb_conv_t *plan, void *output, const void *input, const void *weights,
                             const void *bias, void *cuda_stream);

/* elx_conv with eager_mode = false (src/elx_conv.cpp:228-236): the same work as elb_conv_execute,
 * host or device tensors, but the call returns once the copies and kernels are enqueued on the
 * plan's own streams -- the counterpart of the reference handing the call to its worker thread
 * (src/elx_stream.cpp:54-62).  Calls on one plan run in submission order.  Host tensors must stay
 * valid, and the output must not be read, until elb_conv_wait returns. */
ELB_API int elb_conv_execute_async(elb_conv_t *plan, void *output, const void *input, const void *weights,
                                   const void *bias);

/* Wait for every elb_conv_execute_async issued on this plan -- stream_sync = true
 * (src/elx_conv.cpp:234-235, src/elx_stream.cpp:95-98).  Returns ELB_GENERAL_ERROR when a kernel of
 * one of those calls gave up a bounded wait. */
ELB_API int elb_conv_wait(elb_conv_t *plan);

/* eld_conv_t::name (include/euler.hpp:172): the label of this convolution in the euler-perf line. */
ELB_API int elb_conv_set_name(elb_conv_t *plan, const char *name);

/* Do the first-call weight preparation now -- the `setup_workspace` step of the reference
 * (src/elx_conv.hpp:130-145) made explicit so that callers can keep it out of a timed region. */
ELB_API int elb_conv_prepare(elb_conv_t *plan, const void *weights, const void *bias);

/* Parity hook: when set (device pointer to int32, output-tensor shape nChw16c, or [36][tiles][OC]
 * for Winograd), integer kernels also store their raw int32 accumulators there.  NULL switches it
 * off.  The reference keeps the same values in its `toutput` scratch (src/kernel/elk_u8s8_gemm.hxx:146-166). */
ELB_API int elb_conv_set_accumulator_dump(elb_conv_t *plan, void *device_int32);

/* No counterpart in the reference (its harness feeds a layer's output to the next call,
 * tests/elt_conv.cpp:399-410, and networks subsample between stages): enqueue as elb_conv_enqueue
 * on an already prepared plan, but `input` is a device tensor of src_h x src_w pixels per plane of
 * which the convolution reads every step-th row and column (ceil(src_h / step) == ih, same for w) --
 * a subsample folded into the kernel's own loads instead of a kernel and a tensor of its own.
 * elb_conv_input_step_supported() says whether the plan's kernel can do it (fp32 Winograd
 * F(4x4,3x3) today); otherwise ELB_UNIMPLEMENTED, and elb_subsample_nChw16c does the job. */
ELB_API int elb_conv_input_step_supported(elb_conv_t *plan);
ELB_API int elb_conv_enqueue_strided(elb_conv_t *plan, void *output, const void *input, int src_h, int src_w, int step,
                                     void *cuda_stream);

/* Device-side status word of the last launch: 0 = ok, otherwise the code of the bounded wait that
 * gave up (see csrc/elb_common.cuh).  Also returned as ELB_GENERAL_ERROR by execute. */
ELB_API int elb_conv_device_status(elb_conv_t *plan);

/* Measurement hook, no counterpart in the reference: four cudaEvent_t handles which the Winograd
 * path records before, between and after its three kernels (input transform, batched GEMM,
 * output transform) on every following call; NULL switches it off.  Must be off during CUDA
 * graph capture. */
ELB_API int elb_conv_set_stage_events(elb_conv_t *plan, void **cuda_events4);

/* Debug hook, no counterpart in the reference: per-CTA timeline of the tcgen05 kernels (SM cycle
 * counter), 64 int64 slots per CTA in caller DEVICE memory; NULL switches it off.  While it is on,
 * the Winograd / fp32 GEMM runs its generic kernel instead of the one compiled for its mode (the
 * stamps would slow the specialised role loops down for everybody), so timings taken with a
 * timeline are not the timings of a normal call. */
ELB_API int elb_conv_set_trace(elb_conv_t *plan, void *device_int64);

/* Self test of the bounded waits, no counterpart in the reference: a one-CTA kernel waits on a
 * barrier nobody arrives at, gives up after limit_ns and returns normally.  Returns the status word
 * it wrote (104 = gave up as designed), or a negative number when the test could not run.
 * device = -1: the current device. */
ELB_API int elb_selftest_bounded_wait(int device, unsigned long long limit_ns);

/* Number of kernels this plan has launched since it was created. */
ELB_API uint64_t elb_conv_launch_count(const elb_conv_t *plan);

/* Release the plan and its device memory -- replaces ~eld_conv_t / ~elx_conv_t
 * (src/eld_conv.cpp:52-57, src/elx_conv.cpp:168-188). */
ELB_API void elb_conv_destroy(elb_conv_t *plan);

/* Message of the last failure on the calling thread ("" if none); the text the reference would
 * have printed through el_error / el_warn (src/common/el_log.cpp:7-25). */
ELB_API const char *elb_last_error(void);

/* Library / device probe -- replaces the AVX-512 check in setup (src/eld_conv.cpp:62-72,
 * src/common/el_isa.hpp:31-70): returns ELB_OK when `device` is an sm_100 GPU. */
ELB_API int elb_device_supported(int device);

/* Layout converters on the device -- replace reorder<T, dst, src> (include/euler_reorder.hpp:9-64,
 * src/elx_reorder.cpp:11-207) for the two conversions callers with plain tensors need.
 * elem_bytes is 1 or 4.  Pointers are device pointers; stream may be NULL. */
ELB_API int elb_reorder_nchw_to_nChw16c(void *dst, const void *src, int n, int c, int h, int w,
                                        int elem_bytes, void *cuda_stream);
ELB_API int elb_reorder_nChw16c_to_nchw(void *dst, const void *src, int n, int c, int h, int w,
                                        int elem_bytes, void *cuda_stream);

/* Any layout conversion the reference exports, on the device -- replaces the twelve
 * reorder<T, dst, src> specialisations (src/elx_reorder.cpp:11-207): nchw <-> nhwc, nchw <-> nChw16c,
 * oihw <-> hwio, oihw <-> OIhw16i16o, goihw <-> ghwio, goihw <-> gOIhw16i16o -- and the remaining
 * pairs inside each family (nhwc <-> nChw16c, hwio <-> OIhw16i16o, ghwio <-> gOIhw16i16o).
 * dst_format / src_format are ELB_NCHW ... ELB_GOIHW16I16O; (g, a, b, h, w) are the logical extents
 * (activations: g ignored, a = n, b = c; weights: a = o, b = i; g only for the g* formats).
 * Lanes of a blocked destination past o / i / c are written as zero, as the reference does.
 * elem_bytes is 1 or 4; pointers are device pointers; returns ELB_UNIMPLEMENTED for other pairs. */
ELB_API int elb_reorder(void *dst, int dst_format, const void *src, int src_format, int g, int a, int b,
                        int h, int w, int elem_bytes, void *cuda_stream);

/* Spatial subsample of an nChw16c tensor on the device: dst[n][C/16][ceil(h/step_h)][ceil(w/step_w)][16]
 * = src[n][C/16][y*step_h][x*step_w][16].  The glue between two layers of a stack that the reference's
 * harness leaves to the host (tests/elt_conv.cpp:399-410 feeds a layer's output to the next layer). */
ELB_API int elb_subsample_nChw16c(void *dst, const void *src, int n, int c, int h, int w, int step_h,
                                  int step_w, int elem_bytes, void *cuda_stream);

/* ---- A chain of convolutions that stays on the device --------------------------------------
 * Replaces the layer-to-layer modes of the reference's harness (tests/elt_conv.cpp:399-410:
 * --output_as_input feeds a layer's output tensor to the next call, --dbuffering alternates two
 * buffer sets): layer k's output is layer k+1's input, u8 between int8 layers, fp32 between fp32
 * layers; subsample_after[k] = s > 1 keeps every s-th row and column of layer k's output (the
 * stride-2 stand-in for pooling between the stages of VGG-16).  All descriptors name the same batch
 * n, nChw16c activations and one device (descs[0].device); the FIRST layer's input may instead be
 * the caller's plain image (ELB_NCHW or ELB_NHWC, as the reference's first-layer runs pass it,
 * scripts/regression-fp32.sh: --input-format=nchw).  An fp32 3x3 stride-1 layer with at most four
 * input channels reads an nchw image directly (three planes instead of a 16-channel block of which
 * three channels are real); other plain inputs are converted on the device first. */
typedef struct elb_stack elb_stack_t;
ELB_API int elb_stack_create(const elb_conv_desc_t *descs, const int32_t *subsample_after, int n_layers,
                             elb_stack_t **stack);
/* Weights and bias of one layer (read once, like the first elx_conv of that layer). */
ELB_API int elb_stack_prepare(elb_stack_t *stack, int layer, const void *weights, const void *bias);
/* Enqueue the chain for one batch of n images on cuda_stream; DEVICE pointers; does not wait.
 * May be captured into a CUDA graph by the caller. */
ELB_API int elb_stack_enqueue(elb_stack_t *stack, void *output, const void *input, void *cuda_stream);
/* Run `images` images (a multiple of n) and wait.  Host or device tensors.  Host tensors go through
 * two staging slots: the copy in of batch b+1, the chain of batch b (one CUDA graph launch) and the
 * copy out of batch b-1 overlap. */
ELB_API int elb_stack_execute(elb_stack_t *stack, void *output, const void *input, int64_t images);
/* The plan of one layer (owned by the stack): for elb_conv_info, launch counts, stage events. */
ELB_API int elb_stack_layer(elb_stack_t *stack, int layer, elb_conv_t **plan);
/* Device address and size of layer k's output tensor inside the stack (nChw16c, the whole batch;
 * before any subsample): what the reference's harness would hand to the next call.  Valid until the
 * stack is destroyed; read it only after the run that wrote it has finished.  NULL for the last
 * layer when its output goes straight to the caller's tensor. */
ELB_API int elb_stack_layer_output(elb_stack_t *stack, int layer, void **device_ptr, uint64_t *bytes);
/* Measurement hook, no counterpart in the reference: n_layers + 1 cudaEvent_t handles recorded
 * before every layer and after the last one by elb_stack_enqueue; NULL switches it off (it must be
 * off during stream capture and for elb_stack_execute on host tensors). */
ELB_API int elb_stack_set_layer_events(elb_stack_t *stack, void **cuda_events, int count);
/* Layer count and the byte sizes of one batch of the first input and the last output. */
ELB_API int elb_stack_sizes(const elb_stack_t *stack, int32_t *n_layers, uint64_t *bytes_input, uint64_t *bytes_output);
ELB_API uint64_t elb_stack_launch_count(const elb_stack_t *stack);
ELB_API void elb_stack_destroy(elb_stack_t *stack);

/* ---- One convolution, minibatch split over the GPUs of one box ------------------------------
 * The reference spreads images / tiles over the OpenMP threads of one process
 * (src/elx_conv_wino_xopt.hpp:41-64, src/elx_int8_conv_direct_1x1_xopt.hpp:91-97); here GPU r takes
 * images [r*N/G, (r+1)*N/G) of ONE host tensor.  Every GPU prepares its own copy of the weights on
 * the first call; nothing is exchanged between GPUs, so the result is bit-identical to the
 * one-GPU result.  devices = NULL: GPUs 0..G-1 with G = n_devices if > 0, else EULER_GPUS, else all
 * visible GPUs. */
typedef struct elb_conv_multi elb_conv_multi_t;
ELB_API int elb_conv_multi_create(const elb_conv_desc_t *desc, const int32_t *devices, int n_devices,
                                  elb_conv_multi_t **multi);
/* elx_conv on host tensors of all N images; returns when every slab is back in `output`. */
ELB_API int elb_conv_multi_execute(elb_conv_multi_t *multi, void *output, const void *input, const void *weights,
                                   const void *bias);
/* How the batch was split: in: *n_parts = capacity of the arrays; out: *n_parts = GPUs used. */
ELB_API int elb_conv_multi_parts(const elb_conv_multi_t *multi, int32_t *n_parts, int32_t *devices,
                                 int32_t *first_image, int32_t *image_count);
ELB_API void elb_conv_multi_destroy(elb_conv_multi_t *multi);

/* FP32 Winograd F(4x4,3x3) convolution that allocates nothing -- no counterpart in the reference.
 *
 * For callers that may not allocate device memory at the point where they run a convolution (a
 * server whose GPU memory was handed to a fixed arena at start-up, a latency-critical loop that
 * must stay off the driver's allocation lock, a plug-in confined to its host framework's memory
 * budget).  All transform-domain buffers live in one 64 MiB array that is part of the library
 * image on every GPU; the call uses no cudaMalloc/cudaFree and no allocating library routine.
 *
 *   desc      fp32 in/weights/out/bias, nChw16c / OIhw16i16o, 3x3, stride 1, pad 1, g = 1;
 *             with_bias / with_relu / with_ip_sum are honoured
 *   output, input, weights, bias   DEVICE pointers on the current device, 16-byte aligned; weights
 *             in the caller's OIhw16i16o form (they are transformed on the device in every call)
 *   cuda_stream   cudaStream_t the kernels are enqueued on (NULL = default stream); the call does
 *             not wait for them
 *
 * Limits: problems whose buffers (packed weights + transformed input + transform-domain result)
 * exceed 64 MiB return ELB_UNIMPLEMENTED, message in elb_last_error().  The array is shared by
 * every call in the process and keeps the previous call's contents (this path overwrites all it
 * reads and clears its status word itself): calls that overlap on the GPU race, so serialise
 * them.  The FIRST call on each device resolves the array's device address and sets a kernel
 * attribute; issue it once before any CUDA stream capture starts. */
ELB_API int elb_wino_f32_conv_noalloc(const elb_conv_desc_t *desc, void *output, const void *input,
                                      const void *weights, const void *bias, void *cuda_stream);

/* Verdict of the last elb_wino_f32_conv_noalloc on the current device -- no counterpart in the
 * reference.  The kernels' waits are bounded; one that gives up leaves a code in the first word of
 * the static array, and the output of that call is invalid.  0 = ok, > 0 = the code, -1 = the
 * entry point has not run on this device (or the read failed).  Call it after synchronising the
 * stream the convolution ran on; it copies four bytes to the host and allocates nothing. */
ELB_API int elb_wino_f32_noalloc_status(void);

#ifdef __cplusplus
}
#endif
#endif /* EULER_B200_H_ */
