/*
 * gie_b200 -- C ABI of the B200 (sm_100a) implementation of the fused Conv2D / RMSNorm path.
 *
 * This is the drop-in boundary: plain pointers, fixed-width integers, integer status codes, no C++ types,
 * no exceptions.  The C++ operator layer (gie::Conv2D, gie::ExecutionPlan, gie::rmsnorm_forward, ...) and any
 * foreign-language binding sit on top of exactly these entry points.  Each entry point names the interface of
 * the reference library (lehendo/cuda-inference, paths relative to its root) that it stands in for.
 *
 * Conventions
 *  - Every function returns a gieb_status (numeric values of gie::StatusCode, include/gpu_inference/error.h:16-26);
 *    on failure gieb_last_error() returns a thread-local message.  Nothing is launched when a call fails.
 *  - Tensor pointers are DEVICE pointers owned by the caller: X contiguous NCHW, W contiguous OIHW, bias [O],
 *    Y contiguous NCHW, all in the problem's storage type (include/gpu_inference/conv2d.h:1-7, 66-69).
 *  - `stream` is a cudaStream_t passed as void*.  Launch functions never synchronise, never allocate and are safe
 *    to call while the stream is being captured into a CUDA graph (include/gpu_inference/conv2d.h:100-104,
 *    include/gpu_inference/cuda_graph.h:16).  Plan creation may allocate and synchronise a private stream.
 *  - A plan is immutable after creation and may be used concurrently from many host threads and streams as long
 *    as each concurrent launch has its own workspace (tests/test_runtime_concurrency.cu:110-188).
 */
#ifndef GIE_B200_H_
#define GIE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define GIEB_API
#else
#define GIEB_API __attribute__((visibility("default")))
#endif

/* Numeric values of gie::StatusCode (include/gpu_inference/error.h:16-26). */
typedef enum gieb_status {
  GIEB_OK = 0,
  GIEB_INVALID_ARGUMENT = 1,
  GIEB_UNSUPPORTED = 2,
  GIEB_WORKSPACE_TOO_SMALL = 3,
  GIEB_CUDA_ERROR = 4,
  GIEB_INTERNAL = 7
} gieb_status;

/* Order of gie::Precision (include/gpu_inference/conv2d.h:26).  GIEB_TF32: FP32 tensors (x, w, bias, y), inputs rounded
 * to TF32 (nearest, ties away) and multiplied on the tensor cores (kind::tf32), FP32 accumulation and output; the
 * reference reaches this precision only through cuBLAS (src/kernels/im2col.cu:108-112).  cfg.tile_k counts FP32 values
 * for it (8, 16 or 32 per slab row); routes 1 and 4; no extension flags.
 * GIEB_FP8_E4M3 (an extension: gie::Precision has no such member, so it is reachable through this C ABI only): x and w are
 * FP8 E4M3 bit patterns (1 byte per element, NCHW / OIHW), bias is float[O], y is FP16 NCHW.  Products are exact in the
 * tensor core (kind::f8f6f4), FP32 accumulation, bias + ReLU in FP32, one rounding to FP16.  cfg.tile_k counts FP8 values
 * (32, 64 or 128 per slab row); routes 1 and 4; no extension flags. */
typedef enum gieb_precision { GIEB_FP32 = 0, GIEB_FP16 = 1, GIEB_BF16 = 2, GIEB_TF32 = 3, GIEB_FP8_E4M3 = 4 } gieb_precision;

/* Optional behaviour beyond the reference API (all off by default = exact drop-in behaviour). */
enum {
  GIEB_FLAG_BIAS_FP32 = 1u << 0,        /* bias is float[O] even for 16-bit storage                              */
  GIEB_FLAG_WEIGHTS_PREPACKED = 1u << 1, /* `w` already holds gieb_prepack_weights output (static weights)      */
  /* Channel-contiguous tensors and a fused residual for chains of convolutions (16-bit tensor path only).  The
   * reference keeps every tensor NCHW (include/gpu_inference/conv2d.h:66-69) and has no residual operand; its
   * epilogue hook is src/kernels/fused_epilogue.cuh:11-16.  A chain that stays channel-contiguous needs no layout
   * repack between layers, and the residual add + ReLU of a bottleneck block disappears into the epilogue. */
  GIEB_FLAG_INPUT_NHWC = 1u << 2,   /* x is [B][H][W][C], 16-byte aligned, C a multiple of 16: read in place, no repack */
  GIEB_FLAG_OUTPUT_NHWC = 1u << 3,  /* y (and the residual) are [B][P][Q][O]                                             */
  GIEB_FLAG_RESIDUAL = 1u << 4      /* y = act(conv + bias + residual); launch with gieb_conv_launch_fused               */
};

/* Conv2DParams + ConvProblem (include/gpu_inference/conv2d.h:47-85) as fixed-width fields. */
typedef struct gieb_conv_desc {
  int32_t batch, in_channels, in_h, in_w;
  int32_t out_channels, kernel_h, kernel_w;
  int32_t stride_h, stride_w, pad_h, pad_w;
  int32_t dilation_h, dilation_w, groups;
  int32_t precision; /* gieb_precision */
  int32_t has_bias;
  int32_t relu;      /* Activation::kReLU */
  uint32_t flags;    /* GIEB_FLAG_* */
} gieb_conv_desc;

/* One point of the single sm_100a kernel family; replaces the reference's per-backend template parameter lists
 * (src/kernels/tensor_core_mma.cu:369-388, src/kernels/implicit_gemm.cu:243-266).  Zero / NULL = heuristic. */
typedef struct gieb_conv_cfg {
  int32_t tile_n;   /* output channels per CTA tile: 32, 64, 128 or 256 (tensor path); 0 = auto              */
  int32_t tile_k;   /* reduction slab in channels: 16, 32 or 64; 0 = auto                                    */
  int32_t stages;   /* shared-memory ring depth, 2..8; 0 = auto                                              */
  int32_t split_k;  /* number of reduction splits, >= 1; 0 = auto                                            */
  int32_t variant;  /* 0 = auto; 1 = tensor path, im2col-mode TMA over the channel-contiguous copy (any geometry);
                       4 = tensor path, tiled TMA over that copy (1x1, pad 0; stride 1, or any stride over an NCHW 16-bit
                           input, in which case the copy holds only the pixels the convolution reads);
                       2 = tensor path reading the caller's NCHW activations directly, no activation repack
                           (1x1, stride 1, pad 0, H*W % 8 == 0; a call whose x is not 16-byte aligned takes route 4);
                       3 = FP32 SIMT;
                       5 = tensor path over row-gathered activations for inputs with few channels (NCHW input,
                           kernel_w > 1, kernel_w * C <= 64): the S taps of a filter row become channels, so a 7x7
                           stem over 3 channels reduces over 7 x 32 values instead of 49 x 16 padded ones      */
  int32_t tile_m;   /* output pixels per CTA tile: 128 or 256 (two accumulators share each weight tile); 0 = auto */
  int32_t reduce;   /* how split-K slices are summed: 0 = auto; 1 = FP32 partials in the workspace + a reduction launch;
                       2 = inside the convolution kernel: the slices of a tile form a thread-block cluster and are
                           summed through distributed shared memory (split_k 2, 4 or 8 dividing tile_n / 32,
                           tile_m 128); no partials in the workspace, no extra launch                       */
  int32_t cta_pair; /* 0 = auto; 1 = every tile is computed by one CTA; 2 = 256-pixel tiles computed by pairs of CTAs (clusters
                       of two, tcgen05.mma.cta_group::2): each CTA stages its own 128 pixels and half of the weight tile, so
                       the weight traffic per SM is halved.  FP16 / BF16, tile_n 64, 128 or 256, tile_m 0 or 256, split-K
                       slices through the workspace (reduce 0 or 1)                                                  */
} gieb_conv_cfg;

/* What KernelDesc::supports / workspace_bytes / dynamic_smem_bytes / num_blocks answer
 * (include/gpu_inference/kernel_registry.h:62-70). */
typedef struct gieb_conv_info {
  int32_t supported;
  int32_t variant;
  gieb_conv_cfg cfg;          /* the configuration that would run (heuristic filled in)  */
  uint64_t workspace_bytes;   /* caller-provided per-call scratch                          */
  uint64_t persistent_bytes;  /* plan-owned device memory                                  */
  uint32_t dynamic_smem_bytes;
  uint32_t threads_per_block;
  int64_t num_blocks;
  int32_t launches;           /* kernel launches per forward call                          */
  int32_t padded_channels;    /* C_in rounded up for the channel-contiguous copy           */
  char reason[256];           /* why not, when supported == 0                              */
} gieb_conv_info;

typedef struct gieb_conv_plan gieb_conv_plan;

/* Thread-local text of the last failure on this thread ("" if none). */
GIEB_API const char* gieb_last_error(void);

/* Library identity: kLibraryVersion analogue (include/gpu_inference/kernel_registry.h:24). */
GIEB_API int gieb_version(void);

/* validate_problem (src/runtime/conv2d.cpp:83-109): same checks, same status codes. */
GIEB_API int gieb_conv_validate(const gieb_conv_desc* desc);

/* KernelDesc::supports + workspace_bytes + dynamic_smem_bytes + num_blocks
 * (include/gpu_inference/kernel_registry.h:62-70; src/kernels/tensor_core_mma.cu:280-295,326-330).
 * device < 0 = current device.  Needs no GPU work. */
GIEB_API int gieb_conv_query(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg, int device, gieb_conv_info* out);

/* ExecutionPlan::create (src/runtime/execution_plan.cpp:51-76): capability check, workspace size, plan-owned
 * state (status word), kernel attributes.  May allocate and synchronise a private stream only. */
GIEB_API int gieb_conv_plan_create(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg, int device,
                                   gieb_conv_plan** out);
GIEB_API void gieb_conv_plan_destroy(gieb_conv_plan* plan);
GIEB_API int gieb_conv_plan_info(const gieb_conv_plan* plan, gieb_conv_info* out);

/* ExecutionPlan::execute_unchecked -> KernelDesc::launch (src/runtime/execution_plan.cpp:121-138;
 * src/kernels/tensor_core_mma.cu:297-324): layout repack + weight prepack + implicit-GEMM (+ split-K reduce)
 * on `stream`.  Checks only what it needs to stay memory-safe: non-null pointers, workspace size and 256-byte
 * alignment (src/runtime/execution_plan.cpp:103-108), current device == plan device (:113-117). */
GIEB_API int gieb_conv_launch(const gieb_conv_plan* plan, const void* x, const void* w, const void* bias, void* y,
                              void* workspace, size_t workspace_bytes, void* stream);

/* Static weights (GIEB_FLAG_WEIGHTS_PREPACKED): the layout a plan's kernel reads depends on its route ([O][R*S][Cp]
 * on the repack routes -- what gieb_prepack_weights writes -- and [O][R][padded S*C] on the row-gather route), so the
 * plan itself converts OIHW weights once: size of the converted tensor, and the conversion on `stream` (dst 16-byte
 * aligned).  Stands in for the per-call weight transpose of the reference (src/kernels/tensor_core_mma.cu:310). */
GIEB_API int gieb_conv_plan_prepacked_weight_bytes(const gieb_conv_plan* plan, uint64_t* bytes);
GIEB_API int gieb_conv_plan_prepack_weights(const gieb_conv_plan* plan, const void* w, void* dst, void* stream);

/* gieb_conv_launch with one more operand (no reference counterpart): `residual` has the shape, layout and storage
 * type of y and is added in FP32 before the activation and the single rounding.  Required (non-null) for plans
 * created with GIEB_FLAG_RESIDUAL, refused for others.  `residual` may be the same buffer as y (each element is read
 * by the thread that writes it) but must not overlap x or w. */
GIEB_API int gieb_conv_launch_fused(const gieb_conv_plan* plan, const void* x, const void* w, const void* bias,
                                    const void* residual, void* y, void* workspace, size_t workspace_bytes, void* stream);

/* Measurement helper standing in for the stage_events hook of ExecutionPlan::execute
 * (include/gpu_inference/execution_plan.h:25-31, kernel_registry.h:38-40) and time_stream_work
 * (src/runtime/timing.cpp:21-83): runs `iters` forward calls on `stream` with CUDA events between the stages,
 * synchronises the stream and returns average milliseconds per call of stage_ms[0] = layout repack + weight
 * prepack, [1] = convolution kernel, [2] = split-K reduction.  Creates events and synchronises: not for hot paths. */
GIEB_API int gieb_conv_time_stages(const gieb_conv_plan* plan, const void* x, const void* w, const void* bias, void* y,
                                   void* workspace, size_t workspace_bytes, void* stream, int iters, float* stage_ms);

/* Measurement helper (the stage_events hook again, include/gpu_inference/kernel_registry.h:38-40, in a form that can
 * be captured into a CUDA graph): gieb_conv_launch restricted to the stages in `stage_mask` -- bit 0 = layout repack +
 * weight prepack, bit 1 = convolution kernel, bit 2 = split-K reduction launch.  A call without bit 0 reads the
 * repacked tensors a previous full launch left in `workspace`; a benchmark replays graphs of single-stage calls to
 * time one kernel back to back.  Not for plans with a fused residual. */
GIEB_API int gieb_conv_launch_stages(const gieb_conv_plan* plan, unsigned stage_mask, const void* x, const void* w,
                                     const void* bias, void* y, void* workspace, size_t workspace_bytes, void* stream);

/* No counterpart in the reference.  One-shot forward call for callers that are not allowed to allocate device memory
 * -- code running inside someone else's memory budget (a serving process whose pool owns the whole GPU, a plug-in
 * loaded into a host application, a real-time loop) where cudaMalloc either fails or stalls everything on the device.
 * It does what gieb_conv_plan_create + gieb_conv_launch do, but the scratch the path needs (channel-contiguous copy
 * of X, prepacked W, split-K partials, status word) lives in an 8 MiB array that is part of the library image, so the
 * call performs no cudaMalloc/cudaFree and calls no allocating routine.  Limits and rules:
 *   - problems whose scratch exceeds 8 MiB are refused with GIEB_WORKSPACE_TOO_SMALL (the message says how much is
 *     needed); use the plan API with your own workspace for those;
 *   - every GPU that loads the library carries the 8 MiB + 256 B until the process exits;
 *   - the first call on each device looks up the array's device address (with that device current); make that first
 *     call outside any stream capture;
 *   - all calls on a device share the one array: two calls whose GPU work overlaps (different streams, different
 *     threads) race on it -- serialise them on one stream or with events.  Nothing is carried from call to call:
 *     the status word is cleared and the rest rewritten on every call;
 *   - a bounded device-side wait that runs out leaves y incomplete and is reported only through
 *     gieb_conv_static_status: call it (it waits for the stream) before using y;
 *   - there is no residual operand: GIEB_FLAG_RESIDUAL is refused, sm_100 devices only.
 * Results are bit-identical to gieb_conv_launch with the same configuration. */
GIEB_API int gieb_conv_forward_static(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg, const void* x, const void* w,
                                      const void* bias, void* y, void* stream);

/* No counterpart in the reference.  Companion of gieb_conv_forward_static, equally allocation-free: the kernels
 * report a bounded device-side wait that ran out (the result of that call is then incomplete) in a status word at the
 * head of the built-in scratch; gieb_conv_forward_static clears it at the start of every call.  This copies the word of
 * the current device to *status_out on `stream` and waits for that stream, so pass the stream the forward call ran on:
 * 0 means the last call on this device computed everything.  Check it before trusting y. */
GIEB_API int gieb_conv_static_status(uint32_t* status_out, void* stream);

/* Device-side status word of the plan: 0 = no kernel of this plan ever gave up on a bounded wait.  Synchronises
 * nothing itself; call after the stream has been synchronised.  (No reference counterpart: the reference's
 * kernels have no asynchronous waits.) */
GIEB_API int gieb_conv_plan_device_status(const gieb_conv_plan* plan, uint32_t* status_out);

/* Test hook (no reference counterpart; the reference's kernels cannot stall).  Makes later launches of this plan fail
 * the way a lost TMA completion would, without faulting anything: `roles` bit 0 = the TMA producer warps issue no
 * loads, bit 1 = the MMA warp issues nothing and signals nobody; the warps that wait for them give up after
 * `wait_limit_cycles` SM cycles (at most 2e9, about a second), set their bit in the plan's status word (1 = producer,
 * 2 = MMA issuer, 4 = epilogue), and the kernel ends by itself with its tensor memory freed.  The output of such a
 * launch is garbage by construction.  roles = 0 restores normal behaviour.  Not thread-safe: call it while no other
 * thread uses the plan. */
GIEB_API int gieb_conv_plan_inject_stall(gieb_conv_plan* plan, uint32_t roles, uint64_t wait_limit_cycles);

/* transpose_c_hw as used for X (src/kernels/tensor_core_mma.cu:61-82,309): 16-bit [B][C][HW] -> [B][HW][Cp],
 * Cp = c_padded >= C (extra channels zero).  Bit-exact permutation.  `src` needs only 2-byte alignment,
 * `dst` 16-byte alignment and c_padded % 8 == 0. */
GIEB_API int gieb_repack_nchw_to_nhwc(const void* src, void* dst, int batch, int channels, int hw, int c_padded,
                                      void* stream);

/* transpose_c_hw as used for W (src/kernels/tensor_core_mma.cu:310): 16-bit OIHW [O][C][RS] -> [O][RS][Cp]. */
GIEB_API int gieb_prepack_weights(const void* src, void* dst, int out_channels, int channels, int rs, int c_padded,
                                  void* stream);

/* Channel count of the channel-contiguous copy the tensor path would use for this problem and configuration. */
GIEB_API int gieb_padded_channels(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg);

/* RmsNormParams (include/gpu_inference/rmsnorm.h:17-22). dtype: 0 = FP32, 1 = FP16, 2 = BF16 (gie::DataType). */
typedef struct gieb_rmsnorm_desc {
  int32_t rows, hidden;
  float eps;
  int32_t dtype;
  uint32_t flags;  /* bit 0: gamma is float[hidden] even for 16-bit storage */
} gieb_rmsnorm_desc;

/* rmsnorm_forward (src/transformer/rmsnorm.cu:155-166): y = rmsnorm(x)*gamma, or with both residual pointers
 * res_out = round(x + res_in), y = rmsnorm(res_out)*gamma.  Same argument checks and status codes. */
GIEB_API int gieb_rmsnorm_launch(const gieb_rmsnorm_desc* desc, const void* x, const void* gamma, void* y,
                                 const void* residual_in, void* residual_out, void* stream);

/* launch_bias_act (include/gpu_inference/fused_ops.h:13-19; src/kernels/elementwise.cu:13-55): in-place
 * y = act(y + bias[channel]) on an NCHW tensor; bias may be NULL, relu may be 0. */
GIEB_API int gieb_bias_act_launch(int precision, int batch, int channels, int hw, const void* bias, int relu, void* y,
                                  void* stream);

/* Glue of the ResNet-50-shaped chain; the reference has neither operator (its chain benchmark is conv-only,
 * benchmarks/graph_bench.cpp:84-91).  16-bit NCHW tensors. */
GIEB_API int gieb_maxpool2d_launch(int precision, int batch, int channels, int h, int w, int kernel, int stride, int pad,
                                   const void* x, void* y, void* stream);
/* The same pooling on channel-contiguous [B][H][W][C] tensors (fp16 / bf16, C % 8 == 0, 16-byte aligned). */
GIEB_API int gieb_maxpool2d_nhwc_launch(int precision, int batch, int channels, int h, int w, int kernel, int stride, int pad,
                                        const void* x, void* y, void* stream);
GIEB_API int gieb_add_relu_launch(int precision, int relu, const void* a, const void* b, void* y, int64_t n, void* stream);

/* estimate_kernel (src/runtime/perf_model.cpp:130-174) for this family: the library's own cycle model for the
 * configuration `cfg` (NULL = the one the heuristic picks), in microseconds.  For ranking and pruning tuning candidates;
 * validation and timing of candidates are the reference autotuner's own (src/autotuner/autotuner.cpp:60-117). */
GIEB_API int gieb_conv_estimate_us(const gieb_conv_desc* desc, const gieb_conv_cfg* cfg, double* microseconds);

#ifdef __cplusplus
}
#endif
#endif /* GIE_B200_H_ */
