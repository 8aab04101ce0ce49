/*
 * dnxcu — C ABI of the sm_100a dispatch backend for denox fp16 HWC U-Nets.
 *
 * denox has no C ABI of its own: its hot path sits behind C++ interfaces
 * (variant generator, dispatch record, runtime instance, benchmark database).
 * Each entry point below names the reference interface it stands in for
 * (paths relative to the reference project root).  A maintainer binds these
 * from the reference's C++ with a plain `extern "C"` include; nothing here
 * uses C++ types, exceptions or torch types.
 *
 * Conventions
 *  - every function returns DNXCU_OK (0) or a negative dnxcu_status;
 *    nothing throws, aborts or exits;
 *  - tensors are HWC binary16: index(h,w,c) = (h*W + w)*C + c
 *    (common/src/denox/memory/tensor/ActivationLayout.hpp:38-40);
 *  - "launch" calls are stream ordered and never synchronise; the caller owns
 *    every device buffer it passes in;
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream).
 */
#ifndef DNXCU_H
#define DNXCU_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define DNXCU_API
#else
#define DNXCU_API __attribute__((visibility("default")))
#endif

typedef enum dnxcu_status {
  DNXCU_OK = 0,
  DNXCU_E_BAD_ARG = -1,      /* null pointer, non-positive size, inconsistent channels */
  DNXCU_E_UNSUPPORTED = -2,  /* the variant cannot run this shape / flag combination   */
  DNXCU_E_MISALIGNED = -3,   /* a pointer breaks the variant's alignment rule          */
  DNXCU_E_CUDA = -4,         /* a CUDA runtime call failed; see dnxcu_last_cuda_error  */
  DNXCU_E_DEVICE = -5,       /* a kernel reported a bounded wait that ran out          */
  DNXCU_E_NO_MEMORY = -6,
  DNXCU_E_STATE = -7,        /* object used in the wrong state                         */
  DNXCU_E_IO = -8,           /* database file could not be read or written             */
  DNXCU_E_LIMIT = -9         /* a fixed capacity of the library was exceeded           */
} dnxcu_status;

/* Human readable name of a status code (static string). */
DNXCU_API const char *dnxcu_status_string(int status);
/* cudaError_t of the most recent failing CUDA call on this thread (0 if none). */
DNXCU_API int dnxcu_last_cuda_error(void);

/* ------------------------------------------------------------------------
 * Device capabilities.
 * Stands in for denox::DeviceInfo filled by query_driver_device_info
 * (device_info/src/denox/device_info/DeviceInfo.hpp:12-20), which the variant
 * generators read to prune their configuration space
 * (compiler/src/denox/compiler/implement/shaders/conv/DirectConvShaderCM.cpp:19-28).
 * ---------------------------------------------------------------------- */
typedef struct dnxcu_caps {
  int32_t device;
  int32_t cc_major, cc_minor;
  int32_t sm_count;
  int32_t max_threads_per_block;
  int32_t tmem_columns; /* tensor memory columns per SM (512 on sm_100)  */
  int32_t tcgen05;      /* 1 when the tcgen05/TMEM conv variants can run */
  int32_t reserved;
  uint64_t smem_per_block_optin; /* bytes */
  uint64_t l2_bytes;
  uint64_t global_bytes;
  char name[64];
} dnxcu_caps;

DNXCU_API int dnxcu_get_device_caps(int device, dnxcu_caps *caps);

/* ------------------------------------------------------------------------
 * Kernel variants.
 * A variant is what an IShader configuration is in the reference
 * (compiler/src/denox/compiler/implement/shaders/IShader.hpp:33-71): one
 * kernel family with one fixed set of tuning parameters.  `config` uses the
 * reference's KEY=VAL#KEY=VAL spelling (DirectConvShaderCM.cpp:690-694).
 * ---------------------------------------------------------------------- */
typedef enum dnxcu_op {
  DNXCU_OP_CONV3X3 = 1,    /* direct_conv_cm.comp / concat_conv_cm.comp / direct_conv.comp */
  DNXCU_OP_MAXPOOL2X2 = 2, /* basic_pool.comp      */
  DNXCU_OP_UPSAMPLE2X = 3, /* basic_upsample.comp  */
  DNXCU_OP_CONCAT = 4,     /* copy_transform.comp  */
  DNXCU_OP_RELU = 5,       /* basic_activation.comp */
  DNXCU_OP_PAD_CHANNELS = 6, /* copy_transform.comp used as a layout change: HWC with C channels ->
                                HWC with c_out >= C channels, the new ones zero (what the reference's
                                HWC -> HWC8 / CHWC8 layout specialisation does,
                                specialization/specialization.cpp:183-340) */
  DNXCU_OP_PAD_EDGE = 7,     /* memory_pad.comp: spatial pad, source coordinate clamped to the input
                                (edge replication); pc = {OUT_W, OUT_H},
                                pc_ext = {PAD_LEFT, PAD_RIGHT, PAD_TOP, PAD_BOTTOM} */
  DNXCU_OP_SLICE = 8         /* memory_slice.comp: out[h][w] = in[h + IN_TOP][w + IN_LEFT];
                                pc = {OUT_W, OUT_H}, pc_ext = {IN_LEFT, IN_TOP, IN_W, IN_H} */
} dnxcu_op;

/* dispatch flags (conv only unless noted) */
#define DNXCU_F_RELU 0x01u        /* max(0, x) on the finished sum                          */
#define DNXCU_F_BIAS 0x02u        /* dispatch.bias holds c_out binary16 values              */
#define DNXCU_F_UP2X_A 0x04u      /* operand a is (H/2)x(W/2), read through src = dst/2      */
#define DNXCU_F_POOL_OUT 0x08u    /* also write the 2x2 max pooled result to out_pool       */
#define DNXCU_F_NO_FULL_OUT 0x10u /* with POOL_OUT: do not write the full resolution output */
#define DNXCU_F_LEAKY 0x20u       /* max(x, alpha * x) in binary16 on the finished, rounded sum
                                     (direct_conv_cm.comp:1071-1076, basic_activation.comp:29-30);
                                     alpha = dispatch.leaky_alpha; excludes DNXCU_F_RELU; also the
                                     flag that turns a DNXCU_OP_RELU dispatch into a LeakyReLU */

typedef struct dnxcu_variant_desc {
  int32_t id;          /* index in the table, stable within one build of the library */
  int32_t op;          /* dnxcu_op */
  const char *family;  /* e.g. "direct-conv-tc" (names follow the reference's shaders) */
  const char *config;  /* KEY=VAL#KEY=VAL */
  uint32_t allowed_flags; /* dispatch flags this variant implements */
  int32_t needs_tcgen05;  /* 1: requires dnxcu_caps.tcgen05 */
  int32_t c_align;        /* operand channel counts must be multiples of this, or 1 */
  int32_t k_align;        /* output channel count must be a multiple of this, or 1  */
  int32_t max_c_out;
  int32_t reserved;
} dnxcu_variant_desc;

/* Registration list; stands in for get_all_shaders
 * (compiler/src/denox/compiler/implement/shaders/shaders.cpp:16-50). */
DNXCU_API int dnxcu_variant_count(void);
DNXCU_API const dnxcu_variant_desc *dnxcu_variant(int id);
/* First variant whose family and config match exactly, or DNXCU_E_BAD_ARG. */
DNXCU_API int dnxcu_find_variant(const char *family, const char *config);
/* SHA-256 of (family, config, digest of the kernel sources the library was built from) as 64 hex digits
 * plus NUL: the identity a benchmark database keys on; editing a kernel changes it, so stored timings of
 * an older build are not picked up.  Stands in for GlslCompilerInstance::fast_sha256, the hash of source
 * text and preamble (spirv/src/denox/glsl/GlslCompilerInstance.hpp:73-79). */
DNXCU_API int dnxcu_variant_sha256(int id, char out_hex[65]);

/* ------------------------------------------------------------------------
 * One dispatch.
 * Stands in for ComputeDispatch
 * (compiler/src/denox/compiler/implement/ComputeDispatch.hpp:29-40) and its
 * run-time form InstanceDispatch (runtime/src/denox/runtime/instance.hpp:13-21).
 * pc[] keeps the reference's push constant block {IN_W, IN_H}
 * (DirectConvShaderCM.cpp:628-630): the extent of the tensor the kernel
 * iterates over — the output resolution for a conv, the input resolution for
 * pool / upsample / concat / relu.  Channel counts, which the reference bakes
 * into the shader as #defines, are plain fields.
 * Pointers follow the reference's binding order: inputs, outputs, parameters.
 * ---------------------------------------------------------------------- */
typedef struct dnxcu_dispatch {
  int32_t variant;
  uint32_t flags;
  uint32_t pc[2]; /* IN_W, IN_H */
  int32_t c_a;    /* channels of operand a */
  int32_t c_b;    /* channels of operand b (concat second operand), 0 if none */
  int32_t c_out;  /* output channels (conv); ignored otherwise */
  float leaky_alpha; /* slope of DNXCU_F_LEAKY (rounded to binary16 before use, as the reference's
                        atype(ACTIVATION_LeakyReLU_alpha)); ignored without the flag */
  const void *in_a;
  const void *in_b;
  void *out;
  void *out_pool;      /* (H/2)x(W/2)xc_out, conv with DNXCU_F_POOL_OUT */
  const void *weights; /* blob made by dnxcu_prepare_weights for this variant */
  const void *bias;    /* c_out binary16, or NULL */
  /* Row band execution: one row (W x C binary16, or (W/2) x C for an operand
   * read through UP2X_A) that sits directly above / below this band in the
   * full image, already resident in this device's memory.  NULL = image
   * border (zeros).  Order: a_top, a_bottom, b_top, b_bottom. */
  const void *halo[4];
  int32_t *device_status; /* optional device int: a kernel stores a non-zero code
                             here when one of its bounded waits ran out
                             (1 weights, 2 input row, 3 accumulator block free,
                             4/5 streamed weights, 6 accumulators complete,
                             7 input slot free, 8 raw row of the upsampled
                             operand, 10 halo row of a neighbouring band) or
                             when it met a state it refuses to compute in (9);
                             the launch returns normally and the output is
                             then undefined */
  uint32_t pc_ext[4];     /* further push constants of pad / slice dispatches (see dnxcu_op) */
} dnxcu_dispatch;

/* Checks the dispatch against the variant's rules without launching. */
DNXCU_API int dnxcu_validate(const dnxcu_dispatch *d);
/* Enqueues the kernel on `stream`.  Stands in for the vkCmdDispatch recorded in
 * Instance::infer (runtime/src/denox/runtime/instance.cpp:367-396). */
DNXCU_API int dnxcu_launch(const dnxcu_dispatch *d, void *stream);
/* A dispatch planned once and launched many times: validation, launch geometry and the TMA tensor maps
 * (encoded from the dispatch's pointers and shape) are worked out by dnxcu_plan_create, so that
 * dnxcu_plan_launch only enqueues.  The plan is tied to the pointers, shape and flags it was made from; the
 * caller owns it and keeps one per stream that may launch concurrently.  Stands in for the pipeline +
 * descriptor set objects Instance::make builds once per dispatch (runtime/src/denox/runtime/instance.cpp:25-286). */
typedef struct dnxcu_plan dnxcu_plan;
DNXCU_API int dnxcu_plan_create(const dnxcu_dispatch *d, dnxcu_plan **out);
DNXCU_API int dnxcu_plan_launch(const dnxcu_plan *p, void *stream);
DNXCU_API void dnxcu_plan_destroy(dnxcu_plan *p);
/* Limit of every bounded wait inside the kernels, in microseconds at the device's nominal SM clock
 * (process wide, read when a launch is planned); 0 restores the default of about 1.5 s.  A wait that runs
 * out makes the kernel store its code to dispatch.device_status and return. */
DNXCU_API int dnxcu_set_wait_limit_us(uint32_t microseconds);
/* Grid the launch would use (wgX, wgY, wgZ of the reference's dispatch record). */
DNXCU_API int dnxcu_grid(const dnxcu_dispatch *d, uint32_t grid[3]);
/* Algorithmic cost of the dispatch, the reference's per dispatch metadata
 * (DirectConvShaderCM.cpp:632-644): bytes read, bytes written, flops. */
DNXCU_API int dnxcu_cost(const dnxcu_dispatch *d, uint64_t *bytes_read, uint64_t *bytes_written,
                         uint64_t *flops);

/* ------------------------------------------------------------------------
 * Parameter re-layout (host side).
 * Stands in for the lazy FilterTensor conversion a conv variant registers with
 * OpImpl::createParameter (DirectConvShaderCM.cpp:595-619,
 * ConcatConvCMShader.cpp:832-873; index formulas
 * common/src/denox/memory/tensor/FilterLayout.hpp:36-118).
 * Input: KCRS (= ONNX OIHW) binary16, C = c_a + c_b, R = S = 3.
 * Call with out == NULL to get the blob size in *bytes.
 * ---------------------------------------------------------------------- */
DNXCU_API int dnxcu_prepare_weights(int variant, const void *kcrs_f16, int c_out, int c_a, int c_b,
                                    void *out, size_t *bytes);

/* ------------------------------------------------------------------------
 * conv3x3 (+bias, +ReLU) then 2x2 max pool WITHOUT any device allocation.
 * No counterpart in the reference: its runtime allocates every buffer itself
 * (runtime/src/denox/runtime/instance.cpp:25-286).
 *
 * Who needs it: hosts that run this inside a frame loop or a latency critical
 * render thread, where cudaMalloc / cudaFree are off limits because they
 * serialise the whole device and may block for an unbounded time, and hosts
 * whose memory budget is fixed at start-up and audited, so that a library may
 * not grow it later.  dnxcu_instance_create serves everyone else.
 *
 * The full resolution conv result, which the pool consumes, is kept in a fixed
 * array inside the library (DNXCU_STATIC_SCRATCH_BYTES, held by every device
 * that loads the library until the process exits).  The call fails with
 * DNXCU_E_LIMIT when height * width * c_out * 2 exceeds that size.
 *   in       : height x width x c_in binary16 (device)
 *   weights  : blob from dnxcu_prepare_weights for variant 0 ("direct-conv")
 *   bias     : c_out binary16 (device) when flags has DNXCU_F_BIAS, else NULL
 *   flags    : any of DNXCU_F_RELU, DNXCU_F_BIAS
 *   out_pool : (height/2) x (width/2) x c_out binary16 (device); height, width even
 * The first call on each device looks up the array's device address (a
 * synchronous runtime query): make that call before starting a stream capture.
 * Every call overwrites the array and all calls share it: two calls whose
 * kernels can overlap on the GPU (different streams) race; keep them on one
 * stream or order them with events.
 * ---------------------------------------------------------------------- */
#define DNXCU_STATIC_SCRATCH_BYTES (8u << 20)
DNXCU_API int dnxcu_conv3x3_pool_static(const void *in, int height, int width, int c_in, const void *weights,
                                        const void *bias, int c_out, uint32_t flags, void *out_pool, void *stream);

/* float -> binary16 exactly as the reference converts fp32 model weights:
 * mantissa truncated, sub-normal results flushed to zero
 * (common/src/denox/memory/dtype/f16.cpp:6-20). */
DNXCU_API uint16_t dnxcu_f16_from_float(float f);
DNXCU_API float dnxcu_f16_to_float(uint16_t h);

/* ------------------------------------------------------------------------
 * Model / instance runtime.
 * Stands in for runtime::Model::make, Instance::make, Instance::infer and
 * Instance::bench (runtime/src/denox/runtime/model.hpp:107-168,
 * instance.hpp:44-81).  The model is described as the un-fused node list an
 * ONNX import produces (Conv, Relu, MaxPool, Resize-nearest-2x, Concat);
 * dnxcu_model_create runs the fusion patterns and picks a variant per
 * dispatch (from a benchmark database when one is given).
 * ---------------------------------------------------------------------- */
typedef enum dnxcu_node_kind {
  DNXCU_NODE_CONV = 1,
  DNXCU_NODE_RELU = 2,
  DNXCU_NODE_MAXPOOL = 3,
  DNXCU_NODE_UPSAMPLE = 4,
  DNXCU_NODE_CONCAT = 5,
  DNXCU_NODE_LEAKY_RELU = 6 /* slope in dnxcu_node.alpha (onnx LeakyRelu,
                               frontend/onnx/details/ops/leaky_relu.cpp:9-44) */
} dnxcu_node_kind;

typedef struct dnxcu_node {
  int32_t kind;     /* dnxcu_node_kind */
  int32_t in0;      /* tensor id */
  int32_t in1;      /* tensor id (concat) or -1 */
  int32_t out;      /* tensor id */
  int32_t c_out;    /* conv: output channels */
  float alpha;      /* leaky relu: slope */
  const void *weights_kcrs; /* conv: host binary16 [c_out][c_in][3][3] */
  const void *bias;         /* conv: host binary16 [c_out] or NULL */
} dnxcu_node;

typedef struct dnxcu_model_desc {
  int32_t n_nodes;
  int32_t n_tensors;
  const dnxcu_node *nodes; /* topological order */
  int32_t input_tensor;
  int32_t input_channels;
  int32_t output_tensor;
  uint32_t options; /* DNXCU_OPT_* */
} dnxcu_model_desc;

#define DNXCU_OPT_NO_FUSE_ACTIVATION 0x1u /* reference --ffusion off (Options.hpp:16) */
#define DNXCU_OPT_NO_FUSE_POOL 0x2u
#define DNXCU_OPT_NO_FUSE_UPSAMPLE 0x4u
#define DNXCU_OPT_NO_FUSE_CONCAT 0x8u
#define DNXCU_OPT_NO_TCGEN05 0x10u /* reference --fcoopmat off */
#define DNXCU_OPT_NO_PAD_INPUT 0x20u /* do not copy a ragged input into a zero padded tensor first */
#define DNXCU_OPT_SELECT_BY_COST_ONLY 0x40u /* schedule selection with a database: skip the reference's pre-filter
                                               that keeps only the topologies with the fewest dispatches
                                               (dce/prune_topological.cpp:86-152), so that an un-fused schedule
                                               can win when the database says it is faster */

typedef struct dnxcu_model dnxcu_model;
typedef struct dnxcu_instance dnxcu_instance;
typedef struct dnxcu_db dnxcu_db;

/* db may be NULL: every fusion pattern that applies is taken and variants are picked by a fixed preference
 * order.  With a database, dnxcu_instance_create builds the graph of all candidate dispatches (fused and
 * un-fused, every variant) for its extent, weighs them with the database's latencies (1 hour for a candidate
 * never timed, selection.cpp:21) and runs the minimum cost sub-graph search of the reference
 * (common/src/denox/algorithm/minimum_const_subgraph.hpp:45-353).
 * device < 0: no device is touched and every capability is assumed (a model that is only written to a dnx
 * file); instances of such a model run on device 0. */
DNXCU_API int dnxcu_model_create(const dnxcu_model_desc *desc, const dnxcu_db *db, int device,
                                 dnxcu_model **out);
DNXCU_API void dnxcu_model_destroy(dnxcu_model *m);
/* Tensor ids of the model's input and output and the input's channel count (any pointer may be NULL). */
DNXCU_API int dnxcu_model_io(const dnxcu_model *m, int *input_tensor, int *input_channels, int *output_tensor);
/* Dispatches of the default schedule (what an instance runs when the model has no database). */
DNXCU_API int dnxcu_model_dispatch_count(const dnxcu_model *m);
/* Dispatches of this instance's schedule (may differ from the model's default when a database chose it). */
DNXCU_API int dnxcu_instance_dispatch_count(const dnxcu_instance *inst);
/* The schedule search on a caller-built hypergraph: node ids 0 .. n_nodes-1; edge e reads the nodes
 * srcs[src_off[e] .. src_off[e+1]) and writes dsts[dst_off[e] .. dst_off[e+1]) at cost weight[e].  Writes the
 * chosen edges in an order in which they can fire to chosen[0 .. *n_chosen) (room for n_edges) and their total
 * cost to *cost; DNXCU_E_UNSUPPORTED when the outputs cannot be derived from the inputs.  Stands in for
 * algorithm::minimum_cost_subgraph (common/src/denox/algorithm/minimum_const_subgraph.hpp:45-353); with
 * min_dispatches != 0 the edges are first reduced to those of sub-graphs with the fewest edges
 * (prune_topological.cpp:86-152). */
DNXCU_API int dnxcu_select_min_cost(int n_nodes, int n_edges, const int32_t *src_off, const int32_t *srcs,
                                    const int32_t *dst_off, const int32_t *dsts, const double *weight,
                                    const int32_t *inputs, int n_inputs, const int32_t *outputs, int n_outputs,
                                    int min_dispatches, int32_t *chosen, int32_t *n_chosen, double *cost);

/* A model from the bytes of an ONNX file.  Accepts what the reference's importer accepts of the operators this
 * backend runs (compiler/src/denox/compiler/frontend/onnx/onnx.cpp:32-160, details/ops/{conv,max_pool,resize,
 * concat,relu,leaky_relu}.cpp): Conv 3x3 with stride 1, dilation 1, group 1 and extent preserving padding
 * (OIHW weights, float or float16 constants), Relu, LeakyRelu, MaxPool 2x2 / stride 2 without auto_pad,
 * ceil_mode or indices, Resize / Upsample nearest x2 with asymmetric coordinates and constant scales, Concat of
 * two runtime tensors on the channel axis; one runtime input (NCHW, constant channel count) and one output.
 * Anything else: DNXCU_E_UNSUPPORTED, with the reason in dnxcu_last_error_message().  fp32 weights become
 * binary16 by the reference's truncating conversion.  db / device / options as for dnxcu_model_create. */
DNXCU_API int dnxcu_model_create_from_onnx(const void *bytes, size_t n, const dnxcu_db *db, int device,
                                           uint32_t options, dnxcu_model **out);
/* Text that explains the most recent import failure on this thread (empty if none). */
DNXCU_API const char *dnxcu_last_error_message(void);

/* dnx files (dnx.fbs:1-195 of the reference: tensors with symbolic extents, buffers, parameter initializers,
 * dispatches with bindings and push constants, the symbolic expression list over H and W).
 *   dnxcu_model_write_dnx    : the model's default schedule with the preferred variant per dispatch: a
 *                              compiled model that does not depend on an extent (no device needed);
 *   dnxcu_instance_write_dnx : the instance's own schedule and variants (what a benchmark database chose);
 *   dnxcu_model_create_from_dnx : a model that runs exactly the file's dispatches; instances of it take any
 *                              extent the file's alignment allows.  device < 0: parse only.
 * Call the writers with out == NULL to get the size in *bytes.  Stands in for the reference's serialize step
 * (compiler/src/denox/compiler/serialize/serialize.cpp:1-635) and runtime::Model::make
 * (runtime/src/denox/runtime/model.hpp:109-118).  The `shader_binaries` of these files hold a descriptor of the
 * CUDA kernel variant (first word "DNXC") where the reference holds SPIR-V; a file with SPIR-V binaries is
 * refused with DNXCU_E_UNSUPPORTED. */
DNXCU_API int dnxcu_model_write_dnx(const dnxcu_model *m, void *out, size_t *bytes);
DNXCU_API int dnxcu_instance_write_dnx(const dnxcu_instance *inst, void *out, size_t *bytes);
DNXCU_API int dnxcu_model_create_from_dnx(const void *bytes, size_t n, int device, dnxcu_model **out);

/* Row band of a taller image: band rows [row0, row0+rows) of image height
 * image_h; (0, h, h) = whole image.  All three must be multiples of 16 when
 * the band is a strict part of the image. */
typedef struct dnxcu_band {
  int32_t image_h, row0, rows;
} dnxcu_band;

DNXCU_API int dnxcu_instance_create(const dnxcu_model *m, int height, int width,
                                    const dnxcu_band *band, dnxcu_instance **out);
DNXCU_API void dnxcu_instance_destroy(dnxcu_instance *inst);

/* Host in, host out, synchronous — the contract of Instance::infer
 * (instance.hpp:59; instance.cpp:322-430): input is H x W x C_in binary16,
 * output H x W x C_out binary16, tightly packed. */
DNXCU_API int dnxcu_instance_infer(dnxcu_instance *inst, const void *host_in, void *host_out);
/* Stream ordered form of the same call (no counterpart in the reference, whose infer waits for the queue to
 * idle): enqueues the host->device copy, the schedule and the device->host copy on the instance's own stream
 * and returns; dnxcu_instance_wait blocks until they are done and reports kernel time-outs.  Several instances
 * used round robin overlap the copies of one frame with the kernels of another.  host_in / host_out must stay
 * valid until the wait returns; pinned memory is needed for the copies to overlap. */
DNXCU_API int dnxcu_instance_infer_async(dnxcu_instance *inst, const void *host_in, void *host_out);
DNXCU_API int dnxcu_instance_wait(dnxcu_instance *inst);
/* Device resident form: input/output are device pointers, work is enqueued on
 * `stream`, nothing is synchronised and nothing else runs on the device.  The
 * schedule is replayed from a CUDA graph; the first call with a new (dev_in,
 * dev_out) pair captures one (host work only, no device work outside `stream`)
 * and the instance keeps the graphs of the most recently used pairs (dnxcu_instance_graph_cache). */
DNXCU_API int dnxcu_instance_enqueue(dnxcu_instance *inst, const void *dev_in, void *dev_out,
                                     void *stream);
/* Number of (dev_in, dev_out) pairs whose graph dnxcu_instance_enqueue keeps (default 4, 1 .. 256): a caller
 * that feeds frames from a ring of n buffers sets it to n, so that no frame re-captures. */
DNXCU_API int dnxcu_instance_graph_cache(dnxcu_instance *inst, int pairs);
/* Device pointer and shape of any tensor of the instance after a run (for per
 * layer parity checks): returns the device pointer in *ptr. */
DNXCU_API int dnxcu_instance_tensor(const dnxcu_instance *inst, int tensor_id, void **ptr,
                                    int *h, int *w, int *c);

typedef struct dnxcu_dispatch_info {
  char name[48];   /* reference style dispatch name, e.g. "direct-conv-tc+relu+pool" */
  int32_t variant;
  int32_t src_node; /* first node of the model this dispatch covers */
  uint32_t grid[3];
  uint32_t flags;
  uint64_t bytes_read, bytes_written, flops;
  float ms; /* filled by dnxcu_instance_bench */
  int32_t h, w, c_a, c_b, c_out;
  int32_t out_tensor;
} dnxcu_dispatch_info;

DNXCU_API int dnxcu_instance_dispatch_info(const dnxcu_instance *inst, int i,
                                           dnxcu_dispatch_info *info);
/* `warmup` untimed passes, then `iters` passes with a CUDA event pair around
 * every dispatch; info[i].ms = mean per dispatch.  Stands in for
 * Instance::bench (instance.cpp:432-654: 100 warm-up passes, one timed pass). */
DNXCU_API int dnxcu_instance_bench(dnxcu_instance *inst, int warmup, int iters,
                                   dnxcu_dispatch_info *info, int n_info, float *total_ms);

/* Halo rows of a row band instance.  For every conv dispatch the instance
 * keeps, per operand, one row above and one row below the band.  These calls
 * expose them so that a caller (NCCL, peer copies, or a test on one device)
 * can move rows between neighbouring bands between dispatches.
 *   dnxcu_instance_halo_count: number of exchange points (one per conv operand)
 *   dnxcu_instance_halo: for exchange point e: the dispatch index it precedes,
 *     device pointers of this band's own first/last row of that operand
 *     (send_top / send_bottom), the slabs the neighbour rows must land in
 *     (recv_top / recv_bottom) and the row size in bytes. */
typedef struct dnxcu_halo_point {
  int32_t before_dispatch;
  int32_t tensor;
  const void *send_top, *send_bottom;
  void *recv_top, *recv_bottom;
  uint64_t row_bytes;
} dnxcu_halo_point;
DNXCU_API int dnxcu_instance_halo_count(const dnxcu_instance *inst);
DNXCU_API int dnxcu_instance_halo(const dnxcu_instance *inst, int e, dnxcu_halo_point *p);
/* Direct halo exchange over peer memory, for the row bands of one image on the GPUs of one node (or on one
 * device).  Every band instance keeps its halo slabs and arrival flags in one allocation; a neighbour writes
 * its boundary rows straight into them (plain stores through a peer mapping, then a flag), so no copy engine
 * or collective sits between two convs.  No counterpart in the reference, which runs on one device.
 *   dnxcu_instance_halo_export : a handle of this band's slabs that can be sent to another process
 *     (cudaIpcMemHandle inside) or used in this one;
 *   dnxcu_instance_halo_connect: `up` / `down` are the handles of the bands directly above / below (NULL at
 *     the image border).  Fails with DNXCU_E_BAD_ARG when a neighbour has another band height, width or
 *     model, or is not the adjacent band.  With auto_exchange != 0 every dnxcu_instance_enqueue /
 *     dnxcu_instance_enqueue_range runs the exchange in front of each conv by itself: all bands must then
 *     run the same frames in the same order, each on ONE stream, on different GPUs (a band that waits for a
 *     neighbour queued behind it on the same device would wait until its limit);
 *   dnxcu_instance_halo_step   : with auto_exchange == 0 the caller drives the two halves itself: mode 1
 *     pushes this band's rows for the conv `dispatch`, mode 2 waits for the neighbours' rows, 3 does both.
 *     Bands that share a device push for all bands first and wait afterwards.
 * The wait is bounded (dnxcu_set_wait_limit_us); when it runs out the kernel stores code 10 to the
 * instance's status word, which dnxcu_instance_wait / infer / bench report as DNXCU_E_DEVICE. */
typedef struct dnxcu_peer_handle {
  unsigned char ipc[64];
  uint64_t arena_bytes, layout, local_ptr;
  int64_t pid;
  int32_t device, row0, rows, reserved;
} dnxcu_peer_handle;
DNXCU_API int dnxcu_instance_halo_export(const dnxcu_instance *inst, dnxcu_peer_handle *out);
DNXCU_API int dnxcu_instance_halo_connect(dnxcu_instance *inst, const dnxcu_peer_handle *up,
                                          const dnxcu_peer_handle *down, int auto_exchange);
DNXCU_API int dnxcu_instance_halo_step(dnxcu_instance *inst, int dispatch, uint32_t mode, void *stream);
/* After a wait that ran out the bands no longer agree on how many rows they have swapped.  Once every band
 * of the image is idle, each calls this: its push counts and arrival flags return to zero (synchronous). */
DNXCU_API int dnxcu_instance_halo_reset(dnxcu_instance *inst);
/* Switches the automatic exchange of a connected instance on or off (takes effect for schedules enqueued or
 * captured afterwards; graphs captured before keep what they were captured with). */
DNXCU_API int dnxcu_instance_halo_auto(dnxcu_instance *inst, int on);
/* Runs dispatches [first, last) on `stream` (row band callers interleave this
 * with their halo exchange). */
DNXCU_API int dnxcu_instance_enqueue_range(dnxcu_instance *inst, int first, int last, void *stream);
/* Copies the band's input into the instance's input tensor / the output out. */
DNXCU_API int dnxcu_instance_io(const dnxcu_instance *inst, void **dev_in, void **dev_out);
/* The extent the caller's frames have (h, w) and the extent the schedule runs at
 * (h_run, w_run).  They differ when the instance was created with an extent that is not
 * a multiple of the network's alignment: the instance then pads the frame by edge
 * replication at the right and the bottom before the first dispatch and slices the
 * output back after the last one, as the reference's exported models do
 * (oidn_model.py:334-347: UNetAlignment; memory_pad.comp, memory_slice.comp). */
DNXCU_API int dnxcu_instance_extent(const dnxcu_instance *inst, int *h, int *w, int *h_run, int *w_run);

/* ------------------------------------------------------------------------
 * Benchmark database.
 * Stands in for denox::Db (database/src/denox/db/Db.hpp:15-76) and the
 * sampling loop of runtime::Db::bench (runtime/src/denox/runtime/db.cpp:665-868).
 * Key = (variant sha-256, push constants {IN_W, IN_H}, channel counts, flags);
 * value = every latency sample with its time stamp and benchmark environment,
 * their mean and standard deviation.
 * The file is a FlatBuffer of the reference's schema (db.fbs:1-139, identifier
 * "dbdb"): BenchEnv records, one ShaderBinary per variant identity (src_sha256 =
 * the identity, spirv = a "DNXC" descriptor instead of SPIR-V), one
 * ComputeDispatch per key with the launch grid as workgroup counts, the key's
 * numbers as push_constant bytes, Timing and ComputeDispatchInfo.  A file of
 * the reference itself (SPIR-V binaries) is refused with DNXCU_E_IO: its
 * timings are those of other kernels.  Entries of identities this build does
 * not know are kept and written back as read.
 * ---------------------------------------------------------------------- */
DNXCU_API int dnxcu_db_open(const char *path, dnxcu_db **out); /* missing file = empty db */
DNXCU_API void dnxcu_db_close(dnxcu_db *db);
DNXCU_API int dnxcu_db_size(const dnxcu_db *db);
/* Adds every (dispatch, variant) candidate of the model at H x W that is not
 * in the database yet; returns the number added (denox::populate,
 * compiler/src/denox/compiler/populate.cpp:23-256).  Candidates are those
 * `device` can run; device < 0 enumerates for a device with every capability
 * without touching one. */
DNXCU_API int dnxcu_db_populate(dnxcu_db *db, const dnxcu_model_desc *desc, int height, int width,
                                int device);
/* The same for a model that exists already (imported from ONNX, say). */
DNXCU_API int dnxcu_db_populate_model(dnxcu_db *db, const dnxcu_model *m, int height, int width, int device);
/* Samples un-converged entries until n >= min_samples and
 * sem / mean <= max_relative_error, coldest first then largest relative error
 * (db.cpp:71-175, 630-649); writes back atomically when done. */
DNXCU_API int dnxcu_db_bench(dnxcu_db *db, int device, int min_samples, double max_relative_error,
                             int max_rounds);
DNXCU_API int dnxcu_db_atomic_writeback(dnxcu_db *db); /* tmp file + rename (Db.cpp:270-506) */
/* Latency in ms of the entry matching the dispatch, or DNXCU_E_BAD_ARG when
 * absent / never sampled (Db::query_dispatch_latency). */
DNXCU_API int dnxcu_db_query(const dnxcu_db *db, const dnxcu_dispatch *d, double *mean_ms,
                             double *std_ms, int *samples);
DNXCU_API int dnxcu_db_add_result(dnxcu_db *db, const dnxcu_dispatch *d, const double *samples_ms,
                                  int n);

#ifdef __cplusplus
}
#endif
#endif /* DNXCU_H */
