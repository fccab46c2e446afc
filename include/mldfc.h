/*
 * mldfc - C ABI of the B200-native quantized FullyConnected path.
 *
 * ML Drift has no FFI of its own: the seam it offers is a C++ class hierarchy
 * (GPUOperation / GpuModelBuilder).  This header is the boundary a binding for
 * that seam calls into; every entry point names the ml-drift interface it
 * stands in for (paths relative to ml_drift/).  All pointers are plain device
 * or host pointers, all sizes plain integers; no C++ or torch types appear.
 *
 * Conventions
 *  - every function returns an mld_status (0 = OK); nothing throws or aborts;
 *  - `stream` is a cudaStream_t passed as void* (NULL = default stream); work
 *    is enqueued on it and the call returns without synchronising unless the
 *    function says otherwise;
 *  - the caller owns every buffer it passes; a plan owns only its workspace;
 *  - device layouts are the reference's BUFFER layouts:
 *      activations BHWC(1,1,M,C)  -> [ceil(C/4)][M][4]      (tensor_desc.cc:1852-1860)
 *      weights kOSpatialIOGroupI4O4 -> [I/4][O/4][4 i][4 o], INT8 bytes hold
 *        q+128, INT4 nibbles hold q+8 with element 2j in the low nibble
 *        (weights_conversion.cc:46-87, 1495-1523)
 *      scales / zero points: per-channel [O4]; block-wise [G][O4]
 *        (tensor_desc.cc:266-311, 2245-2257), in the activation type.
 */
#ifndef MLDFC_H_
#define MLDFC_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define MLD_API __attribute__((visibility("default")))
#else
#define MLD_API
#endif

typedef enum mld_status {
  MLD_OK = 0,
  MLD_INVALID_ARGUMENT = 1, /* absl::InvalidArgumentError in the reference */
  MLD_UNIMPLEMENTED = 2,    /* absl::UnimplementedError */
  MLD_CUDA_ERROR = 3,
  MLD_NCCL_ERROR = 4,
  MLD_TIMEOUT = 5,          /* a bounded device-side wait gave up */
  MLD_OUT_OF_RANGE = 6,     /* size beyond a fixed capacity */
  MLD_NOT_FOUND = 7         /* absl::NotFoundError: a weight file is missing */
} mld_status;

/* common/precision.h:25-36 (CalculationsPrecision). */
typedef enum mld_precision {
  MLD_PRECISION_F32 = 0,    /* fp32 tensors, fp32 math */
  MLD_PRECISION_F16 = 1,    /* fp16 tensors, fp16-level math */
  MLD_PRECISION_F32F16 = 2  /* fp16 tensors, fp32 accumulation */
} mld_precision;

/* fc::IsScalarQuantized / IsLinearQuantized / IsBlockQuantized
 * (common/kernels/fully_connected_util.cc:499-513). */
typedef enum mld_scale_mode {
  MLD_SCALE_SCALAR = 0,
  MLD_SCALE_PER_CHANNEL = 1,
  MLD_SCALE_BLOCK = 2
} mld_scale_mode;

typedef enum mld_act_layout {
  MLD_LAYOUT_SLICED = 0,    /* [ceil(C/4)][M][4], the reference buffer layout */
  MLD_LAYOUT_ROW_MAJOR = 1  /* [M][C] */
} mld_act_layout;

/* Elementwise operation fused into the destination write (the reference links
 * elementwise nodes into the FC's dst write, fully_connected_util.cc:356-407,
 * common/task/gpu_operation.cc:1182-1256). */
typedef enum mld_epilogue {
  MLD_EPILOGUE_NONE = 0,
  /* Weight rows alternate gate_i, up_i (N rows -> N/2 outputs):
   * dst[i] = silu(row 2i) * (row 2i+1), the SiluMul of the FFN
   * (samples/llm/qwen3_model_builder.cc:918-932).  Decode kernel only. */
  MLD_EPILOGUE_SWIGLU_PAIRS = 1
} mld_epilogue;

typedef enum mld_weight_source {
  MLD_SRC_INT8 = 0,         /* OHWI, one signed value per byte */
  MLD_SRC_UINT4_PACKED = 1  /* OHWI (IHWO with swap_dims), two's-complement
                               nibbles, element 2j in the low nibble */
} mld_weight_source;

MLD_API const char* mld_status_string(int status);
/* Text of the last CUDA error seen by this thread ("" if none). */
MLD_API const char* mld_last_error(void);
/* Number of kernels this library has launched in the calling process. */
MLD_API int64_t mld_kernel_launch_count(void);

/* ------------------------------------------------------------------------ */
/* Weight conversion                                                         */
/* ------------------------------------------------------------------------ */

/* WeightsDescription + source shape for the one layout the buffer FC path
 * uses (common/task/weights_layout.h:27-93; GetFullyConnectedInt{8,4}
 * WeightsDesc, common/kernels/fully_connected.cc:1218-1246). */
typedef struct mld_pack_desc {
  int32_t o, h, w, i;        /* OHWI source shape */
  int32_t bits;              /* 8 -> kUint8, 4 -> kUint4 destination */
  int32_t out_group_size;    /* 0 = ceil(o/4) (the FC choice) */
  int32_t source;            /* mld_weight_source */
  int32_t swap_dims;         /* packed source only: source is IHWO */
  uint32_t pad_value;        /* 128 for INT8, 8 for INT4 */
} mld_pack_desc;

/* GetTotalElementsCountForLayout (common/task/weights_conversion.cc:1015-1027)
 * times bits/8: bytes of the packed destination. */
MLD_API size_t mld_packed_size_bytes(const mld_pack_desc* d);

/* GetTensorDescriptorForWeightsLayout(int8) -> RearrangeWeightsInt8AsUint8 /
 * AsUint4 (weights_conversion.cc:1672-1713, 1495-1523) for MLD_SRC_INT8, and
 * RearrangeWeightsUInt4Packed (weights_conversion.cc:1604-1620, 631-708) for
 * MLD_SRC_UINT4_PACKED, run as a CUDA kernel like the reference's own
 * ConverterToConvWeights (common/kernels/conv_weights_converter.cc:1114-1400).
 * src/dst are device pointers.  sum_i (device, may be NULL) receives
 * sum_i[o] = sum of the signed weights of output o; it has sum_len >= o
 * entries, of which the first o are cleared first and padded entries receive
 * the (pad_value - 8) terms exactly as the reference does. */
MLD_API int mld_pack_weights(const mld_pack_desc* d, const void* src,
                             void* dst, int32_t* sum_i, int32_t sum_len,
                             void* stream);

/* GetWeightsAccumulatedInputChannels (weights_conversion.cc:1584-1602) from an
 * int8 OHWI source. */
MLD_API int mld_weights_sum_i(const int8_t* src, int32_t o, int32_t hwi,
                              int32_t* sum_i, void* stream);

/* ScaleOrZeroPointToTensorDesc (common/task/tensor_desc.cc:2245-2257):
 * src [o][g] fp32 -> [g][o4], fp16 (IEEE RNE) when dst_f16, zero padded. */
MLD_API int mld_pack_scales(const float* src, int32_t o, int32_t g,
                            int32_t dst_f16, void* dst, void* stream);

/* quantize_tensor_int8_sym / quantize_tensor_int4_sym
 * (samples/llm/extract_weights_hf.py:137-229): w [o][i] fp32 -> q [o][i] int8
 * and scale [o][g] fp32; bits 8 is per-channel (block ignored), bits 4 uses
 * blocks of `block` input channels (0 = per-channel).  optimize_scale must be
 * 0 (scale = absmax / 127 or / 7); 1 asks for the converter's grid search over
 * seven candidate scales (:78-134), which is not built: MLD_UNIMPLEMENTED. */
MLD_API int mld_quantize_weights(const float* w, int32_t o, int32_t i,
                                 int32_t bits, int32_t block,
                                 int32_t optimize_scale, int8_t* q,
                                 float* scale, void* stream);

/* ------------------------------------------------------------------------ */
/* Weight files                                                              */
/* ------------------------------------------------------------------------ */

/* LlmFileTensorLoader (samples/llm/llm_file_tensor_loader.h:34-84) over the
 * file set that samples/llm/extract_weights_hf.py writes (:355-440): one raw
 * little-endian array per checkpoint tensor, `<key>` (float32, int8 [O][I] or
 * INT4 packed two per byte, low nibble first) and `<key>_quantized_scale`
 * (float32 [O][I/block], or an int32 group size followed by int8 / int16 values
 * in units of 1/1024).  The files are read on the host; the rearrangement into
 * the operator's layouts runs in the kernels of "Weight conversion" above, so
 * the destinations are device pointers.  Every load is synchronous. */
typedef struct mld_loader mld_loader;

/* weights_directory is prepended to every tensor name as it is (end it with
 * its separator), llm_file_tensor_loader.cc:145-148. */
MLD_API int mld_loader_open(const char* weights_directory, mld_loader** out);
MLD_API int mld_loader_close(mld_loader* loader);
/* HasTensor (:499-509): 1 when the file can be opened. */
MLD_API int mld_loader_has_tensor(mld_loader* loader, const char* name);
/* GetTensorElementSizeInBits (:511-522): file size * 8 / count, 0 for a
 * missing file; how the samples tell INT4 from INT8 from float files. */
MLD_API int mld_loader_element_bits(mld_loader* loader, const char* name,
                                    int64_t count);
/* GetQuantizationIGroupSize (:399-452): input channels per scale group,
 * deduced from the size (and, for the header form, the first word) of
 * `<base>.weight_quantized_scale`; i when there is no usable scale file. */
MLD_API int mld_loader_group_size(mld_loader* loader, const char* weights_name,
                                  int32_t o, int32_t i);
/* LoadFloat32 (:150-161): count floats into host memory (a short file leaves
 * zeros at the end); MLD_NOT_FOUND when the file is missing. */
MLD_API int mld_loader_load_float32(mld_loader* loader, const char* name,
                                    int64_t count, float* dst);
/* LoadInt8Weights (:260-302) for bits 8, LoadInt4WeightsFast (:351-397) for
 * bits 4: the file's [o][i] values ([i][o] with swap_dims) packed into
 * kOSpatialIOGroupI4O4 at dst (mld_packed_size_bytes bytes on the device), and
 * weights_sum_i into sum_i (device, sum_len >= o entries, may be NULL). */
MLD_API int mld_loader_load_weights(mld_loader* loader, const char* name,
                                    int32_t bits, int32_t o, int32_t i,
                                    int32_t swap_dims, void* dst,
                                    int32_t* sum_i, int32_t sum_len,
                                    void* stream);
/* LoadScale (:454-467): [o][g] values in either file form -> the operator's
 * [g][o4] layout on the device (mld_pack_scales). */
MLD_API int mld_loader_load_scale(mld_loader* loader, const char* name,
                                  int32_t o, int32_t g, int32_t dst_f16,
                                  void* dst, void* stream);
/* LoadZeroPoint (:469-497): the file holds zero_point * scale; the result is
 * divided by the scale again (0 where the scale is 0), all zero when there is
 * no such file. */
MLD_API int mld_loader_load_zero_point(mld_loader* loader,
                                       const char* zero_point_name,
                                       const char* scale_name, int32_t o,
                                       int32_t g, int32_t dst_f16, void* dst,
                                       void* stream);

/* ------------------------------------------------------------------------ */
/* FullyConnected operator                                                   */
/* ------------------------------------------------------------------------ */

/* What CreateFullyConnectedExternalWeights receives
 * (common/kernels/fully_connected.h:155-161; ExternalWeights,
 * common/task/gpu_operation.h:354-363). */
enum mld_prefill_route {
  MLD_PREFILL_ROUTE_AUTO = 0,
  MLD_PREFILL_ROUTE_INLINE = 1,
  MLD_PREFILL_ROUTE_CONVERT = 2,
  MLD_PREFILL_ROUTE_INLINE_SMEM = 3  /* inside the GEMM, through shared memory
                                        instead of tensor memory (the form the
                                        int8-activation route uses; kept
                                        selectable for comparison) */
};

typedef struct mld_fc_desc {
  int32_t n;                 /* weights.shape.o */
  int32_t k;                 /* weights.shape.i */
  int32_t weight_bits;       /* 4 or 8 (2, the reference's kUint2 weights:
                                MLD_UNIMPLEMENTED) */
  int32_t scale_mode;        /* mld_scale_mode */
  int32_t groups;            /* scale_zp_shape.i (1 unless block-wise) */
  float scalar_scale;        /* ExternalWeights::scalar_scale */
  float scalar_zero_point;   /* ExternalWeights::scalar_zero_point */
  int32_t has_zero_point;
  int32_t has_bias;
  int32_t precision;         /* mld_precision */
  int32_t src_layout;        /* mld_act_layout */
  int32_t dst_layout;        /* mld_act_layout */
  int32_t max_tokens;        /* largest M passed to mld_fc_run */
  int32_t force_path;        /* 0 = IsFullyConnectedRecommended rule,
                                1 = decode GEMV kernel, 2 = prefill GEMM */
  int32_t device;            /* CUDA device ordinal, -1 = current */
  int32_t prefill_act_quant; /* prefill GEMM only: 0 = float activations (the
                                convolution that dequantises inline,
                                gpu_model_builder.cc:1128-1173,
                                conv_generic.cc:1553-1640); 1 / 2 = per-token
                                int8 activations x int8 weights
                                (FullyConnectedInt8QuantizedWithSrcQuantization,
                                gpu_model_builder.cc:1325-1431; per-channel
                                INT8 weights only), 1 with the symmetric and 2
                                with the asymmetric quantisation rule
                                (quantize_and_dequantize.cc:355-441; 2 is the
                                builder's default and needs
                                mld_fc_plan_set_weights_sum) */
  int32_t cache_prepared_weights; /* prefill GEMM only: instead of dequantising
                                inside the GEMM, expand the weights to a K-major
                                fp16 (s8) copy in a pass of its own
                                (WeightsConverter + float conv route,
                                gpu_model_builder.cc:1110-1276) and keep the
                                copy between calls while the weights and scale
                                pointers stay the same (the caller promises not
                                to modify them in between) */
  int32_t epilogue;          /* mld_epilogue */
  int32_t prefill_route;     /* prefill GEMM only, mld_prefill_route: 0 = the
                                builder's conversion-cost rule
                                (gpu_model_builder.cc:1132-1173: convert the
                                weights in a pass of their own when that costs
                                little beside the product, dequantise inside
                                the GEMM otherwise; with the costs measured
                                for these kernels the pass pays above 512
                                tokens, with the reference's constants above
                                200), 1 = always inside the GEMM, 2 = always
                                the separate pass */
  /* Features of the reference operator that this library does not serve: a
   * non-zero value makes mld_fc_plan_create return MLD_UNIMPLEMENTED and name
   * the feature in mld_last_error(). */
  int32_t runtime_channel_bounds; /* ConvRuntimeCheckDesc: src / dst channel
                                counts read from a tensor at run time
                                (common/kernels/fully_connected.cc:410-470) */
  int32_t has_batch_ids;     /* per-token weight selection of the mixture-of-
                                experts builder
                                (common/gpu_model_builder_moe_util.cc:200-270) */
  /* Tuning of the streaming decode kernel; 0 everywhere = the defaults. */
  int32_t exact_operands;    /* 1: dequantise to exact fp16 integers before the MMA.
                                0: 4-bit weights with one token multiply the nibbles
                                by the activations as 16-bit fixed point (one power-
                                of-two scale per 32 inputs) in integer MMAs; the other
                                cases feed the raw nibbles / bytes as fp16 subnormals
                                (same results up to fp32 summation order) */
  int32_t no_overlap;        /* 1: do not let consecutive launches overlap
                                (programmatic dependent launch off) */
  int32_t smem_limit_kb;     /* > 0: shared-memory budget of the stage ring */
  int32_t independent_io;    /* 1: the caller promises that neither src nor dst of a
                                call is written or read by the launch ahead of it on
                                the stream (projections of one input, benchmarks over
                                rotating tensors): consecutive decode launches then
                                overlap completely instead of handing over at the
                                activation load; stream order of completion is kept */
} mld_fc_desc;

typedef struct mld_fc_plan mld_fc_plan;

/* IsFullyConnectedRecommended (common/kernels/fully_connected.cc:981-1011) for
 * a desktop GPU: 1 when `tokens` <= 16 (F16) or <= 8 (F32, F32F16). */
MLD_API int mld_fc_is_gemv_recommended(int32_t precision, int32_t tokens);

/* Builds the operator (FullyConnected constructor,
 * common/kernels/fully_connected.cc:351-409): validates the description,
 * picks kernels and allocates the plan's workspace.  Synchronous. */
MLD_API int mld_fc_plan_create(const mld_fc_desc* d, mld_fc_plan** out);
MLD_API int mld_fc_plan_destroy(mld_fc_plan* plan);
/* Bytes of device workspace the plan holds. */
MLD_API size_t mld_fc_plan_workspace_bytes(const mld_fc_plan* plan);
/* Which kernels served the plan's most recent mld_fc_run (mld_fc_route;
 * MLD_ROUTE_NONE before the first run): what the builder's node names tell a
 * reader of the reference's graph (fc1x1_*, fc_prefill_*). */
enum mld_fc_route {
  MLD_ROUTE_NONE = 0,
  MLD_ROUTE_DECODE_STREAMING = 1,   /* the decode GEMV over TMA-staged weights */
  MLD_ROUTE_DECODE_GENERAL = 2,     /* the general decode kernel */
  MLD_ROUTE_PREFILL_INLINE = 3,     /* GEMM that dequantises inside */
  MLD_ROUTE_PREFILL_CONVERTED = 4,  /* conversion pass, then GEMM */
  MLD_ROUTE_PREFILL_CACHED = 5      /* GEMM on the copy kept from an earlier call */
};
MLD_API int mld_fc_plan_last_route(const mld_fc_plan* plan);
/* Synchronous read of the plan's device-side status: *code = 0, or the code of
 * a bounded device-side wait that gave up during an earlier mld_fc_run (then
 * cleared); the function then returns MLD_TIMEOUT.  The kernels never spin
 * without a limit: a wait that runs out makes its CTA stop and record the code. */
MLD_API int mld_fc_plan_device_status(mld_fc_plan* plan, int32_t* code);

/* The weights_sum input of the fused dequantisation of the int8-activation
 * route (CreateDequantization, quantize_and_dequantize.cc:867-964;
 * GetWeightsAccumulatedInputChannels, weights_conversion.cc:1584-1602):
 * sum_i[o] = sum over the inputs of the signed weights of output o, a device
 * array of at least n entries as mld_pack_weights / mld_weights_sum_i produce
 * it.  Borrowed: it must stay valid while the plan runs. */
MLD_API int mld_fc_plan_set_weights_sum(mld_fc_plan* plan, const int32_t* sum_i);

/* Optional hint for the next mld_fc_run on this plan: once that call's decode
 * kernel has requested all of its own data it also asks for `bytes` of
 * `next_weights` (the packed weights of whichever projection runs after it) to
 * be brought into L2, so the bytes travel while the memory system would be
 * idle.  One-shot; has no effect on results.  No counterpart in the reference. */
MLD_API int mld_fc_plan_prefetch_next(mld_fc_plan* plan, const void* next_weights, size_t bytes);

/* Dispatch of one FullyConnected node (ClOperation::AddToQueue,
 * cl/cl_operation.cc:85-89) with the argument order of
 * fc::AddWeightsArguments (fully_connected_util.cc:423-487):
 * src, weights, scale, [zero_point], [bias] -> dst.  All device pointers in
 * the layouts named at the top of this file; `tokens` = B*H*W of src.
 * Small token counts run the decode dequant-GEMV
 * (GetFullyConnectedKernelCode, fully_connected.cc:623-942); larger ones the
 * prefill dequant-GEMM the reference builds from WeightsConverter + ConvGeneric
 * (common/gpu_model_builder.cc:1110-1276). */
MLD_API int mld_fc_run(mld_fc_plan* plan, const void* src, const void* weights,
                       const void* scale, const void* zero_point,
                       const void* bias, void* dst, int32_t tokens,
                       void* stream);

/* ------------------------------------------------------------------------ */
/* Embedding lookup over the same packed table                               */
/* ------------------------------------------------------------------------ */

/* EmbeddingLookupAttributes (common/operations.h) for a quantised table that
 * is stored as FullyConnected weights, O = vocabulary, I = embedding width
 * (common/kernels/embedding_lookup.cc:200-216 builds it with
 * GetFullyConnectedInt{8,4}WeightsDesc), so that one packed tensor serves the
 * lookup and the lm_head projection. */
typedef struct mld_embed_desc {
  int32_t vocab;             /* original_weights_shape.o */
  int32_t dim;               /* original_weights_shape.i */
  int32_t weight_bits;       /* 4 or 8 */
  int32_t scale_mode;        /* MLD_SCALE_PER_CHANNEL or MLD_SCALE_BLOCK */
  int32_t groups;            /* scale groups along dim (block-wise only) */
  int32_t has_zero_point;
  int32_t f16;               /* 1: scales, zero points and dst are fp16; 0: fp32 */
  int32_t dst_layout;        /* mld_act_layout: [dim/4][tokens][4] or [tokens][dim] */
} mld_embed_desc;

/* The generated kernel of EmbeddingLookup (embedding_lookup.cc:44-196): for
 * every token, column ids[token] % 4 of the 4x4 blocks of output slice
 * ids[token] / 4, dequantised in fp32 as u * scale - scale * (shift +
 * zero_point) and converted to the dst type.  Ids are clamped to [0, vocab - 1]
 * as in the reference.  ids: int32 device array [tokens]; weights / scale /
 * zero_point: as for mld_fc_run with n = vocab, k = dim. */
MLD_API int mld_embedding_lookup(const mld_embed_desc* d, const int32_t* ids, const void* weights, const void* scale,
                                 const void* zero_point, void* dst, int32_t tokens, void* stream);

/* ------------------------------------------------------------------------ */
/* A FullyConnected node split over the GPUs of one node                      */
/* ------------------------------------------------------------------------ */

/* The reference is single-device; nothing below has a counterpart in it.
 * Output channels are independent dot products (FullyConnectedReference,
 * common/task/testing_ref_ops.cc:961-988), so rank r of `world` computes the
 * rows [r n, (r+1) n) of a node with world * n outputs from its own packed
 * sub-matrix (a plan with n outputs), and the gathered result is the
 * concatenation of the ranks' blocks.  A shard group owns that gathered tensor
 * on every rank: fp16 in the sliced layout [world * n / 4][tokens][4], where a
 * rank's block is one contiguous range. */
typedef struct mld_shard_group mld_shard_group;

typedef enum mld_gather {
  MLD_GATHER_NCCL = 0,        /* compute into the own range, then one in-place
                                 ncclAllGather (the group needs an NCCL id) */
  MLD_GATHER_PEER_STORES = 1  /* the producing kernel stores its block into every
                                 rank's tensor over NVLink while it computes (the
                                 prefill GEMM does so tile by tile; other kernels
                                 are followed by a copy), then the ranks exchange
                                 completion flags (bounded waits; see
                                 mld_shard_group_device_status).  Needs
                                 mld_shard_group_ipc_export / _import. */
} mld_gather;

/* output_bytes: capacity of the gathered tensor (a multiple of 16).
 * nccl_id128: the 128-byte id from mld_comm_unique_id, distributed by the
 * caller, or NULL when only peer stores will be used.  Collective when an id
 * is given.  Synchronous. */
MLD_API int mld_shard_group_create(int32_t rank, int32_t world, int32_t device, size_t output_bytes,
                                   const void* nccl_id128, mld_shard_group** out);
MLD_API int mld_shard_group_destroy(mld_shard_group* group);
/* Every rank exports a 64-byte handle of its tensor, the caller distributes
 * them (rank order, world x 64 bytes) and every rank imports the table; all
 * ranks must have imported before any of them runs with peer stores. */
MLD_API int mld_shard_group_ipc_export(mld_shard_group* group, void* handle64);
MLD_API int mld_shard_group_ipc_import(mld_shard_group* group, const void* handles);
/* Device pointer of this rank's copy of the gathered tensor. */
MLD_API void* mld_shard_group_output(mld_shard_group* group);
/* mld_fc_run for one rank's shard, followed by the gather: after the work this
 * call enqueues on `stream` has completed, the group's tensor on this rank
 * holds all ranks' blocks.  Every rank calls it with the same `tokens` and
 * `gather`.  With peer stores a run begins with a handshake, so a rank's
 * tensor is not overwritten before that rank's own stream has reached the run. */
MLD_API int mld_fc_run_sharded(mld_fc_plan* plan, mld_shard_group* group, const void* src, const void* weights,
                               const void* scale, const void* zero_point, const void* bias, int32_t tokens,
                               int32_t gather, void* stream);
/* Synchronous: *code = 0, or non-zero when a wait for another rank's flag ran
 * out during an earlier peer-store run (then cleared); returns MLD_TIMEOUT then. */
MLD_API int mld_shard_group_device_status(mld_shard_group* group, int32_t* code);

/* ------------------------------------------------------------------------ */
/* Decode step: the callers of the FullyConnected path                       */
/* ------------------------------------------------------------------------ */

/* Geometry of a Llama-style decoder whose projections are INT4 block-quantized
 * FullyConnected nodes - what samples/llm/qwen3_model_builder.cc:947-1038
 * (SelfAttention, FFLayer, TransformerLayer) builds per layer, for one token.
 * rank/world select the column shard this process holds (world == 1: all). */
typedef struct mld_decoder_desc {
  int32_t layers, d_model, heads, head_dim, ffn, max_seq;
  int32_t block;                 /* INT4 scale block along K (32) */
  float rms_eps;                 /* 1e-6 in the reference builder */
  float rope_min_timescale;      /* 1 */
  float rope_max_timescale;      /* 1e6 */
  int32_t rank, world;
  int32_t device;                /* -1 = current */
  /* How a sharded decoder's matrices are split (world > 1):
   * 0 = by output rows, all four projections (shard outputs are all-gathered);
   * 1 = q/k/v and gate/up by output rows, o and down by INPUT columns (wo:
   *     N = d_model, K = d_model/world, the columns of this rank's heads;
   *     wdown: N = d_model, K = ffn/world, the columns of this rank's FFN
   *     units); their outputs are partial sums that every rank adds up, which
   *     halves the exchanges per layer.  Supported by the single-kernel
   *     decoder only. */
  int32_t shard_layout;
  int32_t mode;                  /* mld_decoder_mode */
  /* Single-kernel decoder, 0 everywhere = the defaults: */
  int32_t handover;              /* how a vector passes from one op to the next:
                                    0 = every value travels with the number of the
                                    op that wrote it and readers poll the words they
                                    need (no barrier; sharded: the writer stores the
                                    words into every rank's copy over NVLink);
                                    1 = grid barriers between ops */
  int32_t grid_limit;            /* > 0: use at most this many CTAs */
  int32_t ring_stages;           /* > 0: use at most this many ring stages */
  int32_t wait_limit_us;         /* > 0: bound, in microseconds, on every device-side
                                    wait of a step (default 2 000 000) */
} mld_decoder_desc;

typedef enum mld_decoder_mode {
  MLD_DECODER_AUTO = 0,          /* one GPU: single kernel when the shape allows it;
                                    sharded: op chain */
  MLD_DECODER_OP_CHAIN = 1,      /* a chain of mld_fc_run / attention kernels */
  MLD_DECODER_SINGLE_KERNEL = 2  /* the whole step as one persistent kernel; sharded
                                    ranks exchange shards with peer stores
                                    (mld_decoder_ipc_export / _import, no NCCL id) */
} mld_decoder_mode;

/* Device tensors of one layer, in the layouts named at the top of this file.
 * Shard-local: wqkv packs the rows [q heads | k heads | v heads] of this rank
 * (N = 3*d_model/world, K = d_model); wo N = d_model/world, K = d_model;
 * wgu packs this rank's FFN rows interleaved gate_i, up_i, gate_i+1, ...
 * (N = 2*ffn/world, K = d_model) for the fused SiLU*mul write;
 * wdown N = d_model/world, K = ffn.  s* are the fp16 block scales [K/block][N].
 * norm1/norm2: fp16 RMSNorm weights [d_model].  kcache/vcache: fp16
 * [max_seq][heads/world * head_dim], updated in place at `pos`. */
typedef struct mld_layer_weights {
  const void *wqkv, *sqkv, *wo, *so, *wgu, *sgu, *wdown, *sdown;
  const void *norm1, *norm2;
  void *kcache, *vcache;
} mld_layer_weights;

/* Decode attention of one query token over an fp16 KV cache: what the
 * reference assembles from FullyConnected(q, K-cache) -> mask -> SoftmaxReduce
 * -> FullyConnected(p, V-cache) (samples/llm/qwen3_model_builder.cc:983-1017),
 * as one split-KV pass.  q: fp16 [heads][128], already scaled and rotated;
 * kcache/vcache: fp16 [n_tokens][heads*128]; out: fp16 [heads][128].  Partial
 * results live in a per-device scratch buffer the library allocates on first
 * use and grows when a larger shape arrives (calls on one device must not
 * overlap on different streams). */
MLD_API int mld_attn_decode(const void* q, const void* kcache, const void* vcache, void* out, int32_t heads,
                            int32_t head_dim, int32_t n_tokens, void* stream);

/* The same attention for callers that must not trigger a device allocation:
 * a host that has handed the whole GPU to its own memory pool, or one that
 * froze its memory plan before the first dispatch, cannot afford a cudaMalloc
 * hidden inside a library call (it may fail, and it stalls the device).  This
 * entry point has no counterpart in the reference.  It allocates nothing: the
 * partial results go to a 2.03 MB array that is part of the library image on
 * every GPU, sized for heads x splits <= 4096 - the split count shrinks to fit,
 * and more than 4096 heads are refused with MLD_OUT_OF_RANGE.  The first call
 * on a device looks up the array's device address (make that call with the
 * device current and before starting any stream capture).  All calls share the
 * one array: two calls that overlap on the GPU, on any streams, corrupt each
 * other; calls ordered on one stream are safe, and no call depends on what an
 * earlier one left behind. */
MLD_API int mld_attn_decode_static(const void* q, const void* kcache, const void* vcache, void* out,
                                   int32_t heads, int32_t head_dim, int32_t n_tokens, void* stream);

typedef struct mld_decoder mld_decoder;

/* 128-byte id shared by all ranks of a sharded decoder (rank 0 creates it and
 * the caller distributes it).  No counterpart in the reference, which is
 * single-device. */
MLD_API int mld_comm_unique_id(void* id128);
/* nccl_id128 may be NULL when world == 1, or when the ranks will exchange
 * shards directly (mld_decoder_ipc_export / _import below).  Collective when
 * an id is given. */
MLD_API int mld_decoder_create(const mld_decoder_desc* d, const void* nccl_id128, mld_decoder** out);
MLD_API int mld_decoder_destroy(mld_decoder* dec);
/* 1 when this decoder runs a step as ONE persistent kernel (single GPU, INT4
 * block scales, head_dim 128): a producer thread per SM streams every weight
 * and KV-cache tile of the step through a shared-memory ring while the other
 * warps compute.  0: the step is a chain of mld_fc_run / attention kernels.
 * mld_decoder_desc.mode chooses. */
MLD_API int mld_decoder_is_single_kernel(const mld_decoder* dec);
/* Synchronous read of the device-side status of the steps run so far: *code =
 * 0, or the code of the bounded wait that gave up (then cleared, with the
 * decoder's hand-over state made consistent so that it can be used again; the
 * ranks of a sharded decoder must all call this before any of them steps
 * again); the function then returns MLD_TIMEOUT. */
MLD_API int mld_decoder_device_status(mld_decoder* dec, int32_t* code);
/* Puts the decoder's hand-over state (launch counters, step counters, the tagged
 * words and completion flags of the vectors that pass between ops and ranks)
 * back to what it was after creation; weights and KV caches are untouched.
 * mld_decoder_device_status does this by itself on the rank that saw a failure.
 * The ranks of a sharded decoder number their steps alike, so after a failure on
 * any rank ALL ranks call this, with no step in flight anywhere, and none steps
 * again before all have returned (the caller synchronises them).  Synchronous.
 * No counterpart in the reference. */
MLD_API int mld_decoder_reset(mld_decoder* dec);
/* Changes the bound on device-side waits (see mld_decoder_desc.wait_limit_us)
 * for the steps enqueued after this call. */
MLD_API int mld_decoder_set_wait_limit(mld_decoder* dec, int32_t wait_limit_us);
/* Direct shard exchange between the ranks of one node, without a collective
 * library: every kernel that produces a shard stores it straight into each
 * rank's copy of the gathered vector (peer stores over NVLink) and raises a
 * completion flag there; the consuming kernel waits for all flags (bounded).
 * Each rank exports a 64-byte handle of its exchange block, the caller
 * distributes them (rank order, world x 64 bytes) and every rank imports the
 * table; all ranks must have imported before any of them steps.  Without this
 * the sharded decoder all-gathers through NCCL.  No counterpart in the
 * reference. */
MLD_API int mld_decoder_ipc_export(mld_decoder* dec, void* handle64);
MLD_API int mld_decoder_ipc_import(mld_decoder* dec, const void* handles);
MLD_API size_t mld_decoder_scratch_bytes(const mld_decoder* dec);
MLD_API int mld_decoder_set_layer(mld_decoder* dec, int32_t layer, const mld_layer_weights* w);
/* One token through all layers (OpenCLLlmModelRunner::Decode,
 * samples/llm/llm_opencl.cc:503-596, minus embedding lookup and sampling):
 * x_in, x_out fp16 [d_model] device vectors; pos = index of the new token in
 * the KV cache.  Enqueues on `stream` and returns. */
MLD_API int mld_decoder_step(mld_decoder* dec, const void* x_in, void* x_out, int32_t pos, void* stream);
/* The same step with host vectors: copies x_host to the device, runs the step,
 * copies the result back and synchronises `stream` (the shape of the
 * reference runner's per-token host round trip, llm_opencl.cc:503-596).
 * Returns MLD_TIMEOUT when a device-side wait of the step gave up (the result
 * is then not valid; call mld_decoder_device_status before stepping again). */
MLD_API int mld_decoder_step_host(mld_decoder* dec, const void* x_host, void* y_host, int32_t pos, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MLDFC_H_ */
