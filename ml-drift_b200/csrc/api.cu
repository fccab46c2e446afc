// C ABI of libmldfc: argument checking, plan objects and dispatch.  There is
// no CPU fallback anywhere in this file: a call either enqueues CUDA work or
// returns an error status.
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace mld {

namespace {
thread_local std::string g_last_error;
std::atomic<int64_t> g_launches{0};
}  // namespace

void set_last_error(const char* what, cudaError_t err) {
  g_last_error = std::string(what) + ": " + cudaGetErrorString(err);
}
void set_last_error_text(const char* what) { g_last_error = what; }
void count_launch(int n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count(int device) {
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
  return n;
}

encode_tiled_fn get_encode_tiled() {
  static encode_tiled_fn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<encode_tiled_fn>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t pitch_bytes,
                 uint32_t box_bytes, uint32_t box_rows, int elem_bytes, CUtensorMapSwizzle swizzle,
                 CUtensorMapDataType dtype_override, bool use_override) {
  encode_tiled_fn enc = get_encode_tiled();
  if (enc == nullptr) {
    set_last_error_text("cuTensorMapEncodeTiled is not available from this driver");
    return MLD_CUDA_ERROR;
  }
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  if (use_override)
    dt = dtype_override;
  else if (elem_bytes == 2)
    dt = CU_TENSOR_MAP_DATA_TYPE_UINT16;
  else if (elem_bytes == 4)
    dt = CU_TENSOR_MAP_DATA_TYPE_UINT32;
  const cuuint64_t dims[2] = {row_bytes / elem_bytes, rows};
  const cuuint64_t strides[1] = {pitch_bytes};
  const cuuint32_t box[2] = {box_bytes / elem_bytes, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    char buf[160];
    snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed (%d): row_bytes=%llu rows=%llu pitch=%llu box=%ux%u",
             static_cast<int>(r), (unsigned long long)row_bytes, (unsigned long long)rows,
             (unsigned long long)pitch_bytes, box_bytes, box_rows);
    set_last_error_text(buf);
    return MLD_CUDA_ERROR;
  }
  return MLD_OK;
}

}  // namespace mld

using namespace mld;

static int gm_stage_rows() { return strip_geometry(4, 64, 64, 1, 8, MLD_SCALE_BLOCK, 1, false).stage_rows; }

// ------------------------------------------------------------------ plan type
struct TmapEntry {
  const void* w;
  const void* s;
  int geom;
  CUtensorMap tw, ts;
};

struct mld_fc_plan {
  mld_fc_desc d;
  int device;
  int sms;
  bool stream_ok;        // the streaming GEMV can serve this operator
  bool subnormal;        // operand encoding of the streaming GEMV
  bool pdl;              // launch GEMVs with programmatic stream serialization
  int group_slices;
  StripGeometry gm;
  int* error;            // device error word written by kernels whose bounded waits ran out
  int* error_shared;     // when set (a decoder's word), the kernels report there instead
  size_t ws_bytes;
  // prefill GEMM workspace (allocated with the plan)
  void* w_kmajor;        // dequantised fp16 / re-biased s8 weights, [N4][kp]
  void* x_kmajor;        // activations, [max_tokens][kp]
  PairSplit split;       // where SM pairs that share a tile of the prefill GEMM combine their partial sums
  int last_route;        // mld_fc_route of the most recent run
  float* a_params;       // per-token {inv_scale, offset, sum}
  const void* prepared_w;
  const void* prepared_s;
  const int32_t* w_sum;  // per-output sums of the signed weights (asymmetric int8 activations), caller-owned
  bool pair_ok;          // the prefill GEMM can read the packed weights directly (tensor-map pitch rule)
  const void* next_w;    // one-shot L2 prefetch hint for the next mld_fc_run on this plan
  size_t next_w_bytes;
  std::vector<TmapEntry> tmaps;  // tensor maps keyed by the (weights, scale) pointers last seen
  std::mutex mu;
};

// Tuning aid, compiled only with -DMLD_TRACE: when set (mld_debug_set_trace), the streaming GEMV records
// per-CTA timestamps.
static unsigned long long* g_trace_buffer = nullptr;

void mld::fc_plan_share_error(mld_fc_plan* plan, int* word) {
  if (plan != nullptr) plan->error_shared = word;
}

extern "C" {

#ifdef MLD_TRACE
__attribute__((visibility("default"))) void mld_debug_set_trace(void* dev_buffer) {
  g_trace_buffer = static_cast<unsigned long long*>(dev_buffer);
}
#endif

const char* mld_status_string(int status) {
  switch (status) {
    case MLD_OK: return "OK";
    case MLD_INVALID_ARGUMENT: return "INVALID_ARGUMENT";
    case MLD_UNIMPLEMENTED: return "UNIMPLEMENTED";
    case MLD_NOT_FOUND: return "NOT_FOUND";
    case MLD_CUDA_ERROR: return "CUDA_ERROR";
    case MLD_NCCL_ERROR: return "NCCL_ERROR";
    case MLD_TIMEOUT: return "TIMEOUT";
    case MLD_OUT_OF_RANGE: return "OUT_OF_RANGE";
  }
  return "UNKNOWN";
}

const char* mld_last_error(void) { return g_last_error.c_str(); }
int64_t mld_kernel_launch_count(void) { return g_launches.load(); }

// ----------------------------------------------------------- weight conversion
static int check_pack_desc(const mld_pack_desc* d) {
  MLD_REQUIRE(d != nullptr, "null pack descriptor");
  MLD_REQUIRE(d->o >= 0 && d->h >= 1 && d->w >= 1 && d->i >= 0, "bad OHWI shape");
  MLD_REQUIRE(d->bits == 8 || d->bits == 4, "bits must be 4 or 8");
  MLD_REQUIRE(d->out_group_size >= 0, "bad out_group_size");
  MLD_REQUIRE(d->source == MLD_SRC_INT8 || d->source == MLD_SRC_UINT4_PACKED, "bad source kind");
  if (d->source == MLD_SRC_UINT4_PACKED) {
    MLD_REQUIRE(d->bits == 4, "a nibble-packed source converts to kUint4 only");
    MLD_REQUIRE(d->pad_value < 16, "pad_value must fit a nibble");
  } else {
    MLD_REQUIRE(d->swap_dims == 0, "swap_dims applies to the nibble-packed source only");
  }
  return MLD_OK;
}

size_t mld_packed_size_bytes(const mld_pack_desc* d) {
  if (check_pack_desc(d) != MLD_OK) return 0;
  const int ds = div_up(d->o, 4);
  const int group = d->out_group_size > 0 ? d->out_group_size : (ds > 0 ? ds : 1);
  const size_t elems =
      static_cast<size_t>(align_n(d->i, 4)) * static_cast<size_t>(align_n(d->o, 4 * group)) * d->h * d->w;
  return d->bits == 8 ? elems : elems / 2;
}

int mld_pack_weights(const mld_pack_desc* d, const void* src, void* dst, int32_t* sum_i, int32_t sum_len,
                     void* stream) {
  int rc = check_pack_desc(d);
  if (rc != MLD_OK) return rc;
  if (d->o == 0 || d->i == 0) return MLD_OK;
  MLD_REQUIRE(src != nullptr && dst != nullptr, "null buffer");
  MLD_REQUIRE((reinterpret_cast<uintptr_t>(dst) & 15) == 0, "dst must be 16-byte aligned");
  MLD_REQUIRE(sum_i == nullptr || sum_len >= d->o, "sum_i needs at least o entries");
  return pack_weights_impl(d, src, dst, sum_i, sum_len, static_cast<cudaStream_t>(stream));
}

int mld_weights_sum_i(const int8_t* src, int32_t o, int32_t hwi, int32_t* sum_i, void* stream) {
  MLD_REQUIRE(o >= 0 && hwi >= 0, "bad shape");
  MLD_REQUIRE(o == 0 || (src != nullptr && sum_i != nullptr), "null buffer");
  return weights_sum_i_impl(src, o, hwi, sum_i, static_cast<cudaStream_t>(stream));
}

int mld_pack_scales(const float* src, int32_t o, int32_t g, int32_t dst_f16, void* dst, void* stream) {
  MLD_REQUIRE(o >= 0 && g >= 0, "bad shape");
  MLD_REQUIRE(o * g == 0 || (src != nullptr && dst != nullptr), "null buffer");
  return pack_scales_impl(src, o, g, dst_f16, dst, static_cast<cudaStream_t>(stream));
}

int mld_quantize_weights(const float* w, int32_t o, int32_t i, int32_t bits, int32_t block, int32_t optimize_scale,
                         int8_t* q, float* scale, void* stream) {
  if (optimize_scale != 0) {
    set_last_error_text("optimize_scale (the converter's grid search for the scale of least squared error) is not implemented");
    return MLD_UNIMPLEMENTED;
  }
  MLD_REQUIRE(bits == 8 || bits == 4, "bits must be 4 or 8");
  MLD_REQUIRE(o >= 0 && i >= 0 && block >= 0, "bad shape");
  if (bits == 4 && block > 0) MLD_REQUIRE(i % block == 0, "input channels not divisible by block size");
  MLD_REQUIRE(o * i == 0 || (w != nullptr && q != nullptr && scale != nullptr), "null buffer");
  return quantize_weights_impl(w, o, i, bits, block, q, scale, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------ operator
int mld_fc_is_gemv_recommended(int32_t precision, int32_t tokens) {
  // GetRecommendedMaxTotalSpatialSize: 4, x2 for kF16, x2 for non-Mali, capped at 16
  const int limit = precision == MLD_PRECISION_F16 ? 16 : 8;
  return tokens <= limit ? 1 : 0;
}

// The builder's conversion-cost rule (gpu_model_builder.cc:1132-1173) weighs the bytes a separate conversion
// pass reads and writes against the flops of the product and converts when the ratio is small, which with its
// constants means from 200 tokens up.  The same rule with this library's measured costs (a 14336 x 4096 INT4
// projection: dequantising inside the GEMM wins by 12 us up to 512 tokens, i.e. two token tiles, and loses by
// 12 us from 640 on) puts the threshold at 512.
static bool convert_pays(int tokens) { return tokens > 512; }

int mld_fc_plan_create(const mld_fc_desc* d, mld_fc_plan** out) {
  MLD_REQUIRE(d != nullptr && out != nullptr, "null argument");
  *out = nullptr;
  MLD_REQUIRE(d->n > 0 && d->k > 0, "weights shape must be positive");
  if (d->weight_bits == 2) {
    set_last_error_text("INT2 weights (kUint2) are not implemented");
    return MLD_UNIMPLEMENTED;
  }
  if (d->runtime_channel_bounds != 0) {
    set_last_error_text("runtime channel bounds (ConvRuntimeCheckDesc) are not implemented");
    return MLD_UNIMPLEMENTED;
  }
  if (d->has_batch_ids != 0) {
    set_last_error_text("batch ids (per-token weights of the mixture-of-experts builder) are not implemented");
    return MLD_UNIMPLEMENTED;
  }
  MLD_REQUIRE(d->weight_bits == 4 || d->weight_bits == 8, "Unsupported WeightsDescription type.");
  MLD_REQUIRE(d->precision >= MLD_PRECISION_F32 && d->precision <= MLD_PRECISION_F32F16, "bad precision");
  MLD_REQUIRE(d->scale_mode >= MLD_SCALE_SCALAR && d->scale_mode <= MLD_SCALE_BLOCK, "bad scale mode");
  MLD_REQUIRE(d->src_layout == MLD_LAYOUT_SLICED || d->src_layout == MLD_LAYOUT_ROW_MAJOR, "bad src layout");
  MLD_REQUIRE(d->dst_layout == MLD_LAYOUT_SLICED || d->dst_layout == MLD_LAYOUT_ROW_MAJOR, "bad dst layout");
  MLD_REQUIRE(d->max_tokens >= 1, "max_tokens must be at least 1");
  MLD_REQUIRE(d->prefill_act_quant >= 0 && d->prefill_act_quant <= 2, "bad prefill_act_quant");
  MLD_REQUIRE(d->epilogue == MLD_EPILOGUE_NONE || d->epilogue == MLD_EPILOGUE_SWIGLU_PAIRS, "bad epilogue");
  MLD_REQUIRE((d->exact_operands | 1) == 1 && (d->no_overlap | 1) == 1 && d->smem_limit_kb >= 0, "bad tuning field");
  if (d->epilogue == MLD_EPILOGUE_SWIGLU_PAIRS)
    MLD_REQUIRE(d->n % 8 == 0 && !d->has_bias, "the SiLU*mul write needs an even row count (n % 8 == 0) and no bias");
  if (d->prefill_act_quant != 0)
    MLD_REQUIRE(d->weight_bits == 8 && d->scale_mode == MLD_SCALE_PER_CHANNEL && !d->has_zero_point,
                "int8-activation prefill needs per-channel INT8 weights without zero points");
  const int src_slices = div_up(d->k, 4);
  int group_slices = src_slices;
  if (d->scale_mode == MLD_SCALE_BLOCK) {
    MLD_REQUIRE(d->groups >= 1, "block-wise scales need groups >= 1");
    group_slices = src_slices / d->groups;  // fully_connected.cc:365-370
    MLD_REQUIRE(group_slices >= 1, "more scale groups than input slices");
  }
  int device = d->device;
  if (device < 0) MLD_CUDA_CHECK(cudaGetDevice(&device));

  mld_fc_plan* p = new mld_fc_plan();
  p->d = *d;
  p->device = device;
  p->sms = sm_count(device);
  p->group_slices = group_slices;
  p->error = nullptr;
  p->error_shared = nullptr;
  p->ws_bytes = 0;
  p->w_kmajor = p->x_kmajor = nullptr;
  p->split = PairSplit{nullptr, nullptr, 0};
  p->last_route = MLD_ROUTE_NONE;
  p->a_params = nullptr;
  p->prepared_w = p->prepared_s = nullptr;
  p->w_sum = nullptr;
  // the packed weight matrix as a TMA tensor: rows of N4 / 4 blocks, pitch a multiple of 16 bytes
  p->pair_ok = ((align_n(d->n, 4) / 4) * (d->weight_bits == 4 ? 8 : 16)) % 16 == 0 && get_encode_tiled() != nullptr;
  p->next_w = nullptr;
  p->next_w_bytes = 0;
  p->subnormal = d->exact_operands == 0;
  p->pdl = d->no_overlap == 0;

  const int N4 = align_n(d->n, 4);
  bool ok = d->precision != MLD_PRECISION_F32 && !d->has_zero_point && (N4 % 8 == 0) && (d->k % 8 == 0) &&
            p->sms > 0 && get_encode_tiled() != nullptr;
  if (d->scale_mode == MLD_SCALE_BLOCK) {
    const bool small = group_slices == 8 || group_slices == 16 || group_slices == 32;
    const bool large = group_slices >= gm_stage_rows() && group_slices % gm_stage_rows() == 0;
    ok = ok && (small || large) && (group_slices * d->groups == src_slices);
  }
  p->stream_ok = ok;
  if (ok) {
    const int max_m = d->max_tokens < 16 ? d->max_tokens : 16;
    p->gm = strip_geometry(d->weight_bits, d->n, d->k, max_m, group_slices, d->scale_mode, p->sms, p->pdl,
                           d->smem_limit_kb);
    if (p->gm.stages < 2) p->stream_ok = false;
  }
  {
    cudaError_t e = cudaSetDevice(device);
    if (e == cudaSuccess) e = cudaMalloc(&p->error, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(p->error, 0, sizeof(int));
    if (e != cudaSuccess) {
      set_last_error("plan workspace", e);
      if (p->error) cudaFree(p->error);
      delete p;
      return MLD_CUDA_ERROR;
    }
    p->ws_bytes = sizeof(int);
  }
  // An operator that may run as the prefill GEMM gets its operand workspace now, so that mld_fc_run never
  // allocates: the K-major copy of the weights, the K-major (optionally quantised) activations and the
  // per-token quantisation parameters.
  MLD_REQUIRE(d->prefill_route >= MLD_PREFILL_ROUTE_AUTO && d->prefill_route <= MLD_PREFILL_ROUTE_INLINE_SMEM,
              "prefill_route out of range");
  const bool may_gemm = d->force_path == 2 || (d->force_path == 0 && !mld_fc_is_gemv_recommended(d->precision, d->max_tokens));
  if (may_gemm && d->precision != MLD_PRECISION_F32 && !d->has_zero_point) {
    const bool i8 = d->prefill_act_quant != 0;
    const size_t esz = i8 ? 1 : 2;
    const GemmGeometry gmax = gemm_geometry(d->max_tokens, d->n, d->k, i8, p->sms);
    // the K-major copy of the weights is needed only by the route that prepares them in a pass of its own
    const bool need_w = d->cache_prepared_weights != 0 || !p->pair_ok || d->prefill_route == MLD_PREFILL_ROUTE_CONVERT ||
                        (d->prefill_route == MLD_PREFILL_ROUTE_AUTO && convert_pays(d->max_tokens));
    const size_t wb = need_w ? (size_t)N4 * gmax.kp * esz : 0, xb = (size_t)d->max_tokens * gmax.kp * esz,
                 pb = (size_t)d->max_tokens * kActParamFloats * sizeof(float);
    cudaError_t e = need_w ? cudaMalloc(&p->w_kmajor, wb) : cudaSuccess;
    if (e == cudaSuccess) e = cudaMalloc(&p->x_kmajor, xb);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&p->a_params), pb);
    const size_t sb = pair_split_bytes(p->sms), fb = pair_split_flags(p->sms) * sizeof(uint32_t);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&p->split.ws), sb);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&p->split.flags), fb);
    if (e == cudaSuccess) e = cudaMemset(p->split.flags, 0, fb);
    if (e != cudaSuccess) {
      set_last_error("prefill workspace", e);
      mld_fc_plan_destroy(p);
      return MLD_CUDA_ERROR;
    }
    p->ws_bytes += wb + xb + pb + sb + fb;
  }
  *out = p;
  return MLD_OK;
}

int mld_fc_plan_destroy(mld_fc_plan* plan) {
  if (plan == nullptr) return MLD_OK;
  if (plan->error) cudaFree(plan->error);
  if (plan->w_kmajor) cudaFree(plan->w_kmajor);
  if (plan->x_kmajor) cudaFree(plan->x_kmajor);
  if (plan->split.ws) cudaFree(plan->split.ws);
  if (plan->split.flags) cudaFree(plan->split.flags);
  if (plan->a_params) cudaFree(plan->a_params);
  delete plan;
  return MLD_OK;
}

size_t mld_fc_plan_workspace_bytes(const mld_fc_plan* plan) { return plan ? plan->ws_bytes : 0; }
int mld_fc_plan_last_route(const mld_fc_plan* plan) { return plan ? plan->last_route : MLD_ROUTE_NONE; }

int mld_fc_plan_device_status(mld_fc_plan* plan, int32_t* code) {
  MLD_REQUIRE(plan != nullptr && code != nullptr, "null argument");
  int c = 0;
  int* word = plan->error_shared != nullptr ? plan->error_shared : plan->error;
  MLD_CUDA_CHECK(cudaMemcpy(&c, word, sizeof(int), cudaMemcpyDeviceToHost));
  *code = c;
  if (c != 0) {
    MLD_CUDA_CHECK(cudaMemset(word, 0, sizeof(int)));
    set_last_error_text("a bounded device-side wait of a FullyConnected kernel gave up");
    return MLD_TIMEOUT;
  }
  return MLD_OK;
}

int mld_fc_plan_set_weights_sum(mld_fc_plan* plan, const int32_t* sum_i) {
  MLD_REQUIRE(plan != nullptr, "null plan");
  plan->w_sum = sum_i;
  return MLD_OK;
}

int mld_fc_plan_prefetch_next(mld_fc_plan* plan, const void* next_weights, size_t bytes) {
  MLD_REQUIRE(plan != nullptr, "null plan");
  MLD_REQUIRE((reinterpret_cast<uintptr_t>(next_weights) & 15) == 0, "prefetch address must be 16-byte aligned");
  plan->next_w = bytes > 0 ? next_weights : nullptr;
  plan->next_w_bytes = bytes;
  return MLD_OK;
}

static int run_generic(mld_fc_plan* p, const void* src, const void* weights, const void* scale, const void* zp,
                       const void* bias, void* dst, int tokens, cudaStream_t stream) {
  const mld_fc_desc& d = p->d;
  GenericArgs a;
  a.x = src;
  a.weights = weights;
  a.scale = scale;
  a.zp = zp;
  a.bias = bias;
  a.y = dst;
  a.M = tokens;
  a.K = d.k;
  a.N = d.n;
  a.src_slices = div_up(d.k, 4);
  a.dst_slices = div_up(d.n, 4);
  a.scale_mode = d.scale_mode;
  a.groups = d.scale_mode == MLD_SCALE_BLOCK ? d.groups : 1;
  a.group_slices = p->group_slices;
  a.scalar_scale = d.scalar_scale;
  a.scalar_zp = d.scalar_zero_point;
  a.has_zp = d.has_zero_point;
  a.src_layout = d.src_layout;
  a.dst_layout = d.dst_layout;
  return launch_fc_generic(a, d.weight_bits, d.precision == MLD_PRECISION_F32, stream);
}

static int run_stream(mld_fc_plan* p, const void* src, const void* weights, const void* scale, const void* bias,
                      void* dst, int tokens, cudaStream_t stream, const PeerScatter* scatter, const PeerWait* wait) {
  const mld_fc_desc& d = p->d;
  const StripGeometry& gm = p->gm;
  const int N4 = align_n(d.n, 4), SS = div_up(d.k, 4), DS = N4 / 4;
  CUtensorMap tw, ts;
  {
    std::lock_guard<std::mutex> lock(p->mu);
    const TmapEntry* te = nullptr;
    for (const TmapEntry& e : p->tmaps)
      if (e.w == weights && e.s == scale) te = &e;
    if (te == nullptr) {
      TmapEntry e;
      e.w = weights;
      e.s = scale;
      e.geom = 0;
      const uint64_t blk = d.weight_bits == 4 ? 8 : 16;
      int rc = make_tmap_2d(&e.tw, weights, (uint64_t)DS * blk, SS, (uint64_t)DS * blk, 128, gm.stage_rows, 1,
                            CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc != MLD_OK) return rc;
      if (gm.scale_rows > 0) {
        const int G = d.scale_mode == MLD_SCALE_BLOCK ? d.groups : 1;
        const int wt = gm.w * (d.weight_bits == 4 ? 64 : 32);
        rc = make_tmap_2d(&e.ts, scale, (uint64_t)N4 * 2, G, (uint64_t)N4 * 2, wt * 2, gm.scale_rows, 2,
                          CU_TENSOR_MAP_SWIZZLE_NONE);
        if (rc != MLD_OK) return rc;
      } else {
        memset(&e.ts, 0, sizeof e.ts);
      }
      if (p->tmaps.size() >= 64) p->tmaps.erase(p->tmaps.begin());
      p->tmaps.push_back(e);
      te = &p->tmaps.back();
    }
    tw = te->tw;
    ts = te->ts;
  }
  StripArgs a;
  a.x = src;
  a.bias = bias;
  a.y = dst;
  a.error = p->error_shared != nullptr ? p->error_shared : p->error;
  a.M_total = tokens;
  a.N = d.n;
  a.N4 = N4;
  a.src_slices = SS;
  a.units = gm.units;
  a.gran = gm.gran;
  a.strips = gm.strips;
  a.ksplit = gm.ksplit;
  a.rows_per_split = gm.rows_per_split;
  a.stages = gm.stages;
  a.stage_bytes = gm.stage_bytes;
  a.scale_stage_bytes = gm.scale_stage_bytes;
  a.scale_rows = gm.scale_rows;
  a.group_slices = gm.group_slices;
  a.gs_shift = gm.gs_shift;
  a.red_m = gm.red_m;
  a.dst_layout = d.dst_layout;
  a.epilogue = d.epilogue;
  a.scalar_scale = d.scalar_scale;
  a.pdl = p->pdl ? (d.independent_io != 0 && scatter == nullptr && wait == nullptr ? 2 : 1) : 0;
  a.trace = g_trace_buffer;
  a.trace_skip_math = 0;
#ifdef MLD_TRACE
  a.trace_skip_math = getenv("MLD_GEMV_SKIP_MATH") != nullptr ? 1 : 0;
#endif
  memset(&a.scatter, 0, sizeof a.scatter);
  memset(&a.wait, 0, sizeof a.wait);
  if (scatter != nullptr) a.scatter = *scatter;
  if (wait != nullptr) a.wait = *wait;
  a.next_w = p->next_w;
  a.next_w_bytes = p->next_w_bytes;
  p->next_w = nullptr;  // the hint is consumed by this call
  for (int tok0 = 0; tok0 < tokens; tok0 += 8) {
    a.tok0 = tok0;
    a.M = tokens - tok0 < 8 ? tokens - tok0 : 8;
    const int rc = launch_fc_strip(d.weight_bits, p->subnormal, tw, ts, a, gm, stream);
    if (rc != MLD_OK) return rc;
  }
  return MLD_OK;
}

// Prefill: the activations are brought into K-major order (and quantised per token for the int8 route),
// then one tcgen05 GEMM.  By default the GEMM reads the packed weights as they are and dequantises them in
// shared memory (gemm_pair_kernel); with cache_prepared_weights, or for a weight matrix whose row pitch a
// tensor map cannot express, the weights are first expanded to a K-major copy (kept between calls when
// cached) and a plain GEMM runs on that.
static int run_gemm(mld_fc_plan* p, const void* src, const void* weights, const void* scale, const void* bias,
                    void* dst, int tokens, cudaStream_t stream, const PeerOutputs* outs, bool* outs_used) {
  const mld_fc_desc& d = p->d;
  const bool i8 = d.prefill_act_quant != 0;
  int* err = p->error_shared != nullptr ? p->error_shared : p->error;
  if (p->x_kmajor == nullptr) {
    set_last_error_text("this operator was not planned for the prefill route (force_path / max_tokens at creation)");
    return MLD_INVALID_ARGUMENT;
  }
  MLD_REQUIRE((reinterpret_cast<uintptr_t>(bias) & 7) == 0, "biases must be 8-byte aligned");
  if (d.prefill_act_quant == 2 && p->w_sum == nullptr) {
    set_last_error_text("asymmetric int8 activations need the weights' per-output sums (mld_fc_plan_set_weights_sum)");
    return MLD_INVALID_ARGUMENT;
  }
  int rc;
  const bool convert = d.cache_prepared_weights != 0 || !p->pair_ok || d.prefill_route == MLD_PREFILL_ROUTE_CONVERT ||
                       (d.prefill_route == MLD_PREFILL_ROUTE_AUTO && convert_pays(tokens));  // (routes 1 and 3: inside)
  if (!convert && !i8 && d.prefill_route != MLD_PREFILL_ROUTE_INLINE_SMEM) {
    // float route: the dequantised weights go to tensor memory
    p->last_route = MLD_ROUTE_PREFILL_INLINE;
    const int mode = d.weight_bits == 4 ? 0 : 1;
    const WtGeometry wg = wtmem_geometry(tokens, d.n, d.k, mode, p->sms, true);
    if (++p->split.epoch == 0) p->split.epoch = 1;
    rc = launch_transpose_x(src, d.src_layout, tokens, d.k, wg.kp, p->x_kmajor, stream);
    if (rc != MLD_OK) return rc;
    return launch_gemm_wtmem(mode, p->x_kmajor, weights, wg, tokens, d.n, d.k, scale, d.scale_mode,
                             d.scale_mode == MLD_SCALE_BLOCK ? d.groups : 1, p->group_slices, d.scalar_scale, bias, dst,
                             d.dst_layout, err, stream, outs, &p->split);
  }
  if (!convert) {
    p->last_route = MLD_ROUTE_PREFILL_INLINE;
    const int mode = i8 ? 2 : (d.weight_bits == 4 ? 0 : 1);
    const PairGeometry pg = pair_geometry(tokens, d.n, d.k, mode, p->sms, true);
    if (++p->split.epoch == 0) p->split.epoch = 1;
    if (i8)
      rc = launch_quantize_act(src, d.src_layout, tokens, d.k, pg.kp, d.prefill_act_quant == 1, p->x_kmajor, p->a_params,
                               stream);
    else
      rc = launch_transpose_x(src, d.src_layout, tokens, d.k, pg.kp, p->x_kmajor, stream);
    if (rc != MLD_OK) return rc;
    return launch_gemm_pair(mode, p->x_kmajor, weights, pg, tokens, d.n, d.k, scale, d.scale_mode,
                            d.scale_mode == MLD_SCALE_BLOCK ? d.groups : 1, p->group_slices, d.scalar_scale, bias,
                            p->a_params, d.prefill_act_quant == 2 ? p->w_sum : nullptr, dst, d.dst_layout, err, stream,
                            outs, &p->split);
  }

  const GemmGeometry g = gemm_geometry(tokens, d.n, d.k, i8, p->sms);
  const bool reuse = d.cache_prepared_weights && p->prepared_w == weights && p->prepared_s == scale;
  bool x_done = false;
  p->last_route = reuse ? MLD_ROUTE_PREFILL_CACHED : MLD_ROUTE_PREFILL_CONVERTED;
  if (!reuse) {
    // float route, sliced activations: their transposition rides along in the conversion launch
    const bool ride = !i8 && d.src_layout == MLD_LAYOUT_SLICED;
    rc = launch_dequant_weights(d.weight_bits, i8, weights, scale, d.scale_mode,
                                d.scale_mode == MLD_SCALE_BLOCK ? d.groups : 1, p->group_slices, d.scalar_scale, d.n,
                                d.k, g.kp, p->w_kmajor, stream, ride ? src : nullptr, tokens, p->x_kmajor);
    if (rc != MLD_OK) return rc;
    p->prepared_w = weights;
    p->prepared_s = scale;
    x_done = ride;
  }
  if (x_done) {
    rc = MLD_OK;
  } else if (i8)
    rc = launch_quantize_act(src, d.src_layout, tokens, d.k, g.kp, d.prefill_act_quant == 1, p->x_kmajor, p->a_params,
                             stream);
  else
    rc = launch_transpose_x(src, d.src_layout, tokens, d.k, g.kp, p->x_kmajor, stream);
  if (rc != MLD_OK) return rc;
  {
    // the multiplication itself: the SM-pair kernel with both operands loaded by TMA
    const int mode = i8 ? 4 : 3;
    const PairGeometry pg = pair_geometry(tokens, d.n, d.k, mode, p->sms, true);
    if (++p->split.epoch == 0) p->split.epoch = 1;
    if (pg.kp == g.kp)
      return launch_gemm_pair(mode, p->x_kmajor, p->w_kmajor, pg, tokens, d.n, d.k, scale, d.scale_mode, 1, 1, 0.0f,
                              bias, p->a_params, d.prefill_act_quant == 2 ? p->w_sum : nullptr, dst, d.dst_layout, err,
                              stream, outs, &p->split);
  }
  if (d.prefill_act_quant == 2) {
    set_last_error_text("asymmetric int8 activations are served by the SM-pair GEMM only");
    return MLD_UNIMPLEMENTED;
  }
  if (outs_used != nullptr) *outs_used = false;  // this kernel writes dst only
  return launch_gemm_umma(i8, p->x_kmajor, p->w_kmajor, g, tokens, d.n, d.k, bias, scale, p->a_params, dst,
                          d.dst_layout, err, stream);
}

int mld_fc_run(mld_fc_plan* plan, const void* src, const void* weights, const void* scale, const void* zero_point,
               const void* bias, void* dst, int32_t tokens, void* stream_v) {
  return mld::fc_run_internal(plan, src, weights, scale, zero_point, bias, dst, tokens, stream_v, nullptr, nullptr);
}

}  // extern "C"

void mld::fc_plan_shape(const mld_fc_plan* plan, int* n, int* dst_layout, int* max_tokens, int* device) {
  *n = plan->d.n;
  *dst_layout = plan->d.dst_layout;
  *max_tokens = plan->d.max_tokens;
  *device = plan->device;
}

int mld::fc_run_internal(mld_fc_plan* plan, const void* src, const void* weights, const void* scale,
                         const void* zero_point, const void* bias, void* dst, int32_t tokens, void* stream_v,
                         const PeerScatter* scatter, const PeerWait* wait, const PeerOutputs* outs, bool* outs_used) {
  MLD_REQUIRE(plan != nullptr, "null plan");
  // outs_used: whether the kernel that ran stored into the peers' tensors itself (only the inline-dequant
  // prefill GEMM does; after any other route the caller distributes dst)
  if (outs_used != nullptr) *outs_used = false;
  const mld_fc_desc& d = plan->d;
  MLD_REQUIRE(tokens >= 0 && tokens <= d.max_tokens, "tokens exceeds the plan's max_tokens");
  if (tokens == 0) return MLD_OK;
  MLD_REQUIRE(src != nullptr && weights != nullptr && dst != nullptr, "null tensor");
  MLD_REQUIRE(d.scale_mode == MLD_SCALE_SCALAR || scale != nullptr, "weights_scale tensor missing");
  MLD_REQUIRE(!d.has_bias || bias != nullptr, "biases tensor missing");
  MLD_REQUIRE((reinterpret_cast<uintptr_t>(weights) & 15) == 0, "weights must be 16-byte aligned");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const void* b = d.has_bias ? bias : nullptr;
  const void* zp = d.has_zero_point ? zero_point : nullptr;

  int path = d.force_path;
  if (path == 0) path = mld_fc_is_gemv_recommended(d.precision, tokens) ? 1 : 2;
  if (path == 2) {
    // the tensor-core route takes fp16 tensors without zero points; anything
    // else is served, correctly but slowly, by the general kernel below
    const bool gemm_ok = d.precision != MLD_PRECISION_F32 && !d.has_zero_point && get_encode_tiled() != nullptr &&
                         (reinterpret_cast<uintptr_t>(src) & 7) == 0;
    if (gemm_ok) {
      if (outs_used != nullptr) *outs_used = outs != nullptr && outs->world > 1 && d.dst_layout == MLD_LAYOUT_SLICED;
      return run_gemm(plan, src, weights, scale, b, dst, tokens, stream, outs, outs_used);
    }
    if (d.prefill_act_quant != 0) {
      set_last_error_text("quantised-activation prefill needs fp16 tensors and no zero points");
      return MLD_UNIMPLEMENTED;
    }
    plan->last_route = MLD_ROUTE_DECODE_GENERAL;
    return run_generic(plan, src, weights, scale, zp, b, dst, tokens, stream);
  }
  if (d.epilogue != MLD_EPILOGUE_NONE && !(path == 1 && plan->stream_ok && tokens <= 16)) {
    set_last_error_text("the fused SiLU*mul write is available on the streaming decode kernel only");
    return MLD_UNIMPLEMENTED;
  }
  const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
                       (scale == nullptr || (reinterpret_cast<uintptr_t>(scale) & 15) == 0);
  const bool layout_ok = d.src_layout == MLD_LAYOUT_SLICED || tokens == 1;
  if (plan->stream_ok && tokens <= 16 && aligned && layout_ok) {
    plan->last_route = MLD_ROUTE_DECODE_STREAMING;
    return run_stream(plan, src, weights, scale, b, dst, tokens, stream, scatter, wait);
  }
  if (d.epilogue != MLD_EPILOGUE_NONE) {
    set_last_error_text("the fused SiLU*mul write needs 16-byte aligned fp16 tensors in the sliced layout");
    return MLD_UNIMPLEMENTED;
  }
  plan->last_route = MLD_ROUTE_DECODE_GENERAL;
  return run_generic(plan, src, weights, scale, zp, b, dst, tokens, stream);
}


