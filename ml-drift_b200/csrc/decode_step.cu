// One decode step of a Llama-style decoder whose seven projections per layer
// are quantized FullyConnected nodes (the callers of the FC hot path in
// ml_drift/samples/llm/qwen3_model_builder.cc:907-1038: Linear, FFLayer,
// SelfAttention, TransformerLayer).  The FullyConnected nodes run through the
// same plans mld_fc_run uses, with the residual adds and SiLU*mul fused into the
// projections' dst writes; the glue around them (RMSNorm, one attention kernel
// doing RoPE + KV-cache update + decode attention) is plain CUDA.
//
// Column sharding: with world > 1 every projection holds the rows of its own
// output shard; shard outputs are concatenated by an all-gather before the next
// full-width consumer (after attention, o_proj, SiLU*mul and down_proj).
#include <cuda_fp16.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "kernels.h"
#include "nccl_lazy.h"

namespace mld {
namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// h = x (+ r); y = h * rsqrt(mean(h^2) + eps) * gamma.  One CTA.
// RMSNormalization with epsilon 1e-6 and a gamma vector
// (qwen3_model_builder.cc:890-902).  gamma == null: only h is written.
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ r,
                                                          const __half* __restrict__ gamma, __half* __restrict__ h_out,
                                                          __half* __restrict__ y, int d, float eps, PeerWait wait) {
  __shared__ float part[32];
  pdl_wait();
  pdl_launch_dependents();
  if (wait.world > 1) {  // x is a vector other ranks contribute to: wait for all of its shards
    if (threadIdx.x == 0 &&
        !wait_peer_flags(wait.flags, wait.world, static_cast<unsigned>(*wait.step * wait.seq_per_step + wait.seq_off),
                         wait.limit_ns))
      atomicExch(wait.error, kErrPeerWait);  // the step goes on with what has arrived; the host sees the code
    __syncthreads();
  }
  float ss = 0.0f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v = __half2float(x[i]);
    if (r != nullptr) v = __half2float(__float2half_rn(v + __half2float(r[i])));
    if (h_out != nullptr) h_out[i] = __float2half_rn(v);
    ss += v * v;
  }
  if (gamma == nullptr) return;
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? part[threadIdx.x] : 0.0f;
    t = warp_sum(t);
    if (threadIdx.x == 0) part[0] = rsqrtf(t / static_cast<float>(d) + eps);
  }
  __syncthreads();
  const float inv = part[0];
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float v;
    if (h_out != nullptr) {
      v = __half2float(h_out[i]);  // written above by this same thread (h_out may alias x)
    } else {
      v = __half2float(x[i]);
      if (r != nullptr) v = __half2float(__float2half_rn(v + __half2float(r[i])));
    }
    y[i] = __float2half_rn(v * inv * __half2float(gamma[i]));
  }
}

// Decode attention for one query token, split over the cached tokens.
// grid (heads, splits), 128 threads.  Eight lanes share a token (16 dims each);
// every 8-lane group keeps its own running max / sum / output and the groups
// are merged at the end.  head_dim is fixed at 128.  Partial results:
// part_o [heads][splits][128] fp32, part_ml [heads][splits][2] (max, sum).
constexpr int kHeadDim = 128;
__global__ void __launch_bounds__(128) attn_decode_kernel(const __half* __restrict__ q, const __half* __restrict__ kcache,
                                                          const __half* __restrict__ vcache, float* __restrict__ part_o,
                                                          float* __restrict__ part_ml, int heads, int n_tokens,
                                                          int splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int head = blockIdx.x, split = blockIdx.y;
  const int per = (n_tokens + splits - 1) / splits;
  const int t0 = split * per, t1 = min(n_tokens, t0 + per);
  const int grp = threadIdx.x >> 3, sub = threadIdx.x & 7;  // 16 groups of 8 lanes
  const int width = heads * kHeadDim;
  float qv[16];
  {
    const __half* qp = q + (size_t)head * kHeadDim + sub * 16;
#pragma unroll
    for (int j = 0; j < 16; ++j) qv[j] = __half2float(qp[j]);
  }
  float m = -INFINITY, l = 0.0f, acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
  const unsigned gmask = 0xFFu << (threadIdx.x & 24);
  for (int t = t0 + grp; t < t1; t += 16) {
    const uint4* kp = reinterpret_cast<const uint4*>(kcache + (size_t)t * width + head * kHeadDim + sub * 16);
    const uint4 k0 = kp[0], k1 = kp[1];
    const __half2* kh = reinterpret_cast<const __half2*>(&k0);
    const __half2* kh2 = reinterpret_cast<const __half2*>(&k1);
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __half22float2(kh[j]), b = __half22float2(kh2[j]);
      s += qv[2 * j] * a.x + qv[2 * j + 1] * a.y + qv[8 + 2 * j] * b.x + qv[8 + 2 * j + 1] * b.y;
    }
    // the eight lanes of a token group run this loop together; other groups of
    // the warp may have a different trip count, so the shuffle names only them
    s += __shfl_xor_sync(gmask, s, 1);
    s += __shfl_xor_sync(gmask, s, 2);
    s += __shfl_xor_sync(gmask, s, 4);
    const float m_new = fmaxf(m, s);
    const float corr = __expf(m - m_new), p = __expf(s - m_new);
    const uint4* vp = reinterpret_cast<const uint4*>(vcache + (size_t)t * width + head * kHeadDim + sub * 16);
    const uint4 v0 = vp[0], v1 = vp[1];
    const __half2* vh = reinterpret_cast<const __half2*>(&v0);
    const __half2* vh2 = reinterpret_cast<const __half2*>(&v1);
    l = l * corr + p;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 a = __half22float2(vh[j]), b = __half22float2(vh2[j]);
      acc[2 * j] = acc[2 * j] * corr + p * a.x;
      acc[2 * j + 1] = acc[2 * j + 1] * corr + p * a.y;
      acc[8 + 2 * j] = acc[8 + 2 * j] * corr + p * b.x;
      acc[8 + 2 * j + 1] = acc[8 + 2 * j + 1] * corr + p * b.y;
    }
    m = m_new;
  }
  // merge the 16 groups
  __shared__ float sm_m[16], sm_l[16], sm_o[16][kHeadDim];
  if (sub == 0) {
    sm_m[grp] = m;
    sm_l[grp] = l;
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) sm_o[grp][sub * 16 + j] = acc[j];
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int g = 0; g < 16; ++g) gm = fmaxf(gm, sm_m[g]);
  const int dim = threadIdx.x;  // 128 threads, one output dim each
  float o = 0.0f, lsum = 0.0f;
#pragma unroll
  for (int g = 0; g < 16; ++g) {
    const float w = sm_m[g] == -INFINITY ? 0.0f : __expf(sm_m[g] - gm);
    o += w * sm_o[g][dim];
    lsum += w * sm_l[g];
  }
  part_o[((size_t)head * splits + split) * kHeadDim + dim] = o;
  if (dim == 0) {
    part_ml[((size_t)head * splits + split) * 2 + 0] = gm;
    part_ml[((size_t)head * splits + split) * 2 + 1] = lsum;
  }
}

__global__ void __launch_bounds__(128) attn_combine_kernel(const float* __restrict__ part_o,
                                                           const float* __restrict__ part_ml, __half* __restrict__ out,
                                                           int splits) {
  pdl_wait();
  pdl_launch_dependents();
  const int head = blockIdx.x, dim = threadIdx.x;
  float gm = -INFINITY;
  for (int s = 0; s < splits; ++s) gm = fmaxf(gm, part_ml[((size_t)head * splits + s) * 2]);
  float o = 0.0f, l = 0.0f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_ml[((size_t)head * splits + s) * 2];
    const float w = ms == -INFINITY ? 0.0f : __expf(ms - gm);
    o += w * part_o[((size_t)head * splits + s) * kHeadDim + dim];
    l += w * part_ml[((size_t)head * splits + s) * 2 + 1];
  }
  out[(size_t)head * kHeadDim + dim] = __float2half_rn(o / l);
}

// The decoder's attention node in one launch: rotary embedding of q and of the
// new token's k (rope.cc:70-89), KV-cache write of the new token, split-KV
// attention, and the merge of the splits by whichever CTA of a head finishes
// last (a ticket per head; nothing waits).  qkv = raw [q | k | v] of the local
// heads as the projection wrote them.
struct AttnStepArgs {
  const __half* qkv;
  __half* kcache;
  __half* vcache;
  float* part_o;
  float* part_ml;
  int* tickets;   // one per head, zero between launches
  __half* out;
  int heads, pos, splits;
  float min_ts, max_ts, q_scale;
  PeerScatter scatter;  // world > 1: the merged head outputs go to every rank's attention vector
};
__global__ void __launch_bounds__(128) attn_step_kernel(AttnStepArgs a) {
  pdl_wait();
  pdl_launch_dependents();
  const int head = blockIdx.x, split = blockIdx.y;
  const int n_tokens = a.pos + 1;
  const int per = (n_tokens + a.splits - 1) / a.splits;
  const int t0 = split * per, t1 = min(n_tokens, t0 + per);
  const int grp = threadIdx.x >> 3, sub = threadIdx.x & 7;
  const int width = a.heads * kHeadDim;
  __shared__ float sq[kHeadDim];
  __shared__ float sm_m[16], sm_l[16], sm_o[16][kHeadDim];
  __shared__ int s_last;
  const bool owns_new = a.pos >= t0 && a.pos < t1;
  if (threadIdx.x < kHeadDim / 2) {
    const int i = threadIdx.x, half = kHeadDim / 2;
    const float fraction = 2.0f * i / static_cast<float>(kHeadDim);
    const float timescale = a.min_ts * powf(a.max_ts / a.min_ts, fraction);
    float sn, cs;
    sincosf(static_cast<float>(a.pos) / timescale, &sn, &cs);
    const __half* qp = a.qkv + (size_t)head * kHeadDim;
    const float q0 = __half2float(qp[i]), q1 = __half2float(qp[i + half]);
    // rounded to fp16 exactly where the unfused graph stores the rotated q
    sq[i] = __half2float(__float2half_rn((q0 * cs - q1 * sn) * a.q_scale));
    sq[i + half] = __half2float(__float2half_rn((q1 * cs + q0 * sn) * a.q_scale));
    if (owns_new) {
      const __half* kp = a.qkv + (size_t)(a.heads + head) * kHeadDim;
      const float k0 = __half2float(kp[i]), k1 = __half2float(kp[i + half]);
      __half* kc = a.kcache + (size_t)a.pos * width + head * kHeadDim;
      kc[i] = __float2half_rn(k0 * cs - k1 * sn);
      kc[i + half] = __float2half_rn(k1 * cs + k0 * sn);
    }
  } else if (owns_new) {
    const int j = threadIdx.x - kHeadDim / 2;  // 64 threads copy the 128 v values
    const __half* vp = a.qkv + (size_t)(2 * a.heads + head) * kHeadDim;
    __half* vc = a.vcache + (size_t)a.pos * width + head * kHeadDim;
    vc[j] = vp[j];
    vc[j + kHeadDim / 2] = vp[j + kHeadDim / 2];
  }
  __syncthreads();  // the new token's cache rows are visible to this CTA, which is the only reader of them
  float qv[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) qv[j] = sq[sub * 16 + j];
  float m = -INFINITY, l = 0.0f, acc[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) acc[j] = 0.0f;
  const unsigned gmask = 0xFFu << (threadIdx.x & 24);
  for (int t = t0 + grp; t < t1; t += 16) {
    const uint4* kp = reinterpret_cast<const uint4*>(a.kcache + (size_t)t * width + head * kHeadDim + sub * 16);
    const uint4 k0 = kp[0], k1 = kp[1];
    const __half2* kh = reinterpret_cast<const __half2*>(&k0);
    const __half2* kh2 = reinterpret_cast<const __half2*>(&k1);
    float s = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x0 = __half22float2(kh[j]), x1 = __half22float2(kh2[j]);
      s += qv[2 * j] * x0.x + qv[2 * j + 1] * x0.y + qv[8 + 2 * j] * x1.x + qv[8 + 2 * j + 1] * x1.y;
    }
    s += __shfl_xor_sync(gmask, s, 1);
    s += __shfl_xor_sync(gmask, s, 2);
    s += __shfl_xor_sync(gmask, s, 4);
    const float m_new = fmaxf(m, s);
    const float corr = __expf(m - m_new), p = __expf(s - m_new);
    const uint4* vp = reinterpret_cast<const uint4*>(a.vcache + (size_t)t * width + head * kHeadDim + sub * 16);
    const uint4 v0 = vp[0], v1 = vp[1];
    const __half2* vh = reinterpret_cast<const __half2*>(&v0);
    const __half2* vh2 = reinterpret_cast<const __half2*>(&v1);
    l = l * corr + p;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x0 = __half22float2(vh[j]), x1 = __half22float2(vh2[j]);
      acc[2 * j] = acc[2 * j] * corr + p * x0.x;
      acc[2 * j + 1] = acc[2 * j + 1] * corr + p * x0.y;
      acc[8 + 2 * j] = acc[8 + 2 * j] * corr + p * x1.x;
      acc[8 + 2 * j + 1] = acc[8 + 2 * j + 1] * corr + p * x1.y;
    }
    m = m_new;
  }
  if (sub == 0) {
    sm_m[grp] = m;
    sm_l[grp] = l;
  }
#pragma unroll
  for (int j = 0; j < 16; ++j) sm_o[grp][sub * 16 + j] = acc[j];
  __syncthreads();
  float gm = -INFINITY;
#pragma unroll
  for (int g = 0; g < 16; ++g) gm = fmaxf(gm, sm_m[g]);
  const int dim = threadIdx.x;
  float o = 0.0f, lsum = 0.0f;
#pragma unroll
  for (int g = 0; g < 16; ++g) {
    const float w = sm_m[g] == -INFINITY ? 0.0f : __expf(sm_m[g] - gm);
    o += w * sm_o[g][dim];
    lsum += w * sm_l[g];
  }
  a.part_o[((size_t)head * a.splits + split) * kHeadDim + dim] = o;
  if (dim == 0) {
    a.part_ml[((size_t)head * a.splits + split) * 2 + 0] = gm;
    a.part_ml[((size_t)head * a.splits + split) * 2 + 1] = lsum;
  }
  // the last CTA of this head to get here merges the splits
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) s_last = atomicAdd(a.tickets + head, 1) == a.splits - 1 ? 1 : 0;
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  float tm = -INFINITY;
  for (int s = 0; s < a.splits; ++s) tm = fmaxf(tm, __ldcg(a.part_ml + ((size_t)head * a.splits + s) * 2));
  float to = 0.0f, tl = 0.0f;
  for (int s = 0; s < a.splits; ++s) {
    const float ms = __ldcg(a.part_ml + ((size_t)head * a.splits + s) * 2);
    const float w = ms == -INFINITY ? 0.0f : __expf(ms - tm);
    to += w * __ldcg(a.part_o + ((size_t)head * a.splits + s) * kHeadDim + dim);
    tl += w * __ldcg(a.part_ml + ((size_t)head * a.splits + s) * 2 + 1);
  }
  const __half res = __float2half_rn(to / tl);
  if (a.scatter.world > 1) {
    for (int pr = 0; pr < a.scatter.world; ++pr)
      static_cast<__half*>(a.scatter.y_peers[pr])[(size_t)head * kHeadDim + dim] = res;
    // second-level ticket over the heads of this rank: the last head raises the flag everywhere
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      a.tickets[head] = 0;
      if (atomicAdd(a.scatter.ticket, 1) == a.heads - 1) {
        *a.scatter.ticket = 0;
        __threadfence_system();
        const unsigned seq = static_cast<unsigned>(*a.scatter.step * a.scatter.seq_per_step + a.scatter.seq_off);
        for (int pr = 0; pr < a.scatter.world; ++pr) st_release_sys(a.scatter.flag_peers[pr], seq);
      }
    }
    return;
  }
  a.out[(size_t)head * kHeadDim + dim] = res;
  if (threadIdx.x == 0) a.tickets[head] = 0;
}

// Step bookkeeping of the peer exchange: bumps the device-side step counter
// (flag values are derived from it, so CUDA-graph replays produce fresh values).
__global__ void bump_step_kernel(int* step) {
  pdl_wait();
  pdl_launch_dependents();
  *step += 1;
}

// Final copy of a gathered vector out of the exchange block, after all shards arrived.
__global__ void __launch_bounds__(256) copy_after_wait_kernel(const __half* __restrict__ src, __half* __restrict__ dst,
                                                              int n, PeerWait wait) {
  pdl_wait();
  pdl_launch_dependents();
  if (wait.world > 1) {
    if (threadIdx.x == 0 &&
        !wait_peer_flags(wait.flags, wait.world, static_cast<unsigned>(*wait.step * wait.seq_per_step + wait.seq_off),
                         wait.limit_ns))
      atomicExch(wait.error, kErrPeerWait);
    __syncthreads();
  }
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) dst[i] = src[i];
}

// Launches a glue kernel so that it may be scheduled while its predecessor in
// the stream drains (programmatic dependent launch); every glue kernel starts
// with griddepcontrol.wait, so it touches memory only after the predecessor
// has completed.
bool g_glue_pdl = true;
template <typename... KArgs, typename... Args>
int launch_glue(void (*kern)(KArgs...), dim3 grid, dim3 block, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_glue_pdl ? 1 : 0;
  MLD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...));
  count_launch();
  return MLD_OK;
}

// Split count that fills the GPU about four CTAs deep.
int attn_splits(int heads, int sms) {
  int splits = (4 * sms) / (heads > 0 ? heads : 1);
  if (splits < 1) splits = 1;
  if (splits > 64) splits = 64;
  return splits;
}

int launch_attn_decode(const __half* q, const __half* kcache, const __half* vcache, float* part_o, float* part_ml,
                       __half* out, int heads, int n_tokens, int splits, cudaStream_t stream) {
  int rc = launch_glue(attn_decode_kernel, dim3(heads, splits), dim3(128), stream, q, kcache, vcache, part_o, part_ml,
                       heads, n_tokens, splits);
  if (rc != MLD_OK) return rc;
  return launch_glue(attn_combine_kernel, dim3(heads), dim3(128), stream, part_o, part_ml, out, splits);
}

// Grow-only per-device scratch of mld_attn_decode.
struct AttnScratch {
  void* ptr = nullptr;
  size_t bytes = 0;
};
AttnScratch g_attn_scratch[64];
std::mutex g_attn_mu;

}  // namespace

Nccl& nccl() {
  static Nccl instance;
  return instance;
}

}  // namespace mld

using namespace mld;

struct mld_decoder {
  mld_decoder_desc d;
  int heads_local, d_local, ffn_local;
  mld_fc_plan *p_qkv, *p_o, *p_gu, *p_down;
  std::vector<mld_layer_weights> layers;
  // scratch (owned)
  __half *xn, *qkv, *attn_local, *attn_full, *o_local, *o_full, *h, *hn, *gu, *act_local, *act_full, *d_full, *x_stage, *y_stage;
  float *part_o, *part_ml;
  int* tickets;
  bool prefetch;
  size_t bytes_qkv, bytes_o, bytes_gu, bytes_down;
  uint8_t* scratch;
  int splits;
  ncclComm_t comm;
  size_t scratch_bytes;
  // peer exchange (world > 1, after mld_decoder_ipc_import): gathered vectors and flags live in one
  // IPC-shared block with the same layout on every rank
  uint8_t* xchg;                 // this rank's block
  uint8_t* xchg_peers[8];        // every rank's block as mapped here (index = rank; own entry = xchg)
  bool peer_mode;
  size_t off_attn, off_h, off_act, off_xa, off_xb, off_flags, xchg_bytes;
  int* peer_tickets;             // local: [4] CTA counters + [1] step counter
  int* error;                    // device error word of the op chain (shared with its four plans)
  int* error_host;               // pinned copy read back by mld_decoder_step_host
  unsigned long long wait_limit_ns;
  // single GPU: the whole step as one persistent kernel (null = op-by-op path)
  mld::MegaDecoder* mega;
};

namespace {

int make_plan(int n, int k, int block, int device, bool residual, int epilogue, int* error_word, mld_fc_plan** out) {
  mld_fc_desc fd;
  memset(&fd, 0, sizeof fd);
  fd.n = n;
  fd.k = k;
  fd.weight_bits = 4;
  fd.scale_mode = MLD_SCALE_BLOCK;
  fd.groups = k / block;
  fd.precision = MLD_PRECISION_F32F16;
  fd.src_layout = MLD_LAYOUT_SLICED;
  fd.dst_layout = MLD_LAYOUT_SLICED;
  fd.max_tokens = 1;
  fd.force_path = 1;
  fd.device = device;
  fd.has_bias = residual ? 1 : 0;  // the residual vector rides in the bias slot of the dst write
  fd.epilogue = epilogue;
  const int rc = mld_fc_plan_create(&fd, out);
  if (rc == MLD_OK) fc_plan_share_error(*out, error_word);
  return rc;
}

int gather(mld_decoder* dec, const __half* send, __half* recv, int count, cudaStream_t stream) {
  if (dec->d.world == 1) return MLD_OK;  // callers alias send == recv
  const int rc = nccl().AllGather(send, recv, static_cast<size_t>(count), kNcclHalf, dec->comm, stream);
  if (rc != 0) {
    set_last_error_text(nccl().GetErrorString ? nccl().GetErrorString(rc) : "ncclAllGather failed");
    return MLD_NCCL_ERROR;
  }
  return MLD_OK;
}

}  // namespace

extern "C" {

int mld_comm_unique_id(void* id128) {
  MLD_REQUIRE(id128 != nullptr, "null id buffer");
  if (!nccl().load()) {
    set_last_error_text("libnccl.so.2 could not be loaded");
    return MLD_NCCL_ERROR;
  }
  ncclUniqueId id;
  if (nccl().GetUniqueId(&id) != 0) return MLD_NCCL_ERROR;
  memcpy(id128, &id, sizeof id);
  return MLD_OK;
}

int mld_attn_decode(const void* q, const void* kcache, const void* vcache, void* out, int32_t heads,
                    int32_t head_dim, int32_t n_tokens, void* stream) {
  MLD_REQUIRE(q != nullptr && kcache != nullptr && vcache != nullptr && out != nullptr, "null tensor");
  MLD_REQUIRE(head_dim == kHeadDim, "head_dim must be 128");
  MLD_REQUIRE(heads > 0 && n_tokens > 0, "bad shape");
  int device = 0;
  MLD_CUDA_CHECK(cudaGetDevice(&device));
  MLD_REQUIRE(device < 64, "device ordinal too large");
  const int splits = attn_splits(heads, sm_count(device));
  const size_t need = (size_t)heads * splits * (kHeadDim + 2) * sizeof(float);
  float* base;
  {
    std::lock_guard<std::mutex> lock(g_attn_mu);
    AttnScratch& sc = g_attn_scratch[device];
    if (sc.bytes < need) {
      if (sc.ptr != nullptr) MLD_CUDA_CHECK(cudaFree(sc.ptr));
      sc.ptr = nullptr;
      sc.bytes = 0;
      MLD_CUDA_CHECK(cudaMalloc(&sc.ptr, need));
      sc.bytes = need;
    }
    base = static_cast<float*>(sc.ptr);
  }
  return launch_attn_decode(static_cast<const __half*>(q), static_cast<const __half*>(kcache),
                            static_cast<const __half*>(vcache), base, base + (size_t)heads * splits * kHeadDim,
                            static_cast<__half*>(out), heads, n_tokens, splits, static_cast<cudaStream_t>(stream));
}

// ------------------------------------------------------------------------
// Allocation-free decode attention.
//
// Some hosts cannot let a library allocate device memory on their behalf: a
// serving process whose own pool already owns the whole GPU (a late cudaMalloc
// then fails, and it stalls every stream while the driver looks), or an
// embedded runtime that fixes its memory plan before the first dispatch, the
// way ML Drift's InferenceContext does.  For them the split-KV partial results
// live in this fixed array, which every GPU that loads the library carries
// until the process exits (2.03 MB).
constexpr int kStaticPairs = 4096;  // (head, split) pairs the array can hold
static __device__ __align__(256) float g_attn_static_scratch[kStaticPairs * (kHeadDim + 2)];

namespace {
// Device address of the array, looked up once per device.  In host code the
// symbol's name is only a handle, never a pointer a kernel could use.
float* g_attn_static_ptr[64] = {nullptr};
std::mutex g_attn_static_mu;
}  // namespace

int mld_attn_decode_static(const void* q, const void* kcache, const void* vcache, void* out, int32_t heads,
                           int32_t head_dim, int32_t n_tokens, void* stream) {
  MLD_REQUIRE(q != nullptr && kcache != nullptr && vcache != nullptr && out != nullptr, "null tensor");
  MLD_REQUIRE(head_dim == kHeadDim, "head_dim must be 128");
  MLD_REQUIRE(heads > 0 && n_tokens > 0, "bad shape");
  if (heads > kStaticPairs) {
    set_last_error_text("mld_attn_decode_static: more than 4096 heads do not fit the fixed scratch array");
    return MLD_OUT_OF_RANGE;
  }
  int device = 0;
  MLD_CUDA_CHECK(cudaGetDevice(&device));
  MLD_REQUIRE(device < 64, "device ordinal too large");
  float* base;
  {
    std::lock_guard<std::mutex> lock(g_attn_static_mu);
    if (g_attn_static_ptr[device] == nullptr) {
      // first call on this device (which is current): resolve the symbol
      void* p = nullptr;
      MLD_CUDA_CHECK(cudaGetSymbolAddress(&p, g_attn_static_scratch));
      g_attn_static_ptr[device] = static_cast<float*>(p);
    }
    base = g_attn_static_ptr[device];
  }
  int splits = attn_splits(heads, sm_count(device));
  if (heads * splits > kStaticPairs) splits = kStaticPairs / heads;
  // every (head, split) slot used below is rewritten by this call, so nothing
  // left from an earlier call can leak into the result
  return launch_attn_decode(static_cast<const __half*>(q), static_cast<const __half*>(kcache),
                            static_cast<const __half*>(vcache), base, base + (size_t)heads * splits * kHeadDim,
                            static_cast<__half*>(out), heads, n_tokens, splits, static_cast<cudaStream_t>(stream));
}

int mld_decoder_create(const mld_decoder_desc* d, const void* nccl_id128, mld_decoder** out) {
  MLD_REQUIRE(d != nullptr && out != nullptr, "null argument");
  *out = nullptr;
  MLD_REQUIRE(d->layers > 0 && d->d_model > 0 && d->heads > 0 && d->ffn > 0 && d->max_seq > 0, "bad decoder shape");
  MLD_REQUIRE(d->head_dim == kHeadDim, "head_dim must be 128");
  MLD_REQUIRE(d->heads * d->head_dim == d->d_model, "heads * head_dim must equal d_model");
  MLD_REQUIRE(d->world >= 1 && d->rank >= 0 && d->rank < d->world, "bad rank/world");
  MLD_REQUIRE(d->heads % d->world == 0 && d->ffn % d->world == 0, "heads and ffn must divide by world");
  MLD_REQUIRE(d->block > 0 && d->d_model % d->block == 0 && d->ffn % d->block == 0, "block must divide K");
  MLD_REQUIRE(d->world <= 8, "at most 8 ranks");
  int device = d->device;
  if (device < 0) MLD_CUDA_CHECK(cudaGetDevice(&device));
  MLD_CUDA_CHECK(cudaSetDevice(device));

  MLD_REQUIRE(d->mode >= MLD_DECODER_AUTO && d->mode <= MLD_DECODER_SINGLE_KERNEL, "bad decoder mode");
  MLD_REQUIRE(d->handover == 0 || d->handover == 1, "bad handover");
  MLD_REQUIRE(d->grid_limit >= 0 && d->ring_stages >= 0 && d->wait_limit_us >= 0, "bad tuning field");
  mld_decoder* dec = new mld_decoder();
  dec->d = *d;
  dec->d.device = device;
  dec->heads_local = d->heads / d->world;
  dec->d_local = d->d_model / d->world;
  dec->ffn_local = d->ffn / d->world;
  dec->layers.resize(d->layers);
  memset(dec->layers.data(), 0, sizeof(mld_layer_weights) * d->layers);
  dec->comm = nullptr;
  dec->scratch = nullptr;
  dec->xchg = nullptr;
  dec->peer_tickets = nullptr;
  dec->error = nullptr;
  dec->error_host = nullptr;
  dec->wait_limit_ns = static_cast<unsigned long long>(d->wait_limit_us > 0 ? d->wait_limit_us : 2000000) * 1000ull;
  dec->peer_mode = false;
  dec->mega = nullptr;
  for (int r = 0; r < 8; ++r) dec->xchg_peers[r] = nullptr;
  dec->p_qkv = dec->p_o = dec->p_gu = dec->p_down = nullptr;
  int rc = MLD_OK;
  if (cudaMalloc(&dec->error, sizeof(int)) != cudaSuccess || cudaMemset(dec->error, 0, sizeof(int)) != cudaSuccess ||
      cudaHostAlloc(&dec->error_host, sizeof(int), cudaHostAllocDefault) != cudaSuccess) {
    set_last_error_text("decoder status word allocation failed");
    rc = MLD_CUDA_ERROR;
  }
  int* ew = dec->error;
  if (rc == MLD_OK) rc = make_plan(3 * dec->d_local, d->d_model, d->block, device, false, MLD_EPILOGUE_NONE, ew, &dec->p_qkv);
  if (rc == MLD_OK) rc = make_plan(dec->d_local, d->d_model, d->block, device, true, MLD_EPILOGUE_NONE, ew, &dec->p_o);
  if (rc == MLD_OK)
    rc = make_plan(2 * dec->ffn_local, d->d_model, d->block, device, false, MLD_EPILOGUE_SWIGLU_PAIRS, ew, &dec->p_gu);
  if (rc == MLD_OK) rc = make_plan(dec->d_local, d->ffn, d->block, device, true, MLD_EPILOGUE_NONE, ew, &dec->p_down);
  // split count: fill the GPU about four CTAs deep
  int sms = sm_count(device);
  {
    dec->prefetch = true;  // every projection asks L2 for the next one's weights behind its own
    dec->bytes_qkv = (size_t)3 * dec->d_local * d->d_model / 2;
    dec->bytes_o = (size_t)dec->d_local * d->d_model / 2;
    dec->bytes_gu = (size_t)2 * dec->ffn_local * d->d_model / 2;
    dec->bytes_down = (size_t)dec->d_local * d->ffn / 2;
  }
  const int splits = attn_splits(dec->heads_local, sms);
  dec->splits = splits;
  const size_t dm = d->d_model, ff = d->ffn;
  auto pad = [](size_t bytes) { return (bytes + 255) & ~size_t(255); };  // bulk copies need 16-byte alignment
  const size_t sizes_h[11] = {dm, 3 * (size_t)dec->d_local, dm, dm, dm, dm, 2 * (size_t)dec->ffn_local, ff, dm, dm, dm};
  size_t total = 0;
  for (size_t n : sizes_h) total += pad(n * 2);
  total += pad((size_t)dec->heads_local * splits * kHeadDim * 4) + pad((size_t)dec->heads_local * splits * 2 * 4) +
           pad((size_t)dec->heads_local * 4);
  dec->scratch_bytes = total;
  dec->scratch = nullptr;
  if (rc == MLD_OK && cudaMalloc(&dec->scratch, total) != cudaSuccess) {
    set_last_error_text("decoder scratch allocation failed");
    rc = MLD_CUDA_ERROR;
  }
  if (rc != MLD_OK) {
    mld_decoder_destroy(dec);
    return rc;
  }
  cudaMemset(dec->scratch, 0, total);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    uint8_t* p = dec->scratch + off;
    off += pad(bytes);
    return p;
  };
  dec->xn = reinterpret_cast<__half*>(take(sizes_h[0] * 2));
  dec->qkv = reinterpret_cast<__half*>(take(sizes_h[1] * 2));
  dec->attn_full = reinterpret_cast<__half*>(take(sizes_h[2] * 2));
  dec->o_full = reinterpret_cast<__half*>(take(sizes_h[3] * 2));
  dec->h = reinterpret_cast<__half*>(take(sizes_h[4] * 2));
  dec->hn = reinterpret_cast<__half*>(take(sizes_h[5] * 2));
  dec->gu = reinterpret_cast<__half*>(take(sizes_h[6] * 2));
  dec->act_full = reinterpret_cast<__half*>(take(sizes_h[7] * 2));
  dec->d_full = reinterpret_cast<__half*>(take(sizes_h[8] * 2));
  dec->x_stage = reinterpret_cast<__half*>(take(sizes_h[9] * 2));
  dec->y_stage = reinterpret_cast<__half*>(take(sizes_h[10] * 2));
  dec->part_o = reinterpret_cast<float*>(take((size_t)dec->heads_local * splits * kHeadDim * 4));
  dec->part_ml = reinterpret_cast<float*>(take((size_t)dec->heads_local * splits * 2 * 4));
  dec->tickets = reinterpret_cast<int*>(take((size_t)dec->heads_local * 4));  // zeroed above
  if (d->world > 1) {
    // Vectors that every rank contributes a shard to live in one block with the same layout on all
    // ranks, so that it can be shared between the processes (IPC) and written by peers.
    size_t xo = 0;
    auto xtake = [&](size_t bytes) {
      const size_t o = xo;
      xo += pad(bytes);
      return o;
    };
    dec->off_attn = xtake(dm * 2);
    dec->off_h = xtake(dm * 2);
    dec->off_act = xtake(ff * 2);
    dec->off_xa = xtake(dm * 2);
    dec->off_xb = xtake(dm * 2);
    dec->off_flags = xtake(4 * 8 * sizeof(unsigned));
    dec->xchg_bytes = xo;
    if (cudaMalloc(&dec->xchg, xo) != cudaSuccess || cudaMalloc(&dec->peer_tickets, 256) != cudaSuccess) {
      set_last_error_text("decoder exchange allocation failed");
      mld_decoder_destroy(dec);
      return MLD_CUDA_ERROR;
    }
    cudaMemset(dec->xchg, 0, xo);
    cudaMemset(dec->peer_tickets, 0, 256);
    dec->xchg_peers[d->rank] = dec->xchg;
    dec->attn_full = reinterpret_cast<__half*>(dec->xchg + dec->off_attn);
    dec->h = reinterpret_cast<__half*>(dec->xchg + dec->off_h);
    dec->act_full = reinterpret_cast<__half*>(dec->xchg + dec->off_act);
    dec->o_full = reinterpret_cast<__half*>(dec->xchg + dec->off_xa);   // layer outputs ping-pong between
    dec->d_full = reinterpret_cast<__half*>(dec->xchg + dec->off_xb);   // these two
  }
  // a rank's shard of a gathered vector is written in place
  dec->attn_local = dec->attn_full + (size_t)d->rank * dec->d_local;
  dec->o_local = dec->o_full + (size_t)d->rank * dec->d_local;
  dec->act_local = dec->act_full + (size_t)d->rank * dec->ffn_local;
  if (d->world > 1 && nccl_id128 != nullptr) {
    if (!nccl().load()) {
      set_last_error_text("libnccl.so.2 could not be loaded");
      mld_decoder_destroy(dec);
      return MLD_NCCL_ERROR;
    }
    ncclUniqueId id;
    memcpy(&id, nccl_id128, sizeof id);
    const int nrc = nccl().CommInitRank(&dec->comm, d->world, id, d->rank);
    if (nrc != 0) {
      set_last_error_text(nccl().GetErrorString ? nccl().GetErrorString(nrc) : "ncclCommInitRank failed");
      dec->comm = nullptr;
      mld_decoder_destroy(dec);
      return MLD_NCCL_ERROR;
    }
  }
  // One GPU: run the step as one persistent kernel when the shape allows it, unless the descriptor asks
  // for the op chain.  A sharded decoder does so when asked to (mode MLD_DECODER_SINGLE_KERNEL) and created
  // without an NCCL id: its ranks exchange shards with peer stores, see mld_decoder_ipc_export.
  const bool forced = d->mode == MLD_DECODER_SINGLE_KERNEL;
  const bool want_mega = d->world == 1 ? d->mode != MLD_DECODER_OP_CHAIN : (forced && nccl_id128 == nullptr);
  if (want_mega) {
    MegaConfig mc = {d->layers, d->d_model, d->heads, d->head_dim, d->ffn, d->max_seq, d->block,
                     d->rms_eps, d->rope_min_timescale, d->rope_max_timescale, device, d->rank, d->world,
                     d->shard_layout, d->handover, d->grid_limit, d->ring_stages, d->wait_limit_us};
    if (mega_supported(mc)) {
      const int mrc = mega_create(mc, &dec->mega);
      if (mrc != MLD_OK) {
        dec->mega = nullptr;
        if (forced) {
          mld_decoder_destroy(dec);
          return mrc;
        }
      }
    } else if (forced) {
      set_last_error_text("decoder shape not supported by the single-kernel decoder");
      mld_decoder_destroy(dec);
      return MLD_UNIMPLEMENTED;
    }
  }
  if (d->world > 1 && d->shard_layout != 0 && dec->mega == nullptr) {
    set_last_error_text("shard_layout 1 (o and down split by input columns) needs the single-kernel decoder: "
                        "mode MLD_DECODER_SINGLE_KERNEL and no NCCL id");
    mld_decoder_destroy(dec);
    return MLD_UNIMPLEMENTED;
  }
  *out = dec;
  return MLD_OK;
}

int mld_decoder_destroy(mld_decoder* dec) {
  if (dec == nullptr) return MLD_OK;
  if (dec->comm != nullptr && nccl().CommDestroy) nccl().CommDestroy(dec->comm);
  mld_fc_plan_destroy(dec->p_qkv);
  mld_fc_plan_destroy(dec->p_o);
  mld_fc_plan_destroy(dec->p_gu);
  mld_fc_plan_destroy(dec->p_down);
  if (dec->scratch != nullptr) cudaFree(dec->scratch);
  if (dec->mega != nullptr) mega_destroy(dec->mega);
  for (int r = 0; r < 8; ++r)
    if (dec->xchg_peers[r] != nullptr && dec->xchg_peers[r] != dec->xchg) cudaIpcCloseMemHandle(dec->xchg_peers[r]);
  if (dec->xchg != nullptr) cudaFree(dec->xchg);
  if (dec->peer_tickets != nullptr) cudaFree(dec->peer_tickets);
  if (dec->error != nullptr) cudaFree(dec->error);
  if (dec->error_host != nullptr) cudaFreeHost(dec->error_host);
  delete dec;
  return MLD_OK;
}

int mld_decoder_ipc_export(mld_decoder* dec, void* handle64) {
  MLD_REQUIRE(dec != nullptr && handle64 != nullptr, "null argument");
  if (dec->mega != nullptr && dec->d.world > 1) return mega_ipc_export(dec->mega, handle64);
  MLD_REQUIRE(dec->xchg != nullptr, "a single-rank decoder has nothing to share");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  MLD_CUDA_CHECK(cudaIpcGetMemHandle(&h, dec->xchg));
  memcpy(handle64, &h, sizeof h);
  return MLD_OK;
}

int mld_decoder_ipc_import(mld_decoder* dec, const void* handles) {
  MLD_REQUIRE(dec != nullptr && handles != nullptr, "null argument");
  if (dec->mega != nullptr && dec->d.world > 1) return mega_ipc_import(dec->mega, handles);
  MLD_REQUIRE(dec->xchg != nullptr, "a single-rank decoder has no peers");
  for (int r = 0; r < dec->d.world; ++r) {
    if (r == dec->d.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * 64, sizeof h);
    void* p = nullptr;
    MLD_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    dec->xchg_peers[r] = static_cast<uint8_t*>(p);
  }
  dec->peer_mode = true;
  return MLD_OK;
}

size_t mld_decoder_scratch_bytes(const mld_decoder* dec) { return dec ? dec->scratch_bytes : 0; }

int mld_decoder_set_layer(mld_decoder* dec, int32_t layer, const mld_layer_weights* w) {
  MLD_REQUIRE(dec != nullptr && w != nullptr, "null argument");
  MLD_REQUIRE(layer >= 0 && layer < dec->d.layers, "layer index out of range");
  MLD_REQUIRE(w->wqkv && w->sqkv && w->wo && w->so && w->wgu && w->sgu && w->wdown && w->sdown && w->norm1 &&
                  w->norm2 && w->kcache && w->vcache,
              "missing layer tensor");
  dec->layers[layer] = *w;
  if (dec->mega != nullptr) {
    MegaLayerPtrs p = {w->wqkv, w->sqkv, w->wo, w->so, w->wgu, w->sgu, w->wdown, w->sdown,
                       w->norm1, w->norm2, w->kcache, w->vcache};
    return mega_set_layer(dec->mega, layer, p);
  }
  return MLD_OK;
}

int mld_decoder_is_single_kernel(const mld_decoder* dec) { return dec != nullptr && dec->mega != nullptr ? 1 : 0; }

#ifdef MLD_TRACE
// Tuning aids, compiled only with -DMLD_TRACE: per-CTA timestamps of the persistent step kernel.
__attribute__((visibility("default"))) int mld_debug_decoder_trace(mld_decoder* dec, int on) {
  if (dec == nullptr || dec->mega == nullptr) return MLD_INVALID_ARGUMENT;
  return mega_enable_trace(dec->mega, on != 0);
}
__attribute__((visibility("default"))) int mld_debug_decoder_read_trace(mld_decoder* dec, unsigned long long* out,
                                                                        size_t count) {
  if (dec == nullptr || dec->mega == nullptr) return MLD_INVALID_ARGUMENT;
  return mega_read_trace(dec->mega, out, count);
}
__attribute__((visibility("default"))) int mld_debug_decoder_grid(mld_decoder* dec) {
  return dec != nullptr && dec->mega != nullptr ? mega_grid(dec->mega) : 0;
}
#endif

int mld_decoder_device_status(mld_decoder* dec, int32_t* code) {
  MLD_REQUIRE(dec != nullptr && code != nullptr, "null argument");
  *code = 0;
  int c = 0;
  if (dec->mega != nullptr) {
    const int rc = mega_device_status(dec->mega, &c);
    if (rc != MLD_OK) return rc;
  } else {
    // the op chain: one word shared by its FullyConnected plans and glue kernels
    MLD_CUDA_CHECK(cudaMemcpy(&c, dec->error, sizeof(int), cudaMemcpyDeviceToHost));
    if (c != 0) {
      const int rc = mld_decoder_reset(dec);
      if (rc != MLD_OK) return rc;
    }
  }
  *code = c;
  if (c != 0) {
    set_last_error_text("a bounded device-side wait of the decode step gave up");
    return MLD_TIMEOUT;
  }
  return MLD_OK;
}

int mld_decoder_reset(mld_decoder* dec) {
  MLD_REQUIRE(dec != nullptr, "null argument");
  MLD_CUDA_CHECK(cudaSetDevice(dec->d.device));
  if (dec->mega != nullptr) return mega_reset(dec->mega);
  MLD_CUDA_CHECK(cudaMemset(dec->error, 0, sizeof(int)));
  MLD_CUDA_CHECK(cudaMemset(dec->tickets, 0, (size_t)dec->heads_local * 4));
  if (dec->peer_tickets != nullptr) MLD_CUDA_CHECK(cudaMemset(dec->peer_tickets, 0, 5 * sizeof(int)));
  if (dec->xchg != nullptr) MLD_CUDA_CHECK(cudaMemset(dec->xchg + dec->off_flags, 0, 4 * 8 * sizeof(unsigned)));
  MLD_CUDA_CHECK(cudaDeviceSynchronize());
  return MLD_OK;
}

int mld_decoder_set_wait_limit(mld_decoder* dec, int32_t wait_limit_us) {
  MLD_REQUIRE(dec != nullptr && wait_limit_us >= 0, "bad argument");
  dec->d.wait_limit_us = wait_limit_us;
  dec->wait_limit_ns = static_cast<unsigned long long>(wait_limit_us > 0 ? wait_limit_us : 2000000) * 1000ull;
  if (dec->mega != nullptr) mega_set_wait_limit(dec->mega, wait_limit_us);
  return MLD_OK;
}

int mld_decoder_step(mld_decoder* dec, const void* x_in, void* x_out, int32_t pos, void* stream_v) {
  MLD_REQUIRE(dec != nullptr && x_in != nullptr && x_out != nullptr, "null argument");
  MLD_REQUIRE(pos >= 0 && pos < dec->d.max_seq, "position beyond the KV cache");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  if (dec->mega != nullptr) return mega_step(dec->mega, x_in, x_out, pos, stream);
  const mld_decoder_desc& d = dec->d;
  const int dm = d.d_model, Hl = dec->heads_local, dl = dm / d.world, fl = dec->ffn_local;
  const float q_scale = 1.0f / sqrtf(static_cast<float>(d.head_dim));
  // Per layer (x = layer input, all vectors fp16):
  //   xn = rmsnorm(x) g1;  qkv = Wqkv xn;  attn = attention(rope(q), cache + rope(k), v)
  //   h  = x + Wo attn            (residual added in the projection's dst write)
  //   hn = rmsnorm(h) g2;  act = silu(Wg hn) * (Wu hn)   (fused into the projection's dst write)
  //   x' = h + Wdown act
  // Sharded: attn, h, act and x' are assembled from every rank's shard, either by an NCCL
  // all-gather after the producing kernel or, in peer mode, by the producing kernel itself.
  const bool peer = d.world > 1 && dec->peer_mode;
  MLD_REQUIRE(d.world == 1 || peer || dec->comm != nullptr, "sharded decoder has neither peers nor an NCCL communicator");
  enum { kAttn = 0, kH = 1, kAct = 2, kX = 3 };
  auto scatter_of = [&](int kind, int layer, size_t vec_off, size_t shard_halves) {
    PeerScatter sc;
    memset(&sc, 0, sizeof sc);
    if (!peer) return sc;
    sc.world = d.world;
    for (int r = 0; r < d.world; ++r) {
      sc.y_peers[r] = dec->xchg_peers[r] + vec_off + (size_t)d.rank * shard_halves * 2;
      sc.flag_peers[r] = reinterpret_cast<unsigned*>(dec->xchg_peers[r] + dec->off_flags) + kind * 8 + d.rank;
    }
    sc.ticket = dec->peer_tickets + kind;
    sc.step = dec->peer_tickets + 4;
    sc.seq_off = 4 * layer + kind + 1;
    sc.seq_per_step = 4 * d.layers;
    return sc;
  };
  auto wait_of = [&](int kind, int layer) {
    PeerWait pw;
    memset(&pw, 0, sizeof pw);
    if (!peer || layer < 0) return pw;
    pw.world = d.world;
    pw.flags = reinterpret_cast<const unsigned*>(dec->xchg + dec->off_flags) + kind * 8;
    pw.step = dec->peer_tickets + 4;
    pw.seq_off = 4 * layer + kind + 1;
    pw.seq_per_step = 4 * d.layers;
    pw.error = dec->error;
    pw.limit_ns = dec->wait_limit_ns;
    return pw;
  };
  const __half* x = static_cast<const __half*>(x_in);
  int rc;
  if (peer) {
    rc = launch_glue(bump_step_kernel, dim3(1), dim3(1), stream, dec->peer_tickets + 4);
    if (rc != MLD_OK) return rc;
  }
  for (int l = 0; l < d.layers; ++l) {
    const mld_layer_weights& w = dec->layers[l];
    MLD_REQUIRE(w.wqkv != nullptr, "layer weights not set");
    const bool last = l + 1 == d.layers;
    // the layer's output vector: the caller's buffer for the last layer (peers cannot write there, so
    // peer mode copies it out at the end), else a ping-pong pair
    __half* x_next = (last && !peer) ? static_cast<__half*>(x_out) : ((l & 1) ? dec->d_full : dec->o_full);
    const size_t off_x_next = (l & 1) ? dec->off_xb : dec->off_xa;
    rc = launch_glue(add_rmsnorm_kernel, dim3(1), dim3(1024), stream, x, static_cast<const __half*>(nullptr),
                     static_cast<const __half*>(w.norm1), static_cast<__half*>(nullptr), dec->xn, dm, d.rms_eps,
                     wait_of(kX, l - 1));
    if (rc != MLD_OK) return rc;
    if (dec->prefetch) mld_fc_plan_prefetch_next(dec->p_qkv, w.wo, dec->bytes_o);
    rc = mld_fc_run(dec->p_qkv, dec->xn, w.wqkv, w.sqkv, nullptr, nullptr, dec->qkv, 1, stream);
    if (rc != MLD_OK) return rc;
    {
      AttnStepArgs aa;
      aa.qkv = dec->qkv;
      aa.kcache = static_cast<__half*>(w.kcache);
      aa.vcache = static_cast<__half*>(w.vcache);
      aa.part_o = dec->part_o;
      aa.part_ml = dec->part_ml;
      aa.tickets = dec->tickets;
      aa.out = dec->attn_local;
      aa.heads = Hl;
      aa.pos = pos;
      aa.splits = dec->splits;
      aa.min_ts = d.rope_min_timescale;
      aa.max_ts = d.rope_max_timescale;
      aa.q_scale = q_scale;
      aa.scatter = scatter_of(kAttn, l, dec->off_attn, dl);
      rc = launch_glue(attn_step_kernel, dim3(Hl, dec->splits), dim3(128), stream, aa);
      if (rc != MLD_OK) return rc;
    }
    if (!peer && (rc = gather(dec, dec->attn_local, dec->attn_full, dl, stream)) != MLD_OK) return rc;
    // h shard = x shard + Wo attn
    __half* h_local = dec->h + (size_t)d.rank * dl;
    {
      const PeerScatter sc = scatter_of(kH, l, dec->off_h, dl);
      const PeerWait pw = wait_of(kAttn, l);
      if (dec->prefetch) mld_fc_plan_prefetch_next(dec->p_o, w.wgu, dec->bytes_gu);
      rc = fc_run_internal(dec->p_o, dec->attn_full, w.wo, w.so, nullptr, x + (size_t)d.rank * dl, h_local, 1, stream,
                           peer ? &sc : nullptr, peer ? &pw : nullptr);
      if (rc != MLD_OK) return rc;
    }
    if (!peer && (rc = gather(dec, h_local, dec->h, dl, stream)) != MLD_OK) return rc;
    rc = launch_glue(add_rmsnorm_kernel, dim3(1), dim3(1024), stream, static_cast<const __half*>(dec->h),
                     static_cast<const __half*>(nullptr), static_cast<const __half*>(w.norm2),
                     static_cast<__half*>(nullptr), dec->hn, dm, d.rms_eps, wait_of(kH, l));
    if (rc != MLD_OK) return rc;
    {
      const PeerScatter sc = scatter_of(kAct, l, dec->off_act, fl);
      if (dec->prefetch) mld_fc_plan_prefetch_next(dec->p_gu, w.wdown, dec->bytes_down);
      rc = fc_run_internal(dec->p_gu, dec->hn, w.wgu, w.sgu, nullptr, nullptr, dec->act_local, 1, stream,
                           peer ? &sc : nullptr, nullptr);
      if (rc != MLD_OK) return rc;
    }
    if (!peer && (rc = gather(dec, dec->act_local, dec->act_full, fl, stream)) != MLD_OK) return rc;
    __half* xn_local = x_next + (size_t)d.rank * dl;
    {
      const PeerScatter sc = scatter_of(kX, l, off_x_next, dl);
      const PeerWait pw = wait_of(kAct, l);
      if (dec->prefetch && !last) mld_fc_plan_prefetch_next(dec->p_down, dec->layers[l + 1].wqkv, dec->bytes_qkv);
      rc = fc_run_internal(dec->p_down, dec->act_full, w.wdown, w.sdown, nullptr, dec->h + (size_t)d.rank * dl, xn_local,
                           1, stream, peer ? &sc : nullptr, peer ? &pw : nullptr);
      if (rc != MLD_OK) return rc;
    }
    if (!peer && (rc = gather(dec, xn_local, x_next, dl, stream)) != MLD_OK) return rc;
    x = x_next;
  }
  if (peer) {
    rc = launch_glue(copy_after_wait_kernel, dim3(4), dim3(256), stream, x, static_cast<__half*>(x_out), dm,
                     wait_of(kX, d.layers - 1));
    if (rc != MLD_OK) return rc;
  }
  return MLD_OK;
}

int mld_decoder_step_host(mld_decoder* dec, const void* x_host, void* y_host, int32_t pos, void* stream_v) {
  MLD_REQUIRE(dec != nullptr && x_host != nullptr && y_host != nullptr, "null argument");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  const size_t bytes = static_cast<size_t>(dec->d.d_model) * 2;
  MLD_CUDA_CHECK(cudaMemcpyAsync(dec->x_stage, x_host, bytes, cudaMemcpyHostToDevice, stream));
  const int rc = mld_decoder_step(dec, dec->x_stage, dec->y_stage, pos, stream);
  if (rc != MLD_OK) return rc;
  MLD_CUDA_CHECK(cudaMemcpyAsync(y_host, dec->y_stage, bytes, cudaMemcpyDeviceToHost, stream));
  // the step's status word travels behind the result in the same stream
  const int* status = dec->mega != nullptr ? mega_error_word(dec->mega) : dec->error;
  MLD_CUDA_CHECK(cudaMemcpyAsync(dec->error_host, status, sizeof(int), cudaMemcpyDeviceToHost, stream));
  MLD_CUDA_CHECK(cudaStreamSynchronize(stream));
  if (*dec->error_host != 0) {
    set_last_error_text("a bounded device-side wait of the decode step gave up");
    return MLD_TIMEOUT;
  }
  return MLD_OK;
}

}  // extern "C"
