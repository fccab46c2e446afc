// One persistent kernel for a whole decode step of the INT4 decoder.
//
// The op-by-op decoder spends most of a step between kernels: every
// projection drains its TMA pipeline, the next one fills it again, and the
// weights of a projection (8-45 MB) stream for only a few microseconds.  Here
// one cooperative grid of one CTA per SM runs all layers:
//   * a producer thread per CTA walks the step's whole list of weight and
//     KV-cache tiles this CTA will need, in order, and keeps a ~185 KB ring of
//     TMA boxes full.  Nothing it loads depends on the step's activations, so
//     it runs ahead across op and layer boundaries: HBM stays busy while the
//     consumers finish an op, cross the grid barrier and load the next input
//     vector;
//   * eight consumer warps per CTA do the arithmetic of every op:
//       qkv  = Wqkv rmsnorm(x) g1                 (RMSNorm fused into the vector load)
//       attn = softmax(rope(q) K^T) V             (new k/v roped, written to the cache)
//       h    = x + Wo attn
//       act  = silu(Wg hn) * (Wu hn), hn = rmsnorm(h) g2
//       x'   = h + Wdown act
//     with a grid barrier after each (five per layer);
//   * work is split in items of one TMA box: a projection's (64-output column,
//     64-k-slice stage) tiles, attention's (head, 32-token tile) pairs.  Every
//     CTA takes a contiguous, balanced range of an op's items.  A column (or
//     head) shared between CTAs is completed by whichever of them finishes
//     last (a ticket); it sums the partial results in CTA order, so results do
//     not depend on arrival order.
//
// Projection arithmetic is the streaming GEMV's (gemv_stream.cu): weights as
// the MMA A operand straight from the packed INT4 bytes (fp16 subnormals),
// fp32 accumulation, one scale multiply per 32-input block.  Restated from
// GetFullyConnectedKernelCode (ml_drift/common/kernels/fully_connected.cc:623-942)
// and the decoder graph of samples/llm/qwen3_model_builder.cc:880-1017.
//
// Every wait (ring barriers, grid barrier) is bounded; when one runs out the
// CTA records an error code, stops waiting and runs to the end.
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace mld {

namespace {

constexpr int kCW = 8;                       // consumer warps
constexpr int kThreads = (kCW + 1) * 32;     // + one producer warp
constexpr int kRows = 64;                    // k-slices (of 4 inputs) per weight box
constexpr int kBox = kRows * 128;            // weight box: 64 rows x 128 bytes = 64 outputs x 256 inputs
constexpr int kScaleBox = 1024;              // up to 8 scale rows x 64 outputs x fp16
constexpr int kStageBytes = kBox + kScaleBox;
constexpr int kHeadDim = 128;
constexpr int kTile = 32;                    // cached tokens per attention item (K box, V box: 8 KB each)
constexpr int kAttSlots = 4;                 // heads a CTA's attention range can touch
constexpr float kOutScale = 16777216.0f;     // subnormal operands carry 2^-24

constexpr int kTraceSlots = 6;                // per (CTA, op): 4 timestamps, wait clocks, stages
enum { kQkv = 0, kAttn = 1, kO = 2, kGu = 3, kDown = 4, kOpsPerLayer = 5 };

struct alignas(128) MegaLayer {
  CUtensorMap w[4];   // weights of qkv, o, gu, down: bytes [K/4][2N], box 128 B x 64 rows, 128B swizzle
  CUtensorMap s[4];   // scales: fp16 [K/block][N], box 64 x (256/block) rows
  CUtensorMap kc, vc; // KV cache: fp16 [max_seq][heads*128], box 128 x 32 rows
  const __half* norm1;
  const __half* norm2;
  __half* kcache;
  __half* vcache;
};

struct MegaArgs {
  const MegaLayer* layers;
  int n_layers, d_model, heads, ffn, pos;
  int gs_shift;        // log2(k-slices per scale block)
  int stages;          // ring depth
  int xs_bytes;        // shared-memory bytes of the input-vector / attention area
  float rms_eps, min_ts, max_ts, q_scale;
  const __half* x_in;
  __half* x_out;
  __half *qkv, *attn, *h, *act, *xa, *xb;
  float* col_part;     // [grid][2][64]
  int* col_tickets;    // [max columns]
  float* att_part;     // [grid][kAttSlots][2 + 128]
  int* att_tickets;    // [heads]
  unsigned* bar;       // [0] arrivals, [1] generation
  int* error;
  unsigned long long* trace;  // optional [grid][ops][kTraceSlots]
};

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory"); }
__device__ __forceinline__ void bar64() { asm volatile("bar.sync 3, 64;" ::: "memory"); }
__device__ __forceinline__ void bar128() { asm volatile("bar.sync 4, 128;" ::: "memory"); }

// Per-CTA state shared by all waits: once any wait of this CTA has run out,
// no later wait blocks.
struct Waiter {
  volatile int* s_fail;
  int* error;
  __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, int code) const {
    if (mbar_try_wait(bar, parity)) return true;
    if (*s_fail) return false;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
      for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
      if (*s_fail) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        *s_fail = 1;
        atomicExch(error, code);
        return false;
      }
    }
  }
};

// Balanced contiguous split of `items` over the grid.
__device__ __forceinline__ int range_start(int cta, int items, int grid) {
  return static_cast<int>((int64_t)cta * items / grid);
}
__device__ __forceinline__ int owner_of(int item, int items, int grid) {
  return static_cast<int>((((int64_t)item + 1) * grid - 1) / items);
}

struct ProjShape {
  int N, K4, C, S, I;
};
__device__ __forceinline__ ProjShape proj_shape(const MegaArgs& a, int kind) {
  ProjShape p;
  const int d = a.d_model;
  p.N = kind == kQkv ? 3 * d : kind == kGu ? 2 * a.ffn : d;
  p.K4 = (kind == kDown ? a.ffn : d) >> 2;
  p.C = (p.N + 63) >> 6;
  p.S = (p.K4 + kRows - 1) / kRows;
  p.I = p.C * p.S;
  return p;
}
__device__ __forceinline__ int map_index(int kind) { return kind == kQkv ? 0 : kind == kO ? 1 : kind == kGu ? 2 : 3; }

// ------------------------------------------------------------------ producer
struct Ring {
  int stage;
  uint32_t phase;
  __device__ __forceinline__ void advance(int stages) {
    if (++stage == stages) {
      stage = 0;
      phase ^= 1;
    }
  }
};

__device__ void producer_loop(const MegaArgs& a, uint8_t* ring, uint64_t* full, uint64_t* empty, const Waiter& w) {
  const int cta = blockIdx.x, G = gridDim.x;
  const uint64_t pol = policy_evict_first();
  Ring r{0, 0};
  const int sr = kRows >> a.gs_shift;  // scale rows per box
  const uint32_t proj_bytes = kBox + static_cast<uint32_t>(sr) * 128u;
  const int nt = a.pos / kTile + 1;
  for (int l = 0; l < a.n_layers; ++l) {
    const MegaLayer* ly = a.layers + l;
    for (int kind = 0; kind < kOpsPerLayer; ++kind) {
      if (kind == kAttn) {
        const int I = a.heads * nt;
        const int i0 = range_start(cta, I, G), i1 = range_start(cta + 1, I, G);
        for (int i = i0; i < i1; ++i) {
          const int head = i / nt, j = i - head * nt;
          for (int kv = 0; kv < 2; ++kv) {
            w.wait(&empty[r.stage], r.phase ^ 1, 10);
            uint8_t* st = ring + (size_t)r.stage * kStageBytes;
            mbar_arrive_expect_tx(&full[r.stage], kBox);
            tma_load_2d_hint(st, kv == 0 ? &ly->kc : &ly->vc, &full[r.stage], head * kHeadDim, j * kTile, pol);
            r.advance(a.stages);
          }
        }
      } else {
        const ProjShape p = proj_shape(a, kind);
        const int mi = map_index(kind);
        const int i0 = range_start(cta, p.I, G), i1 = range_start(cta + 1, p.I, G);
        int col = i0 / p.S, ks = i0 - col * p.S;
        for (int i = i0; i < i1; ++i) {
          w.wait(&empty[r.stage], r.phase ^ 1, 11);
          uint8_t* st = ring + (size_t)r.stage * kStageBytes;
          mbar_arrive_expect_tx(&full[r.stage], proj_bytes);
          tma_load_2d_hint(st, &ly->w[mi], &full[r.stage], col * 128, ks * kRows, pol);
          tma_load_2d_hint(st + kBox, &ly->s[mi], &full[r.stage], col * 64, ks * sr, pol);
          r.advance(a.stages);
          if (++ks == p.S) {
            ks = 0;
            ++col;
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------ consumers
struct Ctx {
  const MegaArgs& a;
  uint8_t* ring;
  uint64_t* full;
  uint64_t* empty;
  __half* xs;      // input vector of the running projection / attention scratch
  float* red;      // [2][kCW][64]
  int* s_int;      // [0] = "this CTA completes the column / head"
  Waiter w;
  Ring r;
  unsigned gen;    // grid-barrier generation this CTA waits for next
  int red_buf;
  int op_index;
};

__device__ __forceinline__ void trace_mark(const Ctx& c, int k) {
  if (c.a.trace != nullptr && threadIdx.x == 0)
    c.a.trace[((size_t)blockIdx.x * c.a.n_layers * kOpsPerLayer + c.op_index) * kTraceSlots + k] = globaltimer_ns();
}

// All consumer threads call this after their last global write of an op.
__device__ void grid_barrier(Ctx& c) {
  consumer_bar();
  if (threadIdx.x == 0) {
    __threadfence();
    unsigned* cnt = c.a.bar;
    unsigned* gen = c.a.bar + 1;
    const unsigned old = atomicAdd(cnt, 1u);
    if (old == gridDim.x - 1) {
      atomicExch(cnt, 0u);
      __threadfence();
      atomicAdd(gen, 1u);
    }
    const unsigned want = c.gen + 1;
    if (!*c.w.s_fail) {
      const unsigned long long t0 = globaltimer_ns();
      while (static_cast<int>(ld_acquire_gpu(gen) - want) < 0) {
        if (globaltimer_ns() - t0 > kWaitLimitNs || *reinterpret_cast<volatile int*>(c.a.error) != 0) {
          *c.w.s_fail = 1;
          atomicCAS(c.a.error, 0, 20);
          break;
        }
      }
    }
  }
  c.gen += 1;
  consumer_bar();
}

// xs = fp16(v * rsqrt(mean(v^2) + eps) * gamma)   (reference RMSNorm, fp32 statistics)
__device__ void load_x_norm(Ctx& c, const __half* x, const __half* gamma, int d) {
  float ss = 0.0f;
  for (int i = threadIdx.x * 8; i < d; i += kCW * 32 * 8) {
    const uint4 v = __ldcg(reinterpret_cast<const uint4*>(x + i));
    *reinterpret_cast<uint4*>(c.xs + i) = v;
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      ss += f.x * f.x + f.y * f.y;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  float* part = c.red + 2 * kCW * 64;  // 8 floats after the reduction buffers
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
  consumer_bar();
  float tot = 0.0f;
#pragma unroll
  for (int wi = 0; wi < kCW; ++wi) tot += part[wi];
  const float inv = rsqrtf(tot / static_cast<float>(d) + c.a.rms_eps);
  for (int i = threadIdx.x * 8; i < d; i += kCW * 32 * 8) {
    uint4 v = *reinterpret_cast<uint4*>(c.xs + i);
    const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gamma + i));
    __half2* h = reinterpret_cast<__half2*>(&v);
    const __half2* gh = reinterpret_cast<const __half2*>(&gv);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      const float2 g = __half22float2(gh[j]);
      h[j] = __floats2half2_rn(f.x * inv * g.x, f.y * inv * g.y);
    }
    *reinterpret_cast<uint4*>(c.xs + i) = v;
  }
  consumer_bar();
}
__device__ void load_x_plain(Ctx& c, const __half* x, int d) {
  for (int i = threadIdx.x * 8; i < d; i += kCW * 32 * 8)
    *reinterpret_cast<uint4*>(c.xs + i) = __ldcg(reinterpret_cast<const uint4*>(x + i));
  consumer_bar();
}

// Threads 0..63 (warps 0 and 1): value `v` of output col*64 + tid summed over
// this CTA's k-stages [ks0, ks1) of the column.
__device__ void finish_column(Ctx& c, int kind, const ProjShape& p, int col, int ks0, int ks1, float v, int i0,
                              const __half* resid, __half* out) {
  const MegaArgs& a = c.a;
  const int tid = threadIdx.x, G = gridDim.x, cta = blockIdx.x;
  if (!(ks0 == 0 && ks1 == p.S)) {
    const int slot = col == i0 / p.S ? 0 : 1;
    a.col_part[((size_t)cta * 2 + slot) * 64 + tid] = v;
    __threadfence();
    bar64();
    const int first = owner_of(col * p.S, p.I, G), last = owner_of(col * p.S + p.S - 1, p.I, G);
    if (tid == 0) {
      int need = 0;  // CTAs between first and last whose range is not empty (grids larger than the item count)
      for (int cc = first; cc <= last; ++cc) need += range_start(cc, p.I, G) != range_start(cc + 1, p.I, G) ? 1 : 0;
      const int t = atomicAdd(a.col_tickets + col, 1);
      const int done = t == need - 1 ? 1 : 0;
      if (done) a.col_tickets[col] = 0;
      c.s_int[0] = done;
    }
    bar64();
    const int done = c.s_int[0];
    bar64();  // s_int may be rewritten by the next column
    if (!done) return;
    __threadfence();
    v = 0.0f;
    for (int cc = first; cc <= last; ++cc) {
      const int c0 = range_start(cc, p.I, G);
      if (c0 == range_start(cc + 1, p.I, G)) continue;
      const int sc = col == c0 / p.S ? 0 : 1;
      v += __ldcg(a.col_part + ((size_t)cc * 2 + sc) * 64 + tid);
    }
  }
  const int n = col * 64 + tid;
  const __half r = __float2half_rn(v * kOutScale);
  if (kind == kGu) {
    // rows interleave gate_i, up_i: even lanes hold the gate, the next lane its up value
    const float gf = __half2float(r);
    const float uf = __shfl_down_sync(0xffffffffu, gf, 1);
    if ((tid & 1) == 0 && n + 1 < p.N) out[n >> 1] = __float2half_rn(gf / (1.0f + __expf(-gf)) * uf);
  } else if (n < p.N) {
    out[n] = resid != nullptr ? __hadd(r, __ldcg(resid + n)) : r;
  }
}

__device__ void run_projection(Ctx& c, int kind, const __half* resid, __half* out) {
  const MegaArgs& a = c.a;
  const ProjShape p = proj_shape(a, kind);
  const int cta = blockIdx.x, G = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int rbase = warp * 8;
  const int gidx = rbase >> a.gs_shift;
  const int i0 = range_start(cta, p.I, G), i1 = range_start(cta + 1, p.I, G);
  int i = i0;
  long long waited = 0;
  const bool tracing = a.trace != nullptr && threadIdx.x == 0;
  while (i < i1) {
    const int col = i / p.S, ks0 = i - col * p.S;
    const int ks1 = min(p.S, ks0 + (i1 - i));
    float tot[4][2];
#pragma unroll
    for (int f = 0; f < 4; ++f) tot[f][0] = tot[f][1] = 0.0f;
    for (int ks = ks0; ks < ks1; ++ks) {
      const long long w0 = tracing ? clock64() : 0;
      c.w.wait(&c.full[c.r.stage], c.r.phase, 12);
      if (tracing) waited += clock64() - w0;
      const uint8_t* st = c.ring + (size_t)c.r.stage * kStageBytes;
      const int row0 = ks * kRows;
      uint32_t bx[2][2];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int row = row0 + rbase + 2 * t + q;
        bx[q][0] = bx[q][1] = 0u;
        if (g == 0 && row < p.K4) {
          const uint2 xv = *reinterpret_cast<const uint2*>(c.xs + (size_t)row * 4);
          bx[q][0] = xv.x;
          bx[q][1] = xv.y;
        }
      }
      // sum of the inputs times the nibble offset 8, as the same subnormal product
      float ones[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      {
        const uint32_t oa[4] = {0x00080008u, 0x00080008u, 0x00080008u, 0x00080008u};
        mma_f16(ones, oa, bx[0][0], bx[0][1]);
        mma_f16(ones, oa, bx[1][0], bx[1][1]);
      }
      float grp[4][4];
#pragma unroll
      for (int f = 0; f < 4; ++f) grp[f][0] = grp[f][1] = grp[f][2] = grp[f][3] = 0.0f;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int r = rbase + 2 * t + q;
        const uint4 wv = *reinterpret_cast<const uint4*>(st + r * 128 + ((g ^ (r & 7)) << 4));
        const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
#pragma unroll
        for (int b = 0; b < 2; ++b) {
          const uint32_t lo = ww[2 * b], hi = ww[2 * b + 1];
          const uint32_t lo8 = lo >> 8, hi8 = hi >> 8;
          const uint32_t a0[4] = {lo & 0x000F000Fu, lo & 0x00F000F0u, hi & 0x000F000Fu, hi & 0x00F000F0u};
          const uint32_t a1[4] = {lo8 & 0x000F000Fu, lo8 & 0x00F000F0u, hi8 & 0x000F000Fu, hi8 & 0x00F000F0u};
          mma_f16(grp[2 * b], a0, bx[q][0], bx[q][1]);
          mma_f16(grp[2 * b + 1], a1, bx[q][0], bx[q][1]);
        }
      }
      // scales of this lane's eight outputs for the block these eight rows are in
      const uint4 sv = *reinterpret_cast<const uint4*>(st + kBox + (gidx * 64 + 8 * g) * 2);
      const __half2* sh = reinterpret_cast<const __half2*>(&sv);
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const float2 s2 = __half22float2(sh[f]);
        // MMA row g = output 2f (low nibbles), row g+8 = output 2f+1 (high nibbles, carried x16)
        tot[f][0] = fmaf(s2.x, grp[f][0] - ones[0], tot[f][0]);
        tot[f][1] = fmaf(s2.y, fmaf(grp[f][2], 0.0625f, -ones[0]), tot[f][1]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&c.empty[c.r.stage]);
      c.r.advance(a.stages);
    }
    // cross-warp sum of the column
    float* red = c.red + c.red_buf * (kCW * 64);
    c.red_buf ^= 1;
    if (t == 0) {
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        red[warp * 64 + 8 * g + 2 * f] = tot[f][0];
        red[warp * 64 + 8 * g + 2 * f + 1] = tot[f][1];
      }
    }
    consumer_bar();
    if (threadIdx.x < 64) {
      float v = 0.0f;
#pragma unroll
      for (int wi = 0; wi < kCW; ++wi) v += red[wi * 64 + threadIdx.x];
      finish_column(c, kind, p, col, ks0, ks1, v, i0, resid, out);
    }
    i += ks1 - ks0;
  }
  if (tracing) {
    unsigned long long* t = a.trace + ((size_t)blockIdx.x * a.n_layers * kOpsPerLayer + c.op_index) * kTraceSlots;
    t[4] = static_cast<unsigned long long>(waited);
    t[5] = static_cast<unsigned long long>(i1 - i0);
  }
}

// Attention over the cached tokens 0..pos-1 plus the new token.  Eight lanes
// share a cached token (16 dims each); each of the 32 eight-lane groups keeps a
// running max / sum / output over its rows of the tiles and the groups are
// merged when the CTA's run over a head ends.
__device__ void run_attention(Ctx& c, const MegaLayer* ly) {
  const MegaArgs& a = c.a;
  const int cta = blockIdx.x, G = gridDim.x, tid = threadIdx.x;
  const int lane = tid & 31;
  const int grp = tid >> 3, sub = tid & 7;
  const int nt = a.pos / kTile + 1;
  const int I = a.heads * nt;
  const int width = a.heads * kHeadDim;
  const int i0 = range_start(cta, I, G), i1 = range_start(cta + 1, I, G);
  float* sq = reinterpret_cast<float*>(c.xs);   // [128] rotated, scaled q
  float* skn = sq + kHeadDim;                   // [128] rotated new k (as stored: fp16 values)
  float* svn = skn + kHeadDim;                  // [128] new v
  float* gm = svn + kHeadDim;                   // [32]
  float* gl = gm + 32;                          // [32]
  float* go = gl + 32;                          // [32][128]
  const unsigned gmask = 0xFFu << (lane & 24);
  int i = i0;
  while (i < i1) {
    const int head = i / nt, j0 = i - head * nt;
    const int j1 = min(nt, j0 + (i1 - i));
    const bool owns_new = j1 == nt;
    consumer_bar();  // the previous head's merge has finished reading this scratch
    if (tid < kHeadDim / 2) {
      const int e = tid, half = kHeadDim / 2;
      const float fraction = 2.0f * e / static_cast<float>(kHeadDim);
      const float timescale = a.min_ts * powf(a.max_ts / a.min_ts, fraction);
      float sn, cs;
      sincosf(static_cast<float>(a.pos) / timescale, &sn, &cs);
      const __half* qp = a.qkv + (size_t)head * kHeadDim;
      const float q0 = __half2float(__ldcg(qp + e)), q1 = __half2float(__ldcg(qp + e + half));
      // rounded to fp16 where the unfused graph stores the rotated, scaled q
      sq[e] = __half2float(__float2half_rn((q0 * cs - q1 * sn) * a.q_scale));
      sq[e + half] = __half2float(__float2half_rn((q1 * cs + q0 * sn) * a.q_scale));
      if (owns_new) {
        const __half* kp = a.qkv + (size_t)(a.heads + head) * kHeadDim;
        const float k0 = __half2float(__ldcg(kp + e)), k1 = __half2float(__ldcg(kp + e + half));
        const __half r0 = __float2half_rn(k0 * cs - k1 * sn), r1 = __float2half_rn(k1 * cs + k0 * sn);
        __half* kc = ly->kcache + (size_t)a.pos * width + head * kHeadDim;
        kc[e] = r0;
        kc[e + half] = r1;
        skn[e] = __half2float(r0);
        skn[e + half] = __half2float(r1);
      }
    } else if (tid < kHeadDim && owns_new) {
      const int e = tid - kHeadDim / 2;
      const __half* vp = a.qkv + (size_t)(2 * a.heads + head) * kHeadDim;
      __half* vc = ly->vcache + (size_t)a.pos * width + head * kHeadDim;
      const __half v0 = __ldcg(vp + e), v1 = __ldcg(vp + e + kHeadDim / 2);
      vc[e] = v0;
      vc[e + kHeadDim / 2] = v1;
      svn[e] = __half2float(v0);
      svn[e + kHeadDim / 2] = __half2float(v1);
    }
    consumer_bar();
    // lane `sub` of a group owns dims 8*sub..+8 and 64+8*sub..+8
    float qv[16];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      qv[e] = sq[sub * 8 + e];
      qv[8 + e] = sq[64 + sub * 8 + e];
    }
    float m = -INFINITY, l = 0.0f, acc[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] = 0.0f;
    for (int j = j0; j < j1; ++j) {
      const int ks = c.r.stage;
      c.w.wait(&c.full[ks], c.r.phase, 13);
      c.r.advance(a.stages);
      const int vs = c.r.stage;
      c.w.wait(&c.full[vs], c.r.phase, 14);
      c.r.advance(a.stages);
      const int token = j * kTile + grp;
      if (token <= a.pos) {
        float kf[16], vf[16];
        if (token == a.pos) {
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            kf[e] = skn[sub * 8 + e];
            kf[8 + e] = skn[64 + sub * 8 + e];
            vf[e] = svn[sub * 8 + e];
            vf[8 + e] = svn[64 + sub * 8 + e];
          }
        } else {
          const uint8_t* kr = c.ring + (size_t)ks * kStageBytes + grp * 256 + sub * 16;
          const uint8_t* vr = c.ring + (size_t)vs * kStageBytes + grp * 256 + sub * 16;
          const uint4 k0 = *reinterpret_cast<const uint4*>(kr), k1 = *reinterpret_cast<const uint4*>(kr + 128);
          const uint4 v0 = *reinterpret_cast<const uint4*>(vr), v1 = *reinterpret_cast<const uint4*>(vr + 128);
          const __half2* kh0 = reinterpret_cast<const __half2*>(&k0);
          const __half2* kh1 = reinterpret_cast<const __half2*>(&k1);
          const __half2* vh0 = reinterpret_cast<const __half2*>(&v0);
          const __half2* vh1 = reinterpret_cast<const __half2*>(&v1);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 a0 = __half22float2(kh0[e]), a1 = __half22float2(kh1[e]);
            const float2 b0 = __half22float2(vh0[e]), b1 = __half22float2(vh1[e]);
            kf[2 * e] = a0.x; kf[2 * e + 1] = a0.y; kf[8 + 2 * e] = a1.x; kf[8 + 2 * e + 1] = a1.y;
            vf[2 * e] = b0.x; vf[2 * e + 1] = b0.y; vf[8 + 2 * e] = b1.x; vf[8 + 2 * e + 1] = b1.y;
          }
        }
        float s = 0.0f;
#pragma unroll
        for (int e = 0; e < 16; ++e) s = fmaf(qv[e], kf[e], s);
        s += __shfl_xor_sync(gmask, s, 1);
        s += __shfl_xor_sync(gmask, s, 2);
        s += __shfl_xor_sync(gmask, s, 4);
        const float m_new = fmaxf(m, s);
        const float corr = __expf(m - m_new), pw = __expf(s - m_new);
        l = l * corr + pw;
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] = fmaf(acc[e], corr, pw * vf[e]);
        m = m_new;
      }
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&c.empty[ks]);
        mbar_arrive(&c.empty[vs]);
      }
    }
    // merge the 32 groups
    if (sub == 0) {
      gm[grp] = m;
      gl[grp] = l;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      go[grp * kHeadDim + sub * 8 + e] = acc[e];
      go[grp * kHeadDim + 64 + sub * 8 + e] = acc[8 + e];
    }
    consumer_bar();
    if (tid < kHeadDim) {
      float M = -INFINITY;
#pragma unroll 8
      for (int q = 0; q < 32; ++q) M = fmaxf(M, gm[q]);
      float o = 0.0f, ls = 0.0f;
#pragma unroll 8
      for (int q = 0; q < 32; ++q) {
        const float wq = gm[q] == -INFINITY ? 0.0f : __expf(gm[q] - M);
        o = fmaf(wq, go[q * kHeadDim + tid], o);
        ls = fmaf(wq, gl[q], ls);
      }
      const int first = owner_of(head * nt, I, G), last = owner_of(head * nt + nt - 1, I, G);
      bool write = true;
      if (first != last) {
        const int slot = head - i0 / nt;
        float* mine = a.att_part + ((size_t)cta * kAttSlots + slot) * (2 + kHeadDim);
        mine[2 + tid] = o;
        if (tid == 0) {
          mine[0] = M;
          mine[1] = ls;
        }
        __threadfence();
        bar128();
        if (tid == 0) {
          int need = 0;
          for (int cc = first; cc <= last; ++cc) need += range_start(cc, I, G) != range_start(cc + 1, I, G) ? 1 : 0;
          const int tk = atomicAdd(a.att_tickets + head, 1);
          const int done = tk == need - 1 ? 1 : 0;
          if (done) a.att_tickets[head] = 0;
          c.s_int[1] = done;
        }
        bar128();
        write = c.s_int[1] != 0;
        bar128();
        if (write) {
          __threadfence();
          float TM = -INFINITY;
          for (int cc = first; cc <= last; ++cc) {
            const int c0 = range_start(cc, I, G);
            if (c0 == range_start(cc + 1, I, G)) continue;
            const int sc = head - c0 / nt;
            TM = fmaxf(TM, __ldcg(a.att_part + ((size_t)cc * kAttSlots + sc) * (2 + kHeadDim)));
          }
          o = 0.0f;
          ls = 0.0f;
          for (int cc = first; cc <= last; ++cc) {
            const int c0 = range_start(cc, I, G);
            if (c0 == range_start(cc + 1, I, G)) continue;
            const int sc = head - c0 / nt;
            const float* pp = a.att_part + ((size_t)cc * kAttSlots + sc) * (2 + kHeadDim);
            const float mc = __ldcg(pp);
            const float wc = mc == -INFINITY ? 0.0f : __expf(mc - TM);
            o = fmaf(wc, __ldcg(pp + 2 + tid), o);
            ls = fmaf(wc, __ldcg(pp + 1), ls);
          }
        }
      }
      if (write) a.attn[(size_t)head * kHeadDim + tid] = __float2half_rn(o / ls);
    }
    i += j1 - j0;
  }
}

__global__ void __launch_bounds__(kThreads, 1) decode_mega_kernel(const __grid_constant__ MegaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  __half* xs = reinterpret_cast<__half*>(ring + (size_t)a.stages * kStageBytes);
  float* red = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xs) + a.xs_bytes);  // [2][kCW][64] + 8
  uint64_t* full = reinterpret_cast<uint64_t*>(red + 2 * kCW * 64 + 8);
  uint64_t* empty = full + a.stages;
  int* s_int = reinterpret_cast<int*>(empty + a.stages);  // [0],[1] tickets' verdicts, [2] failure flag
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kCW);
    }
    s_int[0] = s_int[1] = s_int[2] = 0;
    fence_barrier_init();
  }
  __syncthreads();
  Waiter w{s_int + 2, a.error};

  if (warp == kCW) {
    if (lane == 0) producer_loop(a, ring, full, empty, w);
  } else {
    Ctx c{a, ring, full, empty, xs, red, s_int, w, Ring{0, 0}, 0u, 0, 0};
    if (threadIdx.x == 0) c.gen = ld_acquire_gpu(a.bar + 1);
    c.gen = __shfl_sync(0xffffffffu, c.gen, 0);  // only thread 0 uses it
    const int d = a.d_model;
    for (int l = 0; l < a.n_layers; ++l) {
      const MegaLayer* ly = a.layers + l;
      const __half* x_cur = l == 0 ? a.x_in : (((l - 1) & 1) ? a.xb : a.xa);
      __half* x_next = l + 1 == a.n_layers ? a.x_out : ((l & 1) ? a.xb : a.xa);
      c.op_index = l * kOpsPerLayer;
      trace_mark(c, 0);
      load_x_norm(c, x_cur, ly->norm1, d);
      trace_mark(c, 1);
      run_projection(c, kQkv, nullptr, a.qkv);
      trace_mark(c, 2);
      grid_barrier(c);
      trace_mark(c, 3);

      c.op_index += 1;
      trace_mark(c, 0);
      run_attention(c, ly);
      trace_mark(c, 2);
      grid_barrier(c);
      trace_mark(c, 3);

      c.op_index += 1;
      trace_mark(c, 0);
      load_x_plain(c, a.attn, d);
      trace_mark(c, 1);
      run_projection(c, kO, x_cur, a.h);
      trace_mark(c, 2);
      grid_barrier(c);
      trace_mark(c, 3);

      c.op_index += 1;
      trace_mark(c, 0);
      load_x_norm(c, a.h, ly->norm2, d);
      trace_mark(c, 1);
      run_projection(c, kGu, nullptr, a.act);
      trace_mark(c, 2);
      grid_barrier(c);
      trace_mark(c, 3);

      c.op_index += 1;
      trace_mark(c, 0);
      load_x_plain(c, a.act, a.ffn);
      trace_mark(c, 1);
      run_projection(c, kDown, a.h, x_next);
      trace_mark(c, 2);
      grid_barrier(c);
      trace_mark(c, 3);
    }
  }
  // A CTA that gave up may still have copies in flight: give them time to land
  // before its shared memory is released.
  __syncthreads();
  if (s_int[2] != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

}  // namespace

// ------------------------------------------------------------------ host side
struct MegaDecoder {
  MegaConfig cfg;
  int sms, grid, stages, gs_shift, xs_bytes;
  size_t smem_bytes;
  MegaLayer* d_layers;
  std::vector<MegaLayer> h_layers;
  std::vector<char> layer_set;
  uint8_t* scratch;
  __half *qkv, *attn, *h, *act, *xa, *xb;
  float *col_part, *att_part;
  int *col_tickets, *att_tickets, *error;
  unsigned* bar;
  unsigned long long* trace;
};

bool mega_supported(const MegaConfig& c) {
  if (c.head_dim != kHeadDim || c.heads < 1) return false;
  if (c.d_model != c.heads * kHeadDim) return false;
  if (c.d_model % 64 != 0 || c.ffn % 32 != 0) return false;
  int gs = c.block / 4, shift = 0;
  while ((1 << shift) < gs) ++shift;
  if ((1 << shift) != gs || gs < 8 || gs > kRows) return false;  // blocks of 32..256 inputs
  if (c.d_model % c.block != 0 || c.ffn % c.block != 0) return false;
  return get_encode_tiled() != nullptr;
}

void mega_destroy(MegaDecoder* m) {
  if (m == nullptr) return;
  if (m->d_layers != nullptr) cudaFree(m->d_layers);
  if (m->scratch != nullptr) cudaFree(m->scratch);
  if (m->trace != nullptr) cudaFree(m->trace);
  delete m;
}

int mega_create(const MegaConfig& cfg, MegaDecoder** out) {
  MLD_REQUIRE(mega_supported(cfg), "decoder shape not supported by the persistent step kernel");
  MegaDecoder* m = new MegaDecoder();
  m->cfg = cfg;
  m->d_layers = nullptr;
  m->scratch = nullptr;
  m->trace = nullptr;
  m->sms = sm_count(cfg.device);
  int gs = cfg.block / 4;
  m->gs_shift = 0;
  while ((1 << m->gs_shift) < gs) ++m->gs_shift;
  // shared memory: ring + max(input vector, attention scratch) + reductions + barriers
  const int att_bytes = (3 * kHeadDim + 64 + 32 * kHeadDim) * 4;
  const int vec_bytes = (cfg.d_model > cfg.ffn ? cfg.d_model : cfg.ffn) * 2;
  m->xs_bytes = align_n(att_bytes > vec_bytes ? att_bytes : vec_bytes, 128);
  const int fixed = 1024 + m->xs_bytes + (2 * kCW * 64 + 8) * 4 + 64;
  int max_smem = 0;
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, cfg.device);
  int stages = (max_smem - fixed) / (kStageBytes + 16);
  if (const char* e = getenv("MLD_MEGA_STAGES")) {
    const int v = atoi(e);
    if (v >= 2 && v < stages) stages = v;
  }
  if (stages > 64) stages = 64;
  if (stages < 4) {
    set_last_error_text("not enough shared memory for the persistent step kernel");
    mega_destroy(m);
    return MLD_UNIMPLEMENTED;
  }
  m->stages = stages;
  m->smem_bytes = (size_t)fixed + (size_t)stages * (kStageBytes + 16);
  cudaError_t e = cudaFuncSetAttribute(decode_mega_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(m->smem_bytes));
  int per_sm = 0;
  if (e == cudaSuccess)
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_mega_kernel, kThreads, m->smem_bytes);
  if (e != cudaSuccess || per_sm < 1) {
    set_last_error("persistent step kernel does not fit an SM", e);
    mega_destroy(m);
    return MLD_CUDA_ERROR;
  }
  m->grid = m->sms;
  if (const char* g = getenv("MLD_MEGA_GRID")) {
    const int v = atoi(g);
    if (v >= 1 && v < m->grid) m->grid = v;
  }
  // an attention range must not touch more than kAttSlots heads: ceil(n/nt)+1 with n = ceil(heads*nt/grid)
  // is at most ceil(heads/grid + 1/nt) + 1 <= heads/grid + 3
  if (cfg.heads / m->grid + 3 > kAttSlots) {
    set_last_error_text("too many heads per CTA for the persistent step kernel");
    mega_destroy(m);
    return MLD_UNIMPLEMENTED;
  }
  const int d = cfg.d_model, ffn = cfg.ffn;
  const int max_cols = (3 * d > 2 * ffn ? 3 * d : 2 * ffn) / 64 + 1;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += (bytes + 255) & ~size_t(255);
    return o;
  };
  const size_t o_qkv = take((size_t)3 * d * 2), o_attn = take((size_t)d * 2), o_h = take((size_t)d * 2),
               o_act = take((size_t)ffn * 2), o_xa = take((size_t)d * 2), o_xb = take((size_t)d * 2),
               o_cp = take((size_t)m->grid * 2 * 64 * 4), o_ap = take((size_t)m->grid * kAttSlots * (2 + kHeadDim) * 4),
               o_ct = take((size_t)max_cols * 4), o_at = take((size_t)cfg.heads * 4), o_bar = take(8), o_err = take(4);
  if (cudaMalloc(&m->scratch, off) != cudaSuccess ||
      cudaMalloc(&m->d_layers, sizeof(MegaLayer) * cfg.layers) != cudaSuccess) {
    set_last_error_text("persistent step kernel: device allocation failed");
    mega_destroy(m);
    return MLD_CUDA_ERROR;
  }
  cudaMemset(m->scratch, 0, off);
  m->qkv = reinterpret_cast<__half*>(m->scratch + o_qkv);
  m->attn = reinterpret_cast<__half*>(m->scratch + o_attn);
  m->h = reinterpret_cast<__half*>(m->scratch + o_h);
  m->act = reinterpret_cast<__half*>(m->scratch + o_act);
  m->xa = reinterpret_cast<__half*>(m->scratch + o_xa);
  m->xb = reinterpret_cast<__half*>(m->scratch + o_xb);
  m->col_part = reinterpret_cast<float*>(m->scratch + o_cp);
  m->att_part = reinterpret_cast<float*>(m->scratch + o_ap);
  m->col_tickets = reinterpret_cast<int*>(m->scratch + o_ct);
  m->att_tickets = reinterpret_cast<int*>(m->scratch + o_at);
  m->bar = reinterpret_cast<unsigned*>(m->scratch + o_bar);
  m->error = reinterpret_cast<int*>(m->scratch + o_err);
  m->h_layers.resize(cfg.layers);
  m->layer_set.assign(cfg.layers, 0);
  *out = m;
  return MLD_OK;
}

int mega_set_layer(MegaDecoder* m, int layer, const MegaLayerPtrs& p) {
  const MegaConfig& c = m->cfg;
  MegaLayer& L = m->h_layers[layer];
  memset(&L, 0, sizeof L);
  const int d = c.d_model, ffn = c.ffn;
  const int Ns[4] = {3 * d, d, 2 * ffn, d};
  const int Ks[4] = {d, d, d, ffn};
  const void* ws[4] = {p.wqkv, p.wo, p.wgu, p.wdown};
  const void* ss[4] = {p.sqkv, p.so, p.sgu, p.sdown};
  const int sr = kRows >> m->gs_shift;
  for (int i = 0; i < 4; ++i) {
    const uint64_t row_bytes = (uint64_t)Ns[i] * 2;  // N/4 blocks of 8 bytes
    int rc = make_tmap_2d(&L.w[i], ws[i], row_bytes, Ks[i] / 4, row_bytes, 128, kRows, 1, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != MLD_OK) return rc;
    rc = make_tmap_2d(&L.s[i], ss[i], (uint64_t)Ns[i] * 2, Ks[i] / c.block, (uint64_t)Ns[i] * 2, 128, sr, 2,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
    if (rc != MLD_OK) return rc;
  }
  const uint64_t kv_row = (uint64_t)c.heads * kHeadDim * 2;
  int rc = make_tmap_2d(&L.kc, p.kcache, kv_row, c.max_seq, kv_row, kHeadDim * 2, kTile, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MLD_OK) return rc;
  rc = make_tmap_2d(&L.vc, p.vcache, kv_row, c.max_seq, kv_row, kHeadDim * 2, kTile, 2, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MLD_OK) return rc;
  L.norm1 = static_cast<const __half*>(p.norm1);
  L.norm2 = static_cast<const __half*>(p.norm2);
  L.kcache = static_cast<__half*>(p.kcache);
  L.vcache = static_cast<__half*>(p.vcache);
  MLD_CUDA_CHECK(cudaMemcpy(m->d_layers + layer, &L, sizeof L, cudaMemcpyHostToDevice));
  m->layer_set[layer] = 1;
  return MLD_OK;
}

int mega_enable_trace(MegaDecoder* m, bool on) {
  if (on && m->trace == nullptr) {
    const size_t bytes = (size_t)m->grid * m->cfg.layers * kOpsPerLayer * kTraceSlots * sizeof(unsigned long long);
    MLD_CUDA_CHECK(cudaMalloc(&m->trace, bytes));
    MLD_CUDA_CHECK(cudaMemset(m->trace, 0, bytes));
  } else if (!on && m->trace != nullptr) {
    cudaFree(m->trace);
    m->trace = nullptr;
  }
  return MLD_OK;
}
int mega_read_trace(MegaDecoder* m, unsigned long long* out, size_t count) {
  MLD_REQUIRE(m->trace != nullptr, "trace is not enabled");
  const size_t have = (size_t)m->grid * m->cfg.layers * kOpsPerLayer * kTraceSlots;
  MLD_CUDA_CHECK(cudaMemcpy(out, m->trace, (count < have ? count : have) * sizeof(unsigned long long),
                            cudaMemcpyDeviceToHost));
  return MLD_OK;
}
int mega_grid(const MegaDecoder* m) { return m->grid; }

int mega_device_status(MegaDecoder* m, int* code) {
  MLD_CUDA_CHECK(cudaMemcpy(code, m->error, sizeof(int), cudaMemcpyDeviceToHost));
  if (*code != 0) {
    // leave the barrier and tickets consistent for the next step
    const int zero = 0;
    cudaMemcpy(m->error, &zero, sizeof zero, cudaMemcpyHostToDevice);
    cudaMemset(m->bar, 0, 4);
    cudaMemset(m->col_tickets, 0, (size_t)((3 * m->cfg.d_model > 2 * m->cfg.ffn ? 3 * m->cfg.d_model : 2 * m->cfg.ffn) / 64 + 1) * 4);
    cudaMemset(m->att_tickets, 0, (size_t)m->cfg.heads * 4);
  }
  return MLD_OK;
}

int mega_step(MegaDecoder* m, const void* x_in, void* x_out, int pos, cudaStream_t stream) {
  for (char s : m->layer_set) MLD_REQUIRE(s != 0, "layer weights not set");
  MegaArgs a;
  memset(&a, 0, sizeof a);
  const MegaConfig& c = m->cfg;
  a.layers = m->d_layers;
  a.n_layers = c.layers;
  a.d_model = c.d_model;
  a.heads = c.heads;
  a.ffn = c.ffn;
  a.pos = pos;
  a.gs_shift = m->gs_shift;
  a.stages = m->stages;
  a.xs_bytes = m->xs_bytes;
  a.rms_eps = c.rms_eps;
  a.min_ts = c.rope_min_timescale;
  a.max_ts = c.rope_max_timescale;
  a.q_scale = 1.0f / sqrtf(static_cast<float>(kHeadDim));
  a.x_in = static_cast<const __half*>(x_in);
  a.x_out = static_cast<__half*>(x_out);
  a.qkv = m->qkv;
  a.attn = m->attn;
  a.h = m->h;
  a.act = m->act;
  a.xa = m->xa;
  a.xb = m->xb;
  a.col_part = m->col_part;
  a.col_tickets = m->col_tickets;
  a.att_part = m->att_part;
  a.att_tickets = m->att_tickets;
  a.bar = m->bar;
  a.error = m->error;
  a.trace = m->trace;
  void* params[] = {&a};
  MLD_CUDA_CHECK(cudaLaunchCooperativeKernel(reinterpret_cast<void*>(decode_mega_kernel), dim3(m->grid), dim3(kThreads),
                                             params, m->smem_bytes, stream));
  count_launch();
  return MLD_OK;
}

}  // namespace mld
