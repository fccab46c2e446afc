// One persistent kernel for a whole decode step of the INT4 decoder.
//
// The op-by-op decoder spends most of a step between kernels: every
// projection drains its TMA pipeline, the next one fills it again, and the
// weights of a projection (8-45 MB) stream for only a few microseconds.  Here
// one cooperative grid of one CTA per SM runs all layers:
//   * a producer thread per CTA walks the step's whole list of weight boxes and
//     KV-cache tiles this CTA will need, in order, and keeps a ring of 9 KB
//     stages (about 170 KB) full.  Nothing it loads depends on the step's
//     activations, so it runs ahead across op and layer boundaries;
//   * the consumer warps do the arithmetic of every op:
//       qkv  = Wqkv rmsnorm(x) g1                 (RMSNorm fused into the vector load)
//       attn = softmax(rope(q) K^T) V             (new k/v roped, written to the cache)
//       h    = x + Wo attn
//       act  = silu(Wg hn) * (Wu hn), hn = rmsnorm(h) g2
//       x'   = h + Wdown act
//     with a grid barrier after each (five per layer), after which every CTA
//     loads the op's input vector;
//   * work is split in items of one ring stage, each consumed by one warp: a
//     projection's boxes of 16 outputs x 1024 inputs, attention's (head,
//     32-token tile) pairs.  A CTA owns whole 16-output strips of a projection
//     (all of K), so projections need nothing from other CTAs; a head of
//     attention is shared by a group of CTAs whose partial results are merged in
//     a fixed order, so results do not depend on arrival order;
//   * the decoder keeps its own copy of the projection weights, re-tiled from
//     the reference layout when a layer is set: box after box, 8 KB of nibbles
//     in the order the MMA fragments want them followed by the 1 KB of scales
//     they need, strip after strip.  A box is one contiguous 9 KB bulk copy and a
//     CTA's share of a projection one contiguous stream;
//   * sharded over several GPUs, every rank runs this kernel on its shard,
//     stores what the other ranks need straight into their memory and the
//     barriers after such an exchange span the ranks.
//
// Projection arithmetic: the dequantisation of GetFullyConnectedKernelCode
// (ml_drift/common/kernels/fully_connected.cc:623-942), w = (u - 8) * scale
// per block of 32 inputs, as sum(u * x) - 8 * sum(x) per block times the scale:
// the sums are exact integer MMAs over the nibbles and the input vector in
// 16-bit fixed point (see digitise_x), the scale is applied in fp32.  The
// decoder graph is that of samples/llm/qwen3_model_builder.cc:880-1017.
//
// Every wait (ring barriers, flags, grid barriers) is bounded; when one runs
// out the CTA records an error code, stops waiting and runs to the end.
#include <cuda_fp16.h>

#include <cstdlib>
#include <cstring>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace mld {

namespace {

// Per-CTA timestamps for tuning are compiled in only with -DMLD_TRACE (build.py --trace).
#ifdef MLD_TRACE
#define MLD_TRACING(a) ((a).trace != nullptr)
#else
#define MLD_TRACING(a) false
#endif

constexpr int kCW = 11;                      // consumer warps; every ring stage is consumed by ONE warp
constexpr int kThreads = (kCW + 1) * 32;     // + one producer warp
constexpr int kStripN = 16;                  // outputs per strip (the MMA's M)
constexpr int kBoxK = 1024;                  // inputs per box: 32 units of 32 inputs, 64 MMAs
constexpr int kBox = kStripN * kBoxK / 2;    // 8 KB of nibbles
constexpr int kScaleBox = 1024;              // 32 units x 16 outputs x fp16
constexpr int kStageBytes = kBox + kScaleBox;
constexpr int kHeadDim = 128;
constexpr int kTile = 32;                    // cached tokens per attention item (K box, V box: 8 KB each)
constexpr int kAttSlots = 4;                 // heads a CTA's attention range can touch
constexpr int kProjCounters = 12;            // >= kCW: arrivals of a shared strip are counted at its first warp
constexpr int kAttnSlots = 2;                // head runs likewise
constexpr int kAttDump = kHeadDim + 4;       // 128 outputs, then max and sum (padded: rows stay 16-byte aligned)
constexpr int kDumpFloats = 2 * kCW * kStripN > kAttnSlots * kCW * kAttDump ? 2 * kCW * kStripN : kAttnSlots * kCW * kAttDump;
constexpr int kWarpScratch = 3 * kHeadDim;   // attention: rotated q, new k, new v (floats) per warp
constexpr int kMaxParts = 8;                 // CTAs that share a head at most: the merging part reads all partials in one round
constexpr int kTraceSlots = 12;              // per (CTA, op): 4 timestamps, warp 0's clocks, all-warps-done, last load issued
enum { kQkv = 0, kAttn = 1, kO = 2, kGu = 3, kDown = 4, kOpsPerLayer = 5 };

struct alignas(128) MegaLayer {
  CUtensorMap kc, vc; // KV cache: fp16 [max_seq][heads*128], box 64 dims x 32 rows, 128-byte swizzle
  const uint8_t* w[4];  // re-tiled weights + scales of qkv, o, gu, down: [strip][k box][kStageBytes]
  const __half* norm1;
  const __half* norm2;
  __half* kcache;
  __half* vcache;
};

struct MegaArgs {
  const MegaLayer* layers;
  int n_layers, d_model, heads, ffn, pos;
  int stages;          // ring depth
  int l2_ahead;        // ops by which the L2 prefetch runs ahead of the ring's loads (0 = none)
  int xs_bytes;        // shared-memory bytes of the input-vector / attention scratch area
  int us_floats;       // entries of the per-32-input sums of the input vector
  float rms_eps, min_ts, max_ts, q_scale;
  // Sharding: this rank computes heads [rank * heads, ...), outputs [rank * d_local, ...) of o / down and
  // FFN units [rank * ffn_local, ...); heads is the LOCAL head count, d_model and ffn are global (they are
  // the input lengths of the projections).  The vectors every rank needs in full (attn, h, act, xa, xb)
  // and the cross-rank barrier counter live in an exchange block with the same layout on every rank;
  // peers[r] is rank r's block as mapped here (peers[rank] = the local one).
  int world, rank, d_local, ffn_local;
  int paired;  // 1: o and down are split by INPUT columns; their outputs are partial sums every rank adds up
  uint8_t* peers[8];
  unsigned long long off_attn, off_h, off_act, off_xa, off_xb, off_xbar;  // byte offsets in the exchange block
  unsigned long long off_ph, off_pd;  // paired: fp32 partial sums of o / down, [world][d_model] each
  const __half* x_in;
  __half* x_out;
  __half *qkv, *attn, *h, *act, *xa, *xb;  // local copies (attn .. xb inside the local exchange block)
  // Single GPU: the vectors that pass from op to op are arrays of 32-bit words, fp16 value in the low half
  // and the writing op's tag in the high half; a reader polls a word until it carries the tag it expects,
  // so no barrier separates the ops (tagged != 0).
  // Sharded with tagged vectors: tattn .. txb live in the exchange block (same layout on every rank) and a
  // writer stores each word into every rank's copy (plain peer stores; a word carries its own validity, so no
  // fence, flag or barrier orders the exchange); xoff[i] = byte offset of tattn, th, tact, txa, txb there.
  int tagged;
  uint32_t *tq, *tattn, *th, *tact, *txa, *txb;
  unsigned long long wait_limit_ns;  // bound on every wait of this launch
  float* att_part;     // [grid][kAttSlots][kAttDump]
  int* att_tickets;    // [heads]
  unsigned* att_flags; // [heads][grid / heads]: epoch of the attention whose partial the part has published
  unsigned* bar;       // 64-bit arrival counter of the grid barrier (8-byte aligned)
  int* error;
  unsigned long long* trace;  // optional [grid][ops][kTraceSlots]
};

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mbar_arrive_n(uint64_t* bar, uint32_t n) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(n) : "memory");
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory"); }

// Per-CTA state shared by all waits: once any wait of this CTA has run out,
// no later wait blocks.
struct Waiter {
  volatile int* s_fail;
  int* error;
  unsigned long long limit;  // ns
  bool sys;                  // tagged words may be written by other GPUs: poll them at system scope
  __device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity, int code) const {
    if (mbar_try_wait(bar, parity)) return true;
    if (*s_fail) return false;
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
#pragma unroll 1
      for (int i = 0; i < 64; ++i)
        if (mbar_try_wait(bar, parity)) return true;
      if (*s_fail) return false;
      if (globaltimer_ns() - t0 > limit) {
        *s_fail = 1;
        atomicExch(error, code);
        return false;
      }
    }
  }
  // waits until *counter >= want (a shared-memory counter another warp of this CTA advances)
  __device__ __forceinline__ void wait_count(volatile int* counter, int want, int code) const {
    if (*counter - want >= 0 || *s_fail) return;
    const unsigned long long t0 = globaltimer_ns();
    while (*counter - want < 0) {
      if (*s_fail) return;
      if (globaltimer_ns() - t0 > limit) {
        *s_fail = 1;
        atomicExch(error, code);
        return;
      }
    }
  }
};

// Tag of op number `epoch` (unique over launches): 1 .. 65535, never the 0 of untouched memory.
__device__ __forceinline__ uint32_t op_tag(unsigned epoch) { return epoch % 65535u + 1u; }
__device__ __forceinline__ void st_tagged(uint32_t* p, __half v, uint32_t tag) {
  const uint32_t w = (tag << 16) | static_cast<uint32_t>(__half_as_ushort(v));
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(w) : "memory");
}
__device__ __forceinline__ void st_tagged_sys(uint32_t* p, __half v, uint32_t tag) {
  const uint32_t w = (tag << 16) | static_cast<uint32_t>(__half_as_ushort(v));
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(w) : "memory");
}
__device__ __forceinline__ uint32_t ld_word(const uint32_t* p, bool sys) {
  uint32_t v;
  if (sys)
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  else
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_word4(const uint32_t* p, bool sys) {
  uint4 v;
  if (sys)
    asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  else
    asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// One tagged value, waited for (bounded; code 22).
__device__ __forceinline__ __half ld_tagged(const Waiter& w, const uint32_t* p, uint32_t tag) {
  uint32_t v = ld_word(p, w.sys);
  if ((v >> 16) != tag && !*w.s_fail) {
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
      v = ld_word(p, w.sys);
      if ((v >> 16) == tag || *w.s_fail) break;
      if (globaltimer_ns() - t0 > w.limit) {
        *w.s_fail = 1;
        atomicExch(w.error, 22);
        break;
      }
    }
  }
  return __ushort_as_half(static_cast<unsigned short>(v & 0xFFFFu));
}
// The same for a word already asked for: callers load all their words first, so that the loads overlap,
// and then call this for each.
__device__ __forceinline__ __half tagged_value(const Waiter& w, const uint32_t* p, uint32_t tag, uint32_t v) {
  if ((v >> 16) != tag) return ld_tagged(w, p, tag);
  return __ushort_as_half(static_cast<unsigned short>(v & 0xFFFFu));
}
// Eight consecutive tagged values (32-byte aligned), packed as eight halves.
__device__ __forceinline__ uint4 ld_tagged8(const Waiter& w, const uint32_t* p, uint32_t tag) {
  uint4 a = ld_word4(p, w.sys), b = ld_word4(p + 4, w.sys);
  const uint32_t want = tag * 0x00010001u;  // the tag in both halves of a word
  auto ok = [&](const uint4& u, const uint4& v) {
    return __byte_perm(u.x, u.y, 0x7632) == want && __byte_perm(u.z, u.w, 0x7632) == want &&
           __byte_perm(v.x, v.y, 0x7632) == want && __byte_perm(v.z, v.w, 0x7632) == want;
  };
  if (!ok(a, b) && !*w.s_fail) {
    const unsigned long long t0 = globaltimer_ns();
    for (;;) {
      a = ld_word4(p, w.sys);
      b = ld_word4(p + 4, w.sys);
      if (ok(a, b) || *w.s_fail) break;
      if (globaltimer_ns() - t0 > w.limit) {
        *w.s_fail = 1;
        atomicExch(w.error, 22);
        break;
      }
    }
  }
  return make_uint4(__byte_perm(a.x, a.y, 0x5410), __byte_perm(a.z, a.w, 0x5410), __byte_perm(b.x, b.y, 0x5410),
                    __byte_perm(b.z, b.w, 0x5410));
}

// The rare path of a wait that is nearly always over already, kept out of line so that the loops that
// make it stay small.
__device__ __noinline__ void wait_out_of_line(volatile int* s_fail, int* error, unsigned long long limit, uint64_t* bar,
                                              uint32_t parity, int code) {
  const Waiter w{s_fail, error, limit, false};
  w.wait(bar, parity, code);
}
__device__ __forceinline__ void wait_released(const Waiter& w, uint64_t* bar, uint32_t parity, int code) {
  if (!mbar_try_wait(bar, parity)) wait_out_of_line(w.s_fail, w.error, w.limit, bar, parity, code);
}

// Balanced contiguous split of `items` over the grid (32-bit: the host checks items * grid < 2^31).
__device__ __forceinline__ int range_start(int cta, int items, int grid) {
  return static_cast<int>(static_cast<unsigned>(cta) * static_cast<unsigned>(items) / static_cast<unsigned>(grid));
}
__device__ __forceinline__ int owner_of(int item, int items, int grid) {
  return static_cast<int>(((static_cast<unsigned>(item) + 1u) * static_cast<unsigned>(grid) - 1u) /
                          static_cast<unsigned>(items));
}

struct ProjShape {
  int N, K, C, S, I;  // C strips of 16 outputs, S boxes of 1024 inputs per strip, I = C * S items
};
__device__ __forceinline__ ProjShape proj_shape(const MegaArgs& a, int kind) {
  ProjShape p;
  if (a.paired) {
    p.N = kind == kQkv ? 3 * a.d_local : kind == kGu ? 2 * a.ffn_local : a.d_model;
    p.K = kind == kDown ? a.ffn_local : kind == kO ? a.d_local : a.d_model;
  } else {
    p.N = kind == kQkv ? 3 * a.d_local : kind == kGu ? 2 * a.ffn_local : a.d_local;
    p.K = kind == kDown ? a.ffn : a.d_model;
  }
  p.C = p.N / kStripN;
  p.S = (p.K + kBoxK - 1) / kBoxK;
  p.I = p.C * p.S;
  return p;
}
// A CTA's items of a projection: whole strips, so that nothing has to be
// combined between CTAs.
__device__ __forceinline__ void proj_range(const ProjShape& p, int cta, int G, int& i0, int& i1) {
  i0 = range_start(cta, p.C, G) * p.S;
  i1 = range_start(cta + 1, p.C, G) * p.S;
}
__device__ __forceinline__ int map_index(int kind) { return kind == kQkv ? 0 : kind == kO ? 1 : kind == kGu ? 2 : 3; }
__device__ __forceinline__ void bulk_load_1d_hint(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar,
                                                  uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// A CTA's item range [i0, i1) of an op, cut into runs: the items of one unit
// (a projection's 16-output strip, an attention head; S items each).  A run
// that shares its unit with another CTA needs a round trip through L2 to be
// completed, so such runs come first: the range's last run, when it is cut
// short, is processed before the others.
struct Runs {
  int i0, i1, S, first, R;
  bool rotate;
  __device__ __forceinline__ Runs(int i0_, int i1_, int S_) : i0(i0_), i1(i1_), S(S_) {
    first = i0 / S;
    R = i1 > i0 ? (i1 - 1) / S - first + 1 : 0;
    rotate = R > 1 && (i1 % S) != 0;
  }
  __device__ __forceinline__ void bounds(int rr, int& unit, int& lo, int& hi) const {
    const int r = rotate ? (rr == 0 ? R - 1 : rr - 1) : rr;
    unit = first + r;
    lo = max(i0, unit * S);
    hi = min(i1, (unit + 1) * S);
  }
};

// A CTA's attention items.  With at least as many CTAs as heads, P = grid / heads CTAs share a head
// (CTA c: head c / P, tiles [part nt / P, (part + 1) nt / P)) and every CTA has one run; otherwise the
// items (head-major) are split evenly and a CTA may touch several heads.
struct AttnSplit {
  int nt, I, G, heads, P;
  __device__ __forceinline__ AttnSplit(int heads_, int nt_, int G_) : nt(nt_), I(heads_ * nt_), G(G_), heads(heads_) {
    P = G >= heads ? G / heads : 0;
    if (P > kMaxParts) P = kMaxParts;
  }
  __device__ __forceinline__ void range(int cta, int& i0, int& i1) const {
    if (P > 0) {
      const int head = cta / P, part = cta - head * P;
      if (head >= heads) {
        i0 = i1 = 0;
        return;
      }
      // nt / P tiles each, the remainder one by one to the first parts (the last non-empty part also
      // brings in the new token and merges the head)
      const int base = nt / P, rem = nt - base * P;
      i0 = head * nt + part * base + (part < rem ? part : rem);
      i1 = i0 + base + (part < rem ? 1 : 0);
    } else {
      i0 = range_start(cta, I, G);
      i1 = range_start(cta + 1, I, G);
    }
  }
  // CTAs that may hold items of `head`: first..last (P > 0: exactly the non-empty parts)
  __device__ __forceinline__ void contributors(int head, int& first, int& last) const {
    if (P > 0) {
      first = head * P;
      last = first + (nt < P ? nt : P) - 1;
    } else {
      first = owner_of(head * nt, I, G);
      last = owner_of(head * nt + nt - 1, I, G);
    }
  }
};

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

// Asks L2 for this CTA's whole share of an op: HBM then runs an op ahead of the
// ring, which only has to cover the L2 -> shared memory latency.
__device__ void prefetch_op_l2(const MegaArgs& a, int l, int kind) {
  const int cta = blockIdx.x, G = gridDim.x;
  const MegaLayer* ly = a.layers + l;
  if (kind == kAttn) {
    const int nt = a.pos / kTile + 1;
    const AttnSplit split(a.heads, nt, G);
    int i0, i1;
    split.range(cta, i0, i1);
    for (int i = i0; i < i1; ++i) {
      const int head = i / nt, j = i - head * nt;
      asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                       reinterpret_cast<uint64_t>(&ly->kc)),
                   "r"(head * kHeadDim), "r"(j * kTile)
                   : "memory");
      asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(
                       reinterpret_cast<uint64_t>(&ly->vc)),
                   "r"(head * kHeadDim), "r"(j * kTile)
                   : "memory");
    }
  } else {
    const ProjShape p = proj_shape(a, kind);
    int i0, i1;
    proj_range(p, cta, G, i0, i1);
    const uint8_t* src = ly->w[map_index(kind)] + (size_t)i0 * kStageBytes;
    size_t bytes = (size_t)(i1 - i0) * kStageBytes;
    while (bytes > 0) {
      const uint32_t n = bytes < 18432 ? static_cast<uint32_t>(bytes) : 18432u;
      bulk_prefetch_l2(src, n);
      src += n;
      bytes -= n;
    }
  }
}

__device__ void producer_loop(const MegaArgs& a, uint8_t* ring, uint64_t* full, uint64_t* empty, const Waiter& w) {
  const int cta = blockIdx.x, G = gridDim.x;
  const uint64_t pol = policy_evict_first();
  Ring r{0, 0};
  const int nt = a.pos / kTile + 1;
  for (int l = 0; l < a.n_layers; ++l) {
    const MegaLayer* ly = a.layers + l;
    for (int kind = 0; kind < kOpsPerLayer; ++kind) {
      if (a.l2_ahead > 0) {
        // the op `l2_ahead` ops after this one
        const int o = l * kOpsPerLayer + kind + a.l2_ahead;
        if (o < a.n_layers * kOpsPerLayer) prefetch_op_l2(a, o / kOpsPerLayer, o % kOpsPerLayer);
      }
      if (kind == kAttn) {
        const AttnSplit split(a.heads, nt, G);
        int ai0, ai1;
        split.range(cta, ai0, ai1);
        const Runs runs(ai0, ai1, nt);
        for (int rr = 0; rr < runs.R; ++rr) {
          int head, lo, hi;
          runs.bounds(rr, head, lo, hi);
          for (int i = lo; i < hi; ++i) {
            const int j = i - head * nt;
            for (int kv = 0; kv < 2; ++kv) {
              // a producer whose wait ran out requests nothing more: stages it cannot know to be free stay
              // untouched, and no barrier sees an arrival its phase does not expect
              if (!w.wait(&empty[r.stage], r.phase ^ 1, 10)) return;
              uint8_t* st = ring + (size_t)r.stage * kStageBytes;
              mbar_arrive_expect_tx(&full[r.stage], kBox);
              const CUtensorMap* map = kv == 0 ? &ly->kc : &ly->vc;
              tma_load_2d_hint(st, map, &full[r.stage], head * kHeadDim, j * kTile, pol);
              tma_load_2d_hint(st + 4096, map, &full[r.stage], head * kHeadDim + 64, j * kTile, pol);
              r.advance(a.stages);
            }
          }
        }
      } else {
        const ProjShape p = proj_shape(a, kind);
        const uint8_t* wbase = ly->w[map_index(kind)];
        int pi0, pi1;
        proj_range(p, cta, G, pi0, pi1);
        // boxes are stored strip after strip: the CTA's boxes are one contiguous stream, cut into kCW
        // chunks (one per consumer warp); ring position kCW j + w takes box j of chunk w
        const int B = pi1 - pi0, qn = B / kCW, rn = B % kCW;
        for (int j = 0; j * kCW < B; ++j) {
          const int nw = B - j * kCW < kCW ? B - j * kCW : kCW;
          for (int cw = 0; cw < nw; ++cw) {
            const int i = pi0 + cw * qn + (cw < rn ? cw : rn) + j;
            if (!w.wait(&empty[r.stage], r.phase ^ 1, 11)) return;
            uint8_t* st = ring + (size_t)r.stage * kStageBytes;
            mbar_arrive_expect_tx(&full[r.stage], kStageBytes);
            bulk_load_1d_hint(st, wbase + (size_t)i * kStageBytes, kStageBytes, &full[r.stage], pol);
            r.advance(a.stages);
          }
        }
      }
      // when this op's last load was issued
      if (MLD_TRACING(a) && kind != kAttn)
        a.trace[((size_t)blockIdx.x * a.n_layers * kOpsPerLayer + l * kOpsPerLayer + kind) * kTraceSlots + 11] = globaltimer_ns();
    }
  }
}

// ------------------------------------------------------------------ consumers
struct Ctx {
  const MegaArgs& a;
  uint8_t* ring;
  uint64_t* full;
  uint64_t* empty;
  __half* xs;          // input vector of the running projection / per-warp attention scratch
  int* isum;           // [box][t][set]: scale exponent | 8 * (sum of the integers) of unit 4 set + t of the box, see digitise_x
  const float2* rope;  // [64] (cos, sin) of pos / timescale_i, the rotary embedding of this step
  float* dump;         // per-warp sums: projections [warp][share (2)][kStripN], attention [slot][warp][kAttDump]
  int* s_int;          // [0] failure flag, [1..] run bookkeeping (see below)
  Waiter w;
  int ring_base;       // stages of this CTA consumed by earlier ops (same in every warp)
  int attn_runs;       // head runs started so far
  unsigned long long bar_target;  // arrival count that completes the barrier this CTA waits for next
  unsigned long long xbar_target; // the same for the barrier across ranks
  unsigned epoch_base;            // unique per launch: op k of this launch has epoch epoch_base + k + 1
  int op_index;
  __device__ __forceinline__ int* proj_arrived() const { return s_int + 1; }                  // [kProjCounters]
  __device__ __forceinline__ int* attn_arrived() const { return s_int + 1 + kProjCounters; }  // [kAttnSlots]
  __device__ __forceinline__ volatile int* attn_done() const { return s_int + 1 + kProjCounters + kAttnSlots; }
};
static_assert(kProjCounters >= kCW && kProjCounters % 2 == 0, "one counter per consumer warp, even count");
constexpr int kSharedInts = 1 + kProjCounters + 2 * kAttnSlots;  // (odd) + 5 behind them: pad, two 64-bit barrier bases

__device__ __forceinline__ void trace_mark(const Ctx& c, int k) {
  if (MLD_TRACING(c.a) && threadIdx.x == 0)
    c.a.trace[((size_t)blockIdx.x * c.a.n_layers * kOpsPerLayer + c.op_index) * kTraceSlots + k] = globaltimer_ns();
}

// Grid barrier: one 64-bit arrival counter that only grows (launches leave it
// at a multiple of the grid size).  A CTA adds one with release semantics and
// no return value, then polls until the count reaches the end of the barrier's
// round.  All consumer threads call this after their last global write of an op.
// cross (sharded decoder only): the barrier spans the CTAs of all ranks and orders their peer stores: a
// CTA adds one to the counter in every rank's exchange block (release at system scope) and polls its own.
__device__ void grid_barrier(Ctx& c, bool cross = false) {
  consumer_bar();
  cross = cross && c.a.world > 1;
  if (threadIdx.x == 0) {
    trace_mark(c, 6);
    unsigned long long* cnt = reinterpret_cast<unsigned long long*>(c.a.bar);
    unsigned long long target = c.bar_target + gridDim.x;
    if (cross) {
      cnt = reinterpret_cast<unsigned long long*>(c.a.peers[c.a.rank] + c.a.off_xbar);
      target = c.xbar_target + (unsigned long long)gridDim.x * c.a.world;
      // one system-scope fence (this CTA's stores, the peer stores among them, are performed), then the arrivals
      asm volatile("fence.acq_rel.sys;" ::: "memory");
      for (int r = 0; r < c.a.world; ++r)
        asm volatile("red.relaxed.sys.global.add.u64 [%0], %1;" ::"l"(c.a.peers[r] + c.a.off_xbar), "l"(1ull) : "memory");
    } else {
      asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(cnt), "l"(1ull) : "memory");
    }
    if (!*c.w.s_fail) {
      const unsigned long long t0 = globaltimer_ns();
      for (;;) {
        unsigned long long v;
        if (cross)
          asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(cnt) : "memory");
        else
          asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(cnt) : "memory");
        if (static_cast<long long>(v - target) >= 0) break;
        if (globaltimer_ns() - t0 > c.w.limit || *reinterpret_cast<volatile int*>(c.a.error) != 0) {
          *c.w.s_fail = 1;
          atomicCAS(c.a.error, 0, 20);
          break;
        }
      }
    }
  }
  if (cross)
    c.xbar_target += (unsigned long long)gridDim.x * c.a.world;
  else
    c.bar_target += gridDim.x;
  consumer_bar();
}

// Between two ops: the grid barrier, or (tagged vectors) only this CTA's consumer warps, whose shared
// buffers the next op reuses.
__device__ __forceinline__ void op_boundary(Ctx& c, bool tagged, bool cross) {
  if (tagged) {
    consumer_bar();
    if (threadIdx.x == 0) trace_mark(c, 6);
  } else {
    grid_barrier(c, cross);
  }
}

// The digit scale of a unit of 32 inputs whose largest magnitude is amax: the smallest power of two s with
// amax / s <= 32512, so that round(x / s) fits 16 bits with head-room and 1 / s is exact.  Returns the bits
// of s (a float with an empty mantissa).
__device__ __forceinline__ uint32_t unit_scale_bits(float amax) {
  const float t = amax * (1.0f / 32512.0f);
  uint32_t b = (__float_as_uint(t) + 0x007FFFFFu) & 0x7F800000u;  // next power of two >= t
  if (b < (16u << 23)) b = 16u << 23;                              // an all-zero (or vanishing) unit: any scale does
  return b;
}

// Eight inputs (chunk ci = inputs 8 ci .. 8 ci + 7, fp16 in v) become digits in place.  The four lanes of a
// unit (consecutive chunks, one warp) agree on the unit's scale and add up the unit's integers.  All lanes
// of the warp call.
__device__ __forceinline__ void digitise_chunk(Ctx& c, int ci, const uint4& v) {
  const __half2* h = reinterpret_cast<const __half2*>(&v);
  float2 f[4];
  float amax = 0.0f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    f[j] = __half22float2(h[j]);
    amax = fmaxf(amax, fmaxf(fabsf(f[j].x), fabsf(f[j].y)));
  }
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
  const uint32_t sbits = unit_scale_bits(amax);
  const float inv = __uint_as_float((254u << 23) - sbits);  // 1 / s, exact
  // z = round(x / s) + 128 in the low 16 bits of the float's mantissa: high byte = hi digit, low byte ^ 0x80 = lo digit
  uint32_t z[8];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    z[2 * j] = __float_as_uint(fmaf(f[j].x, inv, 12583040.0f));
    z[2 * j + 1] = __float_as_uint(fmaf(f[j].y, inv, 12583040.0f));
  }
  uint32_t hiw[2], low[2];
#pragma unroll
  for (int e = 0; e < 2; ++e) {
    const uint32_t h01 = __byte_perm(z[4 * e], z[4 * e + 1], 0x0051), h23 = __byte_perm(z[4 * e + 2], z[4 * e + 3], 0x0051);
    const uint32_t l01 = __byte_perm(z[4 * e], z[4 * e + 1], 0x0040), l23 = __byte_perm(z[4 * e + 2], z[4 * e + 3], 0x0040);
    hiw[e] = __byte_perm(h01, h23, 0x5410);
    low[e] = __byte_perm(l01, l23, 0x5410) ^ 0x80808080u;
  }
  int sum = __dp4a(static_cast<int>(hiw[0]), 0x01010101, 0);
  sum = __dp4a(static_cast<int>(hiw[1]), 0x01010101, sum) * 256;
  sum = __dp4a(static_cast<int>(low[0]), 0x01010101, sum);
  sum = __dp4a(static_cast<int>(low[1]), 0x01010101, sum);
  sum += __shfl_xor_sync(0xffffffffu, sum, 1);
  sum += __shfl_xor_sync(0xffffffffu, sum, 2);
  // chunk q of the unit holds inputs 8q..8q+7: half q >> 1, lanes t = 2 (q & 1) and 2 (q & 1) + 1
  const int unit = ci >> 2, q = ci & 3;
  uint32_t* ub = reinterpret_cast<uint32_t*>(c.xs + unit * 32);
  const int w0 = 2 * (2 * (q & 1)) + (q >> 1);  // word index of (t, half): 2 t + half
  ub[w0] = hiw[0];
  ub[w0 + 2] = hiw[1];
  ub[8 + w0] = low[0];
  ub[8 + w0 + 2] = low[1];
  if (q == 0) {
    // |8 sum| <= 8 * 32 * 32512 < 2^23: the offset term and the scale's exponent share one word
    const int m = unit & 31;
    c.isum[(unit >> 5) * 32 + (m & 3) * 8 + (m >> 2)] = static_cast<int>(sbits | (static_cast<uint32_t>(8 * sum) & 0x007FFFFFu));
  }
}

// Turns the fp16 vector in xs into what the integer MMAs read, in place.  Every
// unit of 32 inputs (the span of one weight scale) becomes 16-bit fixed point
// with a scale of its own, x ~ s * (256 hi + lo) with hi, lo in [-128, 127] and
// s a power of two with max|x| / s in (16256, 32512]: 15 significant bits
// against fp16's 11, relative to the unit's own largest element, so an outlier
// channel costs its 31 neighbours nothing worth naming and the rest of the
// vector nothing at all.  The unit (64 bytes either way) is rewritten as
// [hi: 32 bytes][lo: 32 bytes], each in the order the B fragments take them
// (8 bytes per lane t: inputs 4t..4t+3 and 16+4t..16+4t+3).
// isum[box][t][set] = the scale's exponent bits | 23 bits of 8 * (sum of the
// unit's integers), the nibble offset's share.
__device__ void digitise_x(Ctx& c, int d) {
  const int chunks = (d + kBoxK - 1) / kBoxK * kBoxK / 8;  // 8 inputs (16 bytes) per thread and round
  for (int ci = threadIdx.x; ci < chunks; ci += kCW * 32) {
    const uint4 v = *reinterpret_cast<const uint4*>(c.xs + ci * 8);
    __syncwarp();  // rounds are warp-uniform (whole boxes): the unit's four lanes have read before any rewrites
    digitise_chunk(c, ci, v);
  }
}

// Where a projection's input vector comes from: a plain fp16 vector, or (paired sharding) a residual
// plus the ranks' fp32 partial sums of the projection before: v = resid + fp16(sum over ranks, in rank
// order).  CTA 0 also stores the assembled vector (it is the residual of a later sum).
struct Src {
  const __half* x;
  const float* partials;  // [world][stride] or null
  int world, stride;
  __half* store;
  const uint32_t* tx = nullptr;  // the vector as tagged words (then x is unused), written by the op with tag `tag`
  uint32_t tag = 0;
};
__device__ __forceinline__ uint4 fetch8(const Waiter& w, const Src& s, int i) {
  if (s.tx != nullptr) return ld_tagged8(w, s.tx + i, s.tag);
  uint4 xv = __ldcg(reinterpret_cast<const uint4*>(s.x + i));
  if (s.partials == nullptr) return xv;
  float acc[8] = {0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f, 0.0f};
  for (int r = 0; r < s.world; ++r) {
    const float4 p0 = __ldcg(reinterpret_cast<const float4*>(s.partials + (size_t)r * s.stride + i));
    const float4 p1 = __ldcg(reinterpret_cast<const float4*>(s.partials + (size_t)r * s.stride + i + 4));
    acc[0] += p0.x; acc[1] += p0.y; acc[2] += p0.z; acc[3] += p0.w;
    acc[4] += p1.x; acc[5] += p1.y; acc[6] += p1.z; acc[7] += p1.w;
  }
  __half2* h = reinterpret_cast<__half2*>(&xv);
#pragma unroll
  for (int j = 0; j < 4; ++j) h[j] = __hadd2(__floats2half2_rn(acc[2 * j], acc[2 * j + 1]), h[j]);
  if (s.store != nullptr && blockIdx.x == 0) *reinterpret_cast<uint4*>(s.store + i) = xv;
  return xv;
}

constexpr int kRegChunks = 4;  // chunks of 8 inputs a thread can hold: vectors up to 4 * 8 * 32 * kCW inputs

// Block-wide sum of one float per thread over the consumer warps.
__device__ __forceinline__ float consumer_sum(Ctx& c, float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  float* part = c.dump;  // free between ops
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  consumer_bar();
  float r = 0.0f;
#pragma unroll
  for (int wi = 0; wi < kCW; ++wi) r += part[wi];
  return r;
}

// Loads the d-element input vector of a projection and leaves it digitised in xs (digitise_x).
// NORM: the reference RMSNorm first, xs = fp16(v * rsqrt(mean(v^2) + eps) * gamma), fp32 statistics.
// Vectors of up to kRegChunks chunks per thread stay in registers between the passes.
template <bool NORM>
__device__ void load_x(Ctx& c, const Src& src, const __half* gamma, int d) {
  const int padded = (d + kBoxK - 1) / kBoxK * kBoxK;
  const int chunks = padded / 8;
  if (chunks > kRegChunks * kCW * 32) {
    // general path through shared memory
    float ss = 0.0f;
    for (int i = threadIdx.x * 8; i < padded; i += kCW * 32 * 8) {
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (i < d) v = fetch8(c.w, src, i);
      *reinterpret_cast<uint4*>(c.xs + i) = v;
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
    if (NORM) {
      const float inv = rsqrtf(consumer_sum(c, ss) / static_cast<float>(d) + c.a.rms_eps);
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
    }
    consumer_bar();
    digitise_x(c, d);
    consumer_bar();
    return;
  }
  uint4 v[kRegChunks];
  if (NORM) {
    uint4 gv[kRegChunks];
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < kRegChunks; ++r) {
      const int ci = threadIdx.x + r * kCW * 32;
      v[r] = make_uint4(0u, 0u, 0u, 0u);
      gv[r] = make_uint4(0u, 0u, 0u, 0u);
      if (ci * 8 < d) {
        v[r] = fetch8(c.w, src, ci * 8);
        gv[r] = __ldg(reinterpret_cast<const uint4*>(gamma + ci * 8));
      }
      const __half2* h = reinterpret_cast<const __half2*>(&v[r]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
    const float inv = rsqrtf(consumer_sum(c, ss) / static_cast<float>(d) + c.a.rms_eps);
#pragma unroll
    for (int r = 0; r < kRegChunks; ++r) {
      __half2* h = reinterpret_cast<__half2*>(&v[r]);
      const __half2* gh = reinterpret_cast<const __half2*>(&gv[r]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        const float2 g = __half22float2(gh[j]);
        h[j] = __floats2half2_rn(f.x * inv * g.x, f.y * inv * g.y);
      }
    }
  } else {
#pragma unroll
    for (int r = 0; r < kRegChunks; ++r) {
      const int ci = threadIdx.x + r * kCW * 32;
      v[r] = make_uint4(0u, 0u, 0u, 0u);
      if (ci * 8 < d) v[r] = fetch8(c.w, src, ci * 8);
    }
  }
  // the digit scale is per unit of 32 inputs, found by the unit's own four lanes: no block-wide maximum
#pragma unroll
  for (int r = 0; r < kRegChunks; ++r) {
    const int ci = threadIdx.x + r * kCW * 32;
    if (ci < chunks) digitise_chunk(c, ci, v[r]);  // warp-uniform: chunks is a multiple of 32
  }
  consumer_bar();
}

__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One box (16 outputs x 1024 inputs) by one warp.  Lane = 4g + t.  A unit of 32
// inputs (one scale per output) is exactly one integer MMA m16n8k32.  A 32-bit
// word of the re-tiled weights holds four inputs of row g in its low nibbles
// and of row g+8 in its high nibbles; A's rows g take the word as it is (bytes
// u_g + 16 u_g8) and its rows g+8 the word with the low nibbles cleared (bytes
// 16 u_g8), so that row g's sum is the difference of the two results and the
// nibbles are never shifted apart.  B = the digitised inputs; everything is
// exact in int32.  The 32 units of a box go in eight sets
// of four; B column 2j holds the high digit and 2j + 1 the low digit of unit j
// of the set (lane g supplies column g, zero for the other units), so a lane
// ends a set with both digits of unit t for rows g and g+8, combines them,
// takes off the nibble offset and applies the unit's scale.
__device__ __forceinline__ void consume_box(const Ctx& c, const uint8_t* st, int kb, float (&tot)[2]) {
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  // this lane's digit bytes for the eight sets: unit 4 set + (g >> 1), digit g & 1, inputs 4t.. and 16+4t..
  const uint2* xd = reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(c.xs) + (size_t)kb * 2 * kBoxK) + lane;
  uint2 xb[8];
#pragma unroll
  for (int sidx = 0; sidx < 8; ++sidx) xb[sidx] = xd[32 * sidx];
  const uint4* wl = reinterpret_cast<const uint4*>(st) + lane;  // load j of the box: wl[32 j], units 2j and 2j + 1
  int acc[8][4];
#pragma unroll
  for (int sidx = 0; sidx < 8; ++sidx) acc[sidx][0] = acc[sidx][1] = acc[sidx][2] = acc[sidx][3] = 0;
  uint4 wbuf[2][4];
#pragma unroll
  for (int jj = 0; jj < 4; ++jj) wbuf[0][jj] = wl[32 * jj];
#pragma unroll
  for (int bt = 0; bt < 4; ++bt) {  // four loads = eight units = two sets per batch, fetched a batch ahead
    if (bt + 1 < 4) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) wbuf[(bt + 1) & 1][jj] = wl[32 * (4 * (bt + 1) + jj)];
    }
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const uint4 wv = wbuf[bt & 1][jj];
      const int sidx = 2 * bt + (jj >> 1);
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int us = 2 * (jj & 1) + h;  // unit within the set
        const uint32_t w0 = h ? wv.z : wv.x, w1 = h ? wv.w : wv.y;
        // rows g: the whole byte (row g's nibble + 16 x row g+8's); rows g+8: 16 x row g+8's nibble
        const uint32_t af[4] = {w0, w0 & 0xF0F0F0F0u, w1, w1 & 0xF0F0F0F0u};
        const bool mine = (g >> 1) == us;
        mma_u8s8(acc[sidx], af, mine ? xb[sidx].x : 0u, mine ? xb[sidx].y : 0u);
      }
    }
  }
  // unit 4 set + t: scales of rows g and g+8 (16 halves per lane: [set][row]) and the offset term
  const uint4 sc0 = *reinterpret_cast<const uint4*>(st + kBox + lane * 32);
  const uint4 sc1 = *reinterpret_cast<const uint4*>(st + kBox + lane * 32 + 16);
  const int4 of0 = *reinterpret_cast<const int4*>(c.isum + kb * 32 + t * 8);
  const int4 of1 = *reinterpret_cast<const int4*>(c.isum + kb * 32 + t * 8 + 4);
  const __half2* sh0 = reinterpret_cast<const __half2*>(&sc0);
  const __half2* sh1 = reinterpret_cast<const __half2*>(&sc1);
  const int offs[8] = {of0.x, of0.y, of0.z, of0.w, of1.x, of1.y, of1.z, of1.w};
#pragma unroll
  for (int sidx = 0; sidx < 8; ++sidx) {
    const float2 sc = __half22float2(sidx < 4 ? sh0[sidx] : sh1[sidx - 4]);
    // the unit's digit scale (a power of two: the exponent bits) and its offset term (signed, 23 bits)
    const float sxu = __int_as_float(offs[sidx] & 0x7F800000);
    const int off = (offs[sidx] << 9) >> 9;
    // acc: {row g + 16 row g+8, high digit}, {same, low digit}, {16 row g+8, high digit}, {same, low digit};
    // every term is exact in int32 (|acc| <= 32 * 255 * 128)
    const int r0 = (acc[sidx][0] - acc[sidx][2]) * 256 + (acc[sidx][1] - acc[sidx][3]) - off;
    const int r1 = ((acc[sidx][2] * 256 + acc[sidx][3]) >> 4) - off;
    tot[0] = fmaf(sc.x * sxu, static_cast<float>(r0), tot[0]);
    tot[1] = fmaf(sc.y * sxu, static_cast<float>(r1), tot[1]);
  }
}

// Where a projection's outputs go: a local vector, or (sharded, `all`) the same place in every rank's
// exchange block, written with plain peer stores.
struct Dest {
  __half* local;
  unsigned long long off;  // byte offset in the exchange block of output 0 of this rank's shard
  bool all;
  bool partial;  // the outputs are fp32 partial sums (paired sharding): no rounding, no residual here
  uint32_t* tagged = nullptr;  // tagged vectors: the outputs go here as tagged words instead (output 0 of this
  uint32_t tag = 0;            // rank's shard); with `all`, also to the same place in every other rank's block
};
// The place in rank r's exchange block that corresponds to p in this rank's.
template <typename T>
__device__ __forceinline__ T* peer_ptr(const MegaArgs& a, T* p, int r) {
  return reinterpret_cast<T*>(a.peers[r] + (reinterpret_cast<uint8_t*>(p) - a.peers[a.rank]));
}
__device__ __forceinline__ void store_out(const MegaArgs& a, const Dest& dst, int idx, __half v) {
  if (dst.tagged != nullptr) {
    st_tagged(dst.tagged + idx, v, dst.tag);
    if (dst.all)
      for (int r = 0; r < a.world; ++r)
        if (r != a.rank) st_tagged_sys(peer_ptr(a, dst.tagged, r) + idx, v, dst.tag);
  } else if (dst.all) {
    for (int r = 0; r < a.world; ++r) reinterpret_cast<__half*>(a.peers[r] + dst.off)[idx] = v;
  } else {
    dst.local[idx] = v;
  }
}

// Lanes 0..15 of one warp: output strip * 16 + lane, summed over all of K, gets its
// epilogue and is written.
__device__ __forceinline__ void finish_strip(const MegaArgs& a, int kind, int strip, float v, bool has_resid,
                                             __half resid, const Dest& out) {
  const int lane = threadIdx.x & 31;
  const int n = strip * kStripN + lane;
  if (out.partial) {
    if (lane < kStripN)
      for (int r = 0; r < a.world; ++r) reinterpret_cast<float*>(a.peers[r] + out.off)[n] = v;
    return;
  }
  const __half r = __float2half_rn(v);
  if (kind == kGu) {
    // rows interleave gate_i, up_i: even lanes hold the gate, the next lane its up value
    const float gf = __half2float(r);
    const float uf = __shfl_down_sync(0xffffffffu, gf, 1);
    if (lane < kStripN && (lane & 1) == 0) store_out(a, out, n >> 1, __float2half_rn(gf / (1.0f + __expf(-gf)) * uf));
  } else if (lane < kStripN) {
    store_out(a, out, n, has_resid ? __hadd(r, resid) : r);
  }
}

// Which warp's chunk holds box b of an op whose boxes are cut into kCW chunks: the first rn chunks have
// qn + 1 boxes, the others qn.
__device__ __forceinline__ int chunk_owner(int b, int qn, int rn) {
  const int big = rn * (qn + 1);
  if (b < big) return static_cast<int>(static_cast<unsigned>(b) / static_cast<unsigned>(qn + 1));
  return rn + static_cast<int>(static_cast<unsigned>(b - big) / static_cast<unsigned>(qn));  // qn > 0 here
}

// resid / tresid: the vector added to the outputs (element 0 = output 0 of this rank's shard), as halves or as
// tagged words written by the op with tag tresid_tag.
__device__ void run_projection(Ctx& c, int kind, const __half* resid, const Dest& out, const uint32_t* tresid = nullptr,
                               uint32_t tresid_tag = 0) {
  const MegaArgs& a = c.a;
  const ProjShape p = proj_shape(a, kind);
  const int cta = blockIdx.x, G = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  int i0, i1;
  proj_range(p, cta, G, i0, i1);
  const int B = i1 - i0;
  long long waited = 0, boxed = 0, ea = 0, eb = 0, ec = 0;
  const bool tracing = MLD_TRACING(a) && lane == 0;  // every warp keeps its own clocks
  // The op's boxes are cut into kCW contiguous chunks, one per warp (lengths differ by at most one), so
  // that a warp meets few strips; ring position kCW j + w holds box j of warp w's chunk.
  const int qn = B / kCW, rn = B % kCW;
  const int len = qn + (warp < rn ? 1 : 0);
  const int start = warp * qn + (warp < rn ? warp : rn);
  int pos = c.ring_base + warp;
  int stage = pos % a.stages;
  uint32_t phase = static_cast<uint32_t>(pos / a.stages) & 1u;
  int b = start;
  const int b_stop = start + len;
  while (b < b_stop) {
    const int sl = b / p.S;  // strip within the CTA's range
    const int strip = i0 / p.S + sl;
    const int s_lo = sl * p.S, s_hi = s_lo + p.S;
    const int b_end = b_stop < s_hi ? b_stop : s_hi;
    // the strip's residual values are fetched now: whichever warp completes the strip has them at hand
    __half rv = __float2half_rn(0.0f);
    if (tresid != nullptr) {
      if (lane < kStripN) {
        const uint32_t* rp = tresid + strip * kStripN + lane;
        rv = tagged_value(c.w, rp, tresid_tag, ld_word(rp, c.w.sys));
      }
    } else if (resid != nullptr && lane < kStripN) {
      rv = __ldcg(resid + strip * kStripN + lane);
    }
    float tot[2] = {0.0f, 0.0f};
    for (; b < b_end; ++b) {
      const long long w0 = tracing ? clock64() : 0;
      // A parity wait is only right while the barrier is at most one phase behind: the stage's previous
      // use must have been filled before its next filling is waited for.  Its having been released (what
      // the producer also waits for) says so, and that wait cannot itself be a phase off, because
      // everything up to a ring's length before this warp's previous box has been released.  The first
      // ring's length of an op needs none of this: what came before it was used up before the op began.
      if ((b - start) * kCW + warp >= a.stages) wait_released(c.w, &c.empty[stage], phase ^ 1u, 17);
      c.w.wait(&c.full[stage], phase, 12);
      if (tracing) waited += clock64() - w0;
      const long long b0 = tracing ? clock64() : 0;
      consume_box(c, c.ring + (size_t)stage * kStageBytes, b - s_lo, tot);
      __syncwarp();
      if (tracing) boxed += clock64() - b0;
      if (lane == 0) mbar_arrive_n(&c.empty[stage], kCW);
      stage += kCW;
      while (stage >= a.stages) {
        stage -= a.stages;
        phase ^= 1u;
      }
    }
    const long long e0 = tracing ? clock64() : 0;
    // sum the four unit pairs (lanes t)
    tot[0] += __shfl_xor_sync(0xffffffffu, tot[0], 1);
    tot[0] += __shfl_xor_sync(0xffffffffu, tot[0], 2);
    tot[1] += __shfl_xor_sync(0xffffffffu, tot[1], 1);
    tot[1] += __shfl_xor_sync(0xffffffffu, tot[1], 2);
    // the warps that hold boxes of this strip: w_lo .. w_hi
    const int w_lo = chunk_owner(s_lo, qn, rn), w_hi = chunk_owner(s_hi - 1, qn, rn);
    if (w_lo == w_hi) {
      // the strip is this warp's alone: rows g and g+8 sit in lanes t == 0
      const float lo = __shfl_sync(0xffffffffu, tot[0], (lane & 7) * 4);
      const float hi = __shfl_sync(0xffffffffu, tot[1], (lane & 7) * 4);
      finish_strip(a, kind, strip, (lane & 8) ? hi : lo, resid != nullptr || tresid != nullptr, rv, out);
      if (tracing) ec += clock64() - e0;
      continue;
    }
    // A warp shares at most two strips with others: the one its chunk begins in (share 0) and the one it
    // ends in (share 1, where it is w_lo).  Each share is written once per op, so nothing waits for a
    // place; the strip's arrivals are counted at w_lo.
    float* mine = c.dump + (warp * 2 + (warp == w_lo ? 1 : 0)) * kStripN;
    if (t == 0) {
      mine[g] = tot[0];
      mine[g + 8] = tot[1];
    }
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      __threadfence_block();
      last = atomicAdd(c.proj_arrived() + w_lo, 1) == w_hi - w_lo ? 1 : 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    const long long e3 = tracing ? clock64() : 0;
    if (tracing) ea += e3 - e0;
    if (last) {
      // the last warp to get here sums the shares in the order of the inputs and completes the strip
      __threadfence_block();
      float v = c.dump[(w_lo * 2 + 1) * kStripN + (lane & 15)];
      for (int w = w_lo + 1; w <= w_hi; ++w) v += c.dump[w * 2 * kStripN + (lane & 15)];
      if (lane == 0) c.proj_arrived()[w_lo] = 0;  // next used after the op's grid barrier
      finish_strip(a, kind, strip, v, resid != nullptr || tresid != nullptr, rv, out);
    }
    if (tracing) eb += clock64() - e3;
  }
  c.ring_base += B;
  if (tracing && warp == 0) {
    unsigned long long* tr = a.trace + ((size_t)blockIdx.x * a.n_layers * kOpsPerLayer + c.op_index) * kTraceSlots;
    tr[4] = static_cast<unsigned long long>(waited);
    tr[5] = static_cast<unsigned long long>(B);
    tr[7] = static_cast<unsigned long long>(boxed);
    // warp 0's clocks after its boxes: up to the arrival, after it (the sum, when it is the last), own strips
    tr[8] = static_cast<unsigned long long>(ea);
    tr[9] = static_cast<unsigned long long>(eb);
    tr[10] = static_cast<unsigned long long>(ec);
  }
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
// Byte offset of element (row, dim) of a K or V tile in its ring stage: two TMA
// boxes of 64 dims (32 rows x 128 bytes, 128-byte swizzle) behind each other.
__device__ __forceinline__ uint32_t tile_offset(int row, int dim) {
  return static_cast<uint32_t>((dim >> 6) * 4096 + row * 128 + ((((dim & 63) >> 3) ^ (row & 7)) << 4) + (dim & 7) * 2);
}

// Attention over the cached tokens 0..pos-1 plus the new token, on the tensor
// cores.  A warp takes whole (K tile, V tile) pairs of 32 tokens:
//   scores  S[token] = K[token][:] . q     MMA with A = K (tokens x dims, ldmatrix) and q in every B column
//   output  O[dim]  += V[token][dim] p     MMA with A = V^T (ldmatrix.trans) and p in every B column
// with an online softmax between them (p = exp(S - max) in fp16 for the second
// product, running sum and output rescaled when the maximum moves).  Because
// every B column holds the same vector, every accumulator column holds the same
// result and nothing has to be masked.  A warp keeps (max, sum, O[128]) over its
// tiles; warps and finally CTAs are merged when the CTA's run over a head ends.
__device__ void run_attention(Ctx& c, const MegaLayer* ly) {
  const MegaArgs& a = c.a;
  const int cta = blockIdx.x, G = gridDim.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int nt = a.pos / kTile + 1;
  const int width = a.heads * kHeadDim;
  const AttnSplit split(a.heads, nt, G);
  int i0, i1;
  split.range(cta, i0, i1);
  const Runs runs(i0, i1, nt);
  __half* sq = reinterpret_cast<__half*>(reinterpret_cast<float*>(c.xs) + warp * kWarpScratch);  // rotated, scaled q
  const uint32_t qtag = op_tag(c.epoch_base + c.op_index - 1);  // q, k, v come from the op before this one
  long long awaited = 0;
  const bool atracing = MLD_TRACING(a) && threadIdx.x == 0;
  // The first aw warps take every aw-th item of the op's sequence; an item is two ring stages.  A warp's
  // items lie 2 aw stages apart, which must not exceed the ring (2 kCW - 1 stages do for kCW warps: the
  // later stage of an item is waited for after the earlier one): shorter rings put fewer warps to work.
  const int aw = a.stages >= 2 * kCW - 1 ? kCW : a.stages / 2;
  int q = warp < aw ? warp : (1 << 30);
  int pos = c.ring_base + 2 * (warp < aw ? warp : 0);
  int stage = pos % a.stages;
  uint32_t phase = static_cast<uint32_t>(pos / a.stages) & 1u;
  int seq_lo = 0;
  for (int rr = 0; rr < runs.R; ++rr) {
    int head, lo, hi;
    runs.bounds(rr, head, lo, hi);
    const int j0 = lo - head * nt, seq_hi = seq_lo + (hi - lo);
    float m = -INFINITY, l = 0.0f;
    float out[8][4];  // O[16 db + g] in out[db][0], O[16 db + g + 8] in out[db][2] (every column alike)
#pragma unroll
    for (int db = 0; db < 8; ++db) out[db][0] = out[db][1] = out[db][2] = out[db][3] = 0.0f;
    if (q < seq_hi) {
      // rotary embedding of q (rope.cc:70-89), scaled and rounded to fp16 as the unfused graph stores it
      __syncwarp();
      uint32_t qw[4] = {0u, 0u, 0u, 0u};
      if (a.tagged) {  // all four words are asked for before any is looked at
        const uint32_t* qp = a.tq + (size_t)head * kHeadDim;
#pragma unroll
        for (int i = 0; i < 4; ++i) qw[i] = ld_word(qp + lane + 32 * (i >> 1) + (i & 1) * (kHeadDim / 2), false);
      }
#pragma unroll
      for (int rep = 0; rep < 2; ++rep) {
        const int e = lane + 32 * rep, half = kHeadDim / 2;
        const float2 rot = c.rope[e];
        float q0, q1;
        if (a.tagged) {
          const uint32_t* qp = a.tq + (size_t)head * kHeadDim;
          q0 = __half2float(tagged_value(c.w, qp + e, qtag, qw[2 * rep]));
          q1 = __half2float(tagged_value(c.w, qp + e + half, qtag, qw[2 * rep + 1]));
        } else {
          const __half* qp = a.qkv + (size_t)head * kHeadDim;
          q0 = __half2float(__ldcg(qp + e));
          q1 = __half2float(__ldcg(qp + e + half));
        }
        sq[e] = __float2half_rn((q0 * rot.x - q1 * rot.y) * a.q_scale);
        sq[e + half] = __float2half_rn((q1 * rot.x + q0 * rot.y) * a.q_scale);
      }
      __syncwarp();
      // B fragments of q for the eight 16-dim steps: dims 16 ks + 2t, +1 and 16 ks + 2t + 8, +9
      uint32_t qb[8][2];
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        qb[ks][0] = *reinterpret_cast<const uint32_t*>(sq + 16 * ks + 2 * t);
        qb[ks][1] = *reinterpret_cast<const uint32_t*>(sq + 16 * ks + 2 * t + 8);
      }
      for (; q < seq_hi; q += aw) {
        const int j = j0 + (q - seq_lo);
        int vstage = stage + 1;
        uint32_t vphase = phase;
        if (vstage == a.stages) {
          vstage = 0;
          vphase ^= 1u;
        }
        const long long w0 = atracing ? clock64() : 0;
        // (the stages' previous uses released first: see run_projection)
        if (2 * q >= a.stages) wait_released(c.w, &c.empty[stage], phase ^ 1u, 18);
        c.w.wait(&c.full[stage], phase, 13);
        if (2 * q + 1 >= a.stages) wait_released(c.w, &c.empty[vstage], vphase ^ 1u, 18);
        c.w.wait(&c.full[vstage], vphase, 14);
        if (atracing) awaited += clock64() - w0;
        uint8_t* kt = c.ring + (size_t)stage * kStageBytes;
        uint8_t* vt = c.ring + (size_t)vstage * kStageBytes;
        const bool has_new = j == nt - 1;
        if (has_new) {
          // the new token's rotated k and its v enter the cache and take their row of this tile
          const int row = a.pos & (kTile - 1);
          const __half* kp = a.qkv + (size_t)(a.heads + head) * kHeadDim;
          const __half* vp = a.qkv + (size_t)(2 * a.heads + head) * kHeadDim;
          __half* kc = ly->kcache + (size_t)a.pos * width + head * kHeadDim;
          __half* vc = ly->vcache + (size_t)a.pos * width + head * kHeadDim;
          uint32_t kw[4] = {0u, 0u, 0u, 0u}, vw[4] = {0u, 0u, 0u, 0u};
          if (a.tagged) {
            const uint32_t* tk = a.tq + (size_t)(a.heads + head) * kHeadDim;
            const uint32_t* tv = a.tq + (size_t)(2 * a.heads + head) * kHeadDim;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              kw[i] = ld_word(tk + lane + 32 * (i >> 1) + (i & 1) * (kHeadDim / 2), false);
              vw[i] = ld_word(tv + lane + 32 * (i >> 1) + (i & 1) * (kHeadDim / 2), false);
            }
          }
#pragma unroll
          for (int rep = 0; rep < 2; ++rep) {
            const int e = lane + 32 * rep, half = kHeadDim / 2;
            const float2 rot = c.rope[e];
            float k0, k1;
            __half v0, v1;
            if (a.tagged) {
              const uint32_t* tk = a.tq + (size_t)(a.heads + head) * kHeadDim;
              const uint32_t* tv = a.tq + (size_t)(2 * a.heads + head) * kHeadDim;
              k0 = __half2float(tagged_value(c.w, tk + e, qtag, kw[2 * rep]));
              k1 = __half2float(tagged_value(c.w, tk + e + half, qtag, kw[2 * rep + 1]));
              v0 = tagged_value(c.w, tv + e, qtag, vw[2 * rep]);
              v1 = tagged_value(c.w, tv + e + half, qtag, vw[2 * rep + 1]);
            } else {
              k0 = __half2float(__ldcg(kp + e));
              k1 = __half2float(__ldcg(kp + e + half));
              v0 = __ldcg(vp + e);
              v1 = __ldcg(vp + e + half);
            }
            const __half r0 = __float2half_rn(k0 * rot.x - k1 * rot.y), r1 = __float2half_rn(k1 * rot.x + k0 * rot.y);
            kc[e] = r0;
            kc[e + half] = r1;
            vc[e] = v0;
            vc[e + half] = v1;
            *reinterpret_cast<__half*>(kt + tile_offset(row, e)) = r0;
            *reinterpret_cast<__half*>(kt + tile_offset(row, e + half)) = r1;
            *reinterpret_cast<__half*>(vt + tile_offset(row, e)) = v0;
            *reinterpret_cast<__half*>(vt + tile_offset(row, e + half)) = v1;
          }
          // rows past the new token are not tokens yet: whatever the cache holds there must not reach
          // the products (0 * NaN), so they read as zero
          for (int zr = row + 1; zr < kTile; ++zr)
            *reinterpret_cast<uint2*>(vt + tile_offset(zr, 4 * lane)) = make_uint2(0u, 0u);
          __syncwarp();
        }
        // ---- scores: two blocks of 16 tokens, eight steps of 16 dims
        float sc[2][4];
#pragma unroll
        for (int mb = 0; mb < 2; ++mb) {
          sc[mb][0] = sc[mb][1] = sc[mb][2] = sc[mb][3] = 0.0f;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            uint32_t af[4];
            // lane i addresses row (i & 7) of 8x8 matrix i >> 3: rows +8 for odd matrices, dims +8 for matrices 2, 3
            const int row = 16 * mb + ((lane >> 3) & 1) * 8 + (lane & 7);
            const int dim = 16 * ks + (lane >> 4) * 8;
            ldmatrix_x4(af, smem_u32(kt) + tile_offset(row, dim));
            mma_f16(sc[mb], af, qb[ks][0], qb[ks][1]);
          }
        }
        // this lane's tokens: g, g+8 (block 0) and 16+g, 24+g (block 1); every column of S is the same
        float s4[4] = {sc[0][0], sc[0][2], sc[1][0], sc[1][2]};
        float mt = -INFINITY;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int token = j * kTile + g + 8 * e;
          if (token > a.pos) s4[e] = -INFINITY;
          mt = fmaxf(mt, s4[e]);
        }
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 4));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 8));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
        const float m_new = fmaxf(m, mt);  // finite: token 32 j is never beyond pos
        float p4[4], psum = 0.0f;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          p4[e] = __expf(s4[e] - m_new);
          psum += p4[e];
        }
        psum += __shfl_xor_sync(0xffffffffu, psum, 4);
        psum += __shfl_xor_sync(0xffffffffu, psum, 8);
        psum += __shfl_xor_sync(0xffffffffu, psum, 16);
        if (m_new != m) {  // warp-uniform
          const float corr = __expf(m - m_new);
          l *= corr;
#pragma unroll
          for (int db = 0; db < 8; ++db) {
            out[db][0] *= corr;
            out[db][1] *= corr;
            out[db][2] *= corr;
            out[db][3] *= corr;
          }
          m = m_new;
        }
        l += psum;
        // B fragments of p: tokens 16 ts + 2t, +1 (b0) and 16 ts + 2t + 8, +9 (b1), which sit in lanes
        // g' = 2t and 2t + 1 (any t): lanes 8t and 8t + 4
        uint32_t pb[2][2];
#pragma unroll
        for (int ts = 0; ts < 2; ++ts) {
          const float pa = __shfl_sync(0xffffffffu, p4[2 * ts], 8 * t);
          const float pbv = __shfl_sync(0xffffffffu, p4[2 * ts], 8 * t + 4);
          const float pc = __shfl_sync(0xffffffffu, p4[2 * ts + 1], 8 * t);
          const float pd = __shfl_sync(0xffffffffu, p4[2 * ts + 1], 8 * t + 4);
          const __half2 h0 = __floats2half2_rn(pa, pbv), h1 = __floats2half2_rn(pc, pd);
          pb[ts][0] = *reinterpret_cast<const uint32_t*>(&h0);
          pb[ts][1] = *reinterpret_cast<const uint32_t*>(&h1);
        }
        // ---- output: eight blocks of 16 dims, two steps of 16 tokens, A = V^T
#pragma unroll
        for (int db = 0; db < 8; ++db) {
#pragma unroll
          for (int ts = 0; ts < 2; ++ts) {
            uint32_t af[4];
            // source 8x8 blocks (tokens x dims): matrix i >> 3 -> dims +8 for odd matrices, tokens +8 for matrices 2, 3
            const int row = 16 * ts + (lane >> 4) * 8 + (lane & 7);
            const int dim = 16 * db + ((lane >> 3) & 1) * 8;
            ldmatrix_x4_trans(af, smem_u32(vt) + tile_offset(row, dim));
            mma_f16(out[db], af, pb[ts][0], pb[ts][1]);
          }
        }
        if (has_new) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // this warp wrote into the tiles
        __syncwarp();
        if (lane == 0) {
          mbar_arrive_n(&c.empty[stage], kCW);
          mbar_arrive_n(&c.empty[vstage], kCW);
        }
        stage += 2 * aw;
        while (stage >= a.stages) {
          stage -= a.stages;
          phase ^= 1u;
        }
      }
    }
    const int run = c.attn_runs + rr, slot = run % kAttnSlots, use = run / kAttnSlots;
    c.w.wait_count(c.attn_done() + slot, use, 16);
    float* mine = c.dump + ((size_t)slot * kCW + warp) * kAttDump;
    if (t == 0) {
#pragma unroll
      for (int db = 0; db < 8; ++db) {
        mine[16 * db + g] = out[db][0];
        mine[16 * db + g + 8] = out[db][2];
      }
      if (g == 0) {
        mine[kHeadDim] = m;
        mine[kHeadDim + 1] = l;
      }
    }
    __syncwarp();
    int last = 0;
    if (lane == 0) {
      __threadfence_block();
      last = atomicAdd(c.attn_arrived() + slot, 1) == kCW - 1 ? 1 : 0;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    unsigned long long* trs = MLD_TRACING(a) && lane == 0
                                  ? a.trace + ((size_t)blockIdx.x * a.n_layers * kOpsPerLayer + c.op_index) * kTraceSlots
                                  : nullptr;
    if (last) {
      if (trs) trs[8] = globaltimer_ns();
      // the CTA's last warp merges the warps in order; lane owns dims 4*lane..+4
      __threadfence_block();
      const float* all = c.dump + (size_t)slot * kCW * kAttDump;
      float M = -INFINITY;
#pragma unroll
      for (int wi = 0; wi < kCW; ++wi) M = fmaxf(M, all[wi * kAttDump + kHeadDim]);
      float o[4] = {0.0f, 0.0f, 0.0f, 0.0f}, ls = 0.0f;
#pragma unroll
      for (int wi = 0; wi < kCW; ++wi) {
        const float mw = all[wi * kAttDump + kHeadDim];
        const float ww = mw == -INFINITY ? 0.0f : __expf(mw - M);
        ls = fmaf(ww, all[wi * kAttDump + kHeadDim + 1], ls);
#pragma unroll
        for (int e = 0; e < 4; ++e) o[e] = fmaf(ww, all[wi * kAttDump + 4 * lane + e], o[e]);
      }
      __syncwarp();
      if (lane == 0) {
        c.attn_arrived()[slot] = 0;
        __threadfence_block();
        c.attn_done()[slot] = use + 1;
      }
      int first, lastc;
      split.contributors(head, first, lastc);
      bool write = true;
      if (split.P > 1 && lastc > first) {
        // The head's parts publish their partial and a flag; the part with the last tile (which also has
        // the new token, so the most to do) waits for them and merges: parts in order, its own last.
        const unsigned epoch = c.epoch_base + static_cast<unsigned>(c.op_index) + 1u;
        const int part = cta - first, pm = lastc - first;  // pm: the part with the head's last tile
        unsigned* flags = a.att_flags + (size_t)head * split.P;
        if (part < pm) {
          float* pp = a.att_part + (size_t)cta * kAttSlots * kAttDump;
          *reinterpret_cast<float4*>(pp + 4 * lane) = make_float4(o[0], o[1], o[2], o[3]);
          if (lane == 0) {
            pp[kHeadDim] = M;
            pp[kHeadDim + 1] = ls;
          }
          if (trs) trs[9] = globaltimer_ns();
          __syncwarp();  // the release below is cumulative over the other lanes' stores
          if (lane == 0) asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flags + part), "r"(epoch) : "memory");
          if (trs) trs[10] = globaltimer_ns();
          write = false;
        } else {
          if (trs) trs[9] = globaltimer_ns();
          for (int base = 0; base < pm; base += 32) {
            const int u = base + lane;
            if (u < pm && !*c.w.s_fail) {
              const unsigned long long t0 = globaltimer_ns();
              for (;;) {
                unsigned fv;
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(fv) : "l"(flags + u) : "memory");
                if (fv == epoch) break;
                if (globaltimer_ns() - t0 > c.w.limit || *c.w.s_fail) {
                  *c.w.s_fail = 1;
                  atomicCAS(a.error, 0, 21);
                  break;
                }
              }
            }
          }
          __syncwarp();
          if (trs) trs[10] = globaltimer_ns();
          float TM = -INFINITY, po[4] = {0.0f, 0.0f, 0.0f, 0.0f}, pl = 0.0f;
          for (int base = 0; base < pm; base += 8) {
            int myoff = -1;
            {
              const int u = base + (lane & 7);
              if (u < pm) myoff = (first + u) * kAttSlots * kAttDump;
            }
            float mc[8], lc[8];
            float4 oc[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int off = __shfl_sync(0xffffffffu, myoff, u);
              mc[u] = -INFINITY;
              lc[u] = 0.0f;
              oc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
              if (off >= 0) {
                const float* pp = a.att_part + off;
                mc[u] = __ldcg(pp + kHeadDim);
                lc[u] = __ldcg(pp + kHeadDim + 1);
                oc[u] = __ldcg(reinterpret_cast<const float4*>(pp + 4 * lane));
              }
            }
            float NM = TM;
#pragma unroll
            for (int u = 0; u < 8; ++u) NM = fmaxf(NM, mc[u]);
            const float resc = TM == -INFINITY ? 0.0f : __expf(TM - NM);
            po[0] *= resc;
            po[1] *= resc;
            po[2] *= resc;
            po[3] *= resc;
            pl *= resc;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const float wc = mc[u] == -INFINITY ? 0.0f : __expf(mc[u] - NM);
              po[0] = fmaf(wc, oc[u].x, po[0]);
              po[1] = fmaf(wc, oc[u].y, po[1]);
              po[2] = fmaf(wc, oc[u].z, po[2]);
              po[3] = fmaf(wc, oc[u].w, po[3]);
              pl = fmaf(wc, lc[u], pl);
            }
            TM = NM;
          }
          // this part's own share last
          const float FM = fmaxf(TM, M);
          const float wa = TM == -INFINITY ? 0.0f : __expf(TM - FM), wb = M == -INFINITY ? 0.0f : __expf(M - FM);
#pragma unroll
          for (int e = 0; e < 4; ++e) o[e] = po[e] * wa + o[e] * wb;
          ls = pl * wa + ls * wb;
        }
      } else if (split.P == 0 && first != lastc) {
        const int ps = head - i0 / nt;
        float* part = a.att_part + ((size_t)cta * kAttSlots + ps) * kAttDump;
        *reinterpret_cast<float4*>(part + 4 * lane) = make_float4(o[0], o[1], o[2], o[3]);
        if (lane == 0) {
          part[kHeadDim] = M;
          part[kHeadDim + 1] = ls;
        }
        if (trs) trs[9] = globaltimer_ns();
        __threadfence();
        __syncwarp();
        // contributors: the CTAs first..lastc whose range is not empty; lane u looks at CTA base + u
        int need = 0;
        for (int base = first; base <= lastc; base += 32) {
          const int cc = base + lane;
          bool has = false;
          if (cc <= lastc) {
            int c0, c1;
            split.range(cc, c0, c1);
            has = c0 != c1;
          }
          need += __popc(__ballot_sync(0xffffffffu, has));
        }
        int done = 0;
        if (lane == 0) {
          const int tk = atomicAdd(a.att_tickets + head, 1);
          if (trs) trs[10] = globaltimer_ns();
          done = tk == need - 1 ? 1 : 0;
          if (done) a.att_tickets[head] = 0;
        }
        write = __shfl_sync(0xffffffffu, done, 0) != 0;
        if (write) {
          __threadfence();
          float TM = -INFINITY;
          o[0] = o[1] = o[2] = o[3] = 0.0f;
          ls = 0.0f;
          for (int base = first; base <= lastc; base += 8) {
            // lane u < 8 finds the partial of CTA base + u (offset in floats, -1 if none); all lanes then load
            int myoff = -1;
            {
              const int cc = base + (lane & 7);
              if (cc <= lastc) {
                int c0, c1;
                split.range(cc, c0, c1);
                if (c0 != c1) myoff = (cc * kAttSlots + (head - c0 / nt)) * kAttDump;
              }
            }
            float mc[8], lc[8];
            float4 oc[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const int off = __shfl_sync(0xffffffffu, myoff, u);
              mc[u] = -INFINITY;
              lc[u] = 0.0f;
              oc[u] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
              if (off >= 0) {
                const float* pp = a.att_part + off;
                mc[u] = __ldcg(pp + kHeadDim);
                lc[u] = __ldcg(pp + kHeadDim + 1);
                oc[u] = __ldcg(reinterpret_cast<const float4*>(pp + 4 * lane));
              }
            }
            float NM = TM;
#pragma unroll
            for (int u = 0; u < 8; ++u) NM = fmaxf(NM, mc[u]);
            const float resc = TM == -INFINITY ? 0.0f : __expf(TM - NM);
            o[0] *= resc;
            o[1] *= resc;
            o[2] *= resc;
            o[3] *= resc;
            ls *= resc;
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const float wc = mc[u] == -INFINITY ? 0.0f : __expf(mc[u] - NM);
              o[0] = fmaf(wc, oc[u].x, o[0]);
              o[1] = fmaf(wc, oc[u].y, o[1]);
              o[2] = fmaf(wc, oc[u].z, o[2]);
              o[3] = fmaf(wc, oc[u].w, o[3]);
              ls = fmaf(wc, lc[u], ls);
            }
            TM = NM;
          }
        }
      }
      if (write) {
        const float inv = 1.0f / ls;
        __half2 r01 = __floats2half2_rn(o[0] * inv, o[1] * inv), r23 = __floats2half2_rn(o[2] * inv, o[3] * inv);
        uint2 pk;
        pk.x = *reinterpret_cast<uint32_t*>(&r01);
        pk.y = *reinterpret_cast<uint32_t*>(&r23);
        // this rank's heads sit at rank * d_local in the full vector, which every rank needs
        if (a.tagged) {
          const uint32_t tg = op_tag(c.epoch_base + c.op_index) << 16;
          uint32_t* dst = a.tattn + (size_t)a.rank * a.d_local + (size_t)head * kHeadDim + 4 * lane;
          asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(tg | (pk.x & 0xFFFFu)),
                       "r"(tg | (pk.x >> 16)), "r"(tg | (pk.y & 0xFFFFu)), "r"(tg | (pk.y >> 16))
                       : "memory");
          for (int r = 0; r < a.world; ++r)
            if (r != a.rank)
              asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(peer_ptr(a, dst, r)),
                           "r"(tg | (pk.x & 0xFFFFu)), "r"(tg | (pk.x >> 16)), "r"(tg | (pk.y & 0xFFFFu)),
                           "r"(tg | (pk.y >> 16))
                           : "memory");
        } else if (a.paired) {  // o is split by input columns: this rank's heads are all it reads
          *reinterpret_cast<uint2*>(a.attn + (size_t)head * kHeadDim + 4 * lane) = pk;
        } else {
          const size_t at = (size_t)a.rank * a.d_local + (size_t)head * kHeadDim + 4 * lane;
          for (int r = 0; r < a.world; ++r)
            *reinterpret_cast<uint2*>(reinterpret_cast<__half*>(a.peers[r] + a.off_attn) + at) = pk;
        }
        if (trs) trs[11] = globaltimer_ns();
      }
    }
    seq_lo = seq_hi;
  }
  if (atracing) {  // thread 0's time waiting for tiles and the CTA's number of items
    unsigned long long* tr = a.trace + ((size_t)blockIdx.x * a.n_layers * kOpsPerLayer + c.op_index) * kTraceSlots;
    tr[4] = static_cast<unsigned long long>(awaited);
    tr[5] = static_cast<unsigned long long>(i1 - i0);
  }
  c.attn_runs += runs.R;
  c.ring_base += 2 * (i1 - i0);
}

__global__ void __launch_bounds__(kThreads, 1) decode_mega_kernel(const __grid_constant__ MegaArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  __half* xs = reinterpret_cast<__half*>(ring + (size_t)a.stages * kStageBytes);
  float* us = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xs) + a.xs_bytes);
  float* dump = us + a.us_floats;
  float2* rope = reinterpret_cast<float2*>(dump + kDumpFloats);
  uint64_t* full = reinterpret_cast<uint64_t*>(rope + kHeadDim / 2);
  uint64_t* empty = full + a.stages;
  int* s_int = reinterpret_cast<int*>(empty + a.stages);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kCW);  // attention tiles are read by every warp; a weight box's one reader arrives kCW-fold
    }
    for (int i = 0; i < kSharedInts; ++i) s_int[i] = 0;
    // Arrival count of the grid barrier when this launch began (a multiple of the grid size; read before
    // this CTA's first arrival it lies in [base, base + grid)).  base / grid numbers the barriers of all
    // launches so far and gives every op of every launch a unique epoch.
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(a.bar) : "memory");
    v -= v % gridDim.x;
    *reinterpret_cast<unsigned long long*>(s_int + kSharedInts + 1) = v;
    unsigned long long xv = 0;
    if (a.world > 1) {  // the cross-rank counter: arrivals of all ranks' CTAs
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(xv) : "l"(a.peers[a.rank] + a.off_xbar) : "memory");
      xv -= xv % ((unsigned long long)gridDim.x * a.world);
    }
    *reinterpret_cast<unsigned long long*>(s_int + kSharedInts + 3) = xv;
    fence_barrier_init();
  }
  if (threadIdx.x >= 32 && threadIdx.x < 32 + kHeadDim / 2) {
    // rotary embedding of this position (rope.cc:70-89): timescale_i = min * (max / min)^(2i / d)
    const int e = threadIdx.x - 32;
    const float fraction = 2.0f * e / static_cast<float>(kHeadDim);
    const float timescale = a.min_ts * powf(a.max_ts / a.min_ts, fraction);
    float sn, cs;
    sincosf(static_cast<float>(a.pos) / timescale, &sn, &cs);
    rope[e] = make_float2(cs, sn);
  }
  __syncthreads();
  Waiter w{s_int, a.error, a.wait_limit_ns, a.world > 1};

  if (warp == kCW) {
    if (lane == 0) producer_loop(a, ring, full, empty, w);
  } else {
    Ctx c{a, ring, full, empty, xs, reinterpret_cast<int*>(us), rope, dump, s_int, w, 0, 0, 0ull, 0ull, 0u, 0};
    c.bar_target = *reinterpret_cast<const unsigned long long*>(s_int + kSharedInts + 1);
    c.xbar_target = *reinterpret_cast<const unsigned long long*>(s_int + kSharedInts + 3);
    // every launch completes at least one local barrier, so five epochs per barrier keep launches apart
    c.epoch_base = static_cast<unsigned>(c.bar_target / gridDim.x) * kOpsPerLayer * (a.tagged ? a.n_layers : 1);
    const int d = a.d_model;
    const bool sharded = a.world > 1;
    const size_t shard = (size_t)a.rank * a.d_local;  // first output of this rank in h / x
    if (!a.paired) {
      for (int l = 0; l < a.n_layers; ++l) {
        const MegaLayer* ly = a.layers + l;
        const bool last = l + 1 == a.n_layers;
        const __half* x_cur = l == 0 ? a.x_in : (((l - 1) & 1) ? a.xb : a.xa);
        // the last layer writes the caller's vector directly, unless peers have to write it too
        __half* x_next = (last && !sharded) ? a.x_out : ((l & 1) ? a.xb : a.xa);
        Dest d_qkv{a.qkv, 0ull, false, false};
        Dest d_h{a.h + shard, a.off_h + shard * 2, sharded, false};
        Dest d_act{a.act + (size_t)a.rank * a.ffn_local, a.off_act + (size_t)a.rank * a.ffn_local * 2, sharded, false};
        Dest d_x{x_next + shard, ((l & 1) ? a.off_xb : a.off_xa) + shard * 2, sharded, false};
        Src s_x{x_cur, nullptr, 0, 0, nullptr}, s_attn{a.attn, nullptr, 0, 0, nullptr}, s_h{a.h, nullptr, 0, 0, nullptr},
            s_act{a.act, nullptr, 0, 0, nullptr};
        const uint32_t* tres_o = nullptr;
        const uint32_t* tres_down = nullptr;
        uint32_t tres_o_tag = 0, tres_down_tag = 0;
        const bool tg = a.tagged != 0;
        uint32_t* tx_next = (l & 1) ? a.txb : a.txa;
        if (tg) {
          // tagged vectors: every op's outputs carry the op's number, readers wait word by word
          const unsigned e0 = c.epoch_base + l * kOpsPerLayer;
          d_qkv.tagged = a.tq, d_qkv.tag = op_tag(e0 + kQkv);
          d_h.tagged = a.th + shard, d_h.tag = op_tag(e0 + kO);
          d_act.tagged = a.tact + (size_t)a.rank * a.ffn_local, d_act.tag = op_tag(e0 + kGu);
          // (one GPU: the last layer writes the caller's vector directly)
          if (!last || sharded) d_x.tagged = tx_next + shard, d_x.tag = op_tag(e0 + kDown);
          if (l > 0) {
            s_x.tx = ((l - 1) & 1) ? a.txb : a.txa, s_x.tag = op_tag(e0 - 1);  // down of the layer before
            tres_o = s_x.tx + shard, tres_o_tag = s_x.tag;
          }
          s_attn.tx = a.tattn, s_attn.tag = op_tag(e0 + kAttn);
          s_h.tx = a.th, s_h.tag = op_tag(e0 + kO);
          s_act.tx = a.tact, s_act.tag = op_tag(e0 + kGu);
          tres_down = a.th + shard, tres_down_tag = s_h.tag;
        }
        // With tagged vectors a CTA without strips of a projection has no business with its input vector
        // (with barriers every CTA keeps the same sequence of block-wide steps).
        auto has_items = [&](int kind) {
          if (!tg) return true;
          int j0, j1;
          proj_range(proj_shape(a, kind), blockIdx.x, gridDim.x, j0, j1);
          return j1 > j0;
        };
        c.op_index = l * kOpsPerLayer;
        trace_mark(c, 0);
        if (has_items(kQkv)) {
          load_x<true>(c, s_x, ly->norm1, d);
          trace_mark(c, 1);
          run_projection(c, kQkv, nullptr, d_qkv);
        }
        trace_mark(c, 2);
        op_boundary(c, tg, false);  // q, k, v stay on this rank
        trace_mark(c, 3);

        c.op_index += 1;
        trace_mark(c, 0);
        run_attention(c, ly);
        trace_mark(c, 2);
        op_boundary(c, tg, true);
        trace_mark(c, 3);

        c.op_index += 1;
        trace_mark(c, 0);
        if (has_items(kO)) {
          load_x<false>(c, s_attn, nullptr, d);
          trace_mark(c, 1);
          run_projection(c, kO, tres_o != nullptr ? nullptr : x_cur + shard, d_h, tres_o, tres_o_tag);
        }
        trace_mark(c, 2);
        op_boundary(c, tg, true);
        trace_mark(c, 3);

        c.op_index += 1;
        trace_mark(c, 0);
        if (has_items(kGu)) {
          load_x<true>(c, s_h, ly->norm2, d);
          trace_mark(c, 1);
          run_projection(c, kGu, nullptr, d_act);
        }
        trace_mark(c, 2);
        op_boundary(c, tg, true);
        trace_mark(c, 3);

        c.op_index += 1;
        trace_mark(c, 0);
        if (has_items(kDown)) {
          load_x<false>(c, s_act, nullptr, a.ffn);
          trace_mark(c, 1);
          run_projection(c, kDown, tg ? nullptr : a.h + shard, d_x, tres_down, tres_down_tag);
        }
        trace_mark(c, 2);
        if (tg && last)
          grid_barrier(c);  // one barrier per launch keeps the launches' op numbers apart
        else
          op_boundary(c, tg, true);
        trace_mark(c, 3);
        if (last && sharded && blockIdx.x == 0) {
          // the step's result, assembled from all ranks' shards, goes to the caller's vector
          for (int i = threadIdx.x * 8; i < d; i += kCW * 32 * 8) {
            if (tg)
              *reinterpret_cast<uint4*>(a.x_out + i) = ld_tagged8(c.w, tx_next + i, d_x.tag);
            else
              *reinterpret_cast<uint4*>(a.x_out + i) = __ldcg(reinterpret_cast<const uint4*>(x_next + i));
          }
        }
      }
    } else {
      // Paired sharding: q/k/v and gate/up are split by outputs, o and down by inputs, so attention's
      // output and the activations never leave the rank; o and down produce fp32 partial sums of the
      // whole vector, stored on every rank, and the next vector load adds them up (rank order) onto the
      // residual.  Two barriers of a layer span the ranks instead of four.
      const float* ph = reinterpret_cast<const float*>(a.peers[a.rank] + a.off_ph);
      const float* pd = reinterpret_cast<const float*>(a.peers[a.rank] + a.off_pd);
      const Dest d_qkv{a.qkv, 0ull, false, false};
      const Dest d_act{a.act, 0ull, false, false};
      const Dest d_ph{nullptr, a.off_ph + (size_t)a.rank * d * 4, true, true};
      const Dest d_pd{nullptr, a.off_pd + (size_t)a.rank * d * 4, true, true};
      for (int l = 0; l < a.n_layers; ++l) {
        const MegaLayer* ly = a.layers + l;
        // layer input: the caller's vector, or h of the layer before (a.h) plus its down partials; kept in
        // a.xa because it is the residual of this layer's h
        const Src s_x = l == 0 ? Src{a.x_in, nullptr, 0, 0, nullptr} : Src{a.h, pd, a.world, d, a.xa};
        const __half* x_res = l == 0 ? a.x_in : a.xa;
        c.op_index = l * kOpsPerLayer;
        trace_mark(c, 0);
        load_x<true>(c, s_x, ly->norm1, d);
        trace_mark(c, 1);
        run_projection(c, kQkv, nullptr, d_qkv);
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
        load_x<false>(c, Src{a.attn, nullptr, 0, 0, nullptr}, nullptr, a.d_local);
        trace_mark(c, 1);
        run_projection(c, kO, nullptr, d_ph);
        trace_mark(c, 2);
        grid_barrier(c, true);
        trace_mark(c, 3);

        c.op_index += 1;
        trace_mark(c, 0);
        load_x<true>(c, Src{x_res, ph, a.world, d, a.h}, ly->norm2, d);  // h = x + o
        trace_mark(c, 1);
        run_projection(c, kGu, nullptr, d_act);
        trace_mark(c, 2);
        grid_barrier(c);
        trace_mark(c, 3);

        c.op_index += 1;
        trace_mark(c, 0);
        load_x<false>(c, Src{a.act, nullptr, 0, 0, nullptr}, nullptr, a.ffn_local);
        trace_mark(c, 1);
        run_projection(c, kDown, nullptr, d_pd);
        trace_mark(c, 2);
        grid_barrier(c, true);
        trace_mark(c, 3);
      }
      if (blockIdx.x == 0) {
        // the step's result: h of the last layer plus its down partials
        const Src s_out{a.h, pd, a.world, d, a.x_out};
        for (int i = threadIdx.x * 8; i < d; i += kCW * 32 * 8) fetch8(c.w, s_out, i);
      }
    }
  }
  // A CTA that gave up may still have copies in flight: give them time to land
  // before its shared memory is released.
  __syncthreads();
  if (s_int[0] != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
}

// ------------------------------------------------------------ weight re-tiling
// Reference layout in: weights [K/4][N/4] blocks of 4 inputs x 4 outputs, 8
// bytes each (nibble (k%4)*4 + (n%4), even nibbles in the low half of a byte;
// fully_connected_util.cc / tensor_utils.h RearrangeWeights... I4O4 layouts),
// scales fp16 [K/block][N].  Out: [strip][k box] records of kStageBytes, laid
// out as consume_box reads them.  One thread per 32-bit word of the output.
__global__ void __launch_bounds__(256) retile_weights_kernel(const uint8_t* __restrict__ w, const __half* __restrict__ sc,
                                                             uint8_t* __restrict__ out, int N, int K, int block) {
  const int S = (K + kBoxK - 1) / kBoxK;
  const int64_t words_per_box = kStageBytes / 4;
  const int64_t total = (int64_t)(N / kStripN) * S * words_per_box;
  const int N4 = N / 4;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t box = idx / words_per_box;
    const int wi = static_cast<int>(idx - box * words_per_box);
    const int strip = static_cast<int>(box / S), kb = static_cast<int>(box - (int64_t)strip * S);
    uint32_t word = 0;
    if (wi < kBox / 4) {
      // weights: word = [load j][lane][q]; unit 2j + (q >> 1) of the box, inputs 16 (q & 1) + 4t + {0..3} of the
      // unit: byte b = input b, low nibble row g, high nibble row g + 8
      const int j = wi >> 7, lane = (wi >> 2) & 31, q = wi & 3;
      const int g = lane >> 2, t = lane & 3;
      const int unit = 2 * j + (q >> 1);
#pragma unroll
      for (int nib = 0; nib < 8; ++nib) {
        const int row = (nib & 1) ? g + 8 : g;
        const int k = kb * kBoxK + unit * 32 + (q & 1) * 16 + 4 * t + (nib >> 1);
        const int n = strip * kStripN + row;
        uint32_t v = 0;
        if (k < K) {
          const uint8_t* blk = w + ((size_t)(k >> 2) * N4 + (n >> 2)) * 8;
          const int e = (k & 3) * 4 + (n & 3);
          const uint8_t byte = blk[e >> 1];
          v = (e & 1) ? (byte >> 4) : (byte & 15);
        }
        word |= v << (4 * nib);
      }
    } else {
      // scales: [lane][set][row g / g+8] halves (unit 4 set + t), two per word
      const int hi = (wi - kBox / 4) * 2;  // first half index of this word
      uint32_t pair = 0;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int h = hi + q;
        const int lane = h >> 4, r = h & 15;
        const int g = lane >> 2, t = lane & 3;
        const int u = 4 * (r >> 1) + t;
        const int k = kb * kBoxK + u * 32;
        const int n = strip * kStripN + ((r & 1) ? g + 8 : g);
        uint16_t bits = 0;
        if (k < K) bits = __half_as_ushort(sc[(size_t)(k / block) * N + n]);
        pair |= static_cast<uint32_t>(bits) << (16 * q);
      }
      word = pair;
    }
    reinterpret_cast<uint32_t*>(out)[idx] = word;
  }
}

}  // namespace

// ------------------------------------------------------------------ host side
struct MegaDecoder {
  MegaConfig cfg;
  int sms, grid, stages, xs_bytes, us_floats, l2_ahead;
  size_t smem_bytes;
  MegaLayer* d_layers;
  std::vector<MegaLayer> h_layers;
  std::vector<char> layer_set;
  uint8_t* scratch;
  int tagged;
  uint32_t *tq, *tattn, *th, *tact, *txa, *txb;  // tagged-word vectors (tq in scratch, the others in xchg)
  size_t off_tagged, tagged_bytes, tq_bytes, flags_bytes;
  uint8_t* xchg;              // exchange block (vectors every rank needs + the cross-rank barrier counter)
  uint8_t* peers[8];          // every rank's exchange block as mapped here (own entry = xchg)
  size_t off_attn, off_h, off_act, off_xa, off_xb, off_xbar, off_ph, off_pd;
  int heads_local, d_local, ffn_local;
  bool paired;
  bool peers_ready;
  uint8_t* prepared;          // re-tiled weights of all layers
  size_t proj_bytes[4], layer_bytes;
  __half *qkv, *attn, *h, *act, *xa, *xb;
  float* att_part;
  int *att_tickets, *error;
  unsigned* att_flags;
  unsigned* bar;
  unsigned long long* trace;
};

bool mega_supported(const MegaConfig& c) {
  if (c.head_dim != kHeadDim || c.heads < 1) return false;
  if (c.d_model != c.heads * kHeadDim) return false;
  if (c.world < 1 || c.world > 8 || c.rank < 0 || c.rank >= c.world) return false;
  if (c.heads % c.world != 0 || c.ffn % (32 * c.world) != 0) return false;
  if (c.shard_layout == 1 && ((c.d_model / c.world) % c.block != 0 || (c.ffn / c.world) % c.block != 0)) return false;
  if (c.block != 32 && c.block != 64 && c.block != 128 && c.block != 256) return false;
  if (c.d_model % c.block != 0 || c.ffn % c.block != 0) return false;
  return get_encode_tiled() != nullptr;
}

void mega_destroy(MegaDecoder* m) {
  if (m == nullptr) return;
  if (m->d_layers != nullptr) cudaFree(m->d_layers);
  if (m->scratch != nullptr) cudaFree(m->scratch);
  for (int r = 0; r < 8; ++r)
    if (m->peers[r] != nullptr && m->peers[r] != m->xchg) cudaIpcCloseMemHandle(m->peers[r]);
  if (m->xchg != nullptr) cudaFree(m->xchg);
  if (m->prepared != nullptr) cudaFree(m->prepared);
  if (m->trace != nullptr) cudaFree(m->trace);
  delete m;
}

int mega_create(const MegaConfig& cfg, MegaDecoder** out) {
  MLD_REQUIRE(mega_supported(cfg), "decoder shape not supported by the persistent step kernel");
  MegaDecoder* m = new MegaDecoder();
  m->cfg = cfg;
  m->d_layers = nullptr;
  m->scratch = nullptr;
  m->xchg = nullptr;
  for (int r = 0; r < 8; ++r) m->peers[r] = nullptr;
  m->peers_ready = cfg.world == 1;
  m->prepared = nullptr;
  m->trace = nullptr;
  m->heads_local = cfg.heads / cfg.world;
  m->d_local = cfg.d_model / cfg.world;
  m->ffn_local = cfg.ffn / cfg.world;
  m->paired = cfg.world > 1 && cfg.shard_layout == 1;
  m->sms = sm_count(cfg.device);
  // shared memory: ring + max(input vector padded to whole boxes, per-warp attention scratch) + unit sums +
  // run slots + rope table + barriers
  const int att_bytes = kCW * kWarpScratch * 4;
  const int vec_elems = align_n(cfg.d_model > cfg.ffn ? cfg.d_model : cfg.ffn, kBoxK);
  const int vec_bytes = vec_elems * 2;
  m->xs_bytes = align_n(att_bytes > vec_bytes ? att_bytes : vec_bytes, 128);
  m->us_floats = vec_elems / 32;
  const int fixed = 1024 + m->xs_bytes + m->us_floats * 4 + kDumpFloats * 4 + (kHeadDim / 2) * 8 + (kSharedInts + 5) * 4 + 64;
  int max_smem = 0;
  cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, cfg.device);
  int stages = (max_smem - fixed) / (kStageBytes + 16);
  if (cfg.ring_stages >= 2 && cfg.ring_stages < stages) stages = cfg.ring_stages;
  if (stages > 64) stages = 64;
  if (stages < kCW + 1) {  // every consumer warp needs a stage of its own in a round
    set_last_error_text("not enough shared memory for the persistent step kernel");
    mega_destroy(m);
    return MLD_UNIMPLEMENTED;
  }
  m->stages = stages;
  m->l2_ahead = 0;  // measured: asking L2 for the next op ahead of the ring's loads slows the step down
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
  if (cfg.grid_limit >= 1 && cfg.grid_limit < m->grid) m->grid = cfg.grid_limit;
  // an attention range must not touch more than kAttSlots heads: ceil(n/nt)+1 with n = ceil(heads*nt/grid)
  // is at most ceil(heads/grid + 1/nt) + 1 <= heads/grid + 3
  if ((int64_t)m->heads_local * (cfg.max_seq / kTile + 1) * m->grid >= (int64_t(1) << 31) ||
      (int64_t)(3 * cfg.d_model > 2 * cfg.ffn ? 3 * cfg.d_model : 2 * cfg.ffn) / kStripN * m->grid >= (int64_t(1) << 31)) {
    set_last_error_text("decoder too large for the persistent step kernel's 32-bit work split");
    mega_destroy(m);
    return MLD_UNIMPLEMENTED;
  }
  if (m->heads_local / m->grid + 3 > kAttSlots) {
    set_last_error_text("too many heads per CTA for the persistent step kernel");
    mega_destroy(m);
    return MLD_UNIMPLEMENTED;
  }
  const int d = cfg.d_model, ffn = cfg.ffn;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t o = off;
    off += (bytes + 255) & ~size_t(255);
    return o;
  };
  const int dl = m->d_local, fl = m->ffn_local;
  const size_t o_qkv = take((size_t)3 * dl * 2), o_ap = take((size_t)m->grid * kAttSlots * kAttDump * 4),
               o_at = take((size_t)m->heads_local * 4), o_af = take((size_t)(m->grid + m->heads_local) * 4),
               o_bar = take(8), o_err = take(4);
  // the op-to-op vectors as tagged words unless the descriptor asks for grid barriers (the split of o and down
  // by input columns exchanges fp32 partial sums and keeps the barriers)
  m->tagged = (cfg.handover == 0 && !m->paired) ? 1 : 0;
  const size_t o_tq = take(m->tagged ? (size_t)3 * dl * 4 : 0);
  const size_t scratch_bytes = off;
  off = 0;  // the exchange block: same layout on every rank
  m->off_attn = take((size_t)d * 2);
  m->off_h = take((size_t)d * 2);
  m->off_act = take((size_t)ffn * 2);
  m->off_xa = take((size_t)d * 2);
  m->off_xb = take((size_t)d * 2);
  m->off_xbar = take(8);
  m->off_ph = take(m->paired ? (size_t)cfg.world * d * 4 : 0);
  m->off_pd = take(m->paired ? (size_t)cfg.world * d * 4 : 0);
  // the vectors every rank reads in full, as tagged words (peers write their shards into them)
  m->off_tagged = off;
  const size_t o_ta = take(m->tagged ? (size_t)d * 4 : 0), o_th = take(m->tagged ? (size_t)d * 4 : 0),
               o_tact = take(m->tagged ? (size_t)ffn * 4 : 0), o_txa = take(m->tagged ? (size_t)d * 4 : 0),
               o_txb = take(m->tagged ? (size_t)d * 4 : 0);
  m->tagged_bytes = off - m->off_tagged;
  const size_t xchg_bytes = off;
  const int Ns[4] = {3 * dl, m->paired ? d : dl, 2 * fl, m->paired ? d : dl};
  const int Ks[4] = {d, m->paired ? dl : d, d, m->paired ? fl : ffn};
  m->layer_bytes = 0;
  for (int i = 0; i < 4; ++i) {
    m->proj_bytes[i] = (size_t)(Ns[i] / kStripN) * div_up(Ks[i], kBoxK) * kStageBytes;
    m->layer_bytes += m->proj_bytes[i];
  }
  if (cudaMalloc(&m->scratch, scratch_bytes) != cudaSuccess || cudaMalloc(&m->xchg, xchg_bytes) != cudaSuccess ||
      cudaMalloc(&m->d_layers, sizeof(MegaLayer) * cfg.layers) != cudaSuccess ||
      cudaMalloc(&m->prepared, m->layer_bytes * cfg.layers) != cudaSuccess) {
    set_last_error_text("persistent step kernel: device allocation failed");
    mega_destroy(m);
    return MLD_CUDA_ERROR;
  }
  cudaMemset(m->scratch, 0, scratch_bytes);
  cudaMemset(m->xchg, 0, xchg_bytes);
  m->peers[cfg.rank] = m->xchg;
  m->qkv = reinterpret_cast<__half*>(m->scratch + o_qkv);
  m->attn = reinterpret_cast<__half*>(m->xchg + m->off_attn);
  m->h = reinterpret_cast<__half*>(m->xchg + m->off_h);
  m->act = reinterpret_cast<__half*>(m->xchg + m->off_act);
  m->xa = reinterpret_cast<__half*>(m->xchg + m->off_xa);
  m->xb = reinterpret_cast<__half*>(m->xchg + m->off_xb);
  m->tq = reinterpret_cast<uint32_t*>(m->scratch + o_tq);
  m->tq_bytes = m->tagged ? (size_t)3 * dl * 4 : 0;
  m->tattn = reinterpret_cast<uint32_t*>(m->xchg + o_ta);
  m->th = reinterpret_cast<uint32_t*>(m->xchg + o_th);
  m->tact = reinterpret_cast<uint32_t*>(m->xchg + o_tact);
  m->txa = reinterpret_cast<uint32_t*>(m->xchg + o_txa);
  m->txb = reinterpret_cast<uint32_t*>(m->xchg + o_txb);
  m->flags_bytes = (size_t)(m->grid + m->heads_local) * 4;
  m->att_part = reinterpret_cast<float*>(m->scratch + o_ap);
  m->att_tickets = reinterpret_cast<int*>(m->scratch + o_at);
  m->att_flags = reinterpret_cast<unsigned*>(m->scratch + o_af);
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
  const int Ns[4] = {3 * m->d_local, m->paired ? d : m->d_local, 2 * m->ffn_local, m->paired ? d : m->d_local};
  const int Ks[4] = {d, m->paired ? m->d_local : d, d, m->paired ? m->ffn_local : ffn};
  const void* ws[4] = {p.wqkv, p.wo, p.wgu, p.wdown};
  const void* ss[4] = {p.sqkv, p.so, p.sgu, p.sdown};
  uint8_t* dst = m->prepared + (size_t)layer * m->layer_bytes;
  for (int i = 0; i < 4; ++i) {
    const int64_t words = static_cast<int64_t>(m->proj_bytes[i] / 4);
    const int blocks = static_cast<int>(words / 256 < 4096 ? (words + 255) / 256 : 4096);
    retile_weights_kernel<<<blocks, 256>>>(static_cast<const uint8_t*>(ws[i]), static_cast<const __half*>(ss[i]), dst,
                                           Ns[i], Ks[i], c.block);
    MLD_LAUNCH_CHECK();
    L.w[i] = dst;
    dst += m->proj_bytes[i];
  }
  const uint64_t kv_row = (uint64_t)m->heads_local * kHeadDim * 2;
  int rc = make_tmap_2d(&L.kc, p.kcache, kv_row, c.max_seq, kv_row, kHeadDim, kTile, 2, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MLD_OK) return rc;
  rc = make_tmap_2d(&L.vc, p.vcache, kv_row, c.max_seq, kv_row, kHeadDim, kTile, 2, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MLD_OK) return rc;
  L.norm1 = static_cast<const __half*>(p.norm1);
  L.norm2 = static_cast<const __half*>(p.norm2);
  L.kcache = static_cast<__half*>(p.kcache);
  L.vcache = static_cast<__half*>(p.vcache);
  MLD_CUDA_CHECK(cudaMemcpy(m->d_layers + layer, &L, sizeof L, cudaMemcpyHostToDevice));
  m->layer_set[layer] = 1;
  return MLD_OK;
}

int mega_ipc_export(MegaDecoder* m, void* handle64) {
  cudaIpcMemHandle_t h;
  MLD_CUDA_CHECK(cudaIpcGetMemHandle(&h, m->xchg));
  memcpy(handle64, &h, sizeof h);
  return MLD_OK;
}
int mega_ipc_import(MegaDecoder* m, const void* handles) {
  for (int r = 0; r < m->cfg.world; ++r) {
    if (r == m->cfg.rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * 64, sizeof h);
    void* p = nullptr;
    MLD_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    m->peers[r] = static_cast<uint8_t*>(p);
  }
  m->peers_ready = true;
  return MLD_OK;
}

#ifdef MLD_TRACE
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
#endif
int mega_grid(const MegaDecoder* m) { return m->grid; }

const int* mega_error_word(const MegaDecoder* m) { return m->error; }

// Back to the state after creation: counters zero, no tagged word or flag valid.  (Tags and flag epochs
// derive from the launch counter; restarting it is safe only because everything that carries a tag or an
// epoch is cleared with it.)
int mega_reset(MegaDecoder* m) {
  MLD_CUDA_CHECK(cudaMemset(m->error, 0, sizeof(int)));
  MLD_CUDA_CHECK(cudaMemset(m->bar, 0, 8));
  MLD_CUDA_CHECK(cudaMemset(m->xchg + m->off_xbar, 0, 8));
  MLD_CUDA_CHECK(cudaMemset(m->att_tickets, 0, (size_t)m->heads_local * 4));
  MLD_CUDA_CHECK(cudaMemset(m->att_flags, 0, m->flags_bytes));
  if (m->tagged) {
    MLD_CUDA_CHECK(cudaMemset(m->tq, 0, m->tq_bytes));
    MLD_CUDA_CHECK(cudaMemset(m->xchg + m->off_tagged, 0, m->tagged_bytes));
  }
  MLD_CUDA_CHECK(cudaDeviceSynchronize());
  return MLD_OK;
}
void mega_set_wait_limit(MegaDecoder* m, int us) { m->cfg.wait_limit_us = us; }

int mega_device_status(MegaDecoder* m, int* code) {
  MLD_CUDA_CHECK(cudaMemcpy(code, m->error, sizeof(int), cudaMemcpyDeviceToHost));
  if (*code != 0) return mega_reset(m);
  return MLD_OK;
}

int mega_step(MegaDecoder* m, const void* x_in, void* x_out, int pos, cudaStream_t stream) {
  for (char s : m->layer_set) MLD_REQUIRE(s != 0, "layer weights not set");
  MegaArgs a;
  memset(&a, 0, sizeof a);
  const MegaConfig& c = m->cfg;
  a.layers = m->d_layers;
  a.n_layers = c.layers;
  MLD_REQUIRE(m->peers_ready, "sharded decoder: exchange blocks not imported yet (mld_decoder_ipc_import)");
  a.d_model = c.d_model;
  a.heads = m->heads_local;
  a.ffn = c.ffn;
  a.world = c.world;
  a.rank = c.rank;
  a.d_local = m->d_local;
  a.ffn_local = m->ffn_local;
  a.paired = m->paired ? 1 : 0;
  a.off_ph = m->off_ph;
  a.off_pd = m->off_pd;
  for (int r = 0; r < 8; ++r) a.peers[r] = m->peers[r];
  a.off_attn = m->off_attn;
  a.off_h = m->off_h;
  a.off_act = m->off_act;
  a.off_xa = m->off_xa;
  a.off_xb = m->off_xb;
  a.off_xbar = m->off_xbar;
  a.pos = pos;
  a.stages = m->stages;
  a.l2_ahead = m->l2_ahead;
  a.xs_bytes = m->xs_bytes;
  a.us_floats = m->us_floats;
  a.rms_eps = c.rms_eps;
  a.min_ts = c.rope_min_timescale;
  a.max_ts = c.rope_max_timescale;
  a.q_scale = 1.0f / sqrtf(static_cast<float>(kHeadDim));
  a.x_in = static_cast<const __half*>(x_in);
  a.x_out = static_cast<__half*>(x_out);
  a.tagged = m->tagged;
  a.wait_limit_ns = static_cast<unsigned long long>(m->cfg.wait_limit_us > 0 ? m->cfg.wait_limit_us : 2000000) * 1000ull;
  a.tq = m->tq;
  a.tattn = m->tattn;
  a.th = m->th;
  a.tact = m->tact;
  a.txa = m->txa;
  a.txb = m->txb;
  a.qkv = m->qkv;
  a.attn = m->attn;
  a.h = m->h;
  a.act = m->act;
  a.xa = m->xa;
  a.xb = m->xb;
  a.att_part = m->att_part;
  a.att_tickets = m->att_tickets;
  a.att_flags = m->att_flags;
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
