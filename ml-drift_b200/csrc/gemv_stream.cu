// Decode-stage dequant-GEMV, streaming form (1..8 tokens per launch) over the
// reference's packed weight layout [K/4][N/4][4 k][4 n].
//
// The kernel is HBM-bound, so it is organised around keeping the memory system
// busy and the exit path short:
//  * the grid is one CTA per SM; each CTA owns a contiguous strip of output
//    columns (16-byte granularity, so the strips balance to within one chunk)
//    and streams every K row of that strip - no split-K traffic through global
//    memory.  When the matrix is too narrow for 148 useful strips, two CTAs of
//    a thread-block cluster share a strip, take half of K each and combine
//    through distributed shared memory;
//  * packed weights (128-byte-swizzled boxes), block scales and activations are
//    staged by TMA / bulk copies into a ring of shared-memory stages, all
//    completing on one mbarrier per stage;
//  * eight consumer warps dequantise in registers and feed m16n8k16 tensor-core
//    MMAs (weights as the 16-row operand, tokens as columns), fp32 accumulate;
//    4-bit weights with a single token go through integer MMAs on 16-bit
//    fixed-point activations instead (the DIGITS form below);
//  * with programmatic dependent launch the next GEMV starts streaming its
//    weights while this one drains; only the activation loads wait for the
//    predecessor.
//
// Arithmetic restated from GetFullyConnectedKernelCode
// (ml_drift/common/kernels/fully_connected.cc:623-942) and fc:: helpers
// (fully_connected_util.cc:80-229, 356-407); accumulation is fp32 for both
// fp16 precision modes.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "kernels.h"

namespace mld {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kStageRows = kConsumerWarps * 8;  // k-slices per stage (256 input channels)
constexpr int kBoxBytes = kStageRows * 128;     // one weight box: 64 rows x 128 bytes

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8s8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(x), "r"(mask), "r"(orv));  // (x & mask) | orv
  return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// Fragment geometry.  Lane = 4*g + t.  One warp step covers four k-slice rows
// (row of lane = base + 2*t + parity) of one 128-byte box row; lane g owns 16
// bytes (one "chunk") of it.
//   BITS 4: a chunk = two 4x4 blocks (8 outputs) -> 4 MMAs, 64 outputs per box
//   BITS 8: a chunk = one 4x4 block  (4 outputs) -> 2 MMAs, 32 outputs per box
// MMA f of a lane: rows g / g+8 are outputs NPL*g + 2*f + {0,1} of the box; the
// sixteen k columns are (row t: k0 k1) at 2t,2t+1 and (row t: k2 k3) at 2t+8,9.
template <int BITS>
struct Frag {
  static constexpr int NF = BITS == 4 ? 4 : 2;   // MMAs (accumulator fragments) per lane and box
  static constexpr int NPL = BITS == 4 ? 8 : 4;  // outputs per chunk
  static constexpr int BOX_N = NPL * 8;          // outputs per box (64 / 32)
};

// EXACT operands: (1024 + u) with the offset removed by one packed half
// subtract, giving the signed weight exactly (x16 for high nibbles).
// SUBNORMAL operands: the raw masked bits, i.e. fp16 subnormals u * 2^-24 (x16
// for high nibbles); the "- shift * sum(x)" term comes from one extra MMA per
// step against a constant operand, and results carry a 2^-24 factor.
template <int BITS, bool SUBNORMAL>
__device__ __forceinline__ void unpack(const uint4& q, uint32_t (&a)[Frag<BITS>::NF][4]) {
  if constexpr (BITS == 4) {
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};  // blockA.lo(k0k1) blockA.hi(k2k3) blockB.lo blockB.hi
#pragma unroll
    for (int b = 0; b < 2; ++b) {
      const uint32_t lo = w[2 * b], hi = w[2 * b + 1];
      const uint32_t lo8 = lo >> 8, hi8 = hi >> 8;
      if constexpr (SUBNORMAL) {
        a[2 * b][0] = lo & 0x000F000Fu;
        a[2 * b][1] = lo & 0x00F000F0u;
        a[2 * b][2] = hi & 0x000F000Fu;
        a[2 * b][3] = hi & 0x00F000F0u;
        a[2 * b + 1][0] = lo8 & 0x000F000Fu;
        a[2 * b + 1][1] = lo8 & 0x00F000F0u;
        a[2 * b + 1][2] = hi8 & 0x000F000Fu;
        a[2 * b + 1][3] = hi8 & 0x00F000F0u;
      } else {
        const uint32_t kLo = 0x64086408u;  // half2(1032): 1024 + 8
        const uint32_t kHi = 0x64806480u;  // half2(1152): 1024 + 16*8
        a[2 * b][0] = hsub2_u32(lop3_and_or(lo, 0x000F000Fu, 0x64006400u), kLo);
        a[2 * b][1] = hsub2_u32(lop3_and_or(lo, 0x00F000F0u, 0x64006400u), kHi);
        a[2 * b][2] = hsub2_u32(lop3_and_or(hi, 0x000F000Fu, 0x64006400u), kLo);
        a[2 * b][3] = hsub2_u32(lop3_and_or(hi, 0x00F000F0u, 0x64006400u), kHi);
        a[2 * b + 1][0] = hsub2_u32(lop3_and_or(lo8, 0x000F000Fu, 0x64006400u), kLo);
        a[2 * b + 1][1] = hsub2_u32(lop3_and_or(lo8, 0x00F000F0u, 0x64006400u), kHi);
        a[2 * b + 1][2] = hsub2_u32(lop3_and_or(hi8, 0x000F000Fu, 0x64006400u), kLo);
        a[2 * b + 1][3] = hsub2_u32(lop3_and_or(hi8, 0x00F000F0u, 0x64006400u), kHi);
      }
    }
  } else {
    // bytes: q.x = k0:(n0..n3), q.y = k1, q.z = k2, q.w = k3
    const uint32_t p01 = prmt(q.x, q.y, 0x5140u);  // [k0n0 k1n0 k0n1 k1n1]
    const uint32_t p23 = prmt(q.z, q.w, 0x5140u);
    const uint32_t r01 = prmt(q.x, q.y, 0x7362u);  // [k0n2 k1n2 k0n3 k1n3]
    const uint32_t r23 = prmt(q.z, q.w, 0x7362u);
    if constexpr (SUBNORMAL) {
      a[0][0] = prmt(p01, 0u, 0x4140u);
      a[0][1] = prmt(p01, 0u, 0x4342u);
      a[0][2] = prmt(p23, 0u, 0x4140u);
      a[0][3] = prmt(p23, 0u, 0x4342u);
      a[1][0] = prmt(r01, 0u, 0x4140u);
      a[1][1] = prmt(r01, 0u, 0x4342u);
      a[1][2] = prmt(r23, 0u, 0x4140u);
      a[1][3] = prmt(r23, 0u, 0x4342u);
    } else {
      const uint32_t kM = 0x64646464u;
      const uint32_t kOff = 0x64806480u;  // half2(1152) = 1024 + 128
      a[0][0] = hsub2_u32(prmt(p01, kM, 0x4140u), kOff);
      a[0][1] = hsub2_u32(prmt(p01, kM, 0x4342u), kOff);
      a[0][2] = hsub2_u32(prmt(p23, kM, 0x4140u), kOff);
      a[0][3] = hsub2_u32(prmt(p23, kM, 0x4342u), kOff);
      a[1][0] = hsub2_u32(prmt(r01, kM, 0x4140u), kOff);
      a[1][1] = hsub2_u32(prmt(r01, kM, 0x4342u), kOff);
      a[1][2] = hsub2_u32(prmt(r23, kM, 0x4140u), kOff);
      a[1][3] = hsub2_u32(prmt(r23, kM, 0x4342u), kOff);
    }
  }
}

// --------------------------------------------------------- cluster primitives
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_rank(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(addr) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait_cluster(bar, parity)) return true;
    if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
  }
}

#define MLD_CONSUMER_BARRIER() asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory")

// W: weight boxes per stage (strip width up to W * 128 bytes per pass).
// MONE: single-token launch (only token column 0 is kept).
// DIGITS (4-bit weights, one token, a one-token activation vector): integer MMAs instead.  The whole
// activation vector is fetched once, and before the first stage is consumed the warps turn every unit
// of 32 inputs into 16-bit fixed point with a power-of-two scale of its own, x ~ s (256 hi + lo).  One
// m16n8k32 u8 x s8 MMA per 16 outputs and unit then multiplies the nibbles, as the bytes of the reference
// layout that hold two outputs each, by the unit's two digits; four units share accumulators (their
// digits sit in different B columns), so a stage costs 64 MMAs where the fp16 form needs 144, with two
// byte permutes per MMA instead of shifts and masks.  Everything is exact in int32; the error is that
// of the fixed point, at most 2^-16 of the unit's largest input per input.
template <int BITS, int W, bool SUBNORMAL, bool MONE, bool DIGITS = false>
__global__ void __launch_bounds__((kConsumerWarps + 1) * 32, W <= 2 ? 2 : 1)
    fc_strip_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_s,
                    StripArgs a) {
  using F = Frag<BITS>;
  constexpr int WT = W * F::BOX_N;       // outputs per pass
  constexpr int NJ = MONE ? 2 : 4;       // accumulator values kept per fragment
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  float* red = reinterpret_cast<float*>(smem + (size_t)a.stages * a.stage_bytes);  // [warps][WT][red_m]
  float* peer = red + kConsumerWarps * WT * a.red_m;                                // [WT][red_m]
  uint64_t* full = reinterpret_cast<uint64_t*>(peer + ((WT * a.red_m + 1) & ~1));
  uint64_t* empty = full + a.stages;
  uint64_t* peer_bar = empty + a.stages;
  // DIGITS: the activation vector of this CTA's K range, digitised in place ([unit][hi: 8 words][lo: 8 words],
  // word j = the four inputs of k-slice j), then per unit {bits of the digit scale, 8 x the sum of its integers}
  uint64_t* xbar = peer_bar + 1;
  uint8_t* xdig = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(xbar + 1) + 15) & ~uintptr_t(15));
  uint2* xmeta = reinterpret_cast<uint2*>(xdig + (size_t)a.rows_per_split * 8);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kr = a.ksplit > 1 ? static_cast<int>(cluster_ctarank()) : 0;
  const int strip = blockIdx.x / a.ksplit;

  // strip -> chunk range (16-byte chunks of a weight row), balanced to one unit
  const int64_t u_lo = (int64_t)strip * a.units / a.strips, u_hi = (int64_t)(strip + 1) * a.units / a.strips;
  const int cs = static_cast<int>(u_lo) * a.gran, ce = static_cast<int>(u_hi) * a.gran;
  const int passes = (ce - cs + W * 8 - 1) / (W * 8);
  const int r_lo = kr * a.rows_per_split;
  const int r_hi = min(a.src_slices, r_lo + a.rows_per_split);
  const int n_st = (r_hi - r_lo + kStageRows - 1) / kStageRows;

#ifdef MLD_TRACE  // per-CTA timestamps for tuning, compiled in only on request
  unsigned long long* tr = a.trace != nullptr ? a.trace + (size_t)blockIdx.x * 8 : nullptr;
#else
  constexpr unsigned long long* tr = nullptr;
#endif
  // The producer thread initialises the barriers and goes straight on to issue
  // its first loads; the consumers wait for the initialisation on a named
  // barrier the producer warp only arrives at.
  if (warp == kConsumerWarps) {
    if (lane == 0) {
      if (tr) tr[0] = globaltimer_ns();
      for (int s = 0; s < a.stages; ++s) {
        mbar_init(&full[s], 1);
        mbar_init(&empty[s], kConsumerWarps);
      }
      mbar_init(peer_bar, kConsumerWarps * 32);
      if constexpr (DIGITS) mbar_init(xbar, 1);
      fence_barrier_init();
    }
    __syncwarp();
    asm volatile("bar.arrive 2, %0;" ::"n"((kConsumerWarps + 1) * 32) : "memory");
  } else {
    asm volatile("bar.sync 2, %0;" ::"n"((kConsumerWarps + 1) * 32) : "memory");
  }
  // cluster partners: arrive now, wait only before the first remote access
  if (a.ksplit > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  if (a.pdl) pdl_launch_dependents();

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------ producer
    if (n_st > 0) {
      const uint64_t pol = policy_evict_first();
      const int total = passes * n_st;
      const uint32_t s_bytes = a.scale_rows > 0 ? static_cast<uint32_t>(a.scale_rows) * WT * 2u : 0u;
      auto issue_weights = [&](int item, int stage) {
        const int pass = item / n_st, si = item % n_st;
        uint8_t* st = smem + (size_t)stage * a.stage_bytes;
        const int row0 = r_lo + si * kStageRows;
        const int rows = min(kStageRows, r_hi - row0);
        const int chunk0 = cs + pass * W * 8;
        mbar_arrive_expect_tx(&full[stage],
                              W * kBoxBytes + s_bytes + (DIGITS ? 0u : static_cast<uint32_t>(rows) * a.M_total * 8u));
#pragma unroll
        for (int b = 0; b < W; ++b)
          tma_load_2d_hint(st + b * kBoxBytes, &tmap_w, &full[stage], (chunk0 + b * 8) * 16, row0, pol);
        if (a.scale_rows > 0)
          tma_load_2d(st + W * kBoxBytes, &tmap_s, &full[stage], chunk0 * F::NPL, row0 / a.group_slices);
      };
      auto issue_x = [&](int item, int stage) {
        if constexpr (DIGITS) return;  // the whole vector is fetched once, below
        const int si = item % n_st;
        uint8_t* st = smem + (size_t)stage * a.stage_bytes;
        const int row0 = r_lo + si * kStageRows;
        const int rows = min(kStageRows, r_hi - row0);
        bulk_load_1d(st + W * kBoxBytes + a.scale_stage_bytes,
                     static_cast<const uint8_t*>(a.x) + (size_t)row0 * a.M_total * 8,
                     static_cast<uint32_t>(rows) * a.M_total * 8u, &full[stage]);
      };
      // weights and scales are constants: the first ring-full of them is
      // requested before waiting for the preceding kernel; activations after.
      // Launches that overlap completely request the whole ring at once, one lane per stage.  A launch that
      // hands over at the activation load requests it stage by stage: measured, its burst only gets in the way
      // of the launch ahead of it, which is still streaming.
      const int head = total < a.stages ? total : a.stages;
      if (a.pdl == 2) {
        if (lane < head) issue_weights(lane, lane);
        __syncwarp();
      }
      if (lane != 0) return;
      if (a.pdl != 2)
        for (int it = 0; it < head; ++it) issue_weights(it, it);
      if (tr) tr[1] = globaltimer_ns();
      if (a.pdl == 1) pdl_wait();  // pdl == 2: the caller declared x and y untouched by the launch before
      if (a.wait.world > 1) {
        const unsigned seq = static_cast<unsigned>(*a.wait.step * a.wait.seq_per_step + a.wait.seq_off);
        if (!wait_peer_flags(a.wait.flags, a.wait.world, seq, a.wait.limit_ns)) atomicExch(a.error, kErrPeerWait);
      }
      if (tr) tr[2] = globaltimer_ns();
      if constexpr (DIGITS) {
        const uint32_t xbytes = static_cast<uint32_t>(r_hi - r_lo) * 8u;
        mbar_arrive_expect_tx(xbar, xbytes);
        bulk_load_1d(xdig, static_cast<const uint8_t*>(a.x) + (size_t)r_lo * 8, xbytes, xbar);
      }
      for (int it = 0; it < head; ++it) issue_x(it, it);
      int stage = head == a.stages ? 0 : head;
      uint32_t phase = head == a.stages ? 1 : 0;
      for (int it = head; it < total; ++it) {
        if (!mbar_wait(&empty[stage], phase ^ 1)) {
          atomicExch(a.error, 1);
          break;
        }
        issue_weights(it, stage);
        issue_x(it, stage);
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
      // Everything this CTA needs has been requested: use the memory system's
      // idle tail (epilogue, the glue kernels that follow) to pull this CTA's
      // share of the next projection's weights into L2.
      // Launches that did not wait above still complete in stream order: the grid is not done before the
      // grid ahead of it is.
      if (a.pdl == 2) pdl_wait();
      if (a.next_w != nullptr) {
        const unsigned long long per = ((a.next_w_bytes / gridDim.x) + 127ull) & ~127ull;
        unsigned long long lo = per * blockIdx.x, hi = lo + per;
        if (hi > a.next_w_bytes) hi = a.next_w_bytes & ~15ull;
        for (; lo < hi; lo += 16384ull) {
          const unsigned long long n = hi - lo < 16384ull ? hi - lo : 16384ull;
          bulk_prefetch_l2(static_cast<const uint8_t*>(a.next_w) + lo, static_cast<uint32_t>(n & ~15ull));
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int g = lane >> 2, t = lane & 3;
  constexpr uint32_t kOnesA = BITS == 4 ? 0x00080008u : 0x00800080u;  // subnormal 8 / 128
  constexpr float kOdd = BITS == 4 ? 0.0625f : 1.0f;                  // high nibbles are carried x16
  constexpr float kOutScale = (SUBNORMAL && !DIGITS) ? 16777216.0f : 1.0f;
  const int rbase = warp * 8;
  int stage = 0;
  uint32_t phase = 0;
  bool failed = false;
#ifdef MLD_TRACE
  long long tr_wait_cycles = 0, tr_busy_cycles = 0;
#endif

  if constexpr (DIGITS) {
    if (n_st > 0) {
      if (!mbar_wait(xbar, 0)) {
        atomicExch(a.error, 2);
        failed = true;
      }
      // this warp digitises unit si * 8 + warp of every stage si; lane = 4 * (stage of the round) + chunk, a chunk
      // being eight inputs (k-slices 2q and 2q + 1 of the unit)
      for (int si0 = 0; si0 < n_st && !failed; si0 += 8) {
        const int si = si0 + (lane >> 2), q = lane & 3;
        const bool have = si < n_st;
        const int u = si * 8 + warp;
        const int row = r_lo + u * 8 + 2 * q;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (have && row < r_hi) {
          v = *reinterpret_cast<const uint4*>(xdig + (size_t)u * 64 + q * 16);
          if (row + 1 >= r_hi) v.z = v.w = 0u;
        }
        __syncwarp();  // the unit's four lanes have read before any of them rewrites it
        float xf[8];
        {
          const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
          const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
          const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z));
          const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
          xf[0] = f0.x; xf[1] = f0.y; xf[2] = f1.x; xf[3] = f1.y;
          xf[4] = f2.x; xf[5] = f2.y; xf[6] = f3.x; xf[7] = f3.y;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(xf[i]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        // the smallest power of two s with amax / s <= 32512 (a float with an empty mantissa); 1 / s is exact
        uint32_t sbits = (__float_as_uint(amax * (1.0f / 32512.0f)) + 0x007FFFFFu) & 0x7F800000u;
        if (sbits < (16u << 23)) sbits = 16u << 23;
        const float inv = __uint_as_float((254u << 23) - sbits);
        // an infinity or NaN among the unit's inputs (an all-ones fp16 exponent) has no digits: the unit's scale
        // becomes NaN, and with it every output, as the reference arithmetic would make most of them
        const auto non_finite = [](uint32_t w) { return (w & 0x7C00u) == 0x7C00u || (w & 0x7C000000u) == 0x7C000000u; };
        unsigned bad = (non_finite(v.x) || non_finite(v.y) || non_finite(v.z) || non_finite(v.w)) ? 1u : 0u;
        bad |= __shfl_xor_sync(0xffffffffu, bad, 1);
        bad |= __shfl_xor_sync(0xffffffffu, bad, 2);
        // z = round(x / s) + 128 in the low 16 bits of the sum's mantissa: byte 1 = high digit, byte 0 ^ 0x80 = low digit
        uint32_t z[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) z[i] = __float_as_uint(fmaf(xf[i], inv, 12583040.0f));
        uint32_t hiw[2], low[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const uint32_t h01 = prmt(z[4 * e], z[4 * e + 1], 0x0051u), h23 = prmt(z[4 * e + 2], z[4 * e + 3], 0x0051u);
          const uint32_t l01 = prmt(z[4 * e], z[4 * e + 1], 0x0040u), l23 = prmt(z[4 * e + 2], z[4 * e + 3], 0x0040u);
          hiw[e] = prmt(h01, h23, 0x5410u);
          low[e] = prmt(l01, l23, 0x5410u) ^ 0x80808080u;
        }
        int isum = __dp4a(static_cast<int>(hiw[0]), 0x01010101, 0);
        isum = __dp4a(static_cast<int>(hiw[1]), 0x01010101, isum) * 256;
        isum = __dp4a(static_cast<int>(low[0]), 0x01010101, isum);
        isum = __dp4a(static_cast<int>(low[1]), 0x01010101, isum);
        isum += __shfl_xor_sync(0xffffffffu, isum, 1);
        isum += __shfl_xor_sync(0xffffffffu, isum, 2);
        if (have) {
          uint32_t* ud = reinterpret_cast<uint32_t*>(xdig + (size_t)u * 64);
          *reinterpret_cast<uint2*>(ud + 2 * q) = make_uint2(hiw[0], hiw[1]);
          *reinterpret_cast<uint2*>(ud + 8 + 2 * q) = make_uint2(low[0], low[1]);
          if (q == 0) xmeta[u] = make_uint2(bad ? 0x7FC00000u : sbits, static_cast<uint32_t>(8 * isum));  // (nibbles = weights + 8)
        }
      }
    }
    MLD_CONSUMER_BARRIER();  // a warp multiplies by units other warps digitised
  }

  for (int pass = 0; pass < passes && !failed; ++pass) {
    float tot[W][F::NF][NJ];
#pragma unroll
    for (int b = 0; b < W; ++b)
#pragma unroll
      for (int f = 0; f < F::NF; ++f)
#pragma unroll
        for (int j = 0; j < NJ; ++j) tot[b][f][j] = 0.0f;

    for (int si = 0; si < n_st; ++si) {
#ifdef MLD_TRACE
      const long long tw0 = clock64();
#endif
      if (!mbar_wait(&full[stage], phase)) {
        atomicExch(a.error, 2);
        failed = true;
        break;
      }
#ifdef MLD_TRACE
      const long long tw1 = clock64();
      tr_wait_cycles += tw1 - tw0;
      if (a.trace_skip_math) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[stage]);
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1;
        }
        continue;
      }
#endif
      if (tr && threadIdx.x == 0 && pass == 0 && si == 0) tr[3] = globaltimer_ns();
      const uint8_t* st = smem + (size_t)stage * a.stage_bytes;
      const uint8_t* xs = st + W * kBoxBytes + a.scale_stage_bytes;
      const int row0 = r_lo + si * kStageRows;
      if constexpr (DIGITS) {
        static_assert(!DIGITS || (BITS == 4 && MONE), "the digit form is for 4-bit weights and one token");
        // A stage is 2 W tasks: (half of its 64 k-slice rows = four units) x (box of 64 outputs).  The four
        // units of a task share accumulators: B column 2 j holds the high and 2 j + 1 the low digits of unit j
        // (lanes g supply column g, zero for the other units), so after the units' MMAs lane t holds both
        // digit sums of unit t and finishes that unit.  With fewer tasks than warps, groups of warps take
        // the stages in turn; every warp still waits for and releases every stage.
        constexpr int T = W == 3 ? 8 : 2 * W;
        constexpr int GC = kConsumerWarps / T;
        const int task = warp % T, tb = task >> 1, hq = task & 1;
        if (tb < W && si % GC == warp / T) {
          const int ubase = si * 8 + hq * 4;  // the task's first unit within the CTA's K range
          const uint32_t* ud = reinterpret_cast<const uint32_t*>(xdig + (size_t)(ubase + (g >> 1)) * 64) + 8 * (g & 1);
          const uint32_t bm0 = ud[t], bm1 = ud[4 + t];
          int acc[4][4];
#pragma unroll
          for (int f = 0; f < 4; ++f) acc[f][0] = acc[f][1] = acc[f][2] = acc[f][3] = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            // k-slice rows ra and ra + 4 of unit j are what lane t feeds the MMA's K with
            const int ra = 32 * hq + 8 * j + t, rb = ra + 4;
            const uint4 qa = *reinterpret_cast<const uint4*>(st + tb * kBoxBytes + ra * 128 + ((g ^ (ra & 7)) << 4));
            const uint4 qb = *reinterpret_cast<const uint4*>(st + tb * kBoxBytes + rb * 128 + ((g ^ (rb & 7)) << 4));
            const bool mine = (g >> 1) == j;
            const uint32_t b0 = mine ? bm0 : 0u, b1 = mine ? bm1 : 0u;
#pragma unroll
            for (int f = 0; f < 4; ++f) {
              // outputs 2f (low nibbles) and 2f + 1 (high nibbles) of this lane's eight: byte i of a block word is
              // input i / 2, output pair i % 2, so the four inputs of a pair are bytes 0, 2 (or 1, 3) of the two words
              const uint32_t sel = (f & 1) ? 0x7531u : 0x6420u;
              const uint32_t wa = f < 2 ? prmt(qa.x, qa.y, sel) : prmt(qa.z, qa.w, sel);
              const uint32_t wb = f < 2 ? prmt(qb.x, qb.y, sel) : prmt(qb.z, qb.w, sel);
              // rows g take the whole byte (even output + 16 x odd output), rows g + 8 the odd output x 16
              const uint32_t af[4] = {wa, wa & 0xF0F0F0F0u, wb, wb & 0xF0F0F0F0u};
              mma_u8s8(acc[f], af, b0, b1);
            }
          }
          // lane t finishes unit t: its digit scale and offset, the weight scales of its group
          const uint2 meta = xmeta[ubase + t];
          const float sx = __uint_as_float(meta.x);
          const int off = static_cast<int>(meta.y);
          float sc[8];
          if (a.scale_rows > 0) {
            const int gidx = a.gs_shift >= 0 ? ((32 * hq + 8 * t) >> a.gs_shift) : 0;
            const __half* sp = reinterpret_cast<const __half*>(st + W * kBoxBytes) + gidx * WT + tb * F::BOX_N + F::NPL * g;
            const uint4 sv = *reinterpret_cast<const uint4*>(sp);
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&sv.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&sv.y));
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&sv.z));
            const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&sv.w));
            sc[0] = f0.x; sc[1] = f0.y; sc[2] = f1.x; sc[3] = f1.y;
            sc[4] = f2.x; sc[5] = f2.y; sc[6] = f3.x; sc[7] = f3.y;
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) sc[i] = a.scalar_scale;
          }
          // acc: {row g high digit, row g low, row g + 8 high, row g + 8 low} of unit t
#pragma unroll
          for (int f = 0; f < 4; ++f) {
            const int even = (acc[f][0] - acc[f][2]) * 256 + (acc[f][1] - acc[f][3]) - off;
            const int odd = ((acc[f][2] * 256 + acc[f][3]) >> 4) - off;
            tot[0][f][0] = fmaf(sc[2 * f] * sx, static_cast<float>(even), tot[0][f][0]);
            tot[0][f][1] = fmaf(sc[2 * f + 1] * sx, static_cast<float>(odd), tot[0][f][1]);
          }
        }
      } else {
        // activation fragments of this warp's eight rows (two steps)
        uint32_t bx[2][2];
#pragma unroll
        for (int p = 0; p < 2; ++p) {
          const int r = rbase + 2 * t + p;
          bx[p][0] = bx[p][1] = 0u;
          if (row0 + r < r_hi && g < a.M) {
            const uint2 xv = *reinterpret_cast<const uint2*>(xs + ((size_t)r * a.M_total + a.tok0 + g) * 8);
            bx[p][0] = xv.x;
            bx[p][1] = xv.y;
          }
        }
        float ones[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if constexpr (SUBNORMAL) {
          const uint32_t oa[4] = {kOnesA, kOnesA, kOnesA, kOnesA};
          mma_f16(ones, oa, bx[0][0], bx[0][1]);
          mma_f16(ones, oa, bx[1][0], bx[1][1]);
        }
        const int gidx = a.gs_shift >= 0 ? (rbase >> a.gs_shift) : 0;
#pragma unroll
        for (int b = 0; b < W; ++b) {
          float grp[F::NF][4];
#pragma unroll
          for (int f = 0; f < F::NF; ++f) grp[f][0] = grp[f][1] = grp[f][2] = grp[f][3] = 0.0f;
#pragma unroll
          for (int p = 0; p < 2; ++p) {
            const int r = rbase + 2 * t + p;
            const uint4 q = *reinterpret_cast<const uint4*>(st + b * kBoxBytes + r * 128 + ((g ^ (r & 7)) << 4));
            uint32_t av[F::NF][4];
            unpack<BITS, SUBNORMAL>(q, av);
#pragma unroll
            for (int f = 0; f < F::NF; ++f) mma_f16(grp[f], av[f], bx[p][0], bx[p][1]);
          }
          // scales of this lane's outputs for the group these eight rows are in
          float sc[F::NPL];
          if (a.scale_rows > 0) {
            const __half* sp = reinterpret_cast<const __half*>(st + W * kBoxBytes) + gidx * WT + b * F::BOX_N + F::NPL * g;
            if constexpr (BITS == 4) {
              const uint4 sv = *reinterpret_cast<const uint4*>(sp);
              const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&sv.x));
              const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&sv.y));
              const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&sv.z));
              const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&sv.w));
              sc[0] = f0.x; sc[1] = f0.y; sc[2] = f1.x; sc[3] = f1.y;
              sc[4] = f2.x; sc[5] = f2.y; sc[6] = f3.x; sc[7] = f3.y;
            } else {
              const uint2 sv = *reinterpret_cast<const uint2*>(sp);
              const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&sv.x));
              const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&sv.y));
              sc[0] = f0.x; sc[1] = f0.y; sc[2] = f1.x; sc[3] = f1.y;
            }
          } else {
#pragma unroll
            for (int i = 0; i < F::NPL; ++i) sc[i] = a.scalar_scale;
          }
          // row g of MMA f is output 2f, row g+8 is output 2f+1
#pragma unroll
          for (int f = 0; f < F::NF; ++f)
#pragma unroll
            for (int jj = 0; jj < NJ; ++jj) {
              const int j = MONE ? 2 * jj : jj;  // MONE keeps (row g, token 2t) and (row g+8, token 2t)
              const bool odd = (j & 2) != 0;
              float v = grp[f][j];
              if constexpr (SUBNORMAL) {
                v = odd ? fmaf(v, kOdd, -ones[j & 1]) : (v - ones[j & 1]);
              } else {
                if (odd) v *= kOdd;
              }
              tot[b][f][jj] = fmaf(sc[2 * f + (odd ? 1 : 0)], v, tot[b][f][jj]);
            }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[stage]);
#ifdef MLD_TRACE
      tr_busy_cycles += clock64() - tw1;
#endif
      if (++stage == a.stages) {
        stage = 0;
        phase ^= 1;
      }
    }
    if (failed) break;
#ifdef MLD_TRACE
    if (tr && threadIdx.x == 0) {
      tr[6] = static_cast<unsigned long long>(tr_wait_cycles);
      tr[7] = static_cast<unsigned long long>(tr_busy_cycles);
    }
#endif

    // ------------------------------------------------ pass epilogue
    if (tr && threadIdx.x == 0) tr[4] = globaltimer_ns();
    if constexpr (DIGITS) {
      // tot[0] is this warp's box (tb) summed over the units the lane finished: add the four lanes t up; the
      // warp contributes nothing to the other boxes
      constexpr int T = W == 3 ? 8 : 2 * W;
      const int tb = (warp % T) >> 1;
#pragma unroll
      for (int f = 0; f < 4; ++f)
#pragma unroll
        for (int jj = 0; jj < 2; ++jj) {
          float v = tot[0][f][jj];
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          if (t == 0) {
#pragma unroll
            for (int b = 0; b < W; ++b)
              red[(warp * WT + b * F::BOX_N + F::NPL * g + 2 * f + jj) * a.red_m] = b == tb ? v : 0.0f;
          }
        }
    } else {
#pragma unroll
      for (int b = 0; b < W; ++b)
#pragma unroll
        for (int f = 0; f < F::NF; ++f)
#pragma unroll
          for (int jj = 0; jj < NJ; ++jj) {
            const int j = MONE ? 2 * jj : jj;
            const int n_local = b * F::BOX_N + F::NPL * g + 2 * f + ((j >> 1) & 1);
            const int tok = 2 * t + (j & 1);
            if (tok < a.M) red[(warp * WT + n_local) * a.red_m + tok] = tot[b][f][jj];
          }
    }
    MLD_CONSUMER_BARRIER();
    const int chunk0 = cs + pass * W * 8;
    const int n0 = chunk0 * F::NPL;               // first output of this pass
    const int n_end = min(ce * F::NPL, a.N4);      // one past the last output this CTA owns
    const int nvals = WT * a.M;
    uint32_t peer_remote = 0, bar_remote = 0;
    if (a.ksplit > 1 && pass == 0) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    if (a.ksplit > 1 && kr == 1) {
      peer_remote = map_to_rank(smem_u32(peer), 0);
      bar_remote = map_to_rank(smem_u32(peer_bar), 0);
    }
    if (a.ksplit > 1 && kr == 0) {
      if (!mbar_wait_cluster(peer_bar, pass & 1)) {
        atomicExch(a.error, 3);
        failed = true;
      }
    }
    if (a.ksplit > 1 && kr == 1) {
      // upper half of K: hand the sums to the partner
      for (int idx = threadIdx.x; idx < nvals && !failed; idx += kConsumerWarps * 32) {
        const int n_local = idx / a.M, tok = idx - n_local * a.M;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) s += red[(w * WT + n_local) * a.red_m + tok];
        st_cluster_f32(peer_remote + (n_local * a.red_m + tok) * 4, s);
      }
    } else if (a.epilogue == MLD_EPILOGUE_SWIGLU_PAIRS) {
      // rows alternate gate_i, up_i: out[i] = silu(gate_i) * up_i, each rounded to
      // fp16 where the unfused graph would store it
      const int npairs = (WT / 2) * a.M;
      for (int idx = threadIdx.x; idx < npairs && !failed; idx += kConsumerWarps * 32) {
        const int p_local = idx / a.M, tok = idx - p_local * a.M;
        float sg = 0.0f, su = 0.0f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) {
          sg += red[(w * WT + 2 * p_local) * a.red_m + tok];
          su += red[(w * WT + 2 * p_local + 1) * a.red_m + tok];
        }
        if (a.ksplit > 1) {
          sg += peer[(2 * p_local) * a.red_m + tok];
          su += peer[(2 * p_local + 1) * a.red_m + tok];
        }
        const int n = n0 + 2 * p_local;
        if (n + 1 < n_end) {
          const float g = __half2float(__float2half_rn(sg * kOutScale));
          const float u = __half2float(__float2half_rn(su * kOutScale));
          const __half r = __float2half_rn(g / (1.0f + __expf(-g)) * u);
          const int i = n >> 1, tk = a.tok0 + tok;
          const int64_t yi = a.dst_layout == MLD_LAYOUT_SLICED ? (((int64_t)(i >> 2) * a.M_total + tk) * 4 + (i & 3))
                                                               : ((int64_t)tk * (a.N / 2) + i);
          if (a.scatter.world > 1) {
            for (int pr = 0; pr < a.scatter.world; ++pr) static_cast<__half*>(a.scatter.y_peers[pr])[yi] = r;
          } else {
            static_cast<__half*>(a.y)[yi] = r;
          }
        }
      }
    } else {
      for (int idx = threadIdx.x; idx < nvals && !failed; idx += kConsumerWarps * 32) {
        const int n_local = idx / a.M, tok = idx - n_local * a.M;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < kConsumerWarps; ++w) s += red[(w * WT + n_local) * a.red_m + tok];
        if (a.ksplit > 1) s += peer[n_local * a.red_m + tok];  // fixed order: lower half of K first
        const int n = n0 + n_local;
        if (n < n_end) {
          __half r = __float2half_rn(s * kOutScale);
          if (a.bias != nullptr) r = __hadd(r, static_cast<const __half*>(a.bias)[n]);
          const int tk = a.tok0 + tok;
          const int64_t yi = a.dst_layout == MLD_LAYOUT_SLICED ? (((int64_t)(n >> 2) * a.M_total + tk) * 4 + (n & 3))
                                                               : ((int64_t)tk * a.N + n);
          if (a.dst_layout == MLD_LAYOUT_SLICED || n < a.N) {
            if (a.scatter.world > 1) {
              for (int pr = 0; pr < a.scatter.world; ++pr) static_cast<__half*>(a.scatter.y_peers[pr])[yi] = r;
            } else {
              static_cast<__half*>(a.y)[yi] = r;
            }
          }
        }
      }
    }
    if (a.ksplit > 1 && kr == 1) mbar_arrive_cluster(bar_remote);  // release: the stores above are visible
    MLD_CONSUMER_BARRIER();
    if (tr && threadIdx.x == 0) tr[5] = globaltimer_ns();
  }
  if (a.scatter.world > 1) {
    // every CTA: make its peer stores visible, then count in; the last one
    // raises this rank's flag on every rank
    __threadfence_system();
    MLD_CONSUMER_BARRIER();
    if (threadIdx.x == 0) {
      const int t = atomicAdd(a.scatter.ticket, 1);
      if (t == static_cast<int>(gridDim.x) - 1) {
        *a.scatter.ticket = 0;
        __threadfence_system();
        const unsigned seq = static_cast<unsigned>(*a.scatter.step * a.scatter.seq_per_step + a.scatter.seq_off);
        for (int pr = 0; pr < a.scatter.world; ++pr) st_release_sys(a.scatter.flag_peers[pr], seq);
      }
    }
  }
}

template <int BITS, int W, bool SUBNORMAL, bool MONE, bool DIGITS = false>
int launch_strip_t(const CUtensorMap& tw, const CUtensorMap& ts, const StripArgs& a, const StripGeometry& gm,
                   cudaStream_t stream) {
  auto kern = fc_strip_kernel<BITS, W, SUBNORMAL, MONE, DIGITS>;
  static bool configured[kMaxDevices];  // per instantiation and device
  int dev;
  if (needs_configure(configured, &dev)) {
    MLD_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    if (dev >= 0) configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(gm.grid, 1, 1);
  cfg.blockDim = dim3((kConsumerWarps + 1) * 32, 1, 1);
  cfg.dynamicSmemBytes = gm.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  if (gm.ksplit > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = gm.ksplit;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  if (a.pdl) {
    attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[na].val.programmaticStreamSerializationAllowed = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  MLD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tw, ts, a));
  count_launch();
  return MLD_OK;
}

template <int BITS, int W>
int launch_strip_w(bool subnormal, bool mone, const CUtensorMap& tw, const CUtensorMap& ts, const StripArgs& a,
                   const StripGeometry& gm, cudaStream_t stream) {
  if (subnormal) {
    if constexpr (BITS == 4) {
      if (mone && a.M_total == 1 && gm.xdig_bytes > 0) return launch_strip_t<BITS, W, true, true, true>(tw, ts, a, gm, stream);
    }
    if (mone) return launch_strip_t<BITS, W, true, true>(tw, ts, a, gm, stream);
    return launch_strip_t<BITS, W, true, false>(tw, ts, a, gm, stream);
  }
  if (mone) return launch_strip_t<BITS, W, false, true>(tw, ts, a, gm, stream);
  return launch_strip_t<BITS, W, false, false>(tw, ts, a, gm, stream);
}

}  // namespace

StripGeometry strip_geometry(int bits, int N, int K, int m_total, int group_slices, int scale_mode, int sms,
                             bool pdl, int smem_limit_kb) {
  StripGeometry gm;
  memset(&gm, 0, sizeof gm);
  const int N4 = align_n(N, 4), SS = div_up(K, 4);
  const int box_n = bits == 4 ? 64 : 32;
  const int row_bytes = (N4 / 4) * (bits == 4 ? 8 : 16);
  gm.gran = bits == 4 ? 1 : 2;
  const int C = row_bytes / 16;
  gm.units = C / gm.gran;
  // Two CTAs per strip (a cluster splitting K) when single strips would be
  // narrower than 128 bytes and K is long enough to halve.
  gm.ksplit = (C < 8 * sms && SS >= 4 * kStageRows && sms >= 2) ? 2 : 1;
  int strips = sms / gm.ksplit;
  if (strips > gm.units) strips = gm.units;
  if (strips < 1) strips = 1;
  gm.strips = strips;
  gm.grid = strips * gm.ksplit;
  const int max_width = div_up(gm.units, strips) * gm.gran;  // chunks
  int w = div_up(max_width, 8);
  // Overlapping launches need two CTAs per SM, which the register file grants to the instantiations of up
  // to two boxes per stage: wider strips take more column passes instead.
  const int w_max = pdl ? 2 : 4;
  if (gm.ksplit > 1 && w > w_max) {  // a cluster pair runs a single pass
    gm.ksplit = 1;
    strips = sms < gm.units ? sms : gm.units;
    gm.strips = strips;
    gm.grid = strips;
    w = div_up(div_up(gm.units, strips) * gm.gran, 8);
  }
  gm.w = w > w_max ? w_max : w;
  gm.rows_per_split = gm.ksplit == 1 ? align_n(SS, kStageRows) : align_n(div_up(SS, 2), kStageRows);
  if (scale_mode == MLD_SCALE_SCALAR) {
    gm.scale_rows = 0;
    gm.group_slices = 1;
    gm.gs_shift = -1;
  } else {
    gm.group_slices = scale_mode == MLD_SCALE_PER_CHANNEL ? align_n(SS, kStageRows) : group_slices;
    gm.scale_rows = gm.group_slices >= kStageRows ? 1 : kStageRows / gm.group_slices;
    gm.gs_shift = -1;
    if (gm.group_slices < kStageRows)
      for (int sh = 3; sh < 7; ++sh)
        if ((1 << sh) == gm.group_slices) gm.gs_shift = sh;
  }
  const int wt = gm.w * box_n;
  gm.scale_stage_bytes = align_n(gm.scale_rows * wt * 2, 128);
  const int x_bytes = align_n(kStageRows * m_total * 8, 128);
  gm.stage_bytes = align_n(gm.w * kBoxBytes + gm.scale_stage_bytes + x_bytes, 1024);
  gm.red_m = m_total < 8 ? m_total : 8;
  // 4-bit weights: room for a one-token activation vector of this CTA's K range as digits (8 bytes per k-slice,
  // 8 per unit of eight k-slices, a barrier)
  gm.xdig_bytes = bits == 4 ? gm.rows_per_split * 9 + 48 : 0;
  const int fixed = (kConsumerWarps + 1) * wt * gm.red_m * 4 + 8 + (2 * 16 + 1) * 8 + gm.xdig_bytes + 1024 + 64;
  gm.stage_rows = kStageRows;
  // With programmatic dependent launch two consecutive GEMVs share an SM while
  // one drains and the next prefetches, so each takes at most half of it.
  int budget = pdl ? 112 * 1024 : 224 * 1024;
  if (smem_limit_kb >= 32 && smem_limit_kb <= 224) budget = smem_limit_kb * 1024;
  int stages = (budget - fixed) / gm.stage_bytes;
  if (stages > 16) stages = 16;
  if (stages < 2) stages = (227 * 1024 - fixed) / gm.stage_bytes;
  gm.stages = stages;
  gm.smem_bytes = (size_t)stages * gm.stage_bytes + fixed;
  return gm;
}

int launch_fc_strip(int bits, bool subnormal, const CUtensorMap& tw, const CUtensorMap& ts, const StripArgs& a,
                    const StripGeometry& gm, cudaStream_t stream) {
  if (a.M == 0 || gm.grid == 0) return MLD_OK;
  const bool mone = a.M == 1;
#define MLD_W(B, WV) \
  case WV:           \
    return launch_strip_w<B, WV>(subnormal, mone, tw, ts, a, gm, stream)
  if (bits == 4) {
    switch (gm.w) {
      MLD_W(4, 1);
      MLD_W(4, 2);
      MLD_W(4, 3);
      MLD_W(4, 4);
    }
  } else {
    switch (gm.w) {
      MLD_W(8, 1);
      MLD_W(8, 2);
      MLD_W(8, 3);
      MLD_W(8, 4);
    }
  }
#undef MLD_W
  set_last_error_text("bad strip geometry");
  return MLD_INVALID_ARGUMENT;
}

}  // namespace mld
