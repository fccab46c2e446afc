// Shared by the prefill GEMMs that run on pairs of SMs (tcgen05 cta_group::2): the PTX wrappers, the kernel
// arguments and the split of the work over the pairs.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace mld {
namespace {

// 0..2: the weights arrive packed and are transformed in shared memory; 3, 4: the weight operand was prepared
// by a pass of its own (K-major fp16 / s8 rows) and is loaded by TMA like the activations.
enum { kModeInt4F16 = 0, kModeInt8F16 = 1, kModeInt8I8 = 2, kModePreparedF16 = 3, kModePreparedI8 = 4 };

constexpr int kPairThreads = 800;
constexpr int kRowsPerCta = 128;        // tokens per CTA (UMMA M = 256 over the pair)
constexpr int kKBytes = 128;            // one swizzle atom of K per stage
constexpr int kABytes = kRowsPerCta * kKBytes;
constexpr int kBBytes = 128 * kKBytes;  // up to 128 weight rows per CTA
constexpr int kTransformWarps = 8;       // two threads per weight row: chunks 0..3 and 4..7 of its 128 bytes
constexpr int kErrPairBase = 30;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_shared(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ bool try_wait_cluster(uint64_t* bar, uint32_t parity) {
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
__device__ __forceinline__ bool wait_cluster(uint64_t* bar, uint32_t parity) {
  if (try_wait_cluster(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (try_wait_cluster(bar, parity)) return true;
    if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
  }
}
// TMA tile load of a CTA pair: the data lands in this CTA's shared memory, the bytes are counted on a
// barrier that may live in the pair's other CTA (bar_cluster_addr is a shared::cluster address).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int c0,
                                                 int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once every MMA issued so far
// has completed.
__device__ __forceinline__ void commit_pair(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(smem_u32(bar)), "h"(static_cast<uint16_t>(3))
      : "memory");
}
template <bool I8>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  if constexpr (I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
  }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 128-byte rows in the 128-byte swizzle: 8-row
// groups 1024 bytes apart (stride byte offset), descriptor version 1, layout type SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

struct PairArgs {
  int M, N, N4;
  int tile_n;                 // UMMA N of the pair (multiple of 16, <= 256); each CTA transforms tile_n / 2 rows
  int m_tiles, n_tiles, k_blocks;
  int stages;                 // operand ring: activation tile + transformed weight tile
  int w_stages;               // packed-weight ring
  int w_box_bytes;            // bytes of one packed-weight box (rows_per_block slices x (tile_n / 2 / 4) blocks)
  int src_slices;             // K / 4 (rounded up)
  // fp16 routes: scales of the weights
  const __half* scale;        // [G][N4] fp16 (null: scalar_scale)
  int scale_mode, G, group_slices;
  int gs_shift;               // log2(group_slices) when it is a power of two, else -1
  float scalar_scale;
  const void* bias;           // fp16 [N4] or null
  // int8 route
  const float* a_params;      // per token {inv_scale, offset, sum of the codes}
  const int32_t* w_sum;       // per output: sum of the signed weights (null: symmetric activations)
  void* y;                    // fp16
  int dst_layout;
  int* error;
  PeerOutputs outs;           // world > 1: the block is stored into every rank's tensor instead of y
  // Work split.  The first shared_tiles tiles are cut into k-block units, in the order (tile 0, k-block 0),
  // (tile 0, k-block 1), ..., and SM pair p takes the units [p * units_per_pair, (p + 1) * units_per_pair): a
  // range that is not a whole number of tiles makes the pair share its first and / or last tile with a
  // neighbour (each tile with at most one: a range is never shorter than a tile); the partial sums meet
  // through split_ws.  After that the pair takes whole tiles shared_tiles + p, + p + pairs, ...
  // (shared_tiles = 0: whole tiles only.)
  int shared_tiles, units_per_pair;
  float* split_ws;            // [pairs][2 CTAs][4 warps][8 chunks][8][32 lanes] x 16 bytes of raw accumulators
  uint32_t* split_flags;      // [pairs][2 CTAs][4 warps]: = epoch once that warp's share of the slot is written
  uint32_t epoch;             // differs from launch to launch, so the flags never need clearing
  long long* trace;           // tuning builds only: [grid][8] cycle counts per role (waiting / working)
  int skip_transform;         // tuning builds only: leave the operand tiles unwritten (timing of the rest)
};

#ifdef MLD_TRACE
#define MLD_PAIR_CLOCK() clock64()
#else
#define MLD_PAIR_CLOCK() 0ll
#endif

// (1024 + u) - 1024 = u exactly, then u * s + b with separate roundings (the WeightsConverter arithmetic).
__device__ __forceinline__ uint32_t dq2(uint32_t biased, __half2 s2, __half2 b2) {
  const __half2 u = __hsub2(*reinterpret_cast<const __half2*>(&biased), __float2half2_rn(1024.0f));
  const __half2 r = __hadd2(__hmul2(u, s2), b2);
  return *reinterpret_cast<const uint32_t*>(&r);
}

// A pair's work in order: runs of k-blocks of the shared tiles inside [u, u_end), then whole tiles.
struct Segment {
  int tile, kb0, kb1;
};
struct WorkList {
  int u, u_end, tile, tile_end, tile_step, k_blocks;
  __device__ __forceinline__ bool next(Segment& sg) {
    if (u < u_end) {
      sg.tile = u / k_blocks;
      sg.kb0 = u - sg.tile * k_blocks;
      sg.kb1 = min(k_blocks, sg.kb0 + (u_end - u));
      u += sg.kb1 - sg.kb0;
      return true;
    }
    if (tile < tile_end) {
      sg.tile = tile;
      sg.kb0 = 0;
      sg.kb1 = k_blocks;
      tile += tile_step;
      return true;
    }
    return false;
  }
  __device__ __forceinline__ int stages_in_all() const {
    return (u_end - u) + (tile < tile_end ? (tile_end - tile + tile_step - 1) / tile_step : 0) * k_blocks;
  }
};
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

}  // namespace
}  // namespace mld
