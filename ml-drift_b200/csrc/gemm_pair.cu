// Prefill-stage dequant-GEMM with the dequantisation inside the kernel, on pairs
// of SMs (tcgen05 cta_group::2).
//
// The reference runs a prefill FullyConnected either as one convolution that
// reads the packed weights and dequantises them inline
// (ml_drift/common/kernels/conv_generic.cc:1553-1640, chosen by the cost rule of
// common/gpu_model_builder.cc:1128-1173) or as a WeightsConverter pass followed
// by a float convolution (gpu_model_builder.cc:1110-1276,
// common/kernels/conv_weights_converter.cc:248-290); and, for per-channel INT8
// with quantised activations, as an int8 convolution with a fused
// dequantisation (gpu_model_builder.cc:1325-1431,
// common/kernels/quantize_and_dequantize.cc:867-964).  This kernel is the inline
// form: the packed weights never leave their reference layout in HBM.
//
// Y[M x N] = X[M x K] W[N x K]^T.  A cluster of two CTAs owns an output tile of
// 256 tokens x tile_n outputs; each CTA holds its 128 tokens of X and HALF of
// the tile's weights, and one thread of the pair's first CTA issues
// tcgen05.mma.cta_group::2, which reads both halves (so every byte of an operand
// crosses L2 -> shared memory once per pair, not once per SM).  Per CTA:
//   warp 0      TMA producer: the activation tile (K-major, 128-byte swizzle) and
//               the packed weight box of the stage ([K/4] rows of 4x4 blocks)
//   warp 1      tensor-memory owner; in the first CTA also the MMA issuer
//   warps 2..5  epilogue: tcgen05.ld -> convert (-> dequantise) -> global stores
//               in the reference's sliced output layout
//   warps 6..9  transform: one thread per weight row of the CTA's half turns the
//               packed nibbles / bytes of the stage into the K-major,
//               128-byte-swizzled operand tile the MMA reads:
//                 fp16 route  w = half(half(u * scale) + half(-scale * shift)),
//                             the WeightsConverter arithmetic
//                 int8 route  w = u - 128 (exact), for kind::i8
// Accumulators live in tensor memory, double-buffered, so the epilogue of one
// tile overlaps the main loop of the next.  Every wait is bounded.
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace mld {
namespace {

enum { kModeInt4F16 = 0, kModeInt8F16 = 1, kModeInt8I8 = 2 };

constexpr int kPairThreads = 320;
constexpr int kRowsPerCta = 128;        // tokens per CTA (UMMA M = 256 over the pair)
constexpr int kKBytes = 128;            // one swizzle atom of K per stage
constexpr int kABytes = kRowsPerCta * kKBytes;
constexpr int kBBytes = 128 * kKBytes;  // up to 128 weight rows per CTA
constexpr int kTransformWarps = 4;
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
  int tile_n;                 // UMMA N of the pair (multiple of 32, <= 256); each CTA transforms tile_n / 2 rows
  int m_tiles, n_tiles, k_blocks;
  int stages;
  int w_box_bytes;            // bytes of one packed-weight box (rows_per_block slices x (tile_n / 2 / 4) blocks)
  int src_slices;             // K / 4 (rounded up)
  // fp16 routes: scales of the weights
  const __half* scale;        // [G][N4] fp16 (null: scalar_scale)
  int scale_mode, G, group_slices;
  float scalar_scale;
  const void* bias;           // fp16 [N4] or null
  // int8 route
  const float* a_params;      // per token {inv_scale, offset, sum of the codes}
  const int32_t* w_sum;       // per output: sum of the signed weights (null: symmetric activations)
  void* y;                    // fp16
  int dst_layout;
  int* error;
};

// (1024 + u) - 1024 = u exactly, then u * s + b with separate roundings (the WeightsConverter arithmetic).
__device__ __forceinline__ uint32_t dq2(uint32_t biased, __half2 s2, __half2 b2) {
  const __half2 u = __hsub2(*reinterpret_cast<const __half2*>(&biased), __float2half2_rn(1024.0f));
  const __half2 r = __hadd2(__hmul2(u, s2), b2);
  return *reinterpret_cast<const uint32_t*>(&r);
}

template <int MODE>
__global__ void __launch_bounds__(kPairThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, PairArgs a) {
  constexpr bool I8 = MODE == kModeInt8I8;
  constexpr int BLK = MODE == kModeInt4F16 ? 8 : 16;            // bytes of a packed 4x4 block
  constexpr int K_PER_STAGE = I8 ? 128 : 64;                      // elements of K in a 128-byte row
  constexpr int SLICES = K_PER_STAGE / 4;                         // packed rows per stage
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int half_n = a.tile_n / 2;
  const int w_pitch = (half_n / 4) * BLK;                         // bytes of one packed row of the box
  uint8_t* sA = smem;
  uint8_t* sB = sA + (size_t)a.stages * kABytes;
  uint8_t* sW = sB + (size_t)a.stages * kBBytes;
  const int w_stage = (a.w_box_bytes + 127) & ~127;
  uint64_t* full_w = reinterpret_cast<uint64_t*>(sW + (size_t)a.stages * w_stage);
  uint64_t* full_ab = full_w + a.stages;     // used in the pair's first CTA: A of both CTAs landed, B of both transformed
  uint64_t* empty = full_ab + a.stages;      // the stage's MMAs have completed (arrives in both CTAs)
  uint64_t* tmem_full = empty + a.stages;    // [2], arrives in both CTAs
  uint64_t* tmem_empty = tmem_full + 2;      // [2], used in the first CTA: the epilogue warps of both CTAs have drained it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int total_tiles = a.m_tiles * a.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full_w[s], 1);
      mbar_init(&full_ab[s], 1 + 2 * kTransformWarps);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2 * 4);
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, 512);
    tmem_relinquish_pair();
  }
  tc_before();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers are initialised before anything arrives on them
  tc_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t full_ab_lead = map_shared(smem_u32(full_ab), 0);      // the first CTA's barriers, as cluster addresses
  const uint32_t tmem_empty_lead = map_shared(smem_u32(tmem_empty), 0);

  if (warp == 0) {
    // --------------------------------------------------------------- producer
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_w);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
        const int mi = tile % a.m_tiles, ni = tile / a.m_tiles;
        const int m0 = mi * 2 * kRowsPerCta + static_cast<int>(rank) * kRowsPerCta;
        const int nb0 = (ni * a.tile_n + static_cast<int>(rank) * half_n) / 4 * BLK;  // byte column of the box
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicExch(a.error, kErrPairBase + 1);
            ok = false;
            break;
          }
          if (rank == 0) mbar_arrive_expect_tx(&full_ab[stage], 2 * kABytes);
          tma_load_2d_pair(sA + (size_t)stage * kABytes, &tmap_a, full_ab_lead + stage * 8, kb * K_PER_STAGE, m0);
          mbar_arrive_expect_tx(&full_w[stage], static_cast<uint32_t>(a.w_box_bytes));
          tma_load_2d(sW + (size_t)stage * w_stage, &tmap_w, &full_w[stage], nb0 / 4, kb * SLICES);  // 32-bit elements
          if (++stage == a.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (rank == 0 && lane == 0) {
      uint32_t idesc;
      if constexpr (I8)
        idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a.tile_n >> 3) << 17) | (16u << 24);
      else
        idesc = (1u << 4) | (static_cast<uint32_t>(a.tile_n >> 3) << 17) | (16u << 24);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      bool ok = true;
      for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++local) {
        const int acc = local & 1;
        if (!wait_cluster(&tmem_empty[acc], acc_phase[acc] ^ 1)) {
          atomicExch(a.error, kErrPairBase + 2);
          ok = false;
          break;
        }
        acc_phase[acc] ^= 1;
        tc_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * 256);
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!wait_cluster(&full_ab[stage], phase)) {
            atomicExch(a.error, kErrPairBase + 3);
            ok = false;
            break;
          }
          tc_after();
          const uint64_t da = make_desc(smem_u32(sA + (size_t)stage * kABytes));
          const uint64_t db = make_desc(smem_u32(sB + (size_t)stage * kBBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t adv = static_cast<uint64_t>((k * 32) >> 4);  // 32 bytes of K per MMA inside the swizzle atom
            umma_pair<I8>(tmem_d, da + adv, db + adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          commit_pair(&empty[stage]);
          if (++stage == a.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) commit_pair(&tmem_full[acc]);
      }
    }
  } else if (warp < 6) {
    // --------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    bool ok = true;
    for (int tile = pair; tile < total_tiles && ok; tile += n_pairs, ++local) {
      const int acc = local & 1;
      const int mi = tile % a.m_tiles, ni = tile / a.m_tiles;
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc])) {
        atomicExch(a.error, kErrPairBase + 4);
        ok = false;
        break;
      }
      acc_phase[acc] ^= 1;
      tc_after();
      const int m = mi * 2 * kRowsPerCta + static_cast<int>(rank) * kRowsPerCta + quad * 32 + lane;
      const int n0 = ni * a.tile_n;
      float a_scale = 1.0f, a_off = 0.0f;
      if constexpr (I8) {
        if (m < a.M) {
          a_scale = a.a_params[m * 3];
          a_off = a.a_params[m * 3 + 1];
        } else {
          a_scale = 0.0f;
        }
      }
      for (int c0 = 0; c0 < a.tile_n; c0 += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * 256 + c0);
        tmem_ld32(taddr, r);
        tmem_ld_wait();
        if (m < a.M) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int n = n0 + c0 + j;
            if (c0 + j >= a.tile_n || n >= a.N4) break;
            __half h[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              float v;
              if constexpr (I8) {
                // CreateDequantization (quantize_and_dequantize.cc:867-964):
                //   res = float(acc) * (w_scale * src_scale) + w_scale * src_zero_point * weights_sum
                const float ws = (n + e) < a.N ? __half2float(a.scale[n + e]) : 0.0f;
                v = static_cast<float>(static_cast<int32_t>(r[j + e])) * (ws * a_scale);
                if (a.w_sum != nullptr && (n + e) < a.N) v += ws * a_off * static_cast<float>(a.w_sum[n + e]);
              } else {
                v = __uint_as_float(r[j + e]);
              }
              h[e] = __float2half_rn(v);
              if (a.bias != nullptr) h[e] = __hadd(h[e], static_cast<const __half*>(a.bias)[n + e]);
            }
            if (a.dst_layout == MLD_LAYOUT_SLICED) {
              uint2 pk;
              pk.x = static_cast<uint32_t>(__half_as_ushort(h[0])) | (static_cast<uint32_t>(__half_as_ushort(h[1])) << 16);
              pk.y = static_cast<uint32_t>(__half_as_ushort(h[2])) | (static_cast<uint32_t>(__half_as_ushort(h[3])) << 16);
              *reinterpret_cast<uint2*>(static_cast<__half*>(a.y) + ((size_t)(n >> 2) * a.M + m) * 4) = pk;
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e)
                if (n + e < a.N) static_cast<__half*>(a.y)[(size_t)m * a.N + n + e] = h[e];
            }
          }
        }
      }
      tc_before();
      __syncwarp();
      if (lane == 0) arrive_remote(tmem_empty_lead + acc * 8);
    }
  } else {
    // -------------------------------------------------------------- transform
    const int row = (warp - 6) * 32 + lane;          // weight row of this CTA's half of the tile
    const bool active = row < half_n;
    const int col4 = row & 3;                         // column of the row inside its 4x4 blocks
    uint8_t* const b_row = sB + (row >> 3) * 1024 + (row & 7) * 128;
    const int sw = row & 7;                           // 16-byte chunk c of the row sits at chunk c ^ sw
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int tile = pair; tile < total_tiles && ok; tile += n_pairs) {
      const int ni = tile / a.m_tiles;
      const int n = ni * a.tile_n + static_cast<int>(rank) * half_n + row;
      const bool has_n = active && n < a.N4;
      for (int kb = 0; kb < a.k_blocks; ++kb) {
        if (!mbar_wait(&full_w[stage], phase)) {
          atomicExch(a.error, kErrPairBase + 5);
          ok = false;
          break;
        }
        if (active) {
          const uint8_t* wp = sW + (size_t)stage * w_stage + (row >> 2) * BLK;
          uint8_t* bp = b_row + (size_t)stage * kBBytes;
          if constexpr (I8) {
            // bytes (k % 4) * 4 + col4 of each block, re-biased u8 -> s8; 8 slices = 32 bytes of K per two chunks
#pragma unroll 4
            for (int c = 0; c < 8; ++c) {       // chunk c: K elements 16 c .. 16 c + 15 = slices 4 c .. 4 c + 3
              uint32_t o[4];
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 blk = *reinterpret_cast<const uint4*>(wp + (size_t)(4 * c + q) * w_pitch);
                const uint32_t b0 = (blk.x >> (8 * col4)) & 0xFFu, b1 = (blk.y >> (8 * col4)) & 0xFFu;
                const uint32_t b2 = (blk.z >> (8 * col4)) & 0xFFu, b3 = (blk.w >> (8 * col4)) & 0xFFu;
                o[q] = (b0 | (b1 << 8) | (b2 << 16) | (b3 << 24)) ^ 0x80808080u;
              }
              *reinterpret_cast<uint4*>(bp + ((c ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          } else {
            // scales of this row for the groups the stage touches
            const int k_slice0 = kb * SLICES;
#pragma unroll 2
            for (int c = 0; c < 8; ++c) {       // chunk c: K elements 8 c .. 8 c + 7 = slices 2 c, 2 c + 1
              __half sc = __float2half_rn(a.scalar_scale);
              if (a.scale != nullptr && has_n) {
                int g = a.scale_mode == MLD_SCALE_BLOCK ? (k_slice0 + 2 * c) / a.group_slices : 0;
                if (g >= a.G) g = a.G - 1;
                sc = __ldg(a.scale + (size_t)g * a.N4 + n);
              }
              const __half2 s2 = __half2half2(sc);
              const __half shift = __ushort2half_rn(static_cast<unsigned short>(MODE == kModeInt4F16 ? 8 : 128));
              const __half2 b2 = __half2half2(__hmul(__hneg(sc), shift));
              uint32_t o[4];
#pragma unroll
              for (int q = 0; q < 2; ++q) {
                if constexpr (MODE == kModeInt4F16) {
                  const uint2 blk = *reinterpret_cast<const uint2*>(wp + (size_t)(2 * c + q) * w_pitch);
                  // nibble (k % 4) * 4 + col4: k0, k1 in the halves of blk.x, k2, k3 in those of blk.y
                  o[2 * q] = dq2(((blk.x >> (4 * col4)) & 0x000F000Fu) | 0x64006400u, s2, b2);
                  o[2 * q + 1] = dq2(((blk.y >> (4 * col4)) & 0x000F000Fu) | 0x64006400u, s2, b2);
                } else {
                  const uint4 blk = *reinterpret_cast<const uint4*>(wp + (size_t)(2 * c + q) * w_pitch);
                  const uint32_t b0 = (blk.x >> (8 * col4)) & 0xFFu, b1 = (blk.y >> (8 * col4)) & 0xFFu;
                  const uint32_t b2b = (blk.z >> (8 * col4)) & 0xFFu, b3 = (blk.w >> (8 * col4)) & 0xFFu;
                  o[2 * q] = dq2(b0 | (b1 << 16) | 0x64006400u, s2, b2);
                  o[2 * q + 1] = dq2(b2b | (b3 << 16) | 0x64006400u, s2, b2);
                }
              }
              *reinterpret_cast<uint4*>(bp + ((c ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
            }
          }
        }
        // the tile was written through the generic proxy; the MMA reads it through the async proxy
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) arrive_remote(full_ab_lead + stage * 8);
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  }
  // Tear-down: nobody leaves while the partner may still arrive on this CTA's barriers or the pair's MMAs
  // may still write this CTA's tensor memory.
  tc_before();
  __syncthreads();
  cluster_sync_all();
  if (*reinterpret_cast<volatile int*>(a.error) != 0) {
    // a wait ran out somewhere: copies may still be in flight towards this CTA's shared memory
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  if (warp == 1) {
    tc_after();
    tmem_dealloc_pair(tmem_base, 512);
  }
}

}  // namespace

// ------------------------------------------------------------------ host side
PairGeometry pair_geometry(int M, int N, int K, int mode, int sms) {
  PairGeometry g;
  const int N4 = align_n(N, 4);
  const bool i8 = mode == kModeInt8I8;
  g.kp = align_n(K, i8 ? 16 : 8);
  g.m_tiles = div_up(M, 2 * kRowsPerCta);
  const int pairs = sms / 2 > 0 ? sms / 2 : 1;
  // UMMA N of the pair: the widest tile whose wave count wastes least (a tile of width tn costs tn tensor-pipe
  // time units; the last wave is paid in full whether or not it is full).
  int best_n = 256;
  long best_cost = -1;
  for (int tn = 256; tn >= 64; tn -= 32) {
    const long tiles = (long)g.m_tiles * div_up(N4, tn);
    const long waves = (tiles + pairs - 1) / pairs;
    const long cost = waves * tn;
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_n = tn;
    }
  }
  g.tile_n = best_n;
  g.n_tiles = div_up(N4, g.tile_n);
  const int k_per_stage = i8 ? 128 : 64;
  g.k_blocks = div_up(g.kp, k_per_stage);
  const int blk = mode == kModeInt4F16 ? 8 : 16;
  g.w_box_bytes = (k_per_stage / 4) * (g.tile_n / 2 / 4) * blk;
  const int w_stage = (g.w_box_bytes + 127) & ~127;
  const int per_stage = kABytes + kBBytes + w_stage;
  const int fixed = 1024 + (3 * 16 + 4) * 8 + 64;
  int stages = (220 * 1024 - fixed) / per_stage;
  if (stages > 8) stages = 8;
  g.stages = stages;
  g.smem_bytes = (size_t)stages * per_stage + fixed;
  const long tiles = (long)g.m_tiles * g.n_tiles;
  g.grid = 2 * static_cast<int>(tiles < pairs ? tiles : pairs);
  return g;
}

int launch_gemm_pair(int mode, const void* a_mat, const void* packed, const PairGeometry& g, int M, int N, int K,
                     const void* scale, int scale_mode, int G, int group_slices, float scalar_scale, const void* bias,
                     const float* a_params, const int32_t* w_sum, void* y, int dst_layout, int* error,
                     cudaStream_t stream) {
  const int N4 = align_n(N, 4);
  const bool i8 = mode == kModeInt8I8;
  const int esz = i8 ? 1 : 2;
  const int blk = mode == kModeInt4F16 ? 8 : 16;
  const int SS = div_up(K, 4), DS = N4 / 4;
  CUtensorMap ta, tw;
  int rc = make_tmap_2d(&ta, a_mat, (uint64_t)g.kp * esz, M, (uint64_t)g.kp * esz, kKBytes, kRowsPerCta, esz,
                        CU_TENSOR_MAP_SWIZZLE_128B, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        true);
  if (rc != MLD_OK) return rc;
  // packed weights: [K/4] rows of N4/4 blocks; the box is one stage's rows of the CTA's half of the tile
  rc = make_tmap_2d(&tw, packed, (uint64_t)DS * blk, SS, (uint64_t)DS * blk, (g.tile_n / 2 / 4) * blk,
                    (i8 ? 128 : 64) / 4, 4, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MLD_OK) return rc;
  PairArgs a;
  memset(&a, 0, sizeof a);
  a.M = M;
  a.N = N;
  a.N4 = N4;
  a.tile_n = g.tile_n;
  a.m_tiles = g.m_tiles;
  a.n_tiles = g.n_tiles;
  a.k_blocks = g.k_blocks;
  a.stages = g.stages;
  a.w_box_bytes = g.w_box_bytes;
  a.src_slices = SS;
  a.scale = scale_mode == MLD_SCALE_SCALAR ? nullptr : static_cast<const __half*>(scale);
  a.scale_mode = scale_mode;
  a.G = G;
  a.group_slices = group_slices;
  a.scalar_scale = scalar_scale;
  a.bias = bias;
  a.a_params = a_params;
  a.w_sum = w_sum;
  a.y = y;
  a.dst_layout = dst_layout;
  a.error = error;
  void (*kern)(CUtensorMap, CUtensorMap, PairArgs) =
      mode == kModeInt4F16 ? gemm_pair_kernel<kModeInt4F16>
                           : (mode == kModeInt8F16 ? gemm_pair_kernel<kModeInt8F16> : gemm_pair_kernel<kModeInt8I8>);
  static bool configured[3][kMaxDevices];
  int dev;
  if (needs_configure(configured[mode], &dev)) {
    MLD_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    if (dev >= 0) configured[mode][dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(g.grid, 1, 1);
  cfg.blockDim = dim3(kPairThreads, 1, 1);
  cfg.dynamicSmemBytes = g.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  MLD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, ta, tw, a));
  count_launch();
  return MLD_OK;
}

}  // namespace mld
