// Prefill-stage dequant-GEMM on the 5th-generation tensor cores.
//
// The reference runs a prefill FullyConnected as a WeightsConverter pass that
// dequantises the packed weights to fp16, followed by a float convolution
// (ml_drift/common/gpu_model_builder.cc:1110-1276,
// common/kernels/conv_weights_converter.cc:248-290), or - for per-channel INT8
// with quantised activations - as an int8 convolution with a fused
// dequantisation (gpu_model_builder.cc:1325-1431).  Here:
//   * operand preparation kernels produce K-major matrices: the dequantised
//     fp16 weights (or re-biased s8 weights), and the activations transposed
//     out of the reference's sliced layout (optionally quantised per token);
//   * gemm_umma_kernel multiplies them with tcgen05.mma: operands staged by TMA
//     into 128-byte-swizzled shared-memory tiles, accumulators in tensor memory
//     (two buffers, so the epilogue of one tile overlaps the main loop of the
//     next), one elected thread issuing the MMAs, a persistent grid of one CTA
//     per SM walking the output tiles.
//
// Roles inside a CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer
// and tensor-memory owner, warps 2..5 = epilogue (tcgen05.ld -> convert ->
// global stores in the reference's sliced output layout).
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace mld {
namespace {

// ------------------------------------------------------------------ tcgen05
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
template <bool I8>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                     uint32_t accumulate) {
  if constexpr (I8) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
  }
}
// 32 lanes x 32 consecutive 32-bit columns -> 32 registers per thread.
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

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes
// and which TMA wrote with the 128-byte swizzle: 8-row groups 1024 bytes apart
// (stride byte offset), descriptor version 1, layout type SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset (unused with swizzle)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // version
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

constexpr int kTileM = 128;
constexpr int kTileKBytes = 128;       // one swizzle atom of K per stage
constexpr int kUmmaKBytes = 32;        // bytes of K consumed by one tcgen05.mma
constexpr int kGemmThreads = 192;
constexpr int kTmemCols = 512;

struct GemmArgs {
  int M, N, N4, K;            // logical sizes; K in elements
  int tile_n;                 // UMMA N (multiple of 16, <= 256)
  int m_tiles, n_tiles, k_blocks;
  int stages, a_stage_bytes, b_stage_bytes;
  const void* bias;           // fp16 [N4] or null
  const __half* w_scale;      // I8: per-output-channel scale [N4] (fp16, as stored for the operator)
  const float* a_params;      // I8: per-token {inv_scale, offset, sum}
  void* y;                    // fp16
  int dst_layout;
  int* error;
};

template <bool I8>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_umma_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = a.a_stage_bytes + a.b_stage_bytes;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + (size_t)a.stages * stage_bytes);
  uint64_t* empty = full + a.stages;
  uint64_t* tmem_full = empty + a.stages;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;     // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int total_tiles = a.m_tiles * a.n_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 4);  // one arrival per epilogue warp
    }
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_base_slot;

  if (warp == 0) {
    // --------------------------------------------------------------- producer
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      prefetch_tmap(&tmap_b);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int k_elems_per_block = I8 ? kTileKBytes : kTileKBytes / 2;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
        const int mi = tile % a.m_tiles, ni = tile / a.m_tiles;
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicExch(a.error, 11);
            ok = false;
            break;
          }
          uint8_t* st = smem + (size_t)stage * stage_bytes;
          mbar_arrive_expect_tx(&full[stage], a.a_stage_bytes + a.b_stage_bytes);
          tma_load_2d(st, &tmap_a, &full[stage], kb * k_elems_per_block, mi * kTileM);
          tma_load_2d(st + a.a_stage_bytes, &tmap_b, &full[stage], kb * k_elems_per_block, ni * a.tile_n);
          if (++stage == a.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      // instruction descriptor: D = F32 (or S32), A/B = F16 (or signed INT8), both K-major
      uint32_t idesc;
      if constexpr (I8)
        idesc = (2u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(a.tile_n >> 3) << 17) |
                (static_cast<uint32_t>(kTileM >> 4) << 24);
      else
        idesc = (1u << 4) | (static_cast<uint32_t>(a.tile_n >> 3) << 17) | (static_cast<uint32_t>(kTileM >> 4) << 24);
      int stage = 0;
      uint32_t phase = 0;
      uint32_t acc_phase[2] = {0, 0};
      int local = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
        const int acc = local & 1;
        if (!mbar_wait(&tmem_empty[acc], acc_phase[acc] ^ 1)) {
          atomicExch(a.error, 12);
          ok = false;
          break;
        }
        acc_phase[acc] ^= 1;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * a.tile_n);
        for (int kb = 0; kb < a.k_blocks; ++kb) {
          if (!mbar_wait(&full[stage], phase)) {
            atomicExch(a.error, 13);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + (size_t)stage * stage_bytes);
          const uint64_t da = make_desc(sa), db = make_desc(sa + a.a_stage_bytes);
#pragma unroll
          for (int k = 0; k < kTileKBytes / kUmmaKBytes; ++k) {
            // advancing K inside the swizzle atom = advancing the start address
            const uint64_t adv = static_cast<uint64_t>((k * kUmmaKBytes) >> 4);
            umma<I8>(tmem_d, da + adv, db + adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          tc_commit(&empty[stage]);  // the stage is free once these MMAs have read it
          if (++stage == a.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) tc_commit(&tmem_full[acc]);  // the accumulator is complete
      }
    }
  } else {
    // --------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    uint32_t acc_phase[2] = {0, 0};
    int local = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++local) {
      const int acc = local & 1;
      const int mi = tile % a.m_tiles, ni = tile / a.m_tiles;
      if (!mbar_wait(&tmem_full[acc], acc_phase[acc])) {
        atomicExch(a.error, 14);
        ok = false;
        break;
      }
      acc_phase[acc] ^= 1;
      tc_fence_after();
      const int m = mi * kTileM + quad * 32 + lane;
      const int n0 = ni * a.tile_n;
      float a_scale = 1.0f;
      if constexpr (I8) a_scale = m < a.M ? a.a_params[m * 3] : 0.0f;
      for (int c0 = 0; c0 < a.tile_n; c0 += 32) {
        uint32_t r[32];
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) +
                               static_cast<uint32_t>(acc * a.tile_n + c0);
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
                // CreateDequantization: res = float(acc) * (w_scale * src_scale)
                const float ws = (n + e) < a.N ? __half2float(a.w_scale[n + e]) : 0.0f;
                v = static_cast<float>(static_cast<int32_t>(r[j + e])) * (ws * a_scale);
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
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ------------------------------------------------------ operand preparation
// Packed weights [K/4][N/4][4k][4n] -> K-major rows [N4][Kp].
//   fp16 route: w = half(half(u * scale) + half(-scale * shift)), the
//     WeightsConverter arithmetic (conv_weights_converter.cc:248-290);
//   s8 route: w = u - shift (exact).
// A CTA moves a tile of 32 k-slices x 32 output slices: packed rows are read
// coalesced into shared memory, then each thread turns whole 4x4 blocks into
// four K-major pieces with packed-half arithmetic; consecutive lanes take
// consecutive k-slices, so every output row is written in 256-byte runs.
__device__ __forceinline__ uint32_t dq_pair(uint32_t w, int nib, __half2 s2, __half2 b2) {
  // nibbles `nib` of the two halves of w (k even / k odd of one output) -> (1024 + u) -> u -> u*s + b
  const uint32_t m = ((w >> (4 * nib)) & 0x000F000Fu) | 0x64006400u;
  const __half2 u = __hsub2(*reinterpret_cast<const __half2*>(&m), __float2half2_rn(1024.0f));
  const __half2 r = __hadd2(__hmul2(u, s2), b2);
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t dq_pair8(uint32_t bytes2, __half2 s2, __half2 b2) {
  // two bytes (k even in bits 0..7, k odd in bits 16..23) -> halves
  const uint32_t m = (bytes2 & 0x00FF00FFu) | 0x64006400u;
  const __half2 u = __hsub2(*reinterpret_cast<const __half2*>(&m), __float2half2_rn(1024.0f));
  const __half2 r = __hadd2(__hmul2(u, s2), b2);
  return *reinterpret_cast<const uint32_t*>(&r);
}

__device__ __forceinline__ void transpose_sliced_tile(const __half* __restrict__ x, int M, int K, int Kp,
                                                      __half* __restrict__ out, int tile_s, int tile_m);

// The activations of the same call can ride along: rows of blocks past `weight_rows` of the grid transpose
// 32 x 32 tiles of the sliced activation tensor instead (x_src null: none), which saves a launch and hides the
// small transposition behind the conversion.
struct RideAlong {
  const __half* x_src;
  __half* x_out;
  int M, K;
  int weight_rows;  // gridDim.y of the conversion proper
};

template <int BITS, bool TO_S8>
__global__ void __launch_bounds__(256) dequant_weights_kernel(const uint8_t* __restrict__ packed,
                                                             const __half* __restrict__ scale, int scale_mode, int G,
                                                             int group_slices, float scalar_scale, int dst_slices,
                                                             int src_slices, int Kp, void* __restrict__ out,
                                                             RideAlong ride) {
  pdl_launch_dependents();
  pdl_wait();
  if (ride.x_src != nullptr && static_cast<int>(blockIdx.y) >= ride.weight_rows) {
    transpose_sliced_tile(ride.x_src, ride.M, ride.K, Kp, ride.x_out, blockIdx.x, blockIdx.y - ride.weight_rows);
    return;
  }
  constexpr int T = 32;
  constexpr int BLK = BITS == 4 ? 8 : 16;
  constexpr int PITCH = T * BLK + 8;  // +8 bytes: lanes that walk down a column hit distinct banks
  __shared__ __align__(16) uint8_t tile[T * PITCH];
  const int ks0 = blockIdx.x * T, ds0 = blockIdx.y * T;
  const int N4 = dst_slices * 4;
  constexpr int PIECES = T * BLK / 8;
  for (int idx = threadIdx.x; idx < T * PIECES; idx += blockDim.x) {
    const int r = idx / PIECES, pc = idx % PIECES;
    const int ks = ks0 + r;
    const int byte0 = ds0 * BLK + pc * 8;
    uint2 v = make_uint2(0, 0);
    if (ks < src_slices && byte0 < dst_slices * BLK)
      v = *reinterpret_cast<const uint2*>(packed + (size_t)ks * dst_slices * BLK + byte0);
    *reinterpret_cast<uint2*>(&tile[r * PITCH + pc * 8]) = v;
  }
  __syncthreads();
  const int shift = BITS == 8 ? 128 : 8;
  const int r = threadIdx.x & 31;  // k-slice inside the tile (fastest over lanes)
  const int ks = ks0 + r;
  if (ks * 4 >= Kp) return;
  for (int dsl = threadIdx.x >> 5; dsl < T; dsl += 8) {
    const int ds = ds0 + dsl;
    if (ds >= dst_slices) break;
    const int n = ds * 4;
    if constexpr (TO_S8) {
      uint32_t w[4];
      if constexpr (BITS == 8) {
        const uint4 q = make_uint4(*reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 16]),
                                   *reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 16 + 4]),
                                   *reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 16 + 8]),
                                   *reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 16 + 12]));
        // rows of q are k (bytes = outputs); transpose 4x4 bytes and re-bias u8 -> s8
        const uint32_t a = q.x ^ 0x80808080u, b = q.y ^ 0x80808080u, c = q.z ^ 0x80808080u, d = q.w ^ 0x80808080u;
        const uint32_t ab_lo = __byte_perm(a, b, 0x5140), ab_hi = __byte_perm(a, b, 0x7362);
        const uint32_t cd_lo = __byte_perm(c, d, 0x5140), cd_hi = __byte_perm(c, d, 0x7362);
        w[0] = __byte_perm(ab_lo, cd_lo, 0x5410);
        w[1] = __byte_perm(ab_lo, cd_lo, 0x7632);
        w[2] = __byte_perm(ab_hi, cd_hi, 0x5410);
        w[3] = __byte_perm(ab_hi, cd_hi, 0x7632);
      } else {
        const uint32_t lo = *reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 8]);
        const uint32_t hi = *reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 8 + 4]);
#pragma unroll
        for (int o = 0; o < 4; ++o) {
          const int k0 = static_cast<int>((lo >> (4 * o)) & 0xF) - shift, k1 = static_cast<int>((lo >> (16 + 4 * o)) & 0xF) - shift;
          const int k2 = static_cast<int>((hi >> (4 * o)) & 0xF) - shift, k3 = static_cast<int>((hi >> (16 + 4 * o)) & 0xF) - shift;
          w[o] = (k0 & 0xFF) | ((k1 & 0xFF) << 8) | ((k2 & 0xFF) << 16) | ((k3 & 0xFF) << 24);
        }
      }
#pragma unroll
      for (int o = 0; o < 4; ++o)
        *reinterpret_cast<uint32_t*>(static_cast<int8_t*>(out) + (size_t)(n + o) * Kp + ks * 4) = w[o];
    } else {
      __half sc[4];
      if (scale_mode == MLD_SCALE_SCALAR) {
        sc[0] = sc[1] = sc[2] = sc[3] = __float2half_rn(scalar_scale);
      } else {
        int g = scale_mode == MLD_SCALE_BLOCK ? ks / group_slices : 0;
        if (g >= G) g = G - 1;
        const uint2 sv = *reinterpret_cast<const uint2*>(scale + (size_t)g * N4 + n);
        sc[0] = __ushort_as_half(static_cast<unsigned short>(sv.x & 0xFFFF));
        sc[1] = __ushort_as_half(static_cast<unsigned short>(sv.x >> 16));
        sc[2] = __ushort_as_half(static_cast<unsigned short>(sv.y & 0xFFFF));
        sc[3] = __ushort_as_half(static_cast<unsigned short>(sv.y >> 16));
      }
      const __half hshift = __ushort2half_rn(static_cast<unsigned short>(shift));
#pragma unroll
      for (int o = 0; o < 4; ++o) {
        const __half2 s2 = __half2half2(sc[o]);
        const __half2 b2 = __half2half2(__hmul(__hneg(sc[o]), hshift));
        uint2 pk;
        if constexpr (BITS == 4) {
          const uint32_t lo = *reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 8]);
          const uint32_t hi = *reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 8 + 4]);
          pk.x = dq_pair(lo, o, s2, b2);  // (k0, k1) of output o
          pk.y = dq_pair(hi, o, s2, b2);  // (k2, k3)
        } else {
          const uint32_t* q = reinterpret_cast<const uint32_t*>(&tile[r * PITCH + dsl * 16]);
          // byte o of k-row i: gather (k0, k1) and (k2, k3) into the byte lanes dq_pair8 reads
          const uint32_t b01 = ((q[0] >> (8 * o)) & 0xFFu) | (((q[1] >> (8 * o)) & 0xFFu) << 16);
          const uint32_t b23 = ((q[2] >> (8 * o)) & 0xFFu) | (((q[3] >> (8 * o)) & 0xFFu) << 16);
          pk.x = dq_pair8(b01, s2, b2);
          pk.y = dq_pair8(b23, s2, b2);
        }
        *reinterpret_cast<uint2*>(static_cast<__half*>(out) + (size_t)(n + o) * Kp + ks * 4) = pk;
      }
    }
  }
}

// Activations: sliced [K/4][M][4] (or row-major [M][K]) fp16 -> row-major [M][Kp] fp16.
// Sliced source: a 32-token x 32-slice tile goes through shared memory, read with lanes along the tokens
// (8 bytes each, contiguous in the source) and written with lanes along K (contiguous in the destination).
__device__ __forceinline__ void transpose_sliced_tile(const __half* __restrict__ x, int M, int K, int Kp,
                                                      __half* __restrict__ out, int tile_s, int tile_m) {
  __shared__ uint2 tile[32][33];
  const int S = (K + 3) / 4, Sp = Kp / 4;
  const int m0 = tile_m * 32, s0 = tile_s * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 8 rows of the tile per pass
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int sl = s0 + ty + 8 * r, m = m0 + tx;
    uint2 v = make_uint2(0u, 0u);
    if (sl < S && m < M) v = *reinterpret_cast<const uint2*>(x + ((size_t)sl * M + m) * 4);
    tile[ty + 8 * r][tx] = v;  // [slice][token]
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int m = m0 + ty + 8 * r, sl = s0 + tx;
    if (m < M && sl < Sp) {
      uint2 v = tile[tx][ty + 8 * r];
      // a ragged K: the channels past K inside the last slice must read as zero
      if (sl * 4 + 3 >= K) {
        __half* h = reinterpret_cast<__half*>(&v);
        for (int i = 0; i < 4; ++i)
          if (sl * 4 + i >= K) h[i] = __float2half(0.0f);
      }
      *reinterpret_cast<uint2*>(out + (size_t)m * Kp + sl * 4) = v;
    }
  }
}

__global__ void __launch_bounds__(256) transpose_x_kernel(const __half* __restrict__ x, int layout, int M, int K, int Kp,
                                                          __half* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int Sp = Kp / 4;
  if (layout == MLD_LAYOUT_SLICED) {
    transpose_sliced_tile(x, M, K, Kp, out, blockIdx.x, blockIdx.y);
    return;
  }
  const int ks = blockIdx.x * 32 * 8 + threadIdx.x;  // one token row per blockIdx.y, 256 slices per block
  const int m = blockIdx.y;
  if (ks >= Sp || m >= M) return;
  __half h[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = ks * 4 + i < K ? x[(size_t)m * K + ks * 4 + i] : __float2half(0.0f);
  uint2 v;
  v.x = static_cast<uint32_t>(__half_as_ushort(h[0])) | (static_cast<uint32_t>(__half_as_ushort(h[1])) << 16);
  v.y = static_cast<uint32_t>(__half_as_ushort(h[2])) | (static_cast<uint32_t>(__half_as_ushort(h[3])) << 16);
  *reinterpret_cast<uint2*>(out + (size_t)m * Kp + ks * 4) = v;
}

// Per-token quantisation to s8 (CreateQuantization,
// ml_drift/common/kernels/quantize_and_dequantize.cc:355-441, constants :757-784).
// One CTA per token; x ~ q * inv_scale + offset.
//   symmetric   inv_scale = max(min_scale, absmax / 127), scale = 1 / inv_scale, offset = 0,
//               q = clamp(floor(x * scale + 128.5), 0, 255) - 128
//   asymmetric  (the reference builder's default, common/gpu_model_builder.h:236-240)
//               range = max - min, scale = 255 / range, inv_scale = range / 255,
//               offset = min + range * (128 / 255), q = clamp(int((x - min) * scale + 0.5), 0, 255) - 128
//               (a constant token, range 0, gets inv_scale 0: every x equals the offset)
// Output xq row-major [M][Kp] s8 (zero padded), params [M][3] = {inv_scale, offset, sum of the codes}.
__global__ void __launch_bounds__(256) quantize_act_kernel(const __half* __restrict__ x, int layout, int M, int K, int Kp,
                                                           int symmetric, int8_t* __restrict__ xq,
                                                           float* __restrict__ params) {
  pdl_launch_dependents();
  pdl_wait();
  const int m = blockIdx.x;
  __shared__ float red[8], red2[8];
  __shared__ int redi[8];
  auto load = [&](int k) -> float {
    const size_t idx = layout == MLD_LAYOUT_SLICED ? (((size_t)(k >> 2) * M + m) * 4 + (k & 3)) : ((size_t)m * K + k);
    return __half2float(x[idx]);
  };
  float vmin = INFINITY, vmax = -INFINITY;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const float v = load(k);
    vmin = fminf(vmin, v);
    vmax = fmaxf(vmax, v);
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, off));
    vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, off));
  }
  if ((threadIdx.x & 31) == 0) {
    red[threadIdx.x >> 5] = vmin;
    red2[threadIdx.x >> 5] = vmax;
  }
  __syncthreads();
  vmin = INFINITY;
  vmax = -INFINITY;
  for (int w = 0; w < 8; ++w) {
    vmin = fminf(vmin, red[w]);
    vmax = fmaxf(vmax, red2[w]);
  }
  float inv_scale = 0.0f, scale = 0.0f, offset = 0.0f;
  if (symmetric) {
    const float amax = fmaxf(fabsf(vmin), fabsf(vmax));
    if (amax > 0.0f) {
      inv_scale = fmaxf(6.103515625e-05f, __fdiv_rn(amax, 127.0f));
      scale = __fdiv_rn(1.0f, inv_scale);
    }
  } else {
    const float range = __fsub_rn(vmax, vmin);
    offset = vmin;
    if (range > 0.0f) {
      scale = __fdiv_rn(255.0f, range);
      inv_scale = __fdiv_rn(range, 255.0f);
      offset = __fadd_rn(offset, __fmul_rn(range, __fdiv_rn(128.0f, 255.0f)));
    }
  }
  int sum = 0;
  for (int k = threadIdx.x; k < Kp; k += blockDim.x) {
    int q = 0;
    if (k < K) {
      if (symmetric) {
        float r = floorf(__fadd_rn(__fmul_rn(load(k), scale), 128.5f));
        r = fminf(255.0f, fmaxf(0.0f, r));
        q = static_cast<int>(r) - 128;
      } else {
        const float r = __fadd_rn(__fmul_rn(__fsub_rn(load(k), vmin), scale), 0.5f);
        q = min(255, max(0, static_cast<int>(r))) - 128;
      }
    }
    xq[(size_t)m * Kp + k] = static_cast<int8_t>(q);
    sum += q;
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if ((threadIdx.x & 31) == 0) redi[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    int t = 0;
    for (int w = 0; w < 8; ++w) t += redi[w];
    params[m * 3 + 0] = inv_scale;
    params[m * 3 + 1] = offset;
    params[m * 3 + 2] = static_cast<float>(t);
  }
}

// The same quantisation for the sliced source layout [K/4][M][4], where a token's channels lie M * 8 bytes
// apart: two passes with lanes along the tokens (contiguous 8-byte pieces), the second one turning a
// 32-token x 32-slice tile through shared memory so that the K-major rows are written in 128-byte runs.
//   pass 1: per-token minimum / maximum over one of kStatSplits ranges of the slices -> part [split][M][2]
//   pass 2: folds the partial extremes, derives the token's parameters (params [M][3] = {inv_scale, offset, 0},
//           written by the first column of blocks) and the codes (the arithmetic of quantize_act_kernel, bit
//           for bit)
// The sum of a token's codes (params[2]) is not produced: only a weight zero point would use it
// (quantize_and_dequantize.cc:927-936), and that route takes none.
__global__ void __launch_bounds__(256) act_stats_sliced_kernel(const __half* __restrict__ x, int M, int K,
                                                               float* __restrict__ part) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float smin[8][33], smax[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int m = blockIdx.x * 32 + tx;
  const int S = (K + 3) / 4;
  const int per = (S + kStatSplits - 1) / kStatSplits;
  const int s_begin = blockIdx.y * per, s_end = min(S, s_begin + per);
  float vmin = INFINITY, vmax = -INFINITY;
  if (m < M) {
#pragma unroll 4
    for (int sl = s_begin + ty; sl < s_end; sl += 8) {
      const uint2 v = *reinterpret_cast<const uint2*>(x + ((size_t)sl * M + m) * 4);
      const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        if (sl * 4 + i < K) {
          const float f = __half2float(h[i]);
          vmin = fminf(vmin, f);
          vmax = fmaxf(vmax, f);
        }
      }
    }
  }
  smin[ty][tx] = vmin;
  smax[ty][tx] = vmax;
  __syncthreads();
  if (ty == 0 && m < M) {
#pragma unroll
    for (int r = 1; r < 8; ++r) {
      vmin = fminf(vmin, smin[r][tx]);
      vmax = fmaxf(vmax, smax[r][tx]);
    }
    part[((size_t)blockIdx.y * M + m) * 2 + 0] = vmin;
    part[((size_t)blockIdx.y * M + m) * 2 + 1] = vmax;
  }
}

__global__ void __launch_bounds__(256) act_quantize_sliced_kernel(const __half* __restrict__ x, int M, int K, int Kp,
                                                                  int symmetric, const float* __restrict__ part,
                                                                  float* __restrict__ params,
                                                                  int8_t* __restrict__ xq) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ uint32_t tile[32][33];
  const int S = (K + 3) / 4, Sp = Kp / 4;
  const int m0 = blockIdx.y * 32, s0 = blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int m = m0 + tx;
  float scale = 0.0f, vmin = 0.0f;
  if (m < M) {
    float vmax = -INFINITY;
    vmin = INFINITY;
#pragma unroll
    for (int y = 0; y < kStatSplits; ++y) {
      vmin = fminf(vmin, part[((size_t)y * M + m) * 2 + 0]);
      vmax = fmaxf(vmax, part[((size_t)y * M + m) * 2 + 1]);
    }
    float inv_scale = 0.0f, offset = 0.0f;
    if (symmetric) {
      const float amax = fmaxf(fabsf(vmin), fabsf(vmax));
      if (amax > 0.0f) inv_scale = fmaxf(6.103515625e-05f, __fdiv_rn(amax, 127.0f));
      if (inv_scale > 0.0f) scale = __fdiv_rn(1.0f, inv_scale);
    } else {
      const float range = __fsub_rn(vmax, vmin);
      offset = vmin;
      if (range > 0.0f) {
        inv_scale = __fdiv_rn(range, 255.0f);
        offset = __fadd_rn(offset, __fmul_rn(range, __fdiv_rn(128.0f, 255.0f)));
        scale = __fdiv_rn(255.0f, range);
      }
    }
    if (blockIdx.x == 0 && ty == 0) {
      params[m * 3 + 0] = inv_scale;
      params[m * 3 + 1] = offset;
      params[m * 3 + 2] = 0.0f;
    }
  }
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int sl = s0 + ty + 8 * r;
    uint32_t packed = 0;
    if (sl < S && m < M) {
      const uint2 v = *reinterpret_cast<const uint2*>(x + ((size_t)sl * M + m) * 4);
      const __half* h = reinterpret_cast<const __half*>(&v);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        int q = 0;
        if (sl * 4 + i < K) {
          const float f = __half2float(h[i]);
          if (symmetric) {
            float t = floorf(__fadd_rn(__fmul_rn(f, scale), 128.5f));
            t = fminf(255.0f, fmaxf(0.0f, t));
            q = static_cast<int>(t) - 128;
          } else {
            const float t = __fadd_rn(__fmul_rn(__fsub_rn(f, vmin), scale), 0.5f);
            q = min(255, max(0, static_cast<int>(t))) - 128;
          }
        }
        packed |= static_cast<uint32_t>(q & 0xFF) << (8 * i);
      }
    }
    tile[ty + 8 * r][tx] = packed;  // [slice][token]
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int mm = m0 + ty + 8 * r, sl = s0 + tx;
    if (mm < M && sl < Sp) *reinterpret_cast<uint32_t*>(xq + (size_t)mm * Kp + sl * 4) = tile[tx][ty + 8 * r];
  }
}

}  // namespace

// ------------------------------------------------------------------ host side
GemmGeometry gemm_geometry(int M, int N, int K, bool i8, int sms) {
  GemmGeometry g;
  const int N4 = align_n(N, 4);
  g.kp = align_n(K, i8 ? 16 : 8);  // K-major row pitch must be a multiple of 16 bytes
  g.m_tiles = div_up(M, kTileM);
  // Choose the UMMA N.  A tile costs 2*N tensor-pipe cycles per 64-wide K block
  // and pulls (128 + N) * 128 bytes of operands through L2 for it; with one CTA
  // per tile the L2 -> SM traffic, not the tensor pipe, bounds narrow tiles, so
  // the estimate is the larger of the two over all waves (L2 feed taken as
  // 6.5 KB per cycle across the GPU, the rate this kernel was measured to draw).
  int best_n = 256;
  double best_cost = -1.0;
  for (int tn = 256; tn >= 64; tn -= 16) {
    const double tiles = (double)g.m_tiles * div_up(N4, tn);
    const double waves = (double)(((long)tiles + sms - 1) / sms);
    const double mma = waves * 2.0 * tn;
    const double l2 = tiles * (128.0 + tn) * 128.0 / 6500.0;
    const double cost = mma > l2 ? mma : l2;
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_n = tn;
    }
  }
  g.tile_n = best_n;
  g.n_tiles = div_up(N4, g.tile_n);
  const int k_elems = i8 ? kTileKBytes : kTileKBytes / 2;
  g.k_blocks = div_up(g.kp, k_elems);
  g.a_stage_bytes = kTileM * kTileKBytes;
  g.b_stage_bytes = align_n(g.tile_n * kTileKBytes, 1024);
  const int fixed = 1024 + 64 * 8 + 64;
  int stages = (220 * 1024 - fixed) / (g.a_stage_bytes + g.b_stage_bytes);
  if (stages > 8) stages = 8;
  g.stages = stages;
  g.smem_bytes = (size_t)stages * (g.a_stage_bytes + g.b_stage_bytes) + fixed;
  const long tiles = (long)g.m_tiles * g.n_tiles;
  g.grid = static_cast<int>(tiles < sms ? tiles : sms);
  return g;
}

int launch_dequant_weights(int bits, bool to_s8, const void* packed, const void* scale, int scale_mode, int G,
                           int group_slices, float scalar_scale, int N, int K, int Kp, void* out, cudaStream_t stream,
                           const void* x_sliced, int M, void* x_kmajor) {
  const int dst_slices = div_up(N, 4), src_slices = div_up(K, 4);
  dim3 grid(div_up(div_up(Kp, 4), 32), div_up(dst_slices, 32));
  RideAlong ride;
  ride.x_src = static_cast<const __half*>(x_sliced);
  ride.x_out = static_cast<__half*>(x_kmajor);
  ride.M = M;
  ride.K = K;
  ride.weight_rows = static_cast<int>(grid.y);
  if (x_sliced != nullptr) grid.y += div_up(M, 32);
  const uint8_t* p = static_cast<const uint8_t*>(packed);
  const __half* s = static_cast<const __half*>(scale);
#define MLD_DQ(B, S8)                                                                                              \
  MLD_CUDA_CHECK(launch_overlapped(dequant_weights_kernel<B, S8>, grid, dim3(256), 0, stream, p, s, scale_mode, G, \
                                   group_slices, scalar_scale, dst_slices, src_slices, Kp, out, ride))
  if (bits == 4) {
    if (to_s8) MLD_DQ(4, true); else MLD_DQ(4, false);
  } else {
    if (to_s8) MLD_DQ(8, true); else MLD_DQ(8, false);
  }
#undef MLD_DQ
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

int launch_transpose_x(const void* x, int layout, int M, int K, int Kp, void* out, cudaStream_t stream) {
  dim3 grid(div_up(div_up(Kp, 4), 256), M);
  if (layout == MLD_LAYOUT_SLICED) grid = dim3(div_up(div_up(Kp, 4), 32), div_up(M, 32));
  MLD_CUDA_CHECK(launch_overlapped(transpose_x_kernel, grid, dim3(256), 0, stream, static_cast<const __half*>(x), layout,
                                   M, K, Kp, static_cast<__half*>(out)));
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

int launch_quantize_act(const void* x, int layout, int M, int K, int Kp, bool symmetric, void* xq, float* params,
                        cudaStream_t stream) {
  if (layout == MLD_LAYOUT_SLICED) {
    // params holds [M][3] parameters followed by the partial extremes [kStatSplits][M][2]
    // (kActParamFloats floats per token in all)
    float* part = params + (size_t)M * 3;
    MLD_CUDA_CHECK(launch_overlapped(act_stats_sliced_kernel, dim3(div_up(M, 32), kStatSplits), dim3(256), 0, stream,
                                     static_cast<const __half*>(x), M, K, part));
    MLD_LAUNCH_CHECK();
    dim3 grid(div_up(Kp / 4, 32), div_up(M, 32));
    MLD_CUDA_CHECK(launch_overlapped(act_quantize_sliced_kernel, grid, dim3(256), 0, stream,
                                     static_cast<const __half*>(x), M, K, Kp, symmetric ? 1 : 0,
                                     static_cast<const float*>(part), params, static_cast<int8_t*>(xq)));
    MLD_LAUNCH_CHECK();
    return MLD_OK;
  }
  MLD_CUDA_CHECK(launch_overlapped(quantize_act_kernel, dim3(M), dim3(256), 0, stream, static_cast<const __half*>(x),
                                   layout, M, K, Kp, symmetric ? 1 : 0, static_cast<int8_t*>(xq), params));
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

int launch_gemm_umma(bool i8, const void* a_mat, const void* b_mat, const GemmGeometry& g, int M, int N, int K,
                     const void* bias, const void* w_scale, const float* a_params, void* y, int dst_layout, int* error,
                     cudaStream_t stream) {
  (void)K;
  const int N4 = align_n(N, 4);
  const int esz = i8 ? 1 : 2;
  CUtensorMap ta, tb;
  // K-major matrices: rows of kp elements; boxes of one swizzle atom (128 bytes of K) x tile rows
  int rc = make_tmap_2d(&ta, a_mat, (uint64_t)g.kp * esz, M, (uint64_t)g.kp * esz, kTileKBytes, kTileM, esz,
                        CU_TENSOR_MAP_SWIZZLE_128B, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        true);
  if (rc != MLD_OK) return rc;
  rc = make_tmap_2d(&tb, b_mat, (uint64_t)g.kp * esz, N4, (uint64_t)g.kp * esz, kTileKBytes, g.tile_n, esz,
                    CU_TENSOR_MAP_SWIZZLE_128B, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                    true);
  if (rc != MLD_OK) return rc;
  GemmArgs a;
  a.M = M;
  a.N = N;
  a.N4 = N4;
  a.K = g.kp;
  a.tile_n = g.tile_n;
  a.m_tiles = g.m_tiles;
  a.n_tiles = g.n_tiles;
  a.k_blocks = g.k_blocks;
  a.stages = g.stages;
  a.a_stage_bytes = g.a_stage_bytes;
  a.b_stage_bytes = g.b_stage_bytes;
  a.bias = bias;
  a.w_scale = static_cast<const __half*>(w_scale);
  a.a_params = a_params;
  a.y = y;
  a.dst_layout = dst_layout;
  a.error = error;
  static bool configured[2][kMaxDevices];
  int dev;
  if (i8) {
    if (needs_configure(configured[1], &dev)) {
      MLD_CUDA_CHECK(cudaFuncSetAttribute(gemm_umma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      if (dev >= 0) configured[1][dev] = true;
    }
    gemm_umma_kernel<true><<<g.grid, kGemmThreads, g.smem_bytes, stream>>>(ta, tb, a);
  } else {
    if (needs_configure(configured[0], &dev)) {
      MLD_CUDA_CHECK(cudaFuncSetAttribute(gemm_umma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
      if (dev >= 0) configured[0][dev] = true;
    }
    gemm_umma_kernel<false><<<g.grid, kGemmThreads, g.smem_bytes, stream>>>(ta, tb, a);
  }
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

}  // namespace mld
