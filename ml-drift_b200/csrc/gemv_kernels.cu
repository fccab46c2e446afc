// Decode-stage dequant-GEMV kernels (1..16 tokens) over the reference's packed
// weight layout [K/4][N/4][4 k][4 n].
//
//  * fc_stream_kernel: the production kernel.  HBM-bound: packed weights,
//    block scales and activations are staged by TMA into a ring of shared
//    memory stages; eight consumer warps dequantise in registers and feed
//    m16n8k16 tensor-core MMAs (weights as the 16-row operand, up to 8/16
//    tokens as columns) with fp32 accumulation; work is split over the grid in
//    (output tile x K chunk) items, with split-K partials combined in a fixed
//    order by the last CTA to finish a tile (deterministic).
//  * fc_generic_kernel: covers every remaining case of the operator (fp32
//    tensors, zero points, scalar scale, ragged shapes, odd group sizes) with
//    plain loads; one warp per output slice.
//
// Arithmetic restated from GetFullyConnectedKernelCode
// (ml_drift/common/kernels/fully_connected.cc:623-942) and fc:: helpers
// (fully_connected_util.cc:80-229, 356-407).
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace mld {

// ===================================================================== generic
namespace {

template <typename T>
struct ActOps;
template <>
struct ActOps<float> {
  static __device__ __forceinline__ float load(const void* p, int64_t i) { return static_cast<const float*>(p)[i]; }
  static __device__ __forceinline__ void store(void* p, int64_t i, float v) { static_cast<float*>(p)[i] = v; }
};
template <>
struct ActOps<__half> {
  static __device__ __forceinline__ __half load(const void* p, int64_t i) { return static_cast<const __half*>(p)[i]; }
  static __device__ __forceinline__ void store(void* p, int64_t i, __half v) { static_cast<__half*>(p)[i] = v; }
};

__device__ __forceinline__ int64_t act_index(int layout, int M, int C, int m, int c) {
  return layout == MLD_LAYOUT_SLICED ? (((int64_t)(c >> 2) * M + m) * 4 + (c & 3)) : ((int64_t)m * C + c);
}

constexpr int kGenTokens = 4;  // tokens per pass of the generic kernel

// One warp per output slice; lanes stride over input slices; shuffle-tree sum.
// T = float: the kF32 arithmetic (separate multiply and add, fp32).
// T = __half: the kF32F16 arithmetic (dequantise and multiply in half, sum of
// four products in half, accumulate in fp32); kF16 requests use it too.
template <typename T, int BITS>
__global__ void __launch_bounds__(128) fc_generic_kernel(GenericArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int dst_s = blockIdx.x * 4 + warp;
  if (dst_s >= a.dst_slices) return;
  const int shift = BITS == 8 ? 128 : 8;
  const int N4 = a.dst_slices * 4;
  const uint8_t* wp = static_cast<const uint8_t*>(a.weights);
  for (int m0 = 0; m0 < a.M; m0 += kGenTokens) {
    float acc[kGenTokens][4];
#pragma unroll
    for (int m = 0; m < kGenTokens; ++m)
#pragma unroll
      for (int o = 0; o < 4; ++o) acc[m][o] = 0.0f;
    int cached_g = -1;
    T ws[4], wb[4];
    for (int src_s = lane; src_s < a.src_slices; src_s += 32) {
      int g = 0;
      if (a.scale_mode == MLD_SCALE_BLOCK) {
        g = src_s / a.group_slices;
        if (g >= a.groups) g = a.groups - 1;
      }
      if (g != cached_g) {
        cached_g = g;
#pragma unroll
        for (int o = 0; o < 4; ++o) {
          T s, z = T(0.0f);
          if (a.scale_mode == MLD_SCALE_SCALAR) {
            s = T(a.scalar_scale);
            if (a.has_zp) z = T(a.scalar_zp);
          } else {
            const int64_t idx = (int64_t)g * N4 + dst_s * 4 + o;
            s = ActOps<T>::load(a.scale, idx);
            if (a.zp != nullptr) z = ActOps<T>::load(a.zp, idx);
          }
          T sh = T(static_cast<float>(shift));
          if (a.has_zp) sh = sh + z;
          ws[o] = s;
          wb[o] = -s * sh;
        }
      }
      uint8_t u[4][4];
      const int64_t lin = (int64_t)src_s * a.dst_slices + dst_s;
      if (BITS == 8) {
        const uint4 q = *reinterpret_cast<const uint4*>(wp + lin * 16);
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int o = 0; o < 4; ++o) u[i][o] = (w[i] >> (8 * o)) & 0xFF;
      } else {
        const uint2 q = *reinterpret_cast<const uint2*>(wp + lin * 8);
        const uint32_t w[2] = {q.x, q.y};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int o = 0; o < 4; ++o) u[i][o] = (w[i >> 1] >> (16 * (i & 1) + 4 * o)) & 0xF;
      }
      T wv[4][4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int o = 0; o < 4; ++o) {
          if constexpr (sizeof(T) == 4) {
            wv[i][o] = __fadd_rn(__fmul_rn(static_cast<float>(u[i][o]), ws[o]), wb[o]);
          } else {
            wv[i][o] = __hadd(__hmul(__ushort2half_rn(u[i][o]), ws[o]), wb[o]);
          }
        }
#pragma unroll
      for (int m = 0; m < kGenTokens; ++m) {
        if (m0 + m >= a.M) break;
        T v[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = src_s * 4 + i;
          v[i] = c < a.K ? ActOps<T>::load(a.x, act_index(a.src_layout, a.M, a.K, m0 + m, c)) : T(0.0f);
        }
#pragma unroll
        for (int o = 0; o < 4; ++o) {
          if constexpr (sizeof(T) == 4) {
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[m][o] = __fadd_rn(acc[m][o], __fmul_rn(v[i], wv[i][o]));
          } else {
            __half t = __hmul(v[0], wv[0][o]);
            t = __hadd(t, __hmul(v[1], wv[1][o]));
            t = __hadd(t, __hmul(v[2], wv[2][o]));
            t = __hadd(t, __hmul(v[3], wv[3][o]));
            acc[m][o] += __half2float(t);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < kGenTokens; ++m)
#pragma unroll
      for (int o = 0; o < 4; ++o)
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc[m][o] += __shfl_xor_sync(0xffffffffu, acc[m][o], off);
    if (lane == 0) {
      for (int m = 0; m < kGenTokens && m0 + m < a.M; ++m)
        for (int o = 0; o < 4; ++o) {
          const int n = dst_s * 4 + o;
          if (a.dst_layout == MLD_LAYOUT_ROW_MAJOR && n >= a.N) continue;
          T r = T(acc[m][o]);
          if (a.bias != nullptr) r = r + ActOps<T>::load(a.bias, n);
          ActOps<T>::store(a.y, act_index(a.dst_layout, a.M, a.N, m0 + m, n), r);
        }
    }
  }
}

}  // namespace

int launch_fc_generic(const GenericArgs& a, int bits, bool f32, cudaStream_t stream) {
  const int grid = div_up(a.dst_slices, 4);
  if (grid == 0 || a.M == 0) return MLD_OK;
  if (f32) {
    if (bits == 8)
      fc_generic_kernel<float, 8><<<grid, 128, 0, stream>>>(a);
    else
      fc_generic_kernel<float, 4><<<grid, 128, 0, stream>>>(a);
  } else {
    if (bits == 8)
      fc_generic_kernel<__half, 8><<<grid, 128, 0, stream>>>(a);
    else
      fc_generic_kernel<__half, 4><<<grid, 128, 0, stream>>>(a);
  }
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

// ================================================================== streaming
namespace {

constexpr int kConsumerWarps = 8;
constexpr int kStageRows = 128;                       // k-slices per stage (512 input channels)
constexpr int kWarpRows = kStageRows / kConsumerWarps;  // 16
constexpr int kWBytes = kStageRows * 128;             // weight box: 128 rows x 128 bytes

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
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

// Fragment geometry.  Lane = 4*g + t.  A warp step covers four k-slice rows
// (row of lane = base + 2*t + parity) and one 128-byte row segment; lane g
// owns 16 bytes of it.
//   BITS 4: 16 bytes = two 4x4 blocks (8 outputs) -> 4 MMAs, tile of 64 outputs
//   BITS 8: 16 bytes = one 4x4 block  (4 outputs) -> 2 MMAs, tile of 32 outputs
// MMA f of a lane: rows g / g+8 are outputs n_local = NPL*g + 2*f + {0,1}; the
// sixteen k columns are (row t: k0 k1) at 2t,2t+1 and (row t: k2 k3) at 2t+8,9.
template <int BITS>
struct Frag {
  static constexpr int NF = BITS == 4 ? 4 : 2;    // MMAs (accumulator fragments) per lane
  static constexpr int NPL = BITS == 4 ? 8 : 4;   // outputs per lane
  static constexpr int TILE_N = NPL * 8;          // outputs per tile (64 / 32)
};

// EXACT mode: operands are (1024 + u) with the offset removed by one packed
// half subtract, giving the signed weight exactly (x16 for high nibbles).
// SUBNORMAL mode: operands are the raw masked bits, i.e. fp16 subnormals
// u * 2^-24 (x16 for high nibbles); the "- shift * sum(x)" term comes from one
// extra MMA against a constant operand, and results carry a 2^-24 factor.
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

struct Range {
  int64_t lo, hi;
};
__host__ __device__ __forceinline__ Range cta_range(int64_t total, int P, int c) {
  return Range{(int64_t)c * total / P, (int64_t)(c + 1) * total / P};
}
// The CTA whose range holds work item u.
__host__ __device__ __forceinline__ int cta_of(int64_t u, int64_t total, int P) {
  int c = static_cast<int>(u * P / total);
  while ((int64_t)(c + 1) * total / P <= u) ++c;
  return c;
}

template <int BITS, int NB, bool SUBNORMAL>
__global__ void __launch_bounds__((kConsumerWarps + 1) * 32, 1)
    fc_stream_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_s,
                     StreamArgs a) {
  using F = Frag<BITS>;
  constexpr int MTOK = 8 * NB;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // carve: stages | reduction buffer | barriers
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stage_bytes = a.stage_bytes;
  float* red = reinterpret_cast<float*>(smem + (size_t)a.stages * stage_bytes);
  uint64_t* full = reinterpret_cast<uint64_t*>(red + kConsumerWarps * F::TILE_N * MTOK);
  uint64_t* empty = full + a.stages;
  int* flag = reinterpret_cast<int*>(empty + a.stages);  // [0] ticket broadcast, [1] error broadcast

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t total = (int64_t)a.n_tiles * a.n_chunks;
  const Range rg = cta_range(total, gridDim.x, blockIdx.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    flag[0] = 0;
    flag[1] = 0;
    fence_barrier_init();
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      prefetch_tmap(&tmap_w);
      if (a.scale_rows > 0) prefetch_tmap(&tmap_s);
      const uint64_t pol = policy_evict_first();
      int stage = 0;
      uint32_t phase = 0;
      int tile = static_cast<int>(rg.lo / a.n_chunks), chunk = static_cast<int>(rg.lo % a.n_chunks);
      for (int64_t it = rg.lo; it < rg.hi; ++it, ++chunk) {
        if (chunk == a.n_chunks) {
          chunk = 0;
          ++tile;
        }
        if (!mbar_wait(&empty[stage], phase ^ 1)) {
          atomicExch(a.error, 1);
          break;
        }
        uint8_t* st = smem + (size_t)stage * stage_bytes;
        const int row0 = chunk * kStageRows;
        const int rows = min(kStageRows, a.src_slices - row0);
        const uint32_t x_bytes = static_cast<uint32_t>(rows) * a.M * 8u;
        const uint32_t s_bytes = a.scale_rows > 0 ? static_cast<uint32_t>(a.scale_rows) * F::TILE_N * 2u : 0u;
        mbar_arrive_expect_tx(&full[stage], kWBytes + s_bytes + x_bytes);
        tma_load_2d_hint(st, &tmap_w, &full[stage], tile * 128, row0, pol);
        if (a.scale_rows > 0) {
          tma_load_2d(st + kWBytes, &tmap_s, &full[stage], tile * F::TILE_N * 2, row0 / a.group_slices);
        }
        bulk_load_1d(st + kWBytes + a.scale_stage_bytes,
                     static_cast<const uint8_t*>(a.x) + (size_t)row0 * a.M * 8, x_bytes, &full[stage]);
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------- consumers
  const int g = lane >> 2, t = lane & 3;
  float tot[F::NF][4 * NB];
  float grp[F::NF][4 * NB];
  float ones[4 * NB];  // SUBNORMAL: shift * sum(x) per token column, same 2^-24 scale
#pragma unroll
  for (int f = 0; f < F::NF; ++f)
#pragma unroll
    for (int j = 0; j < 4 * NB; ++j) tot[f][j] = grp[f][j] = 0.0f;
#pragma unroll
  for (int j = 0; j < 4 * NB; ++j) ones[j] = 0.0f;
  int stage = 0;
  uint32_t phase = 0;
  bool failed = false;
  constexpr uint32_t kOnesA = BITS == 4 ? 0x00080008u : 0x00800080u;  // subnormal 8 / 128

  int tile = static_cast<int>(rg.lo / a.n_chunks), chunk = static_cast<int>(rg.lo % a.n_chunks);
  int first_chunk = chunk;  // first chunk of the current tile handled by this CTA
  for (int64_t it = rg.lo; it < rg.hi && !failed; ++it, ++chunk) {
    if (chunk == a.n_chunks) {
      chunk = 0;
      first_chunk = 0;
      ++tile;
    }
    if (!mbar_wait(&full[stage], phase)) {
      atomicExch(a.error, 2);
      failed = true;
      break;
    }
    const uint8_t* st = smem + (size_t)stage * stage_bytes;
    const uint8_t* xs = st + kWBytes + a.scale_stage_bytes;
    const int row0 = chunk * kStageRows;
    // large groups (multiples of a stage) and scalar scales flush once per
    // group / per range; computed once per stage
    const bool range_ends = (it + 1 == rg.hi) || (chunk + 1 == a.n_chunks);
    const bool stage_group_end =
        range_ends || (a.scale_rows > 0 && a.gs_shift < 0 && ((row0 + kStageRows) % a.group_slices) == 0);
#pragma unroll
    for (int u = 0; u < kWarpRows / 8; ++u) {
      const int rbase = warp * kWarpRows + 8 * u;
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        const int r = rbase + 2 * t + p;
        const uint4 q = *reinterpret_cast<const uint4*>(st + r * 128 + ((g ^ (r & 7)) << 4));
        uint32_t b[NB][2];
        const bool row_ok = row0 + r < a.src_slices;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          b[nb][0] = b[nb][1] = 0u;
          const int tok = g + 8 * nb;
          if (row_ok && tok < a.M) {
            const uint2 xv = *reinterpret_cast<const uint2*>(xs + ((size_t)r * a.M + tok) * 8);
            b[nb][0] = xv.x;
            b[nb][1] = xv.y;
          }
        }
        uint32_t av[F::NF][4];
        unpack<BITS, SUBNORMAL>(q, av);
#pragma unroll
        for (int f = 0; f < F::NF; ++f)
#pragma unroll
          for (int nb = 0; nb < NB; ++nb)
            mma_f16(*reinterpret_cast<float(*)[4]>(&grp[f][4 * nb]), av[f], b[nb][0], b[nb][1]);
        if constexpr (SUBNORMAL) {
          const uint32_t oa[4] = {kOnesA, kOnesA, kOnesA, kOnesA};
#pragma unroll
          for (int nb = 0; nb < NB; ++nb)
            mma_f16(*reinterpret_cast<float(*)[4]>(&ones[4 * nb]), oa, b[nb][0], b[nb][1]);
        }
      }
      // Flush the group accumulator when the next rows this warp will see belong
      // to another scale group, or when this CTA's share of the tile ends.
      const int row_cur = row0 + rbase;
      bool boundary;
      if (u + 1 < kWarpRows / 8) {
        boundary = a.gs_shift >= 0 && (((row_cur ^ (row_cur + 8)) >> a.gs_shift) != 0);
      } else {
        boundary = a.gs_shift >= 0 || stage_group_end;
      }
      if (boundary) {
        // scale row inside this stage's scale box
        float sc[F::NPL];
        if (a.scale_rows > 0) {
          const int gidx = a.gs_shift >= 0 ? ((row_cur >> a.gs_shift) - (row0 >> a.gs_shift)) : 0;
          const __half* sp = reinterpret_cast<const __half*>(st + kWBytes) + gidx * F::TILE_N + F::NPL * g;
          if constexpr (BITS == 4) {
            const uint4 sv = *reinterpret_cast<const uint4*>(sp);
            const __half2 h0 = *reinterpret_cast<const __half2*>(&sv.x), h1 = *reinterpret_cast<const __half2*>(&sv.y);
            const __half2 h2 = *reinterpret_cast<const __half2*>(&sv.z), h3 = *reinterpret_cast<const __half2*>(&sv.w);
            const float2 f0 = __half22float2(h0), f1 = __half22float2(h1), f2 = __half22float2(h2), f3 = __half22float2(h3);
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
        // row g of MMA f is output 2f, row g+8 is output 2f+1 (a high nibble,
        // carried x16, for INT4)
        constexpr float kOdd = BITS == 4 ? 0.0625f : 1.0f;
#pragma unroll
        for (int f = 0; f < F::NF; ++f)
#pragma unroll
          for (int j = 0; j < 4 * NB; ++j) {
            const bool odd = (j & 2) != 0;
            float v = grp[f][j];
            if constexpr (SUBNORMAL) {
              v = odd ? fmaf(v, kOdd, -ones[j & ~2]) : (v - ones[j & ~2]);
            } else {
              if (odd) v *= kOdd;
            }
            tot[f][j] = fmaf(sc[2 * f + (odd ? 1 : 0)], v, tot[f][j]);
            grp[f][j] = 0.0f;
          }
        if constexpr (SUBNORMAL) {
#pragma unroll
          for (int j = 0; j < 4 * NB; ++j) ones[j] = 0.0f;
        }
      }
    }
    // release the stage
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[stage]);
    if (++stage == a.stages) {
      stage = 0;
      phase ^= 1;
    }

    if (!range_ends) continue;

    // ------------------------------------------------ tile epilogue
    // 1. cross-warp reduction through shared memory (fixed order)
#pragma unroll
    for (int f = 0; f < F::NF; ++f)
#pragma unroll
      for (int j = 0; j < 4 * NB; ++j) {
        const int n_local = F::NPL * g + 2 * f + ((j >> 1) & 1);
        const int tok = 2 * t + (j & 1) + 8 * (j >> 2);
        red[(warp * F::TILE_N + n_local) * MTOK + tok] = tot[f][j];
        tot[f][j] = 0.0f;
      }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
    const bool whole = first_chunk == 0 && chunk == a.n_chunks - 1;
    const int first_cta = cta_of((int64_t)tile * a.n_chunks, total, gridDim.x);
    const int last_cta = cta_of((int64_t)tile * a.n_chunks + a.n_chunks - 1, total, gridDim.x);
    const int pieces = last_cta - first_cta + 1;
    const int piece = blockIdx.x - first_cta;
    const int nvals = F::TILE_N * a.M;
    constexpr float kOutScale = SUBNORMAL ? 16777216.0f : 1.0f;
    float* ws = a.partials + ((size_t)tile * a.max_pieces) * (F::TILE_N * MTOK);
    for (int idx = threadIdx.x; idx < nvals; idx += kConsumerWarps * 32) {
      const int n_local = idx / a.M, tok = idx % a.M;
      float s = 0.0f;
#pragma unroll
      for (int w = 0; w < kConsumerWarps; ++w) s += red[(w * F::TILE_N + n_local) * MTOK + tok];
      if (whole) {
        const int n = tile * F::TILE_N + n_local;
        if (n < a.N4) {
          __half r = __float2half_rn(s * kOutScale);
          if (a.bias != nullptr) r = __hadd(r, static_cast<const __half*>(a.bias)[n]);
          const int64_t yi = a.dst_layout == MLD_LAYOUT_SLICED ? (((int64_t)(n >> 2) * a.M + tok) * 4 + (n & 3))
                                                               : ((int64_t)tok * a.N + n);
          if (a.dst_layout == MLD_LAYOUT_SLICED || n < a.N) static_cast<__half*>(a.y)[yi] = r;
        }
      } else {
        __stcg(ws + (size_t)piece * (F::TILE_N * MTOK) + idx, s);
      }
    }
    if (!whole) {
      // 2. split-K: the last CTA to arrive sums the pieces in piece order
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
      if (threadIdx.x == 0) flag[0] = atomicAdd(a.tickets + tile, 1);
      asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
      if (flag[0] == pieces - 1) {
        __threadfence();
        for (int idx = threadIdx.x; idx < nvals; idx += kConsumerWarps * 32) {
          const int n_local = idx / a.M, tok = idx % a.M;
          float s = 0.0f;
          for (int pc = 0; pc < pieces; ++pc) s += __ldcg(ws + (size_t)pc * (F::TILE_N * MTOK) + idx);
          const int n = tile * F::TILE_N + n_local;
          if (n < a.N4) {
            __half r = __float2half_rn(s * kOutScale);
            if (a.bias != nullptr) r = __hadd(r, static_cast<const __half*>(a.bias)[n]);
            const int64_t yi = a.dst_layout == MLD_LAYOUT_SLICED ? (((int64_t)(n >> 2) * a.M + tok) * 4 + (n & 3))
                                                                 : ((int64_t)tok * a.N + n);
            if (a.dst_layout == MLD_LAYOUT_SLICED || n < a.N) static_cast<__half*>(a.y)[yi] = r;
          }
        }
        if (threadIdx.x == 0) a.tickets[tile] = 0;  // ready for the next launch
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerWarps * 32) : "memory");
  }
}

template <int BITS, int NB, bool SUBNORMAL>
int launch_stream_t(const CUtensorMap& tw, const CUtensorMap& ts, const StreamArgs& a, int grid, size_t smem,
                    cudaStream_t stream) {
  auto kern = fc_stream_kernel<BITS, NB, SUBNORMAL>;
  static bool configured = false;  // per instantiation
  if (!configured) {
    MLD_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    configured = true;
  }
  kern<<<grid, (kConsumerWarps + 1) * 32, smem, stream>>>(tw, ts, a);
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

}  // namespace

StreamGeometry stream_geometry(int bits, int N, int K, int M, int group_slices, int scale_mode, int sms) {
  StreamGeometry gm;
  const int tile_n = bits == 4 ? 64 : 32;
  const int N4 = align_n(N, 4), SS = div_up(K, 4);
  gm.nb = M > 8 ? 2 : 1;
  gm.tile_n = tile_n;
  gm.n_tiles = div_up(N4, tile_n);
  gm.n_chunks = div_up(SS, kStageRows);
  if (scale_mode == MLD_SCALE_SCALAR) {
    gm.scale_rows = 0;
    gm.group_slices = 0;
  } else if (scale_mode == MLD_SCALE_PER_CHANNEL) {
    gm.scale_rows = 1;
    gm.group_slices = gm.n_chunks * kStageRows;  // one group spanning all rows
  } else {
    gm.group_slices = group_slices;
    gm.scale_rows = group_slices >= kStageRows ? 1 : kStageRows / group_slices;
  }
  gm.gs_shift = -1;
  if (gm.scale_rows > 0 && gm.group_slices <= kStageRows) {
    for (int sh = 3; sh <= 7; ++sh)
      if ((1 << sh) == gm.group_slices) gm.gs_shift = sh;
  }
  gm.scale_stage_bytes = align_n(gm.scale_rows * tile_n * 2, 128);
  const int x_bytes = align_n(kStageRows * M * 8, 128);
  gm.stage_bytes = align_n(kWBytes + gm.scale_stage_bytes + x_bytes, 1024);
  const int mtok = 8 * gm.nb;
  const int fixed = kConsumerWarps * tile_n * mtok * 4 + 2 * 16 * 8 + 64 + 1024;
  int stages = (227 * 1024 - fixed) / gm.stage_bytes;
  if (stages > 12) stages = 12;
  gm.stages = stages;
  gm.smem_bytes = (size_t)stages * gm.stage_bytes + fixed;
  const int64_t total = (int64_t)gm.n_tiles * gm.n_chunks;
  gm.grid = static_cast<int>(total < sms ? total : sms);
  // worst-case pieces per tile for this grid
  int max_pieces = 1;
  for (int tile = 0; tile < gm.n_tiles; ++tile) {
    const int fc = cta_of((int64_t)tile * gm.n_chunks, total, gm.grid);
    const int lc = cta_of((int64_t)tile * gm.n_chunks + gm.n_chunks - 1, total, gm.grid);
    if (lc - fc + 1 > max_pieces) max_pieces = lc - fc + 1;
  }
  gm.max_pieces = max_pieces;
  gm.partial_floats = (size_t)gm.n_tiles * max_pieces * tile_n * mtok;
  return gm;
}

int launch_fc_stream(int bits, bool subnormal, const CUtensorMap& tw, const CUtensorMap& ts, const StreamArgs& a,
                     const StreamGeometry& gm, cudaStream_t stream) {
  if (a.M == 0 || gm.grid == 0) return MLD_OK;
#define MLD_DISPATCH(B, NBV, SUB) return launch_stream_t<B, NBV, SUB>(tw, ts, a, gm.grid, gm.smem_bytes, stream)
  if (bits == 4) {
    if (gm.nb == 1) {
      if (subnormal) MLD_DISPATCH(4, 1, true);
      MLD_DISPATCH(4, 1, false);
    } else {
      if (subnormal) MLD_DISPATCH(4, 2, true);
      MLD_DISPATCH(4, 2, false);
    }
  } else {
    if (gm.nb == 1) {
      if (subnormal) MLD_DISPATCH(8, 1, true);
      MLD_DISPATCH(8, 1, false);
    } else {
      if (subnormal) MLD_DISPATCH(8, 2, true);
      MLD_DISPATCH(8, 2, false);
    }
  }
#undef MLD_DISPATCH
}

}  // namespace mld
