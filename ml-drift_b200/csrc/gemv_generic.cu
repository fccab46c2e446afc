// Decode-stage dequant-GEMV, general form: covers every case of the operator
// the streaming kernel does not take (fp32 tensors, zero points, ragged shapes,
// odd scale-group sizes, row-major multi-token activations) with plain loads.
// A CTA owns four output slices (16 outputs); a lane owns one of them and every
// 128th input slice, so that four lanes read 64 (32) neighbouring bytes of a
// weight row and even a 2048 x 2048 matrix is spread over 128 CTAs of 16 warps; a
// lane asks for four weight blocks before it uses the first; the lanes and warps
// that share an output slice are summed at the end.
//
// Arithmetic restated from GetFullyConnectedKernelCode
// (ml_drift/common/kernels/fully_connected.cc:623-942) and fc:: helpers
// (fully_connected_util.cc:80-229, 356-407).
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace mld {

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
constexpr int kGenWarps = 16;  // warps of a CTA
constexpr int kGenSlices = 4;  // output slices of a CTA
constexpr int kGenPhases = 32 / kGenSlices;  // input-slice phases of a warp

// Lane = kGenSlices * (input-slice phase within the warp) + output slice within the CTA.
// T = float: the kF32 arithmetic (separate multiply and add, fp32).
// T = __half: the kF32F16 arithmetic (dequantise and multiply in half, sum of
// four products in half, accumulate in fp32); kF16 requests use it too.
template <typename T, int BITS>
__global__ void __launch_bounds__(kGenWarps * 32) fc_generic_kernel(GenericArgs a) {
  __shared__ float part[kGenWarps][kGenSlices][kGenTokens][4];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ds = lane % kGenSlices, sp = lane / kGenSlices;
  const int dst_raw = blockIdx.x * kGenSlices + ds;
  const bool live = dst_raw < a.dst_slices;
  const int dst_s = live ? dst_raw : a.dst_slices - 1;  // (idle lanes repeat the last slice and store nothing)
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
    constexpr int kAhead = 4;  // weight loads in flight per lane
    constexpr int kStep = kGenPhases * kGenWarps;  // input slices between two of a lane's
    for (int src0 = warp * kGenPhases + sp; src0 < a.src_slices; src0 += kStep * kAhead) {
      uint4 qw[kAhead];
#pragma unroll
      for (int h = 0; h < kAhead; ++h) {
        const int ss = src0 + h * kStep;
        qw[h] = make_uint4(0u, 0u, 0u, 0u);
        if (ss < a.src_slices) {
          const int64_t lin = (int64_t)ss * a.dst_slices + dst_s;
          if (BITS == 8) {
            qw[h] = *reinterpret_cast<const uint4*>(wp + lin * 16);
          } else {
            const uint2 q2 = *reinterpret_cast<const uint2*>(wp + lin * 8);
            qw[h].x = q2.x;
            qw[h].y = q2.y;
          }
        }
      }
#pragma unroll
      for (int h = 0; h < kAhead; ++h) {
      const int src_s = src0 + h * kStep;
      if (src_s >= a.src_slices) break;
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
      if (BITS == 8) {
        const uint4 q = qw[h];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int o = 0; o < 4; ++o) u[i][o] = (w[i] >> (8 * o)) & 0xFF;
      } else {
        const uint32_t w[2] = {qw[h].x, qw[h].y};
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
    }
    // the phases of a warp, then the warps (in order), share an output slice
#pragma unroll
    for (int m = 0; m < kGenTokens; ++m)
#pragma unroll
      for (int o = 0; o < 4; ++o) {
#pragma unroll
        for (int off = kGenSlices; off < 32; off <<= 1) acc[m][o] += __shfl_xor_sync(0xffffffffu, acc[m][o], off);
        if (sp == 0) part[warp][ds][m][o] = acc[m][o];
      }
    __syncthreads();
    if (warp == 0 && live) {
      // the warp's lane groups take a token each
      for (int m = sp; m < kGenTokens && m0 + m < a.M; m += kGenPhases)
        for (int o = 0; o < 4; ++o) {
          const int n = dst_s * 4 + o;
          if (a.dst_layout == MLD_LAYOUT_ROW_MAJOR && n >= a.N) continue;
          float sum = 0.0f;
#pragma unroll
          for (int w = 0; w < kGenWarps; ++w) sum += part[w][ds][m][o];
          T r = T(sum);
          if (a.bias != nullptr) r = r + ActOps<T>::load(a.bias, n);
          ActOps<T>::store(a.y, act_index(a.dst_layout, a.M, a.N, m0 + m, n), r);
        }
    }
    __syncthreads();
  }
}

}  // namespace

int launch_fc_generic(const GenericArgs& a, int bits, bool f32, cudaStream_t stream) {
  const int grid = div_up(a.dst_slices, kGenSlices);
  if (grid == 0 || a.M == 0) return MLD_OK;
  if (f32) {
    if (bits == 8)
      fc_generic_kernel<float, 8><<<grid, kGenWarps * 32, 0, stream>>>(a);
    else
      fc_generic_kernel<float, 4><<<grid, kGenWarps * 32, 0, stream>>>(a);
  } else {
    if (bits == 8)
      fc_generic_kernel<__half, 8><<<grid, kGenWarps * 32, 0, stream>>>(a);
    else
      fc_generic_kernel<__half, 4><<<grid, kGenWarps * 32, 0, stream>>>(a);
  }
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

}  // namespace mld
