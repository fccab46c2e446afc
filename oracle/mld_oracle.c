/*
 * CPU oracle for the quantized FullyConnected path of ML Drift.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference (google-ai-edge/ml-drift, paths relative to ml_drift/).  It is
 * the checker for the CUDA kernels and the timed CPU baseline; nothing in the
 * shipped library links or calls it.
 *
 * Parity status: PINNED.  The packers are checked byte-for-byte against the
 * known-answer tests of common/task/weights_conversion_test.cc, the quantisers
 * against vectors produced by importing samples/llm/extract_weights_hf.py, and
 * the forward pass against the hand-computed answers of
 * common/kernels/tests/fully_connected_test_util.cc (see tests/).
 *
 * Every function cites the reference lines it follows.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* IEEE binary16 helpers (round-to-nearest-even), common/types.h:28-48 uses   */
/* the fp16 header library which is IEEE RNE; any correct RNE matches.        */
/* ------------------------------------------------------------------------- */

static inline float orc_h2f(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu;
  uint32_t man = h & 0x3FFu;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      /* subnormal: normalise */
      int e = -1;
      do {
        man <<= 1;
        ++e;
      } while ((man & 0x400u) == 0);
      man &= 0x3FFu;
      bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112u) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* double -> binary16, one rounding (RNE).  Used for f32 inputs too (f32->f64 is
 * exact), so a sum or product formed exactly in double is rounded only once. */
static inline uint16_t orc_d2h(double d) {
  uint64_t bits;
  memcpy(&bits, &d, 8);
  uint16_t sign = (uint16_t)((bits >> 48) & 0x8000u);
  int64_t exp = (int64_t)((bits >> 52) & 0x7FF);
  uint64_t man = bits & 0xFFFFFFFFFFFFFull;
  if (exp == 0x7FF) { /* inf / nan */
    return (uint16_t)(sign | 0x7C00u | (man ? 0x200u : 0));
  }
  if (exp == 0 && man == 0) return sign;
  int64_t e = exp - 1023; /* unbiased */
  if (e > 15) return (uint16_t)(sign | 0x7C00u);
  uint64_t sig = man | (1ull << 52); /* 53-bit significand, value = sig*2^(e-52) */
  int shift;                         /* bits to drop */
  uint16_t hexp;
  if (e >= -14) {
    shift = 52 - 10;
    hexp = (uint16_t)(e + 15);
  } else {
    /* subnormal half: value = m * 2^-24, m = sig * 2^(e-52+24) */
    shift = (int)(52 - 10 + (-14 - e));
    hexp = 0;
    if (shift > 63) return sign; /* far below half the smallest subnormal */
  }
  uint64_t q = sig >> shift;
  uint64_t rem = sig & ((1ull << shift) - 1);
  uint64_t half = 1ull << (shift - 1);
  if (rem > half || (rem == half && (q & 1))) ++q;
  if (hexp == 0) {
    /* q may reach 0x400 -> smallest normal, encoding is still q */
    return (uint16_t)(sign | (uint16_t)q);
  }
  /* q has the implicit bit at position 10 */
  uint32_t out = ((uint32_t)hexp << 10) + (uint32_t)(q - 0x400u);
  if (out >= 0x7C00u) return (uint16_t)(sign | 0x7C00u);
  return (uint16_t)(sign | out);
}

static inline uint16_t orc_f2h(float f) { return orc_d2h((double)f); }
static inline uint16_t h_mul(uint16_t a, uint16_t b) {
  return orc_d2h((double)orc_h2f(a) * (double)orc_h2f(b));
}
static inline uint16_t h_add(uint16_t a, uint16_t b) {
  return orc_d2h((double)orc_h2f(a) + (double)orc_h2f(b));
}

ORC_API void orc_f32_to_f16(const float* src, uint16_t* dst, int64_t n) {
  /* common/task/tensor_reorder_cpu.h:60-62 ConvertF32ToF16Cpu (IEEE RNE). */
  for (int64_t i = 0; i < n; ++i) dst[i] = orc_f2h(src[i]);
}
ORC_API void orc_f16_to_f32(const uint16_t* src, float* dst, int64_t n) {
  for (int64_t i = 0; i < n; ++i) dst[i] = orc_h2f(src[i]);
}

static inline int div_up(int a, int b) { return (a + b - 1) / b; }
static inline int align_n(int a, int n) { return div_up(a, n) * n; }

/* ------------------------------------------------------------------------- */
/* Quantisers: samples/llm/extract_weights_hf.py                              */
/* ------------------------------------------------------------------------- */

/* quantize_tensor_int8_sym, optimize_scale=False branch
 * (extract_weights_hf.py:156-164), quant_axis = the input-channel axis of an
 * [O][I] matrix: scale = absmax/127 (0 -> 1), q = clip(rint(w/scale),-128,127).
 * All arithmetic in float32, rounding half-to-even like np.round. */
ORC_API void orc_quantize_int8_sym(const float* w, int O, int I, int8_t* q,
                                   float* scale) {
#pragma omp parallel for schedule(static)
  for (int o = 0; o < O; ++o) {
    const float* row = w + (size_t)o * I;
    float bound = 0.0f;
    for (int i = 0; i < I; ++i) bound = fmaxf(bound, fabsf(row[i]));
    float s = bound / 127.0f;
    if (s == 0.0f) s = 1.0f;
    for (int i = 0; i < I; ++i) {
      float v = rintf(row[i] / s);
      v = fminf(fmaxf(v, -128.0f), 127.0f);
      q[(size_t)o * I + i] = (int8_t)v;
    }
    scale[o] = s;
  }
}

/* quantize_tensor_int4_sym, optimize_scale=False (extract_weights_hf.py:200-208
 * block branch, :221-229 per-channel branch).  block == 0 means per-channel.
 * scale out: [O][G], G = I/block (1 when per-channel). */
ORC_API int orc_quantize_int4_sym(const float* w, int O, int I, int block,
                                  int8_t* q, float* scale) {
  if (block <= 0) block = I;
  if (I % block != 0) return -1; /* :171-175 raises ValueError */
  const int G = I / block;
#pragma omp parallel for schedule(static)
  for (int o = 0; o < O; ++o) {
    for (int g = 0; g < G; ++g) {
      const float* blk = w + (size_t)o * I + (size_t)g * block;
      float bound = 0.0f;
      for (int i = 0; i < block; ++i) bound = fmaxf(bound, fabsf(blk[i]));
      float s = bound / 7.0f;
      if (s == 0.0f) s = 1.0f;
      for (int i = 0; i < block; ++i) {
        float v = rintf(blk[i] / s);
        v = fminf(fmaxf(v, -8.0f), 7.0f);
        q[(size_t)o * I + (size_t)g * block + i] = (int8_t)v;
      }
      scale[(size_t)o * G + g] = s;
    }
  }
  return 0;
}

/* pack_int4 (extract_weights_hf.py:232-241): element 2j in the low nibble. */
ORC_API int orc_pack_int4_dense(const int8_t* q, int64_t n, uint8_t* out) {
  if (n % 2 != 0) return -1;
  for (int64_t j = 0; j < n / 2; ++j) {
    uint8_t lo = (uint8_t)q[2 * j] & 0x0F;
    uint8_t hi = (uint8_t)(((uint8_t)q[2 * j + 1] & 0x0F) << 4);
    out[j] = lo | hi;
  }
  return 0;
}

/* ------------------------------------------------------------------------- */
/* Packers: common/task/weights_conversion.cc                                 */
/* ------------------------------------------------------------------------- */

/* GetTotalElementsCountForLayout, kOSpatialIOGroupI4O4 case
 * (weights_conversion.cc:1015-1027). */
ORC_API int64_t orc_total_elements_i4o4(int O, int H, int W, int I,
                                        int out_group_size) {
  return (int64_t)align_n(I, 4) * align_n(O, 4 * out_group_size) * H * W;
}

/* RearrangeWeights(uint8) for kOSpatialIOGroupI4O4
 * (weights_conversion.cc:1425-1437, 1491-1492).  The aligned case goes through
 * Reshape (:46-87) = pad + 6-D transpose of {dst_groups, group, 4o, HW,
 * src_slices, 4i} by {0,3,4,1,5,2}; the ragged case through
 * RearrangeWeightsToOHWIOGroupI4O4 (:139-185).  Both produce the element order
 * [dst_groups][H][W][src_slices][group][4 i][4 o]; this loop is that order. */
ORC_API void orc_rearrange_u8_i4o4(const uint8_t* src, int O, int H, int W,
                                   int I, int out_group_size, uint8_t pad_value,
                                   uint8_t* dst) {
  const int dst_slices = div_up(O, 4);
  const int src_slices = div_up(I, 4);
  const int dst_groups = div_up(dst_slices, out_group_size);
  uint8_t* p = dst;
  for (int d = 0; d < dst_groups; ++d)
    for (int y = 0; y < H; ++y)
      for (int x = 0; x < W; ++x)
        for (int s = 0; s < src_slices; ++s)
          for (int dg = 0; dg < out_group_size; ++dg)
            for (int s_ch = 4 * s; s_ch < 4 * s + 4; ++s_ch)
              for (int j = 0; j < 4; ++j) {
                const int d_ch = 4 * (d * out_group_size + dg) + j;
                const int64_t f =
                    (((int64_t)d_ch * H + y) * W + x) * I + s_ch;
                *p++ = (s_ch < I && d_ch < O) ? src[f] : pad_value;
              }
}

/* RearrangeWeightsInt8AsUint8 (weights_conversion.cc:1495-1508): add the shift
 * (128 for INT8), then rearrange with pad_value. */
ORC_API void orc_rearrange_int8_as_uint8(const int8_t* src, int O, int H, int W,
                                         int I, int out_group_size,
                                         int shift_value, unsigned pad_value,
                                         uint8_t* dst) {
  const int64_t n = (int64_t)O * H * W * I;
  uint8_t* tmp = (uint8_t*)malloc((size_t)(n > 0 ? n : 1));
  for (int64_t i = 0; i < n; ++i) tmp[i] = (uint8_t)(src[i] + shift_value);
  orc_rearrange_u8_i4o4(tmp, O, H, W, I, out_group_size, (uint8_t)pad_value,
                        dst);
  free(tmp);
}

/* RearrangeWeightsInt8AsUint4 (weights_conversion.cc:1510-1523): as above with
 * shift 8, then two consecutive elements per byte, first one in the low
 * nibble.  dst holds total_elements/2 bytes. */
ORC_API void orc_rearrange_int8_as_uint4(const int8_t* src, int O, int H, int W,
                                         int I, int out_group_size,
                                         int shift_value, unsigned pad_value,
                                         uint8_t* dst) {
  const int64_t total = orc_total_elements_i4o4(O, H, W, I, out_group_size);
  uint8_t* tmp = (uint8_t*)malloc((size_t)(total > 0 ? total : 1));
  orc_rearrange_int8_as_uint8(src, O, H, W, I, out_group_size, shift_value,
                              pad_value, tmp);
  for (int64_t i = 0; i < total / 2; ++i) {
    uint32_t v0 = tmp[2 * i], v1 = tmp[2 * i + 1];
    dst[i] = (uint8_t)((v1 << 4) | v0);
  }
  free(tmp);
}

static inline uint8_t get_u4(uint8_t v, int msb) {
  return msb ? (uint8_t)(v >> 4) : (uint8_t)(v & 0xF);
}

/* RearrangeWeightsUInt4Packed -> Uint4PackedkOSpatialIOGroupI4O4
 * (weights_conversion.cc:1604-1612, 631-708).  src holds two's-complement
 * nibbles packed low-nibble-first in OHWI order (IHWO when swap_dims).
 * sum_i has sum_len entries (>= O); only the first O are zeroed, as in the
 * reference (:643-645). */
ORC_API void orc_rearrange_uint4_packed(const uint8_t* src, int O, int H, int W,
                                        int I, int out_group_size, uint8_t* dst,
                                        int32_t* sum_i, int sum_len,
                                        unsigned pad_value, int swap_dims) {
  const int dst_slices = div_up(O, 4);
  const int src_slices = div_up(I, 4);
  const int dst_groups = div_up(dst_slices, out_group_size);
  const int64_t df_index = swap_dims ? 1 : (int64_t)H * W * I;
  for (int i = 0; i < O && i < sum_len; ++i) sum_i[i] = 0;
  const uint8_t double_pad = (uint8_t)(pad_value | (pad_value << 4));
  pad_value ^= 0x8;
  uint8_t* p = dst;
  for (int d = 0; d < dst_groups; ++d)
    for (int y = 0; y < H; ++y)
      for (int x = 0; x < W; ++x)
        for (int s = 0; s < src_slices; ++s)
          for (int dg = 0; dg < out_group_size; ++dg) {
            const int d_ch = 4 * (d * out_group_size + dg);
            const int d_ch_diff = O - d_ch;
            for (int s_ch = 4 * s; s_ch < 4 * s + 4; ++s_ch) {
              if (s_ch >= I) {
                *p++ = double_pad;
                *p++ = double_pad;
                continue;
              }
              int64_t f = swap_dims
                              ? (((int64_t)s_ch * H + y) * W + x) * O + d_ch
                              : (((int64_t)d_ch * H + y) * W + x) * I + s_ch;
              uint8_t v[4];
              for (int j = 0; j < 4; ++j) {
                v[j] = d_ch_diff > j ? get_u4(src[f >> 1], (int)(f & 1))
                                     : (uint8_t)pad_value;
                f += df_index;
              }
              *p++ = (uint8_t)(((v[1] << 4) | v[0]) ^ 0x88);
              *p++ = (uint8_t)(((v[3] << 4) | v[2]) ^ 0x88);
              for (int j = 0; j < 4; ++j)
                if (d_ch + j < sum_len) sum_i[d_ch + j] += (v[j] ^ 0x8) - 8;
            }
          }
}

/* GetWeightsAccumulatedInputChannels (weights_conversion.cc:1584-1602). */
ORC_API void orc_weights_sum_i(const int8_t* src, int O, int H, int W, int I,
                               int32_t* sum_i) {
  for (int o = 0; o < O; ++o) {
    int32_t s = 0;
    const int8_t* row = src + (size_t)o * H * W * I;
    for (int64_t k = 0; k < (int64_t)H * W * I; ++k) s += row[k];
    sum_i[o] = s;
  }
}

/* ScaleOrZeroPointToTensorDesc (common/task/tensor_desc.cc:2245-2257):
 *  - OHWI(O,1,1,1)  -> linear vector, channels padded to 4 with zeros;
 *  - OHWI(O,1,1,G)  -> OHIToHOIO4 (:266-292) = HWC(1, ceil(O/4), 4G) with
 *    c = g*4 + o%4, which in BUFFER storage (DSHWBC4, :1852-1860) is
 *    idx = g * 4*ceil(O/4) + o, i.e. [G][O padded to 4].
 * src is [O][G] floats.  dst_f16 selects the stored type.  Returns the number
 * of elements written. */
ORC_API int64_t orc_scale_layout(const float* src, int O, int G, int dst_f16,
                                 void* dst) {
  const int O4 = align_n(O, 4);
  for (int g = 0; g < G; ++g)
    for (int o = 0; o < O4; ++o) {
      const float v = o < O ? src[(size_t)o * G + g] : 0.0f;
      const size_t idx = (size_t)g * O4 + o;
      if (dst_f16)
        ((uint16_t*)dst)[idx] = orc_f2h(v);
      else
        ((float*)dst)[idx] = v;
    }
  return (int64_t)G * O4;
}

/* Activation / output tensors BHWC(1,1,M,C) in BUFFER storage are DSHWBC4
 * (tensor_desc.cc:1852-1860): idx = (s*M + m)*4 + c%4, s = c/4, channels
 * padded to 4 with zeros (DataFromBHWDC, tensor_desc.h:540-600). */
ORC_API void orc_rowmajor_to_sliced_f32(const float* src, int M, int C,
                                        float* dst) {
  const int S = div_up(C, 4);
  for (int s = 0; s < S; ++s)
    for (int m = 0; m < M; ++m)
      for (int j = 0; j < 4; ++j) {
        const int c = 4 * s + j;
        dst[((size_t)s * M + m) * 4 + j] = c < C ? src[(size_t)m * C + c] : 0.f;
      }
}
ORC_API void orc_sliced_to_rowmajor_f32(const float* src, int M, int C,
                                        float* dst) {
  for (int m = 0; m < M; ++m)
    for (int c = 0; c < C; ++c)
      dst[(size_t)m * C + c] = src[((size_t)(c / 4) * M + m) * 4 + (c % 4)];
}

/* ------------------------------------------------------------------------- */
/* Forward: the generated FC kernel, restated                                 */
/* ------------------------------------------------------------------------- */

enum { ORC_F32 = 0, ORC_F16 = 1, ORC_F32F16 = 2 };     /* precision.h:25-36  */
enum { ORC_SCALE_SCALAR = 0, ORC_SCALE_CHANNEL = 1, ORC_SCALE_BLOCK = 2 };

/* Unpack one 4x4 block of the packed buffer.  Order = generic branch of
 * PerformU32x2ToU4x16AsVec4x4 (common/task/util.cc:773-790) and
 * PerformU32x4ToU8x16AsVec4x4 (:603-641): w[i][o] with the 4 outputs of input
 * channel i adjacent; INT4 nibble 2j in the low half of byte j. */
static inline void unpack_block(const uint8_t* packed, int bits,
                                int64_t linear_i4o4, uint8_t u[4][4]) {
  if (bits == 8) {
    const uint8_t* b = packed + linear_i4o4 * 16;
    for (int i = 0; i < 4; ++i)
      for (int o = 0; o < 4; ++o) u[i][o] = b[i * 4 + o];
  } else {
    const uint8_t* b = packed + linear_i4o4 * 8;
    for (int i = 0; i < 4; ++i) {
      u[i][0] = b[2 * i] & 0xF;
      u[i][1] = b[2 * i] >> 4;
      u[i][2] = b[2 * i + 1] & 0xF;
      u[i][3] = b[2 * i + 1] >> 4;
    }
  }
}

/* The decode dequant-GEMV/GEMM-let of GetFullyConnectedKernelCode
 * (common/kernels/fully_connected.cc:623-942) with helpers
 * fc::ReadScaleZeroPoint{Block,Linear,Scalar} (fully_connected_util.cc:80-140),
 * WeightsScaleAddBias (:142-165, non-FMA form: UseFMA() is false for NVIDIA,
 * :538-542), AccumulateFloat (:167-203), GenerateDstWrite (:356-407).
 *
 * Layouts are the device layouts:
 *   x      : sliced activations [K/4][M][4], fp32 (F32) or fp16 (F16, F32F16)
 *   packed : [K/4][N/4][4 i][4 o] u8 (+128) or u4 (+8)  (linear_i4o4 =
 *            src_s * dst_slices + dst_s, fully_connected.cc:492)
 *   scale/zp: scalar (value in scalar_scale/scalar_zp), linear [N4], or block
 *            [G][N4]; stored in the activation type
 *   bias   : linear [N4] in the activation type, or NULL
 *   y      : sliced [N/4][M][4] in the activation type
 * The K loop runs in order with no work-group split (WG_SIZE_Y == 1); the
 * reference's K-split tree reduction only reorders the same partial sums.
 * Half arithmetic rounds after every operation. */
ORC_API int orc_fc_forward(int precision, int bits, int M, int K, int N,
                           const void* x, const uint8_t* packed,
                           int scale_mode, int G, const void* scale,
                           const void* zp, float scalar_scale, float scalar_zp,
                           int has_scalar_zp, const void* bias, void* y) {
  if (bits != 4 && bits != 8) return -1;
  const int src_slices = div_up(K, 4), dst_slices = div_up(N, 4);
  const int N4 = dst_slices * 4;
  const int shift = bits == 8 ? 128 : 8;
  const int is_h = precision != ORC_F32;
  const int has_zp = (zp != NULL) || has_scalar_zp;
  int src_groups = 1, src_group_size = src_slices;
  if (scale_mode == ORC_SCALE_BLOCK) {
    src_groups = G;                       /* fully_connected.cc:365-370 */
    src_group_size = src_slices / src_groups;
  }
#pragma omp parallel for schedule(static)
  for (int dst_s = 0; dst_s < dst_slices; ++dst_s) {
    for (int m = 0; m < M; ++m) {
      float accf[4] = {0, 0, 0, 0};
      uint16_t acch[4] = {0, 0, 0, 0};
      float wsf[4], wbf[4];
      uint16_t wsh[4], wbh[4];
      for (int g = 0; g < src_groups; ++g) {
        /* scale / bias for this (group, slice) */
        for (int o = 0; o < 4; ++o) {
          if (is_h) {
            uint16_t s, z = 0;
            if (scale_mode == ORC_SCALE_SCALAR) {
              s = orc_f2h(scalar_scale);
              if (has_zp) z = orc_f2h(scalar_zp);
            } else {
              const size_t idx = (scale_mode == ORC_SCALE_BLOCK
                                      ? (size_t)g * N4
                                      : 0) + (size_t)dst_s * 4 + o;
              s = ((const uint16_t*)scale)[idx];
              if (zp) z = ((const uint16_t*)zp)[idx];
            }
            /* w_bias = -w_scale * (shift [+ w_zp]) */
            uint16_t sh = orc_f2h((float)shift);
            if (has_zp) sh = h_add(sh, z);
            wsh[o] = s;
            wbh[o] = h_mul((uint16_t)(s ^ 0x8000u), sh);
          } else {
            float s, z = 0.f;
            if (scale_mode == ORC_SCALE_SCALAR) {
              s = scalar_scale;
              if (has_zp) z = scalar_zp;
            } else {
              const size_t idx = (scale_mode == ORC_SCALE_BLOCK
                                      ? (size_t)g * N4
                                      : 0) + (size_t)dst_s * 4 + o;
              s = ((const float*)scale)[idx];
              if (zp) z = ((const float*)zp)[idx];
            }
            float sh = (float)shift;
            if (has_zp) sh = sh + z;
            wsf[o] = s;
            wbf[o] = -s * sh;
          }
        }
        for (int sub = 0; sub < src_group_size; ++sub) {
          const int src_s = g * src_group_size + sub;
          uint8_t u[4][4];
          unpack_block(packed, bits, (int64_t)src_s * dst_slices + dst_s, u);
          const size_t xi = ((size_t)src_s * M + m) * 4;
          if (precision == ORC_F32) {
            const float* v = (const float*)x + xi;
            for (int i = 0; i < 4; ++i)
              for (int o = 0; o < 4; ++o) {
                float w = (float)u[i][o] * wsf[o];
                w = w + wbf[o];
                float p = v[i] * w;
                accf[o] = accf[o] + p;
              }
          } else {
            const uint16_t* v = (const uint16_t*)x + xi;
            uint16_t w[4][4];
            for (int i = 0; i < 4; ++i)
              for (int o = 0; o < 4; ++o)
                w[i][o] = h_add(h_mul(orc_f2h((float)u[i][o]), wsh[o]), wbh[o]);
            if (precision == ORC_F16) {
              for (int i = 0; i < 4; ++i)
                for (int o = 0; o < 4; ++o)
                  acch[o] = h_add(acch[o], h_mul(v[i], w[i][o]));
            } else {
              /* r += convert_float4(v.x*w0 + v.y*w1 + v.z*w2 + v.w*w3) */
              for (int o = 0; o < 4; ++o) {
                uint16_t t = h_mul(v[0], w[0][o]);
                t = h_add(t, h_mul(v[1], w[1][o]));
                t = h_add(t, h_mul(v[2], w[2][o]));
                t = h_add(t, h_mul(v[3], w[3][o]));
                accf[o] = accf[o] + orc_h2f(t);
              }
            }
          }
        }
      }
      /* dst write: convert to the tensor type, then add the bias */
      const size_t yi = ((size_t)dst_s * M + m) * 4;
      for (int o = 0; o < 4; ++o) {
        if (!is_h) {
          float r = accf[o];
          if (bias) r = r + ((const float*)bias)[dst_s * 4 + o];
          ((float*)y)[yi + o] = r;
        } else {
          uint16_t r = precision == ORC_F16 ? acch[o] : orc_f2h(accf[o]);
          if (bias) r = h_add(r, ((const uint16_t*)bias)[dst_s * 4 + o]);
          ((uint16_t*)y)[yi + o] = r;
        }
      }
    }
  }
  return 0;
}

/* FullyConnectedReference over MakeWeightsFromInt8
 * (common/task/testing_ref_ops.cc:961-988, 2715-2742): the mathematically
 * plain version the reference's own big tests compare against.
 * q [N][K] int8, scale/zp [N][G] float (zp may be NULL), x [M][K], y [M][N]. */
ORC_API void orc_fc_plain_reference(const int8_t* q, int N, int K,
                                    const float* scale, const float* zp, int G,
                                    const float* bias, const float* x, int M,
                                    float* y) {
  const int gsz = K / G;
#pragma omp parallel for schedule(static)
  for (int d = 0; d < N; ++d)
    for (int m = 0; m < M; ++m) {
      float sum = bias ? bias[d] : 0.0f;
      for (int s = 0; s < K; ++s) {
        const int g = s / gsz;
        const float z = zp ? zp[(size_t)d * G + g] : 0.0f;
        const float w = ((float)q[(size_t)d * K + s] - z) *
                        scale[(size_t)d * G + g];
        sum += x[(size_t)m * K + s] * w;
      }
      y[(size_t)m * N + d] = sum;
    }
}

/* ------------------------------------------------------------------------- */
/* Integer-activation path (W8A8 prefill)                                     */
/* ------------------------------------------------------------------------- */

/* Symmetric per-token quantisation to signed int8, restating the generated
 * kernel of CreateQuantization (common/kernels/quantize_and_dequantize.cc:
 * 355-378 scale, 421-441 rounding) with the constants of the Quantization
 * constructor (:757-784): range 256, symmetric_half_range 127,
 * zero_point_plus_half 128.5, min_scale = smallest normal half when the source
 * is fp16 else 1e-30, signed destination so offset = 0.
 * x: row-major [M][K], fp16 when src_f16 else fp32.  Outputs: q [M][K] int8,
 * params [M][3] = {inv_scale, offset, sum}. */
ORC_API void orc_quantize_act_sym(const void* x, int src_f16, int M, int K,
                                  int8_t* q, float* params) {
  const float min_scale = src_f16 ? 6.103515625e-05f : 1.0e-30f;
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float abs_max = 0.0f;
    for (int k = 0; k < K; ++k) {
      const float v = src_f16 ? orc_h2f(((const uint16_t*)x)[(size_t)m * K + k])
                              : ((const float*)x)[(size_t)m * K + k];
      abs_max = fmaxf(abs_max, fabsf(v));
    }
    float inv_scale = 0.0f, scale = 0.0f;
    if (abs_max > 0.0f) {
      inv_scale = fmaxf(min_scale, abs_max / 127.0f);
      scale = 1.0f / inv_scale;
    }
    int sum = 0;
    for (int k = 0; k < K; ++k) {
      const float v = src_f16 ? orc_h2f(((const uint16_t*)x)[(size_t)m * K + k])
                              : ((const float*)x)[(size_t)m * K + k];
      float t = v * scale;
      float r = floorf(t + 128.5f);
      r = fminf(255.0f, fmaxf(0.0f, r));
      const int qi = (int)r - 128;
      q[(size_t)m * K + k] = (int8_t)qi;
      sum += qi;
    }
    params[m * 3 + 0] = inv_scale;
    params[m * 3 + 1] = 0.0f;
    params[m * 3 + 2] = (float)sum;
  }
}

/* Asymmetric per-token quantisation to signed int8, the other branch of the
 * same generated kernel (quantize_and_dequantize.cc:379-437; it is the model
 * builder's default, common/gpu_model_builder.h:236-240): src_range = max - min,
 * offset = min, scale = dst_range / src_range, inv_scale = src_range / dst_range,
 * and for a signed destination offset += src_range * src_range_middle with
 * src_range_middle = (range / 2) / (range - 1) = 128 / 255 (:778-781);
 * q = clamp(int((x - min) * scale + 0.5), 0, 255) - 128.  A constant token
 * (src_range 0) is given scale = inv_scale = 0 here (the generated kernel would
 * divide by zero): every x then equals the offset.  Same outputs as the
 * symmetric form. */
ORC_API void orc_quantize_act_asym(const void* x, int src_f16, int M, int K,
                                   int8_t* q, float* params) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    float vmin = INFINITY, vmax = -INFINITY;
    for (int k = 0; k < K; ++k) {
      const float v = src_f16 ? orc_h2f(((const uint16_t*)x)[(size_t)m * K + k])
                              : ((const float*)x)[(size_t)m * K + k];
      vmin = fminf(vmin, v);
      vmax = fmaxf(vmax, v);
    }
    const float src_range = vmax - vmin;
    float offset = vmin, scale = 0.0f, inv_scale = 0.0f;
    if (src_range > 0.0f) {
      scale = 255.0f / src_range;
      inv_scale = src_range / 255.0f;
      const float middle = 128.0f / 255.0f;
      const float t = src_range * middle;
      offset = offset + t;
    }
    int sum = 0;
    for (int k = 0; k < K; ++k) {
      const float v = src_f16 ? orc_h2f(((const uint16_t*)x)[(size_t)m * K + k])
                              : ((const float*)x)[(size_t)m * K + k];
      float t = v - vmin;
      t = t * scale;
      t = t + 0.5f;
      int qi = (int)t;
      qi = qi > 255 ? 255 : qi;
      qi = qi < 0 ? 0 : qi;
      qi -= 128;
      q[(size_t)m * K + k] = (int8_t)qi;
      sum += qi;
    }
    params[m * 3 + 0] = inv_scale;
    params[m * 3 + 1] = offset;
    params[m * 3 + 2] = (float)sum;
  }
}

/* int8 x int8 -> int32 GEMM, the exact reference the Si8Wi8 tests use
 * (common/task/testing_ref_ops.cc:1069-1098).  xq [M][K], wq [N][K]. */
ORC_API void orc_gemm_s8s8_s32(const int8_t* xq, const int8_t* wq, int M, int K,
                               int N, int32_t* acc) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      int32_t s = 0;
      const int8_t* a = xq + (size_t)m * K;
      const int8_t* b = wq + (size_t)n * K;
      for (int k = 0; k < K; ++k) s += (int32_t)a[k] * (int32_t)b[k];
      acc[(size_t)m * N + n] = s;
    }
}

/* The same product through the FC kernel's unsigned-weight form
 * (fully_connected_util.cc:205-229): acc = sum(x * u) - shift * sum(x), with u
 * the packed unsigned weights.  Exact in int32; equals orc_gemm_s8s8_s32. */
ORC_API void orc_fc_forward_i8(int bits, int M, int K, int N, const int8_t* xq,
                               const uint8_t* packed, int32_t* acc) {
  const int src_slices = div_up(K, 4), dst_slices = div_up(N, 4);
  const int shift = bits == 8 ? 128 : 8;
  for (int dst_s = 0; dst_s < dst_slices; ++dst_s)
    for (int m = 0; m < M; ++m) {
      int32_t r[4] = {0, 0, 0, 0};
      int32_t xs = 0;
      for (int src_s = 0; src_s < src_slices; ++src_s) {
        uint8_t u[4][4];
        unpack_block(packed, bits, (int64_t)src_s * dst_slices + dst_s, u);
        for (int i = 0; i < 4; ++i) {
          const int k = 4 * src_s + i;
          const int32_t xv = k < K ? xq[(size_t)m * K + k] : 0;
          xs += xv;
          for (int o = 0; o < 4; ++o) r[o] += xv * (int32_t)u[i][o];
        }
      }
      for (int o = 0; o < 4; ++o) {
        const int n = dst_s * 4 + o;
        if (n < N) acc[(size_t)m * N + n] = r[o] - xs * shift;
      }
    }
}

/* CreateDequantization epilogue (quantize_and_dequantize.cc:867-925) for the
 * no-weight-zero-point case: res = float(acc); res *= w_scale * src_scale;
 * res += w_scale * src_zero_point * weights_sum; convert to the output type.
 * params [M][3] from orc_quantize_act_sym; w_scale [N], w_sum [N] (as float,
 * like the reference's Convert<float4>).  y row-major [M][N]; fp16 when
 * dst_f16.  Bias is a separate add node in the reference
 * (gpu_model_builder.cc:1426-1428) applied in the output type. */
ORC_API void orc_dequant_epilogue(const int32_t* acc, int M, int N,
                                  const float* params, const float* w_scale,
                                  const int32_t* w_sum, const void* bias,
                                  int dst_f16, void* y) {
#pragma omp parallel for schedule(static)
  for (int m = 0; m < M; ++m) {
    const float src_scale = params[m * 3 + 0];
    const float src_zp = params[m * 3 + 1];
    for (int n = 0; n < N; ++n) {
      float res = (float)acc[(size_t)m * N + n];
      float f = w_scale[n] * src_scale;
      res = res * f;
      float t = w_scale[n] * src_zp;
      float t2 = t * (float)(w_sum ? w_sum[n] : 0);
      res = res + t2;
      if (dst_f16) {
        uint16_t h = orc_f2h(res);
        if (bias) h = h_add(h, ((const uint16_t*)bias)[n]);
        ((uint16_t*)y)[(size_t)m * N + n] = h;
      } else {
        if (bias) res = res + ((const float*)bias)[n];
        ((float*)y)[(size_t)m * N + n] = res;
      }
    }
  }
}

/* ------------------------------------------------------------------------- */
/* Prefill dequant-GEMM for block-quantised INT4 (float path)                 */
/* ------------------------------------------------------------------------- */

/* The reference's prefill route for block-quantised weights
 * (common/gpu_model_builder.cc:1110-1276): a WeightsConverter pass dequantises
 * the packed weights to fp16 (common/kernels/conv_weights_converter.cc:248-290:
 * w = u * scale + bias with bias = -scale * shift, in half), then a float
 * convolution multiplies fp16 activations by them with fp32 accumulation
 * (F32F16).  Restated here as: wd[n][k] = half(half(u*s) + half(-s*shift));
 * y[m][n] = half(sum_k float(x[m][k]) * float(wd[n][k])), accumulated in fp32
 * in k order.  x row-major [M][K] fp16, y row-major [M][N] fp16. */
ORC_API void orc_prefill_gemm_int4(const uint16_t* x, int M, int K, int N,
                                   const uint8_t* packed, int bits,
                                   const uint16_t* scale_gn, int G,
                                   uint16_t* y) {
  const int dst_slices = div_up(N, 4), src_slices = div_up(K, 4);
  const int N4 = dst_slices * 4;
  const int shift = bits == 8 ? 128 : 8;
  const int gsz = src_slices / G; /* slices per group */
  float* wd = (float*)malloc((size_t)N4 * src_slices * 4 * sizeof(float));
#pragma omp parallel for schedule(static)
  for (int dst_s = 0; dst_s < dst_slices; ++dst_s)
    for (int src_s = 0; src_s < src_slices; ++src_s) {
      uint8_t u[4][4];
      unpack_block(packed, bits, (int64_t)src_s * dst_slices + dst_s, u);
      const int g = src_s / gsz;
      for (int o = 0; o < 4; ++o) {
        const uint16_t s = scale_gn[(size_t)g * N4 + dst_s * 4 + o];
        const uint16_t b =
            h_mul((uint16_t)(s ^ 0x8000u), orc_f2h((float)shift));
        for (int i = 0; i < 4; ++i) {
          const uint16_t w = h_add(h_mul(orc_f2h((float)u[i][o]), s), b);
          wd[((size_t)(dst_s * 4 + o)) * (src_slices * 4) + src_s * 4 + i] =
              orc_h2f(w);
        }
      }
    }
  float* xf = (float*)malloc((size_t)M * K * sizeof(float));
  for (int64_t i = 0; i < (int64_t)M * K; ++i) xf[i] = orc_h2f(x[i]);
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const float* wr = wd + (size_t)n * (src_slices * 4);
    for (int m = 0; m < M; ++m) {
      const float* xr = xf + (size_t)m * K;
      float acc = 0.0f;
      for (int k = 0; k < K; ++k) acc += xr[k] * wr[k];
      y[(size_t)m * N + n] = orc_f2h(acc);
    }
  }
  free(xf);
  free(wd);
}

/* ------------------------------------------------------------------------- */
/* Fast fp32 GEMV over the packed layout: the timed CPU baseline              */
/* ------------------------------------------------------------------------- */

/* Same data, same layout and same per-element arithmetic as orc_fc_forward in
 * F32 mode for M == 1 (activations and scales given as fp32), written so the
 * compiler can vectorise over the four outputs of a slice and OpenMP can
 * spread slices over cores.  x [K], scale [G][N4] (or [N4] when G == 1),
 * y [N4]. */
ORC_API void orc_gemv_f32_fast(int bits, int K, int N, const float* x,
                               const uint8_t* packed, int G, const float* scale,
                               const float* bias, float* y) {
  const int src_slices = div_up(K, 4), dst_slices = div_up(N, 4);
  const int N4 = dst_slices * 4;
  const int gsz = src_slices / G;
  const float shift = bits == 8 ? 128.0f : 8.0f;
#pragma omp parallel for schedule(static)
  for (int dst_s = 0; dst_s < dst_slices; ++dst_s) {
    float acc[4] = {0, 0, 0, 0};
    for (int g = 0; g < G; ++g) {
      float ws[4], wb[4];
      for (int o = 0; o < 4; ++o) {
        ws[o] = scale[(size_t)g * N4 + dst_s * 4 + o];
        wb[o] = -ws[o] * shift;
      }
      for (int sub = 0; sub < gsz; ++sub) {
        const int src_s = g * gsz + sub;
        const int64_t lin = (int64_t)src_s * dst_slices + dst_s;
        if (bits == 8) {
          const uint8_t* b = packed + lin * 16;
          for (int i = 0; i < 4; ++i)
            for (int o = 0; o < 4; ++o)
              acc[o] += x[4 * src_s + i] * ((float)b[i * 4 + o] * ws[o] + wb[o]);
        } else {
          const uint8_t* b = packed + lin * 8;
          for (int i = 0; i < 4; ++i) {
            const float xv = x[4 * src_s + i];
            acc[0] += xv * ((float)(b[2 * i] & 0xF) * ws[0] + wb[0]);
            acc[1] += xv * ((float)(b[2 * i] >> 4) * ws[1] + wb[1]);
            acc[2] += xv * ((float)(b[2 * i + 1] & 0xF) * ws[2] + wb[2]);
            acc[3] += xv * ((float)(b[2 * i + 1] >> 4) * ws[3] + wb[3]);
          }
        }
      }
    }
    for (int o = 0; o < 4; ++o)
      y[dst_s * 4 + o] = acc[o] + (bias ? bias[dst_s * 4 + o] : 0.0f);
  }
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
#else
  (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}
