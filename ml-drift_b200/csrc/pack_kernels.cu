// Weight conversion kernels: quantisation, rearrangement into the reference's
// kOSpatialIOGroupI4O4 buffer layout, scale layout.  All integer/byte work is
// bit-exact with the CPU rearrangers of ml-drift
// (common/task/weights_conversion.cc); these kernels are HBM-bound, so they
// read rows coalesced, transpose in registers (or, for ragged shapes, through
// shared memory) and write whole 4x4 blocks with vector stores.
#include "common.cuh"

namespace mld {

namespace {

constexpr int kTileSlices = 32;                  // 32 x 32 blocks of 4x4 per CTA
constexpr int kTileCh = kTileSlices * 4;         // 128 channels each way
constexpr int kRowPitch = kTileSlices * 16 + 4;  // bytes per src-slice row of the staged tile (+4: bank spread)

// Position of element (o_local, i_local) inside the staged tile, which is kept
// in destination order: [src slice][dst slice][4 i][4 o], one byte per element.
__device__ __forceinline__ int tile_pos(int o_local, int i_local) {
  return (i_local >> 2) * kRowPitch + (o_local >> 2) * 16 + (i_local & 3) * 4 + (o_local & 3);
}

struct PackArgs {
  const uint8_t* src;
  uint8_t* dst;
  int32_t* sum_i;
  int O, HW, I;
  int group;       // out_group_size
  int dst_slices;  // ceil(O/4)
  int src_slices;  // ceil(I/4)
  int total_ds;    // dst_groups * group (>= dst_slices)
  int sum_len;
  int shift;       // added to int8 sources (128 / 8)
  uint32_t pad;    // pad value as the reference passes it
  int swap_dims;
};

// Writes the staged tile to global memory.  BITS == 8: 16 bytes per block;
// BITS == 4: consecutive element pairs share a byte, first in the low nibble
// (RearrangeWeightsInt8AsUint4, weights_conversion.cc:1510-1523).
template <int BITS>
__device__ __forceinline__ void store_tile(const uint8_t* tile, const PackArgs& a, int hw, int s0, int d0) {
  for (int blk = threadIdx.x; blk < kTileSlices * kTileSlices; blk += blockDim.x) {
    const int ss = blk / kTileSlices, dsl = blk % kTileSlices;
    const int s = s0 + ss, ds = d0 + dsl;
    if (s >= a.src_slices || ds >= a.total_ds) continue;
    const int d = ds / a.group, dg = ds % a.group;
    // [dst_groups][HW][src_slices][group] blocks
    const int64_t block_index = (((int64_t)d * a.HW + hw) * a.src_slices + s) * a.group + dg;
    const uint32_t* w = reinterpret_cast<const uint32_t*>(tile + ss * kRowPitch + dsl * 16);
    const uint32_t w0 = w[0], w1 = w[1], w2 = w[2], w3 = w[3];
    if (BITS == 8) {
      *reinterpret_cast<uint4*>(a.dst + block_index * 16) = make_uint4(w0, w1, w2, w3);
    } else {
      // bytes v0 v1 v2 v3 of a word -> (v1<<4|v0), (v3<<4|v2), truncated to 8 bits
      auto squeeze = [](uint32_t x) -> uint32_t {
        const uint32_t b0 = x & 0xFF, b1 = (x >> 8) & 0xFF, b2 = (x >> 16) & 0xFF, b3 = x >> 24;
        return (((b1 << 4) | b0) & 0xFF) | ((((b3 << 4) | b2) & 0xFF) << 8);
      };
      const uint32_t lo = squeeze(w0) | (squeeze(w1) << 16);
      const uint32_t hi = squeeze(w2) | (squeeze(w3) << 16);
      *reinterpret_cast<uint2*>(a.dst + block_index * 8) = make_uint2(lo, hi);
    }
  }
}

// int8 OHWI source -> staged tile of (q + shift) bytes.  One warp reads 128
// consecutive input channels of one output row per step (coalesced).
template <int BITS>
__global__ void __launch_bounds__(256) pack_from_int8_kernel(PackArgs a) {
  __shared__ __align__(16) uint8_t tile[kTileSlices * kRowPitch];
  const int s0 = blockIdx.x * kTileSlices, d0 = blockIdx.y * kTileSlices, hw = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int8_t* src = reinterpret_cast<const int8_t*>(a.src);
  const uint8_t padv = static_cast<uint8_t>(a.pad);
  const bool vec = (a.I % 4 == 0) && ((reinterpret_cast<uintptr_t>(src) & 3) == 0);
  for (int r = warp; r < kTileCh; r += 8) {
    const int o = d0 * 4 + r;
    const int i = s0 * 4 + lane * 4;
    uint8_t v[4];
    int32_t rowsum = 0;
    if (o < a.O) {
      const int64_t base = ((int64_t)o * a.HW + hw) * a.I + i;
      if (vec && i + 3 < a.I) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(src + base);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int8_t q = static_cast<int8_t>((w >> (8 * j)) & 0xFF);
          v[j] = static_cast<uint8_t>(q + a.shift);
          rowsum += q;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (i + j < a.I) {
            const int8_t q = src[base + j];
            v[j] = static_cast<uint8_t>(q + a.shift);
            rowsum += q;
          } else {
            v[j] = padv;
          }
        }
      }
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) v[j] = padv;
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) tile[tile_pos(r, lane * 4 + j)] = v[j];
    if (a.sum_i != nullptr) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) rowsum += __shfl_xor_sync(0xffffffffu, rowsum, off);
      if (lane == 0 && o < a.O && o < a.sum_len && rowsum != 0) atomicAdd(a.sum_i + o, rowsum);
    }
  }
  __syncthreads();
  store_tile<BITS>(tile, a, hw, s0, d0);
}

// Dense two's-complement nibble source (Uint4PackedkOSpatialIOGroupI4O4,
// weights_conversion.cc:631-708).  The staged byte is the *destination nibble*
// (source nibble ^ 8, or the pad rules of the reference), the store step packs
// pairs.  sum_i receives (nibble ^ 8) - 8 per element, and pad - 8 for padded
// output channels of valid input channels, as the reference does.
__global__ void __launch_bounds__(256) pack_from_u4_kernel(PackArgs a) {
  __shared__ __align__(16) uint8_t tile[kTileSlices * kRowPitch];
  const int s0 = blockIdx.x * kTileSlices, d0 = blockIdx.y * kTileSlices, hw = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint8_t pad_nib = static_cast<uint8_t>(a.pad & 0xFF);              // "double_pad" nibble (s_ch >= I)
  const uint8_t pad_dst = static_cast<uint8_t>(((a.pad ^ 0x8) ^ 0x8) & 0xF);  // padded output channel
  for (int r = warp; r < kTileCh; r += 8) {
    const int o = d0 * 4 + r;
    const int i = s0 * 4 + lane * 4;
    int32_t rowsum = 0;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint8_t out;
      if (i + j >= a.I) {
        // both nibbles of the byte are the raw pad value (weights_conversion.cc:660-664)
        out = pad_nib & 0xF;
      } else if (o >= a.O) {
        out = pad_dst;
        rowsum += static_cast<int32_t>(static_cast<uint8_t>((a.pad ^ 0x8) & 0xFF) ^ 0x8) - 8;
      } else {
        const int64_t f = a.swap_dims ? (((int64_t)(i + j) * a.HW + hw) * a.O + o)
                                      : (((int64_t)o * a.HW + hw) * a.I + (i + j));
        const uint8_t b = a.src[f >> 1];
        const uint8_t nib = (f & 1) ? (b >> 4) : (b & 0xF);
        out = nib ^ 0x8;
        rowsum += static_cast<int32_t>(nib ^ 0x8) - 8;
      }
      tile[tile_pos(r, lane * 4 + j)] = out;
    }
    if (a.sum_i != nullptr) {
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) rowsum += __shfl_xor_sync(0xffffffffu, rowsum, off);
      // padded channels exist only inside the last, partly filled slice
      if (lane == 0 && o < a.dst_slices * 4 && o < a.sum_len && rowsum != 0) atomicAdd(a.sum_i + o, rowsum);
    }
  }
  __syncthreads();
  store_tile<4>(tile, a, hw, s0, d0);
}

// The common case without shared memory: int8 source, one output group (the FullyConnected choice), input
// channels a multiple of 16, 16-byte aligned rows.  A warp takes 16 output rows x 128 input channels.  Per
// step it reads four rows, eight lanes to a row and 16 bytes to a lane; the four lanes that hold the same 16
// input channels of the four rows exchange words so that each ends up with the four rows of ONE group of four
// input channels, i.e. one 4x4 block, which it transposes byte-wise in registers.  After four steps a lane
// holds four blocks that are neighbours in the destination (same input slice, four consecutive output
// slices) and writes them as one 64-byte (32-byte for 4 bits) run.
template <int BITS>
__global__ void __launch_bounds__(256) pack_rows_kernel(PackArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hw = blockIdx.z;
  const int r = lane >> 3, c = lane & 7;                 // row of the step's four, 16-byte chunk of the 128 inputs
  const int i0 = blockIdx.x * 128 + c * 16;              // first input channel of this lane's chunk
  const int o0 = (blockIdx.y * 8 + warp) * 16;           // first of the warp's 16 output rows
  if (o0 >= a.dst_slices * 4) return;
  const int8_t* src = reinterpret_cast<const int8_t*>(a.src);
  const uint32_t padw = (a.pad & 0xFFu) * 0x01010101u;
  uint32_t blk[4][4];                                     // [step = output slice][word k = input channel of the block]
#pragma unroll
  for (int st = 0; st < 4; ++st) {
    const int o = o0 + st * 4 + r;
    uint4 v = make_uint4(padw, padw, padw, padw);
    int32_t rowsum = 0;
    if (o < a.O && i0 < a.I) {
      v = *reinterpret_cast<const uint4*>(src + ((int64_t)o * a.HW + hw) * a.I + i0);
      rowsum = __dp4a(static_cast<int>(v.x), 0x01010101, 0);
      rowsum = __dp4a(static_cast<int>(v.y), 0x01010101, rowsum);
      rowsum = __dp4a(static_cast<int>(v.z), 0x01010101, rowsum);
      rowsum = __dp4a(static_cast<int>(v.w), 0x01010101, rowsum);
      // q + shift, byte-wise: +128 is a flip of the top bit; +8 on values in [-8, 7] likewise, kept to 4 bits
      const uint32_t flip = BITS == 8 ? 0x80808080u : 0x08080808u, keep = BITS == 8 ? 0xFFFFFFFFu : 0x0F0F0F0Fu;
      v.x = (v.x ^ flip) & keep;
      v.y = (v.y ^ flip) & keep;
      v.z = (v.z ^ flip) & keep;
      v.w = (v.w ^ flip) & keep;
    }
    if (a.sum_i != nullptr) {
      rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 1);
      rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 2);
      rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 4);
      if (c == 0 && o < a.O && o < a.sum_len && rowsum != 0) atomicAdd(a.sum_i + o, rowsum);
    }
    // lane (r, c) collects word r of the rows 0..3 held by lanes (0..3, c): row n's word comes from lane 8n + c
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t rows[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int offer = (r + j) & 3;                       // as a source: serve destination row (r + j) & 3
      const uint32_t mine = offer == 0 ? w[0] : offer == 1 ? w[1] : offer == 2 ? w[2] : w[3];
      const int from_row = (r - j) & 3;                    // as a destination: read source row (r - j) & 3
      const uint32_t got = __shfl_sync(0xffffffffu, mine, from_row * 8 + c);
      if (from_row == 0) rows[0] = got;
      else if (from_row == 1) rows[1] = got;
      else if (from_row == 2) rows[2] = got;
      else rows[3] = got;
    }
    // rows[n] = bytes (k = 0..3) of output n; the block wants word k = bytes (n = 0..3)
    const uint32_t t0 = __byte_perm(rows[0], rows[1], 0x5140), t1 = __byte_perm(rows[2], rows[3], 0x5140);
    const uint32_t t2 = __byte_perm(rows[0], rows[1], 0x7362), t3 = __byte_perm(rows[2], rows[3], 0x7362);
    blk[st][0] = __byte_perm(t0, t1, 0x5410);
    blk[st][1] = __byte_perm(t0, t1, 0x7632);
    blk[st][2] = __byte_perm(t2, t3, 0x5410);
    blk[st][3] = __byte_perm(t2, t3, 0x7632);
  }
  const int s = (i0 >> 2) + r;                             // this lane's input slice
  if (s >= a.src_slices) return;
  const int ds0 = o0 >> 2;
  const int64_t block_index = ((int64_t)hw * a.src_slices + s) * a.group + ds0;
  if (BITS == 8) {
    uint4* dst = reinterpret_cast<uint4*>(a.dst + block_index * 16);
#pragma unroll
    for (int st = 0; st < 4; ++st)
      if (ds0 + st < a.total_ds) dst[st] = make_uint4(blk[st][0], blk[st][1], blk[st][2], blk[st][3]);
  } else {
    uint2* dst = reinterpret_cast<uint2*>(a.dst + block_index * 8);
#pragma unroll
    for (int st = 0; st < 4; ++st) {
      // bytes v0 v1 v2 v3 of a word (each < 16) -> v0 | v1 << 4, v2 | v3 << 4
      const uint32_t y0 = blk[st][0] | (blk[st][0] >> 4), y1 = blk[st][1] | (blk[st][1] >> 4);
      const uint32_t y2 = blk[st][2] | (blk[st][2] >> 4), y3 = blk[st][3] | (blk[st][3] >> 4);
      if (ds0 + st < a.total_ds) dst[st] = make_uint2(__byte_perm(y0, y1, 0x6420), __byte_perm(y2, y3, 0x6420));
    }
  }
}

// The same for the dense nibble source (two's-complement nibbles, two input channels per byte, the form the
// converter's INT4 files have), input channels a multiple of 32 and output channels a multiple of 4: a lane reads
// 32 input channels (16 bytes) of one output row, the four lanes that hold the same channels of four rows exchange
// words, and each transposes the 4 x 4 nibbles of two input slices in registers (bytes first, then nibbles).
__global__ void __launch_bounds__(256) pack_rows_u4_kernel(PackArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hw = blockIdx.z;
  const int r = lane >> 3, c = lane & 7;
  const int i0 = blockIdx.x * 256 + c * 32;              // first input channel of this lane's 16 bytes
  const int o0 = (blockIdx.y * 8 + warp) * 16;           // first of the warp's 16 output rows
  if (o0 >= a.O) return;
  uint2 blk_a[4], blk_b[4];                              // [output slice of the four]: input slices i0/4 + 2r, + 2r + 1
#pragma unroll
  for (int st = 0; st < 4; ++st) {
    const int o = o0 + st * 4 + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    int32_t rowsum = 0;
    if (o < a.O && i0 < a.I) {
      v = *reinterpret_cast<const uint4*>(a.src + ((((int64_t)o * a.HW + hw) * a.I + i0) >> 1));
      // destination nibble = source nibble ^ 8 (two's complement -> offset by 8); its value is nibble - 8
      v.x ^= 0x88888888u;
      v.y ^= 0x88888888u;
      v.z ^= 0x88888888u;
      v.w ^= 0x88888888u;
      const uint32_t m = 0x0F0F0F0Fu;
      rowsum = __dp4a(static_cast<int>((v.x & m) + ((v.x >> 4) & m)), 0x01010101, -64 * 4);
      rowsum = __dp4a(static_cast<int>((v.y & m) + ((v.y >> 4) & m)), 0x01010101, rowsum);
      rowsum = __dp4a(static_cast<int>((v.z & m) + ((v.z >> 4) & m)), 0x01010101, rowsum);
      rowsum = __dp4a(static_cast<int>((v.w & m) + ((v.w >> 4) & m)), 0x01010101, rowsum);
    }
    if (a.sum_i != nullptr) {
      rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 1);
      rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 2);
      rowsum += __shfl_xor_sync(0xffffffffu, rowsum, 4);
      if (c == 0 && o < a.O && o < a.sum_len && rowsum != 0) atomicAdd(a.sum_i + o, rowsum);
    }
    // lane (r, c) collects word r (input channels i0 + 8 r .. + 7) of the rows held by lanes (0..3, c)
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t rows[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int offer = (r + j) & 3;
      const uint32_t mine = offer == 0 ? w[0] : offer == 1 ? w[1] : offer == 2 ? w[2] : w[3];
      const int from_row = (r - j) & 3;
      const uint32_t got = __shfl_sync(0xffffffffu, mine, from_row * 8 + c);
      if (from_row == 0) rows[0] = got;
      else if (from_row == 1) rows[1] = got;
      else if (from_row == 2) rows[2] = got;
      else rows[3] = got;
    }
    // rows[n]: low half = nibbles k0..k3 of output n in the first slice, high half = the second slice.
    // bytes first: b0 = (k0 k1) of outputs 0, 2; b1 = of outputs 1, 3; b2, b3 = (k2 k3) likewise
    const uint32_t b0 = __byte_perm(rows[0], rows[2], 0x6240), b2 = __byte_perm(rows[0], rows[2], 0x7351);
    const uint32_t b1 = __byte_perm(rows[1], rows[3], 0x6240), b3 = __byte_perm(rows[1], rows[3], 0x7351);
    // then nibbles: c_k = outputs 0..3 of input channel k (both slices at once)
    const uint32_t m = 0x0F0F0F0Fu;
    const uint32_t c0 = (b0 & m) | ((b1 & m) << 4), c1 = ((b0 >> 4) & m) | (b1 & ~m);
    const uint32_t c2 = (b2 & m) | ((b3 & m) << 4), c3 = ((b2 >> 4) & m) | (b3 & ~m);
    blk_a[st] = make_uint2(__byte_perm(c0, c1, 0x5410), __byte_perm(c2, c3, 0x5410));
    blk_b[st] = make_uint2(__byte_perm(c0, c1, 0x7632), __byte_perm(c2, c3, 0x7632));
  }
  const int s = (i0 >> 2) + 2 * r;                       // this lane's first input slice
  const int ds0 = o0 >> 2;
  const int n_ds = min(4, a.dst_slices - ds0);           // (output channels are a multiple of 4 here)
  if (s < a.src_slices) {
    uint2* dst = reinterpret_cast<uint2*>(a.dst + (((int64_t)hw * a.src_slices + s) * a.group + ds0) * 8);
    for (int st = 0; st < n_ds; ++st) dst[st] = blk_a[st];
  }
  if (s + 1 < a.src_slices) {
    uint2* dst = reinterpret_cast<uint2*>(a.dst + (((int64_t)hw * a.src_slices + s + 1) * a.group + ds0) * 8);
    for (int st = 0; st < n_ds; ++st) dst[st] = blk_b[st];
  }
}

__global__ void sum_i_kernel(const int8_t* src, int O, int64_t hwi, int32_t* sum_i) {
  const int o = blockIdx.x;
  if (o >= O) return;
  const int8_t* row = src + (int64_t)o * hwi;
  int32_t s = 0;
  for (int64_t k = threadIdx.x; k < hwi; k += blockDim.x) s += row[k];
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  __shared__ int32_t part[8];
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    int32_t t = 0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += part[w];
    sum_i[o] = t;
  }
}

// [O][G] fp32 -> [G][O4] fp16/fp32, zero padded (OHIToHOIO4 in buffer storage).
__global__ void pack_scales_kernel(const float* src, int O, int G, int O4, int dst_f16, void* dst) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)G * O4) return;
  const int g = static_cast<int>(idx / O4), o = static_cast<int>(idx % O4);
  const float v = o < O ? src[(int64_t)o * G + g] : 0.0f;
  if (dst_f16)
    reinterpret_cast<__half*>(dst)[idx] = __float2half_rn(v);
  else
    reinterpret_cast<float*>(dst)[idx] = v;
}

// One warp per (row, block): absmax -> scale -> round-half-even -> clip.
// IEEE division (__fdiv_rn) and rintf reproduce numpy's float32 results.
__global__ void __launch_bounds__(128) quantize_kernel(const float* w, int O, int I, int block, int G,
                                                       float qmax, float qlo, float qhi, int8_t* q,
                                                       float* scale) {
  const int o = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int g = warp + blockIdx.y * nwarps; g < G; g += nwarps * gridDim.y) {
    const float* blk = w + (int64_t)o * I + (int64_t)g * block;
    float bound = 0.0f;
    for (int i = lane; i < block; i += 32) bound = fmaxf(bound, fabsf(blk[i]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) bound = fmaxf(bound, __shfl_xor_sync(0xffffffffu, bound, off));
    float s = __fdiv_rn(bound, qmax);
    if (s == 0.0f) s = 1.0f;
    int8_t* qb = q + (int64_t)o * I + (int64_t)g * block;
    for (int i = lane; i < block; i += 32) {
      float v = rintf(__fdiv_rn(blk[i], s));
      v = fminf(fmaxf(v, qlo), qhi);
      qb[i] = static_cast<int8_t>(v);
    }
    if (lane == 0) scale[(int64_t)o * G + g] = s;
  }
}

// The same arithmetic with 32-byte loads: the tensor is a flat sequence of blocks of 8 * LPB values (rows are
// whole numbers of blocks), LPB lanes to a block, eight consecutive values to a lane.
template <int LPB>
__global__ void __launch_bounds__(256) quantize_blocks_kernel(const float* __restrict__ w, int64_t chunks, float qmax,
                                                              float qlo, float qhi, int8_t* __restrict__ q,
                                                              float* __restrict__ scale) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const int64_t rounds = (chunks + stride - 1) / stride;  // whole warps stay together for the shuffles
  int64_t ch = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (int64_t it = 0; it < rounds; ++it, ch += stride) {
    const bool has = ch < chunks;
    float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f), b = a;
    if (has) {
      a = *reinterpret_cast<const float4*>(w + ch * 8);
      b = *reinterpret_cast<const float4*>(w + ch * 8 + 4);
    }
    float bound = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))),
                        fmaxf(fmaxf(fabsf(b.x), fabsf(b.y)), fmaxf(fabsf(b.z), fabsf(b.w))));
#pragma unroll
    for (int off = 1; off < LPB; off <<= 1) bound = fmaxf(bound, __shfl_xor_sync(0xffffffffu, bound, off));
    float sc = __fdiv_rn(bound, qmax);
    if (sc == 0.0f) sc = 1.0f;
    if (has) {
      auto one = [&](float x) -> uint32_t {
        const float v = fminf(fmaxf(rintf(__fdiv_rn(x, sc)), qlo), qhi);
        return static_cast<uint32_t>(static_cast<int>(v)) & 0xFFu;
      };
      uint2 out;
      out.x = one(a.x) | (one(a.y) << 8) | (one(a.z) << 16) | (one(a.w) << 24);
      out.y = one(b.x) | (one(b.y) << 8) | (one(b.z) << 16) | (one(b.w) << 24);
      *reinterpret_cast<uint2*>(q + ch * 8) = out;
      if ((ch & (LPB - 1)) == 0) scale[ch / LPB] = sc;
    }
  }
}

// One CTA per row for long blocks (per-channel quantisation): the row is read twice, the second time from
// L2 / L1, 16 bytes per lane.
__global__ void __launch_bounds__(256) quantize_rows_kernel(const float* __restrict__ w, int I, float qmax, float qlo,
                                                            float qhi, int8_t* __restrict__ q, float* __restrict__ scale) {
  __shared__ float red[8];
  const float* row = w + (int64_t)blockIdx.x * I;
  float bound = 0.0f;
  for (int i = threadIdx.x * 4; i < I; i += 1024) {
    const float4 v = *reinterpret_cast<const float4*>(row + i);
    bound = fmaxf(bound, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
  }
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) bound = fmaxf(bound, __shfl_xor_sync(0xffffffffu, bound, off));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = bound;
  __syncthreads();
  bound = red[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) bound = fmaxf(bound, red[k]);
  float sc = __fdiv_rn(bound, qmax);
  if (sc == 0.0f) sc = 1.0f;
  int8_t* qr = q + (int64_t)blockIdx.x * I;
  for (int i = threadIdx.x * 4; i < I; i += 1024) {
    const float4 v = *reinterpret_cast<const float4*>(row + i);
    auto one = [&](float x) -> uint32_t {
      const float t = fminf(fmaxf(rintf(__fdiv_rn(x, sc)), qlo), qhi);
      return static_cast<uint32_t>(static_cast<int>(t)) & 0xFFu;
    };
    *reinterpret_cast<uint32_t*>(qr + i) = one(v.x) | (one(v.y) << 8) | (one(v.z) << 16) | (one(v.w) << 24);
  }
  if (threadIdx.x == 0) scale[blockIdx.x] = sc;
}

}  // namespace

int pack_weights_impl(const mld_pack_desc* d, const void* src, void* dst, int32_t* sum_i, int32_t sum_len,
                      cudaStream_t stream) {
  PackArgs a;
  a.src = static_cast<const uint8_t*>(src);
  a.dst = static_cast<uint8_t*>(dst);
  a.sum_i = sum_i;
  a.O = d->o;
  a.HW = d->h * d->w;
  a.I = d->i;
  a.dst_slices = div_up(d->o, 4);
  a.src_slices = div_up(d->i, 4);
  a.group = d->out_group_size > 0 ? d->out_group_size : a.dst_slices;
  a.total_ds = div_up(a.dst_slices, a.group) * a.group;
  a.sum_len = sum_len;
  a.shift = d->bits == 8 ? 128 : 8;
  a.pad = d->pad_value;
  a.swap_dims = d->swap_dims;
  if (sum_i != nullptr) {
    const int n = sum_len < d->o ? sum_len : d->o;
    if (n > 0) MLD_CUDA_CHECK(cudaMemsetAsync(sum_i, 0, sizeof(int32_t) * n, stream));
  }
  dim3 grid(div_up(a.src_slices, kTileSlices), div_up(a.total_ds, kTileSlices), a.HW);
  if (grid.x == 0 || grid.y == 0 || grid.z == 0) return MLD_OK;
  const bool rows_fit = d->source == MLD_SRC_INT8 && a.I % 16 == 0 && a.group == a.dst_slices &&
                        (reinterpret_cast<uintptr_t>(src) & 15) == 0 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
  if (rows_fit) {
    dim3 rgrid(div_up(a.I, 128), div_up(a.dst_slices * 4, 128), a.HW);
    if (d->bits == 8)
      pack_rows_kernel<8><<<rgrid, 256, 0, stream>>>(a);
    else
      pack_rows_kernel<4><<<rgrid, 256, 0, stream>>>(a);
  } else if (d->source == MLD_SRC_UINT4_PACKED && a.I % 32 == 0 && a.O % 4 == 0 && !a.swap_dims &&
             a.group == a.dst_slices && (reinterpret_cast<uintptr_t>(src) & 15) == 0 &&
             (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
    dim3 rgrid(div_up(a.I, 256), div_up(a.O, 128), a.HW);
    pack_rows_u4_kernel<<<rgrid, 256, 0, stream>>>(a);
  } else if (d->source == MLD_SRC_INT8) {
    if (d->bits == 8)
      pack_from_int8_kernel<8><<<grid, 256, 0, stream>>>(a);
    else
      pack_from_int8_kernel<4><<<grid, 256, 0, stream>>>(a);
  } else {
    pack_from_u4_kernel<<<grid, 256, 0, stream>>>(a);
  }
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

int weights_sum_i_impl(const int8_t* src, int32_t o, int32_t hwi, int32_t* sum_i, cudaStream_t stream) {
  if (o == 0) return MLD_OK;
  sum_i_kernel<<<o, 256, 0, stream>>>(src, o, hwi, sum_i);
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

int pack_scales_impl(const float* src, int32_t o, int32_t g, int32_t dst_f16, void* dst, cudaStream_t stream) {
  const int O4 = align_n(o, 4);
  const int64_t n = (int64_t)g * O4;
  if (n == 0) return MLD_OK;
  pack_scales_kernel<<<static_cast<unsigned>(div_up64(n, 256)), 256, 0, stream>>>(src, o, g, O4, dst_f16, dst);
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

int quantize_weights_impl(const float* w, int32_t o, int32_t i, int32_t bits, int32_t block, int8_t* q,
                          float* scale, cudaStream_t stream) {
  if (o == 0 || i == 0) return MLD_OK;
  if (bits == 8 || block <= 0) block = i;
  const int G = i / block;
  const float qmax = bits == 8 ? 127.0f : 7.0f;
  const float qlo = bits == 8 ? -128.0f : -8.0f;
  const float qhi = bits == 8 ? 127.0f : 7.0f;
  const bool aligned = (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(q) & 7) == 0;
  const int lpb = block / 8;
  if (aligned && block % 8 == 0 && lpb >= 1 && lpb <= 32 && (lpb & (lpb - 1)) == 0) {
    const int64_t chunks = (int64_t)o * i / 8;
    int64_t blocks = (chunks + 255) / 256;
    if (blocks > 148 * 32) blocks = 148 * 32;
    const unsigned gb = static_cast<unsigned>(blocks);
    switch (lpb) {
      case 1: quantize_blocks_kernel<1><<<gb, 256, 0, stream>>>(w, chunks, qmax, qlo, qhi, q, scale); break;
      case 2: quantize_blocks_kernel<2><<<gb, 256, 0, stream>>>(w, chunks, qmax, qlo, qhi, q, scale); break;
      case 4: quantize_blocks_kernel<4><<<gb, 256, 0, stream>>>(w, chunks, qmax, qlo, qhi, q, scale); break;
      case 8: quantize_blocks_kernel<8><<<gb, 256, 0, stream>>>(w, chunks, qmax, qlo, qhi, q, scale); break;
      case 16: quantize_blocks_kernel<16><<<gb, 256, 0, stream>>>(w, chunks, qmax, qlo, qhi, q, scale); break;
      default: quantize_blocks_kernel<32><<<gb, 256, 0, stream>>>(w, chunks, qmax, qlo, qhi, q, scale); break;
    }
  } else if (aligned && G == 1 && i % 4 == 0) {
    quantize_rows_kernel<<<o, 256, 0, stream>>>(w, i, qmax, qlo, qhi, q, scale);
  } else {
    dim3 grid(o, G >= 64 ? 4 : 1);
    quantize_kernel<<<grid, 128, 0, stream>>>(w, o, i, block, G, qmax, qlo, qhi, q, scale);
  }
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

}  // namespace mld
