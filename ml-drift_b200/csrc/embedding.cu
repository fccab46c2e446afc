// Quantised embedding lookup over the FullyConnected weight layout.
//
// The reference stores the embedding table as FullyConnected weights (O = vocabulary, I = embedding
// width, layout kOSpatialIOGroupI4O4 from GetFullyConnectedInt{8,4}WeightsDesc) so that the table can be
// shared with the lm_head projection, and looks a token up by reading column `id % 4` of the 4x4 blocks
// (input slice S, output slice id / 4) and dequantising in fp32:
//   value = u * scale + (-scale * (shift + zero_point)), shift = 128 (INT8) / 8 (INT4)
// (ml_drift/common/kernels/embedding_lookup.cc:44-216; ids are clamped to [0, vocab - 1] as there).
// One thread per (token, input slice): 4 outputs, one 8- or 16-byte block read.  HBM-bound and tiny
// (dim * bits / 8 bytes per token).
#include <cuda_fp16.h>

#include "common.cuh"
#include "kernels.h"

namespace mld {
namespace {

struct EmbedArgs {
  const int32_t* ids;
  const uint8_t* weights;
  const void* scale;
  const void* zp;
  void* dst;
  int tokens, vocab, dim, src_slices, out_slices;
  int bits, block_mode, groups, group_slices;
  int f16, dst_layout;
};

__device__ __forceinline__ float load_param(const void* p, size_t i, int f16) {
  return f16 ? __half2float(static_cast<const __half*>(p)[i]) : static_cast<const float*>(p)[i];
}

__global__ void __launch_bounds__(256) embedding_lookup_kernel(EmbedArgs a) {
  const int S = blockIdx.x * blockDim.x + threadIdx.x;
  const int tok = blockIdx.y;
  if (S >= a.src_slices) return;
  int index = a.ids[tok];
  index = max(index, 0);
  index = min(index, a.vocab - 1);
  const int os = index >> 2, sub = index & 3;
  const size_t blk = (size_t)S * a.out_slices + os;
  float v[4];
  if (a.bits == 8) {
    const uint4 w = *reinterpret_cast<const uint4*>(a.weights + blk * 16);
    v[0] = static_cast<float>((w.x >> (8 * sub)) & 0xFFu);
    v[1] = static_cast<float>((w.y >> (8 * sub)) & 0xFFu);
    v[2] = static_cast<float>((w.z >> (8 * sub)) & 0xFFu);
    v[3] = static_cast<float>((w.w >> (8 * sub)) & 0xFFu);
  } else {
    const uint2 w = *reinterpret_cast<const uint2*>(a.weights + blk * 8);
    v[0] = static_cast<float>((w.x >> (4 * sub)) & 0xFu);
    v[1] = static_cast<float>((w.x >> (16 + 4 * sub)) & 0xFu);
    v[2] = static_cast<float>((w.y >> (4 * sub)) & 0xFu);
    v[3] = static_cast<float>((w.y >> (16 + 4 * sub)) & 0xFu);
  }
  const int g = a.block_mode ? min(S / a.group_slices, a.groups - 1) : 0;
  const size_t si = (size_t)g * a.out_slices * 4 + index;
  const float scale = load_param(a.scale, si, a.f16);
  const float zero_point = a.zp != nullptr ? load_param(a.zp, si, a.f16) : 0.0f;
  const float shift = a.bits == 8 ? 128.0f : 8.0f;
  const float bias = __fmul_rn(-scale, __fadd_rn(shift, zero_point));
  float o[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) o[i] = __fadd_rn(__fmul_rn(v[i], scale), bias);
  const size_t at = a.dst_layout == MLD_LAYOUT_SLICED ? ((size_t)S * a.tokens + tok) * 4 : (size_t)tok * a.dim + (size_t)S * 4;
  if (a.dst_layout == MLD_LAYOUT_SLICED || S * 4 + 3 < a.dim) {
    if (a.f16) {
      const __half2 h0 = __floats2half2_rn(o[0], o[1]), h1 = __floats2half2_rn(o[2], o[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<const uint32_t*>(&h0);
      pk.y = *reinterpret_cast<const uint32_t*>(&h1);
      if ((at & 3) == 0) {
        *reinterpret_cast<uint2*>(static_cast<__half*>(a.dst) + at) = pk;
      } else {
        for (int i = 0; i < 4; ++i) static_cast<__half*>(a.dst)[at + i] = __float2half_rn(o[i]);
      }
    } else {
      for (int i = 0; i < 4; ++i) static_cast<float*>(a.dst)[at + i] = o[i];
    }
  } else {
    for (int i = 0; i < 4 && S * 4 + i < a.dim; ++i) {
      if (a.f16)
        static_cast<__half*>(a.dst)[at + i] = __float2half_rn(o[i]);
      else
        static_cast<float*>(a.dst)[at + i] = o[i];
    }
  }
}

}  // namespace
}  // namespace mld

using namespace mld;

extern "C" int mld_embedding_lookup(const mld_embed_desc* d, const int32_t* ids, const void* weights, const void* scale,
                                    const void* zero_point, void* dst, int32_t tokens, void* stream) {
  MLD_REQUIRE(d != nullptr, "null descriptor");
  MLD_REQUIRE(d->vocab > 0 && d->dim > 0, "bad table shape");
  MLD_REQUIRE(d->weight_bits == 4 || d->weight_bits == 8, "Unsupported WeightsDescription type.");
  MLD_REQUIRE(d->scale_mode == MLD_SCALE_PER_CHANNEL || d->scale_mode == MLD_SCALE_BLOCK, "bad scale mode");
  MLD_REQUIRE(d->dst_layout == MLD_LAYOUT_SLICED || d->dst_layout == MLD_LAYOUT_ROW_MAJOR, "bad dst layout");
  MLD_REQUIRE(tokens >= 0, "bad token count");
  if (tokens == 0) return MLD_OK;
  MLD_REQUIRE(ids != nullptr && weights != nullptr && scale != nullptr && dst != nullptr, "null tensor");
  MLD_REQUIRE(!d->has_zero_point || zero_point != nullptr, "weights_zero_point tensor missing");
  MLD_REQUIRE((reinterpret_cast<uintptr_t>(weights) & 15) == 0, "weights must be 16-byte aligned");
  EmbedArgs a;
  a.ids = ids;
  a.weights = static_cast<const uint8_t*>(weights);
  a.scale = scale;
  a.zp = d->has_zero_point ? zero_point : nullptr;
  a.dst = dst;
  a.tokens = tokens;
  a.vocab = d->vocab;
  a.dim = d->dim;
  a.src_slices = div_up(d->dim, 4);
  a.out_slices = div_up(d->vocab, 4);
  a.bits = d->weight_bits;
  a.block_mode = d->scale_mode == MLD_SCALE_BLOCK ? 1 : 0;
  a.groups = a.block_mode ? d->groups : 1;
  MLD_REQUIRE(a.groups >= 1 && a.groups <= a.src_slices, "bad group count");
  a.group_slices = a.src_slices / a.groups;  // embedding_lookup.cc: (input channels / groups) / 4
  a.f16 = d->f16 ? 1 : 0;
  a.dst_layout = d->dst_layout;
  dim3 grid(div_up(a.src_slices, 256), tokens);
  embedding_lookup_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}
