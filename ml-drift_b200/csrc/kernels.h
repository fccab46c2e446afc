// Internal launch interfaces shared by the mldfc CUDA translation units.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "mldfc.h"

namespace mld {

// ------------------------------------------------------------ weight conversion
int pack_weights_impl(const mld_pack_desc* d, const void* src, void* dst, int32_t* sum_i, int32_t sum_len,
                      cudaStream_t stream);
int weights_sum_i_impl(const int8_t* src, int32_t o, int32_t hwi, int32_t* sum_i, cudaStream_t stream);
int pack_scales_impl(const float* src, int32_t o, int32_t g, int32_t dst_f16, void* dst, cudaStream_t stream);
int quantize_weights_impl(const float* w, int32_t o, int32_t i, int32_t bits, int32_t block, int8_t* q,
                          float* scale, cudaStream_t stream);

// ------------------------------------------------------------------ decode GEMV
struct GenericArgs {
  const void* x;
  const void* weights;
  const void* scale;
  const void* zp;
  const void* bias;
  void* y;
  int M, K, N;
  int src_slices, dst_slices;
  int scale_mode, groups, group_slices;
  float scalar_scale, scalar_zp;
  int has_zp;
  int src_layout, dst_layout;
};
int launch_fc_generic(const GenericArgs& a, int bits, bool f32, cudaStream_t stream);

// Sharded decoding without a separate collective: a kernel stores its output
// shard straight into every rank's copy of the gathered vector (plain peer
// stores over NVLink) and the last CTA to finish raises this rank's completion
// flag on every rank; the kernel that consumes the gathered vector waits
// (bounded) for the flags of all ranks.  world <= 1 disables both.
struct PeerScatter {
  int world;
  void* y_peers[8];          // base of the gathered vector in every rank's memory (index = rank)
  unsigned* flag_peers[8];   // this rank's flag for that vector in every rank's memory
  int* ticket;               // local CTA counter, zero between launches
  const int* step;           // device-side step counter
  int seq_off, seq_per_step; // flag value = *step * seq_per_step + seq_off
};
struct PeerWait {
  int world;
  const unsigned* flags;     // local flags, one per rank
  const int* step;
  int seq_off, seq_per_step;
  int* error;                // device error word: receives code 4 when the wait runs out
  unsigned long long limit_ns;
};
enum { kErrPeerWait = 4 };

// A sharded operator whose output block goes straight into every rank's copy of the gathered tensor:
// y[r] = where this rank's block starts in rank r's tensor (plain peer stores; y[rank] is local).
struct PeerOutputs {
  int world;
  void* y[8];
};

struct StripArgs {
  const void* x;      // fp16, sliced [K/4][M_total][4] (for one token a plain vector)
  const void* bias;   // fp16 [N4] or null
  void* y;            // fp16
  int* error;         // device error word (0 = ok)
  int M;              // tokens handled by this launch (1..8)
  int M_total;        // tokens in the x / y tensors
  int tok0;           // first token handled by this launch
  int N, N4;
  int src_slices;
  int units, gran;    // strip granularity: `units` units of `gran` 16-byte chunks per weight row
  int strips, ksplit;
  int rows_per_split;
  int stages, stage_bytes, scale_stage_bytes;
  int scale_rows;     // rows of the per-stage scale box (0 = scalar scale)
  int group_slices;   // k-slices per scale group
  int gs_shift;       // log2(group_slices) when it is a power of two below a stage, else -1
  int red_m;          // token stride of the reduction buffers
  int dst_layout;
  int epilogue;       // mld_epilogue
  float scalar_scale;
  int pdl;            // launched with programmatic stream serialization
  PeerScatter scatter;  // world <= 1: outputs go to y only
  PeerWait wait;        // world <= 1: no flag wait before the activations are read
  const void* next_w;  // optional: weights of the projection that runs next, pulled into L2 behind this one
  unsigned long long next_w_bytes;
  unsigned long long* trace;  // optional [grid][8] timestamps (ns) for tuning; null in normal use
  int trace_skip_math;        // tuning builds only: consume the stages without computing
};

struct StripGeometry {
  int gran, units, strips, ksplit, grid, w;
  int rows_per_split;
  int scale_rows, group_slices, gs_shift;
  int scale_stage_bytes, stage_bytes, stages, red_m, stage_rows;
  int xdig_bytes;  // shared memory kept for the digitised activation vector (4-bit weights), else 0
  size_t smem_bytes;
};
StripGeometry strip_geometry(int bits, int N, int K, int m_total, int group_slices, int scale_mode, int sms,
                             bool pdl, int smem_limit_kb = 0);
// Makes the plan's kernels report their bounded waits that ran out in `word` (a device int the caller
// owns and reads) instead of the plan's own word.
void fc_plan_share_error(mld_fc_plan* plan, int* word);
// mld_fc_run with the sharded-decoder hooks (null = none); not part of the C ABI.
int fc_run_internal(mld_fc_plan* plan, const void* src, const void* weights, const void* scale, const void* zero_point,
                    const void* bias, void* dst, int32_t tokens, void* stream, const PeerScatter* scatter,
                    const PeerWait* wait, const PeerOutputs* outs = nullptr, bool* outs_used = nullptr);
// Shape facts of a plan the sharded entry points need.
void fc_plan_shape(const mld_fc_plan* plan, int* n, int* dst_layout, int* max_tokens, int* device);
int launch_fc_strip(int bits, bool subnormal, const CUtensorMap& tw, const CUtensorMap& ts, const StripArgs& a,
                    const StripGeometry& gm, cudaStream_t stream);

// ------------------------------------------------- persistent decode-step kernel
struct MegaConfig {
  int layers, d_model, heads, head_dim, ffn, max_seq, block;
  float rms_eps, rope_min_timescale, rope_max_timescale;
  int device;
  int rank, world;  // sharding: heads, o/down outputs and FFN units are split evenly over the ranks
  int shard_layout; // 0: every projection split by output rows; 1: o and down split by input columns
  int handover;     // 0: op-to-op vectors as tagged words; 1: grid barriers between ops
  int grid_limit;   // > 0: at most this many CTAs
  int ring_stages;  // > 0: at most this many ring stages
  int wait_limit_us;  // > 0: bound on every device-side wait, microseconds (default 2 000 000)
};
struct MegaLayerPtrs {
  const void *wqkv, *sqkv, *wo, *so, *wgu, *sgu, *wdown, *sdown, *norm1, *norm2;
  void *kcache, *vcache;
};
struct MegaDecoder;
bool mega_supported(const MegaConfig& c);
int mega_create(const MegaConfig& c, MegaDecoder** out);
void mega_destroy(MegaDecoder* m);
int mega_set_layer(MegaDecoder* m, int layer, const MegaLayerPtrs& p);
int mega_step(MegaDecoder* m, const void* x_in, void* x_out, int pos, cudaStream_t stream);
// Reads (and clears) the kernel's error word: 0 = every wait of the last steps was satisfied.
int mega_device_status(MegaDecoder* m, int* code);
const int* mega_error_word(const MegaDecoder* m);
int mega_reset(MegaDecoder* m);
void mega_set_wait_limit(MegaDecoder* m, int us);
// Sharded: every rank exports its exchange block (64-byte IPC handle) and imports all of them (rank order).
int mega_ipc_export(MegaDecoder* m, void* handle64);
int mega_ipc_import(MegaDecoder* m, const void* handles);
#ifdef MLD_TRACE
int mega_enable_trace(MegaDecoder* m, bool on);
int mega_read_trace(MegaDecoder* m, unsigned long long* out, size_t count);
#endif
int mega_grid(const MegaDecoder* m);

// ----------------------------------------------------------------- prefill GEMM
struct GemmGeometry {
  int kp;              // K rounded up so that a K-major row is a multiple of 16 bytes
  int tile_n;          // UMMA N
  int m_tiles, n_tiles, k_blocks;
  int stages, a_stage_bytes, b_stage_bytes;
  size_t smem_bytes;
  int grid;
};
GemmGeometry gemm_geometry(int M, int N, int K, bool i8, int sms);
// x_sliced != null: the same launch also brings M tokens of sliced fp16 activations into K-major order (x_kmajor)
int launch_dequant_weights(int bits, bool to_s8, const void* packed, const void* scale, int scale_mode, int G,
                           int group_slices, float scalar_scale, int N, int K, int Kp, void* out, cudaStream_t stream,
                           const void* x_sliced = nullptr, int M = 0, void* x_kmajor = nullptr);
int launch_transpose_x(const void* x, int layout, int M, int K, int Kp, void* out, cudaStream_t stream);
// Per-token workspace of launch_quantize_act: {inv_scale, offset, sum} followed by the partial extremes of
// kStatSplits ranges of the input channels.
constexpr int kStatSplits = 16;
constexpr int kActParamFloats = 3 + 2 * kStatSplits;
int launch_quantize_act(const void* x, int layout, int M, int K, int Kp, bool symmetric, void* xq, float* params,
                        cudaStream_t stream);
int launch_gemm_umma(bool i8, const void* a_mat, const void* b_mat, const GemmGeometry& g, int M, int N, int K,
                     const void* bias, const void* w_scale, const float* a_params, void* y, int dst_layout, int* error,
                     cudaStream_t stream);

// ------------------------------------------- prefill GEMM, dequantisation inside (SM pairs)
struct PairGeometry {
  int kp, tile_n, m_tiles, n_tiles, k_blocks, stages, w_stages, w_box_bytes, grid;
  int shared_tiles;    // the first so many tiles are cut along K and dealt out evenly over the SM pairs ...
  int units_per_pair;  // ... so many k-blocks to each; the other tiles go out whole
  bool shares_tiles;   // shared_tiles > 0: neighbouring pairs meet through a PairSplit workspace
  size_t smem_bytes;
};
// Workspace through which two SM pairs that share a tile combine their partial sums.
struct PairSplit {
  float* ws;         // pair_split_bytes(sms) bytes
  uint32_t* flags;   // pair_split_flags(sms) words, zeroed once
  uint32_t epoch;    // a value no earlier launch on this workspace used (never 0)
};
inline size_t pair_split_bytes(int sms) { return (size_t)(sms / 2 > 0 ? sms / 2 : 1) * 2 * 4 * 8 * 8 * 32 * 16; }
inline size_t pair_split_flags(int sms) { return (size_t)(sms / 2 > 0 ? sms / 2 : 1) * 2 * 4 * 8; }
// mode: 0 = INT4 weights -> fp16 MMA, 1 = INT8 weights -> fp16 MMA, 2 = INT8 weights x int8 activations (packed
// weights, transformed in shared memory); 3 / 4 = weights prepared as K-major fp16 / s8 rows [N4][kp] by
// launch_dequant_weights (then `packed` is that matrix)
// may_share: a PairSplit workspace will be passed to the launch, so tile waves need not be whole
PairGeometry pair_geometry(int M, int N, int K, int mode, int sms, bool may_share = false);
int launch_gemm_pair(int mode, const void* a_mat, const void* packed, const PairGeometry& g, int M, int N, int K,
                     const void* scale, int scale_mode, int G, int group_slices, float scalar_scale, const void* bias,
                     const float* a_params, const int32_t* w_sum, void* y, int dst_layout, int* error,
                     cudaStream_t stream, const PeerOutputs* outs = nullptr, const PairSplit* split = nullptr);

// ------------------------------------------- prefill GEMM, dequantised weights in tensor memory (SM pairs)
struct WtGeometry {
  int kp, tile_tok, tok_tiles, n_tiles, k_blocks, w_stages, grid;
  int shared_tiles, units_per_pair;
  bool shares_tiles;
  size_t smem_bytes;
};
// mode: 0 = INT4 weights, 1 = INT8 weights, both dequantised to fp16 inside the kernel (float activations)
WtGeometry wtmem_geometry(int M, int N, int K, int mode, int sms, bool may_share = false);
int launch_gemm_wtmem(int mode, const void* x_kmajor, const void* packed, const WtGeometry& g, int M, int N, int K,
                      const void* scale, int scale_mode, int G, int group_slices, float scalar_scale, const void* bias,
                      void* y, int dst_layout, int* error, cudaStream_t stream, const PeerOutputs* outs = nullptr,
                      const PairSplit* split = nullptr);

}  // namespace mld
