// Prefill-stage dequant-GEMM with the dequantised weights in TENSOR MEMORY, on pairs of SMs
// (tcgen05 cta_group::2, A operand from tensor memory).
//
// Same contract as gemm_pair_kernel's inline modes (the packed weights never leave their reference layout in
// HBM; arithmetic of the WeightsConverter, ml_drift/common/kernels/conv_weights_converter.cc:248-290, followed
// by an fp16 x fp16 -> fp32 product as the float convolution of common/gpu_model_builder.cc:1110-1276 computes
// it), but with the operand roles turned round:
//
//   Y^T[N x M] = W[N x K] X[M x K]^T
//
// The weights are the MMA's M-side operand and sit in tensor memory; the activations are the N-side operand in
// shared memory.  A dequantised weight tile is then written once, by tcgen05.st, into the memory the tensor
// core reads it from, instead of being written to shared memory by the transform warps and read back from
// there by the tensor core beside their own traffic - which is what held gemm_pair_kernel's inline modes at
// about 1000 cycles per 64-wide K stage against 560 with prepared operands.
//
// A cluster of two CTAs owns a tile of 256 output channels x tile_tok tokens (tile_tok <= 256).  Per CTA:
//   warp 0       TMA producer of the activation tiles: this CTA's half of the tile's tokens, K-major rows of
//                128 bytes in the 128-byte swizzle, eight stages
//   warp 24      TMA producer of the packed weight boxes ([K/4] rows of 4x4 blocks) of this CTA's 128 channels
//   warps 6..21  transform: two groups of eight warps on alternate stages; a thread owns one output channel
//                (= one TMEM lane; a warp can only address the lane quarter 32 * (warp % 4)) and half of the
//                stage's 64 input channels, dequantises them to 16 registers of two halves and stores them to
//                the stage's 32 tensor-memory columns
//   warps 22,23  forwarders: tell the pair's first CTA that this CTA's half of a stage is in place
//   warp 1       tensor-memory owner; in the first CTA also the MMA issuer: four tcgen05.mma per stage (K = 16
//                each, A = 8 TMEM columns, B = 32 bytes further into the swizzled rows)
//   warps 2..5   epilogue: a thread reads its output channel's accumulators (one TMEM lane, a column per token),
//                adds the bias, and four neighbouring lanes exchange values so that each holds the four channels
//                of one output slice for two tokens, a 16-byte piece of the sliced output layout
// Tensor memory: columns 0..255 accumulators (one buffer: reading a tile's accumulators is not overlapped with
// the next tile's MMAs, so the transform warps, idle meanwhile, share the reading with the epilogue warps),
// columns 256..511 the weight ring (8 stages x 32 columns).
// The split of the work over the pairs (tiles of the last wave shared along K) is gemm_pair_kernel's.
// Every wait is bounded.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "pair_common.cuh"

namespace mld {
namespace {

constexpr int kWtStages = 8;          // operand ring: activation tile in shared memory + weight tile in TMEM
constexpr int kWtRows = 128;          // output channels per CTA
constexpr int kWtTokBytes = 128 * kKBytes;  // up to 128 token rows per CTA and stage
constexpr uint32_t kWtACol = 256;     // first TMEM column of the weight ring
constexpr int kErrWtBase = 50;
constexpr int kDrainParts = 5;        // warps that read one lane quarter's accumulators: one epilogue + four transform

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
// D[tmem_d] (+)= A[tmem_a] B[desc_b]^T over the pair; A: 16 halves per lane in 8 columns of both CTAs' tensor memory.
__device__ __forceinline__ void umma_pair_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u)
      : "memory");
}

struct WtArgs {
  PairArgs p;       // M, N, N4, k_blocks, scales, bias, y, dst_layout, error, outs, split, work list, w ring
  int tile_tok;     // tokens per tile (UMMA N), a multiple of 16
  int tok_tiles;    // ceil(M / tile_tok)
  long long* trace; // tuning builds only: [grid][8] cycle counts
  int trace_flags;  // tuning builds only: 1 = no output stores, 2 = no lane exchange either
};

template <int MODE>
__global__ void __launch_bounds__(kPairThreads, 1)
    gemm_wtmem_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w, WtArgs wa) {
  const PairArgs& a = wa.p;
  constexpr int BLK = MODE == kModeInt4F16 ? 8 : 16;   // bytes of a packed 4x4 block
  constexpr int SLICES = 16;                            // packed rows per stage (64 input channels)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int half_tok = wa.tile_tok / 2;
  constexpr int w_pitch = (kWtRows / 4) * BLK;          // bytes of one packed row of the box
  constexpr int w_stage = SLICES * w_pitch;             // 4 KB / 8 KB
  uint8_t* sX = smem;
  uint8_t* sW = sX + (size_t)kWtStages * kWtTokBytes;
  uint64_t* full_w = reinterpret_cast<uint64_t*>(sW + (size_t)a.w_stages * w_stage);  // [w_stages]
  uint64_t* w_empty = full_w + a.w_stages;            // [w_stages]: the transform warps have read the box
  uint64_t* full_ab = w_empty + a.w_stages;           // [stages], first CTA: tokens of both CTAs landed, weights of both in TMEM
  uint64_t* empty = full_ab + kWtStages;              // [stages]: the stage's MMAs have completed (arrives in both CTAs)
  uint64_t* tmem_full = empty + kWtStages;            // [1], arrives in both CTAs
  uint64_t* tmem_empty = tmem_full + 1;               // [1], first CTA: the epilogue warps of both CTAs have drained it
  uint64_t* xf_done = tmem_empty + 1;                 // [stages]: this CTA's transform warps have stored their half
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xf_done + kWtStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  WorkList work0;
  {
    const int shared_units = a.shared_tiles * a.k_blocks;
    work0.u = min(shared_units, pair * a.units_per_pair);
    work0.u_end = min(shared_units, work0.u + a.units_per_pair);
    work0.tile = a.shared_tiles + pair;
    work0.tile_end = a.m_tiles * a.n_tiles;
    work0.tile_step = n_pairs;
    work0.k_blocks = a.k_blocks;
  }

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    for (int s = 0; s < a.w_stages; ++s) {
      mbar_init(&full_w[s], 1);
      mbar_init(&w_empty[s], kTransformWarps);
    }
    for (int s = 0; s < kWtStages; ++s) {
      mbar_init(&full_ab[s], 1 + 2);  // the producer's expect_tx, + one arrival per CTA for its weights
      mbar_init(&empty[s], 1);
      mbar_init(&xf_done[s], kTransformWarps);
    }
    mbar_init(tmem_full, 1);
    mbar_init(tmem_empty, 2 * 4 * kDrainParts);
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
  pdl_wait();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t full_ab_lead = map_shared(smem_u32(full_ab), 0);
  const uint32_t tmem_empty_lead = map_shared(smem_u32(tmem_empty), 0);
  // tile -> (token tile, channel tile): the token tiles of one channel tile follow each other
  auto tile_tok0 = [&](int tile) { return (tile % a.m_tiles) * wa.tile_tok; };
  auto tile_n0 = [&](int tile) { return (tile / a.m_tiles) * 2 * kWtRows; };

  // Accumulators -> outputs, the share `part` of kDrainParts of the warps that can address this lane quarter
  // (one epilogue warp and the quarter's four transform warps, which have nothing to transform while the only
  // accumulator buffer is being read): pieces of 16 token columns, part, part + kDrainParts, ...  A tile shared
  // with a neighbouring pair (see gemm_pair_kernel): the pair that holds the tile's last k-blocks leaves its raw
  // accumulators in the workspace slot of the pair before it, which adds them to its own and writes the outputs.
  auto drain = [&](const Segment& sg, int part) -> bool {
    const int quad = warp & 3;  // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    const bool hands_over = sg.kb0 > 0, takes_over = sg.kb1 < a.k_blocks;
    const int slot = hands_over ? pair - 1 : pair;
    uint4* const slot_rows =
        reinterpret_cast<uint4*>(a.split_ws) + ((size_t)(slot * 2 + static_cast<int>(rank)) * 4 + quad) * (8 * 8 * 32) + lane;
    uint32_t* const slot_flag = a.split_flags + ((slot * 2 + static_cast<int>(rank)) * 4 + quad) * 8 + part;
    const uint32_t lane_base = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const int n_pieces = wa.tile_tok >> 4;
    if (hands_over) {
      for (int pc = part; pc < n_pieces; pc += kDrainParts) {
        uint32_t r[16];
        tmem_ld16(lane_base + static_cast<uint32_t>(16 * pc), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) slot_rows[(pc * 4 + j) * 32] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
      }
      __threadfence();
      tc_before();
      __syncwarp();
      if (lane == 0) {
        st_release_gpu(slot_flag, a.epoch);
        arrive_remote(tmem_empty_lead);
      }
      return true;
    }
    if (takes_over) {
      uint32_t seen = 0;
      if (lane == 0) {
        const unsigned long long t0 = globaltimer_ns();
        while ((seen = ld_acquire_gpu(slot_flag)) != a.epoch && globaltimer_ns() - t0 <= kWaitLimitNs) __nanosleep(64);
      }
      seen = __shfl_sync(0xffffffffu, seen, 0);
      if (seen != a.epoch) {
        atomicExch(a.error, kErrWtBase + 8);
        return false;
      }
    }
    const int n = (sg.tile / a.m_tiles) * 2 * kWtRows + static_cast<int>(rank) * kWtRows + quad * 32 + lane;  // output channel
    const int m_first = (sg.tile % a.m_tiles) * wa.tile_tok;
    const bool has_n = n < a.N4;
    __half bias_h = __float2half_rn(0.0f);
    if (a.bias != nullptr && has_n) bias_h = static_cast<const __half*>(a.bias)[n];
    const int q = lane & 3;  // place among the four channels of the output slice n >> 2
    for (int pc = part; pc < n_pieces; pc += kDrainParts) {
      const int c0 = 16 * pc;
      uint32_t r[16];
      tmem_ld16(lane_base + static_cast<uint32_t>(c0), r);
      tmem_ld_wait();
      if (takes_over) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint4 o = __ldcg(&slot_rows[(pc * 4 + j) * 32]);
          r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + __uint_as_float(o.x));
          r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + __uint_as_float(o.y));
          r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + __uint_as_float(o.z));
          r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + __uint_as_float(o.w));
        }
      }
      // token pairs as packed halves: h2[i] = tokens c0 + 2i, c0 + 2i + 1 of channel n
      uint32_t h2[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        __half2 v = __floats2half2_rn(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        if (a.bias != nullptr) v = __hadd2(v, __half2half2(bias_h));
        h2[i] = *reinterpret_cast<const uint32_t*>(&v);
      }
      if (a.dst_layout == MLD_LAYOUT_SLICED) {
        // Eight tokens at a time: the four lanes of a slice exchange token pairs so that lane q holds tokens
        // 2q, 2q + 1 (of the eight) of all four channels, 16 contiguous bytes of [slice][token][4 channels].
#pragma unroll
        for (int grp = 0; grp < 2; ++grp) {
          // 4 x 4 transpose over the slice's four lanes in two butterfly steps (lanes 2 apart, then 1 apart):
          // lane q starts with its channel's pairs p0..p3 and ends with pair q of channels 0..3
          uint32_t x0 = h2[4 * grp], x1 = h2[4 * grp + 1], x2 = h2[4 * grp + 2], x3 = h2[4 * grp + 3];
          {
            const bool up = (q & 2) != 0;
            const uint32_t s0 = up ? x0 : x2, s1 = up ? x1 : x3;  // what the lane 2 away needs
            const uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 2), r1 = __shfl_xor_sync(0xffffffffu, s1, 2);
            if (up) {
              x0 = r0;
              x1 = r1;
            } else {
              x2 = r0;
              x3 = r1;
            }
          }
          {
            const bool up = (q & 1) != 0;
            const uint32_t s0 = up ? x0 : x1, s1 = up ? x2 : x3;  // what the lane 1 away needs
            const uint32_t r0 = __shfl_xor_sync(0xffffffffu, s0, 1), r1 = __shfl_xor_sync(0xffffffffu, s1, 1);
            if (up) {
              x0 = r0;
              x2 = r1;
            } else {
              x1 = r0;
              x3 = r1;
            }
          }
          const int m = m_first + c0 + 8 * grp + 2 * q;  // first of this lane's two tokens
          uint4 pk;
          pk.x = __byte_perm(x0, x1, 0x5410);  // token m: channels 0, 1
          pk.y = __byte_perm(x2, x3, 0x5410);  //          channels 2, 3
          pk.z = __byte_perm(x0, x1, 0x7632);  // token m + 1
          pk.w = __byte_perm(x2, x3, 0x7632);
          if (has_n && m < a.M) {
            const size_t at = ((size_t)(n >> 2) * a.M + m) * 4;  // in halves
            const bool both = m + 1 < a.M && ((at * 2) & 15) == 0;
            const int world = a.outs.world > 1 ? a.outs.world : 1;
            for (int pr = 0; pr < world; ++pr) {
              __half* base = static_cast<__half*>(a.outs.world > 1 ? a.outs.y[pr] : a.y) + at;
              if (both) {
                *reinterpret_cast<uint4*>(base) = pk;
              } else {
                *reinterpret_cast<uint2*>(base) = make_uint2(pk.x, pk.y);
                if (m + 1 < a.M) *reinterpret_cast<uint2*>(base + 4) = make_uint2(pk.z, pk.w);
              }
            }
          }
        }
      } else if (n < a.N) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int m = m_first + c0 + 2 * i;
          if (m < a.M) static_cast<__half*>(a.y)[(size_t)m * a.N + n] = __ushort_as_half(static_cast<unsigned short>(h2[i] & 0xFFFFu));
          if (m + 1 < a.M)
            static_cast<__half*>(a.y)[(size_t)(m + 1) * a.N + n] = __ushort_as_half(static_cast<unsigned short>(h2[i] >> 16));
        }
      }
    }
    tc_before();
    __syncwarp();
    if (lane == 0) arrive_remote(tmem_empty_lead);
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------ producer of the activation tiles
    if (lane == 0) {
      prefetch_tmap(&tmap_x);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      WorkList work = work0;
      Segment sg;
      while (ok && work.next(sg)) {
        const int m0 = tile_tok0(sg.tile) + static_cast<int>(rank) * half_tok;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicExch(a.error, kErrWtBase + 1);
            ok = false;
            break;
          }
          if (rank == 0) mbar_arrive_expect_tx(&full_ab[stage], 2u * static_cast<uint32_t>(half_tok) * kKBytes);
          tma_load_2d_pair(sX + (size_t)stage * kWtTokBytes, &tmap_x, full_ab_lead + stage * 8, kb * 64, m0);
          if (++stage == kWtStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------- MMA issuer
    if (rank == 0 && lane == 0) {
      const uint32_t idesc = (1u << 4) | (static_cast<uint32_t>(wa.tile_tok >> 3) << 17) | (16u << 24);
      int stage = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      WorkList work = work0;
      Segment sg;
      [[maybe_unused]] long long tr_acc = 0, tr_ab = 0;
      [[maybe_unused]] const long long tr_start = MLD_PAIR_CLOCK();
      while (ok && work.next(sg)) {
        [[maybe_unused]] const long long t0 = MLD_PAIR_CLOCK();
        if (!wait_cluster(tmem_empty, acc_phase ^ 1)) {
          atomicExch(a.error, kErrWtBase + 2);
          break;
        }
        tr_acc += MLD_PAIR_CLOCK() - t0;
        acc_phase ^= 1;
        tc_after();
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          [[maybe_unused]] const long long t1 = MLD_PAIR_CLOCK();
          if (!wait_cluster(&full_ab[stage], phase)) {
            atomicExch(a.error, kErrWtBase + 3);
            ok = false;
            break;
          }
          tr_ab += MLD_PAIR_CLOCK() - t1;
          tc_after();
          const uint64_t db = make_desc(smem_u32(sX + (size_t)stage * kWtTokBytes));
          const uint32_t ta = tmem_base + kWtACol + static_cast<uint32_t>(stage * 32);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_pair_ts(tmem_base, ta + 8u * k, db + static_cast<uint64_t>((k * 32) >> 4), idesc,
                         (kb > sg.kb0 || k > 0) ? 1u : 0u);
          commit_pair(&empty[stage]);
          if (++stage == kWtStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) commit_pair(tmem_full);
      }
#ifdef MLD_TRACE
      if (wa.trace != nullptr) {
        wa.trace[blockIdx.x * 8 + 2] = tr_acc;
        wa.trace[blockIdx.x * 8 + 3] = tr_ab;
        wa.trace[blockIdx.x * 8 + 4] = MLD_PAIR_CLOCK() - tr_start;
      }
#endif
    }
  } else if (warp < 6) {
    // --------------------------------------------------------------------- epilogue
    uint32_t acc_phase = 0;
    WorkList work = work0;
    Segment sg;
    while (work.next(sg)) {
      if (!mbar_wait(tmem_full, acc_phase)) {
        atomicExch(a.error, kErrWtBase + 4);
        break;
      }
      acc_phase ^= 1;
      tc_after();
      if (!drain(sg, 0)) break;
    }
    if (a.outs.world > 1) __threadfence_system();  // the peer stores are performed before the kernel ends
  } else if (warp == 24) {
    // ------------------------------------------------- producer of the packed weight boxes
    if (lane == 0) {
      prefetch_tmap(&tmap_w);
      int ws = 0;
      uint32_t wphase = 0;
      bool ok = true;
      WorkList work = work0;
      Segment sg;
      while (ok && work.next(sg)) {
        const int nb0 = (tile_n0(sg.tile) + static_cast<int>(rank) * kWtRows) / 4 * BLK;  // byte column of the box
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(&w_empty[ws], wphase ^ 1)) {
            atomicExch(a.error, kErrWtBase + 7);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_w[ws], static_cast<uint32_t>(w_stage));
          tma_load_2d(sW + (size_t)ws * w_stage, &tmap_w, &full_w[ws], nb0 / 4, kb * SLICES);  // 32-bit elements
          if (++ws == a.w_stages) {
            ws = 0;
            wphase ^= 1;
          }
        }
      }
    }
  } else if (warp >= 22) {
    // ------------------------------------------------------------------- forwarders
    if (lane == 0) {
      const int parity_of_mine = warp - 22;  // stages of even / odd iterations
      int stage = 0, iter = 0;
      uint32_t phase = 0;
      const int n_iter = work0.stages_in_all();
      for (; iter < n_iter; ++iter) {
        if ((iter & 1) == parity_of_mine) {
          if (!mbar_wait(&xf_done[stage], phase)) {
            atomicExch(a.error, kErrWtBase + 6);
            break;
          }
          arrive_remote(full_ab_lead + stage * 8);
        }
        if (++stage == kWtStages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // -------------------------------------------------------------------- transform
    const int group = (warp - 6) >> 3;            // this group takes the iterations of its parity
    const int half = ((warp - 6) & 7) >> 2;       // which 32 of the stage's 64 input channels
    const int quad = warp & 3;                     // the TMEM lane quarter this warp can address
    const int row = quad * 32 + lane;              // output channel of the CTA's 128 = TMEM lane
    const int col4 = row & 3;                      // column of the row inside its 4x4 blocks
    const uint32_t sel8 = static_cast<uint32_t>(col4) | (static_cast<uint32_t>(4 + col4) << 8);
    int stage = 0, ws = 0;
    uint32_t phase = 0, wphase = 0;
    auto advance = [&](int n) {
      for (int i = 0; i < n; ++i) {
        if (++stage == kWtStages) {
          stage = 0;
          phase ^= 1;
        }
        if (++ws == a.w_stages) {
          ws = 0;
          wphase ^= 1;
        }
      }
    };
    bool ok = true;
    int xf_iter = 0;
    uint32_t acc_phase = 0;
    WorkList work = work0;
    Segment sg;
    [[maybe_unused]] long long tr_wait = 0, tr_work = 0, tr_st = 0;
    [[maybe_unused]] const long long tr_start = MLD_PAIR_CLOCK();
    while (ok && work.next(sg)) {
      const int n = tile_n0(sg.tile) + static_cast<int>(rank) * kWtRows + row;
      const bool has_n = n < a.N4;
      // this thread's 32 input channels of a stage are one scale group whenever groups are whole multiples of 32
      // inputs, the usual case: one load per stage then, issued a stage ahead
      const bool one_group = a.scale_mode != MLD_SCALE_BLOCK || (a.group_slices & 7) == 0;
      auto scale_at = [&](int slice) -> __half {
        if (!has_n) return __float2half_rn(0.0f);
        if (a.scale == nullptr) return __float2half_rn(a.scalar_scale);
        int g = a.scale_mode != MLD_SCALE_BLOCK ? 0 : (a.gs_shift >= 0 ? slice >> a.gs_shift : slice / a.group_slices);
        if (g >= a.G) g = a.G - 1;
        return __ldg(a.scale + (size_t)g * a.N4 + n);
      };
      int kb = sg.kb0 + ((xf_iter ^ group) & 1);
      if (kb != sg.kb0) advance(1);  // skip the other group's stage
      __half sc_next = __float2half_rn(0.0f);
      if (kb < sg.kb1) sc_next = scale_at(kb * SLICES + 8 * half);
      for (; kb < sg.kb1; kb += 2) {
        const __half sc_cur = sc_next;
        if (kb + 2 < sg.kb1) sc_next = scale_at((kb + 2) * SLICES + 8 * half);
        // the packed box has landed, and the stage's tensor-memory columns are free again (their MMAs completed)
        [[maybe_unused]] const long long t0 = MLD_PAIR_CLOCK();
        if (!mbar_wait(&full_w[ws], wphase) || !mbar_wait(&empty[stage], phase ^ 1)) {
          atomicExch(a.error, kErrWtBase + 5);
          ok = false;
          break;
        }
        [[maybe_unused]] const long long t1 = MLD_PAIR_CLOCK();
        tr_wait += t1 - t0;
        tc_after();
        const uint8_t* wp = sW + (size_t)ws * w_stage + (row >> 2) * BLK;
        const __half shift = __ushort2half_rn(static_cast<unsigned short>(MODE == kModeInt4F16 ? 8 : 128));
        uint32_t o[16];  // o[j] = input channels 32 half + 2j, 2j + 1 of the stage
        if constexpr (MODE == kModeInt4F16) {
          uint2 blk[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) blk[i] = *reinterpret_cast<const uint2*>(wp + (size_t)(8 * half + i) * w_pitch);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const __half scc = one_group ? sc_cur : scale_at(kb * SLICES + 2 * (4 * half + c));
            const __half2 s2 = __half2half2(scc);
            const __half2 b2 = __half2half2(__hmul(__hneg(scc), shift));
#pragma unroll
            for (int qq = 0; qq < 2; ++qq) {
              // nibble (k % 4) * 4 + col4: k0, k1 in the halves of .x, k2, k3 in those of .y
              o[4 * c + 2 * qq] = dq2(((blk[2 * c + qq].x >> (4 * col4)) & 0x000F000Fu) | 0x64006400u, s2, b2);
              o[4 * c + 2 * qq + 1] = dq2(((blk[2 * c + qq].y >> (4 * col4)) & 0x000F000Fu) | 0x64006400u, s2, b2);
            }
          }
        } else {
          uint4 blk[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) blk[i] = *reinterpret_cast<const uint4*>(wp + (size_t)(8 * half + i) * w_pitch);
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const __half scc = one_group ? sc_cur : scale_at(kb * SLICES + 2 * (4 * half + c));
            const __half2 s2 = __half2half2(scc);
            const __half2 b2 = __half2half2(__hmul(__hneg(scc), shift));
#pragma unroll
            for (int qq = 0; qq < 2; ++qq) {
              const uint4 v = blk[2 * c + qq];
              o[4 * c + 2 * qq] = dq2((__byte_perm(v.x, v.y, sel8) & 0x00FF00FFu) | 0x64006400u, s2, b2);
              o[4 * c + 2 * qq + 1] = dq2((__byte_perm(v.z, v.w, sel8) & 0x00FF00FFu) | 0x64006400u, s2, b2);
            }
          }
        }
        [[maybe_unused]] const long long t2 = MLD_PAIR_CLOCK();
        tr_work += t2 - t1;
        tmem_st16(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + kWtACol + static_cast<uint32_t>(stage * 32 + 16 * half), o);
        tmem_st_wait();
        tr_st += MLD_PAIR_CLOCK() - t2;
        tc_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&w_empty[ws]);     // the box may be overwritten
          mbar_arrive(&xf_done[stage]);  // local; a forwarder passes it on to the pair's first CTA
        }
        advance(kb + 1 < sg.kb1 ? 2 : 1);
      }
      xf_iter += sg.kb1 - sg.kb0;
      if (!ok) break;
      // This segment's accumulators: the transform warps share the reading with the epilogue warp of their
      // quarter.  (Measured: reading them only when the ring is full and the next stage blocked, so that the next
      // tile's first stages are transformed beforehand, costs more in polling than the refill costs here.)
      if (!mbar_wait(tmem_full, acc_phase)) {
        atomicExch(a.error, kErrWtBase + 9);
        break;
      }
      acc_phase ^= 1;
      tc_after();
      if (!drain(sg, 1 + group * 2 + half)) break;
    }
#ifdef MLD_TRACE
    if (wa.trace != nullptr && warp == 6 && lane == 0) {
      wa.trace[blockIdx.x * 8 + 5] = tr_wait;
      wa.trace[blockIdx.x * 8 + 6] = MLD_PAIR_CLOCK() - tr_start;
      wa.trace[blockIdx.x * 8 + 7] = tr_work;
      wa.trace[blockIdx.x * 8 + 0] = tr_st;
    }
#endif
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
#ifdef MLD_TRACE
static long long* g_wt_trace = nullptr;
extern "C" __attribute__((visibility("default"))) void mld_debug_set_wt_trace(void* p) {
  g_wt_trace = static_cast<long long*>(p);
}
#endif

WtGeometry wtmem_geometry(int M, int N, int K, int mode, int sms, bool may_share) {
  WtGeometry g;
  const int N4 = align_n(N, 4);
  g.kp = align_n(K, 8);
  g.k_blocks = div_up(g.kp, 64);
  g.n_tiles = div_up(N4, 2 * kWtRows);
  g.tile_tok = M >= 256 ? 256 : align_n(M, 16);
#ifdef MLD_TRACE
  if (const char* e = getenv("MLD_WT_TOK")) g.tile_tok = atoi(e);
#endif
  g.tok_tiles = div_up(M, g.tile_tok);
  const int pairs = sms / 2 > 0 ? sms / 2 : 1;
  const long tiles = (long)g.n_tiles * g.tok_tiles;
  g.shares_tiles = may_share && tiles > pairs && tiles % pairs != 0;
  if (g.shares_tiles) {
    g.shared_tiles = static_cast<int>(pairs + tiles % pairs);
    g.units_per_pair = static_cast<int>(((long)g.shared_tiles * g.k_blocks + pairs - 1) / pairs);
    g.grid = 2 * pairs;
  } else {
    g.shared_tiles = 0;
    g.units_per_pair = 0;
    g.grid = 2 * static_cast<int>(tiles < pairs ? tiles : pairs);
  }
  const int blk = mode == kModeInt4F16 ? 8 : 16;
  const int w_stage = 16 * (kWtRows / 4) * blk;
  const int fixed = 1024 + (2 * 24 + 3 * kWtStages + 2) * 8 + 64;
  int ws = (226 * 1024 - fixed - kWtStages * kWtTokBytes) / w_stage;
  if (ws > 16) ws = 16;
  g.w_stages = ws;
  g.smem_bytes = (size_t)kWtStages * kWtTokBytes + (size_t)ws * w_stage + fixed;
  return g;
}

int launch_gemm_wtmem(int mode, const void* x_kmajor, const void* packed, const WtGeometry& g, int M, int N, int K,
                      const void* scale, int scale_mode, int G, int group_slices, float scalar_scale, const void* bias,
                      void* y, int dst_layout, int* error, cudaStream_t stream, const PeerOutputs* outs,
                      const PairSplit* split) {
  if (mode != kModeInt4F16 && mode != kModeInt8F16) {
    set_last_error_text("bad GEMM mode");
    return MLD_INVALID_ARGUMENT;
  }
  if (g.shares_tiles && (split == nullptr || split->ws == nullptr || split->flags == nullptr || split->epoch == 0)) {
    set_last_error_text("this GEMM geometry shares tiles between SM pairs and needs a split workspace");
    return MLD_INVALID_ARGUMENT;
  }
  const int N4 = align_n(N, 4);
  const int blk = mode == kModeInt4F16 ? 8 : 16;
  const int SS = div_up(K, 4), DS = N4 / 4;
  CUtensorMap tx, tw;
  // activations: K-major rows [M][kp]; box = one swizzle atom of K x this CTA's half of the tile's tokens
  int rc = make_tmap_2d(&tx, x_kmajor, (uint64_t)g.kp * 2, M, (uint64_t)g.kp * 2, kKBytes, g.tile_tok / 2, 2,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, true);
  if (rc != MLD_OK) return rc;
  // packed weights: [K/4] rows of N4/4 blocks; box = one stage's 16 rows x the CTA's 32 blocks, in 32-bit elements
  rc = make_tmap_2d(&tw, packed, (uint64_t)DS * blk, SS, (uint64_t)DS * blk, (kWtRows / 4) * blk, 16, 4,
                    CU_TENSOR_MAP_SWIZZLE_NONE);
  if (rc != MLD_OK) return rc;
  WtArgs wa;
  memset(&wa, 0, sizeof wa);
  PairArgs& a = wa.p;
  a.M = M;
  a.N = N;
  a.N4 = N4;
  a.m_tiles = g.tok_tiles;  // the work list's "tile % m_tiles" runs over the token tiles
  a.n_tiles = g.n_tiles;
  a.k_blocks = g.k_blocks;
  a.w_stages = g.w_stages;
  a.scale = scale_mode == MLD_SCALE_SCALAR ? nullptr : static_cast<const __half*>(scale);
  a.scale_mode = scale_mode;
  a.G = G;
  a.group_slices = group_slices;
  a.gs_shift = -1;
  for (int sh = 0; sh < 24; ++sh)
    if ((1 << sh) == group_slices) a.gs_shift = sh;
  a.scalar_scale = scalar_scale;
  a.bias = bias;
  a.y = y;
  a.dst_layout = dst_layout;
  a.error = error;
  a.shared_tiles = g.shared_tiles;
  a.units_per_pair = g.units_per_pair;
  if (g.shares_tiles) {
    a.split_ws = split->ws;
    a.split_flags = split->flags;
    a.epoch = split->epoch;
  }
  if (outs != nullptr && outs->world > 1 && dst_layout == MLD_LAYOUT_SLICED) a.outs = *outs;
  wa.tile_tok = g.tile_tok;
  wa.tok_tiles = g.tok_tiles;
#ifdef MLD_TRACE
  wa.trace = g_wt_trace;
  wa.trace_flags = getenv("MLD_WT_FLAGS") != nullptr ? atoi(getenv("MLD_WT_FLAGS")) : 0;
#endif
  void (*kern)(CUtensorMap, CUtensorMap, WtArgs) =
      mode == kModeInt4F16 ? gemm_wtmem_kernel<kModeInt4F16> : gemm_wtmem_kernel<kModeInt8F16>;
  static bool configured[2][kMaxDevices];
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
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  MLD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, tx, tw, wa));
  count_launch();
  return MLD_OK;
}

}  // namespace mld
