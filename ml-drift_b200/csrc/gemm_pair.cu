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
//   warp 0      TMA producer of the activation tiles (K-major, 128-byte swizzle)
//   warp 24     TMA producer of the packed weight boxes ([K/4] rows of 4x4 blocks),
//               in a ring of its own that is deeper than the operand ring: the
//               boxes are small, and a box that is already in shared memory when
//               its operand stage comes free takes the load's latency off the
//               path stage free -> transformed -> multiplied
//   warp 1      tensor-memory owner; in the first CTA also the MMA issuer
//   warps 2..5  epilogue: tcgen05.ld -> convert (-> dequantise) -> global stores
//               in the reference's sliced output layout
//   warps 22,23 forwarders: a thread each tells the pair's first CTA that this
//               CTA's half of a stage has been transformed (the arrival on
//               another SM's barrier takes several hundred cycles to return,
//               so it is kept off the transform warps' path; the two threads
//               take alternate stages)
//   warps 6..21 transform, two groups of eight warps that take alternate stages
//               (a stage is a chain of dependent steps - wait, load, convert,
//               store, fence, signal - and two chains in flight hide each
//               other's latencies): two threads per weight row of the CTA's half turn the
//               packed nibbles / bytes of the stage into the K-major,
//               128-byte-swizzled operand tile the MMA reads:
//                 fp16 route  w = half(half(u * scale) + half(-scale * shift)),
//                             the WeightsConverter arithmetic
//                 int8 route  w = u - 128 (exact), for kind::i8
// Accumulators live in tensor memory, double-buffered, so the epilogue of one
// tile overlaps the main loop of the next.  Every wait is bounded.
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.cuh"
#include "pair_common.cuh"

namespace mld {
namespace {

template <int MODE>
__global__ void __launch_bounds__(kPairThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w, PairArgs a) {
  constexpr bool I8 = MODE == kModeInt8I8 || MODE == kModePreparedI8;
  constexpr bool PREPARED = MODE >= kModePreparedF16;
  // Epilogue warps: four (one per quarter of the TMEM lanes) while the transform warps are at work; with
  // prepared weights those warps are free, and sixteen share a tile, four taking every fourth 32-column chunk
  // of each lane quarter.
  constexpr int EPI_PARTS = PREPARED ? 4 : 1;
  constexpr int EPI_WARPS = 4 * EPI_PARTS;
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
  uint64_t* full_w = reinterpret_cast<uint64_t*>(sW + (size_t)a.w_stages * w_stage);  // [w_stages]: the box has landed
  uint64_t* w_empty = full_w + a.w_stages;   // [w_stages]: the transform warps have read the box
  uint64_t* full_ab = w_empty + a.w_stages;  // used in the pair's first CTA: A of both CTAs landed, B of both transformed
  uint64_t* empty = full_ab + a.stages;      // the stage's MMAs have completed (arrives in both CTAs)
  uint64_t* tmem_full = empty + a.stages;    // [2], arrives in both CTAs
  uint64_t* tmem_empty = tmem_full + 2;      // [2], used in the first CTA: the epilogue warps of both CTAs have drained it
  uint64_t* xf_done = tmem_empty + 2;        // [stages]: this CTA's transform warps have written their half of the stage
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xf_done + a.stages);

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
    for (int s = 0; s < a.stages; ++s) {
      // the producer's expect_tx, + one arrival per CTA for its transformed half
      mbar_init(&full_ab[s], PREPARED ? 1 : 1 + 2);
      mbar_init(&empty[s], 1);
      mbar_init(&xf_done[s], kTransformWarps);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&tmem_full[b], 1);
      mbar_init(&tmem_empty[b], 2 * EPI_WARPS);
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
  pdl_wait();  // everything above overlapped the tail of the kernel before; the operands are its outputs
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t full_ab_lead = map_shared(smem_u32(full_ab), 0);      // the first CTA's barriers, as cluster addresses
  const uint32_t tmem_empty_lead = map_shared(smem_u32(tmem_empty), 0);

  if (warp == 0) {
    // --------------------------------------------------------------- producer
    if (lane == 0) {
      prefetch_tmap(&tmap_a);
      if constexpr (PREPARED) prefetch_tmap(&tmap_w);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      long long tr_wait = 0;
      [[maybe_unused]] const long long tr_start = MLD_PAIR_CLOCK();
      WorkList work = work0;
      Segment sg;
      while (ok && work.next(sg)) {
        const int mi = sg.tile % a.m_tiles, ni = sg.tile / a.m_tiles;
        const int m0 = mi * 2 * kRowsPerCta + static_cast<int>(rank) * kRowsPerCta;
        (void)ni;
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          const long long t0 = MLD_PAIR_CLOCK();
          if (!mbar_wait(&empty[stage], phase ^ 1)) {
            atomicExch(a.error, kErrPairBase + 1);
            ok = false;
            break;
          }
          tr_wait += MLD_PAIR_CLOCK() - t0;
          const uint32_t b_bytes = PREPARED ? static_cast<uint32_t>(half_n) * kKBytes : 0u;
          if (rank == 0) mbar_arrive_expect_tx(&full_ab[stage], 2 * (kABytes + b_bytes));
          tma_load_2d_pair(sA + (size_t)stage * kABytes, &tmap_a, full_ab_lead + stage * 8, kb * K_PER_STAGE, m0);
          if constexpr (PREPARED)  // this CTA's half of the tile's weight rows, K-major like the activations
            tma_load_2d_pair(sB + (size_t)stage * kBBytes, &tmap_w, full_ab_lead + stage * 8, kb * K_PER_STAGE,
                             ni * a.tile_n + static_cast<int>(rank) * half_n);
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
      uint32_t acc_phase0 = 0, acc_phase1 = 0;  // (scalars: a run-time index would put an array in local memory)
      int local = 0;
      bool ok = true;
      long long tr_wait_acc = 0, tr_wait_ab = 0;
      [[maybe_unused]] const long long tr_start = MLD_PAIR_CLOCK();
      WorkList work = work0;
      Segment sg;
      for (; ok && work.next(sg); ++local) {
        const int acc = local & 1;
        const long long t0 = MLD_PAIR_CLOCK();
        if (!wait_cluster(&tmem_empty[acc], (acc ? acc_phase1 : acc_phase0) ^ 1)) {
          atomicExch(a.error, kErrPairBase + 2);
          ok = false;
          break;
        }
        if (acc) acc_phase1 ^= 1; else acc_phase0 ^= 1;
        tr_wait_acc += MLD_PAIR_CLOCK() - t0;
        tc_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * 256);
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          const long long t1 = MLD_PAIR_CLOCK();
          if (!wait_cluster(&full_ab[stage], phase)) {
            atomicExch(a.error, kErrPairBase + 3);
            ok = false;
            break;
          }
          tr_wait_ab += MLD_PAIR_CLOCK() - t1;
          tc_after();
          const uint64_t da = make_desc(smem_u32(sA + (size_t)stage * kABytes));
          const uint64_t db = make_desc(smem_u32(sB + (size_t)stage * kBBytes));
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint64_t adv = static_cast<uint64_t>((k * 32) >> 4);  // 32 bytes of K per MMA inside the swizzle atom
            umma_pair<I8>(tmem_d, da + adv, db + adv, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
          }
          commit_pair(&empty[stage]);
          if (++stage == a.stages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (ok) commit_pair(&tmem_full[acc]);
      }
#ifdef MLD_TRACE
      if (a.trace != nullptr) {
        a.trace[blockIdx.x * 8 + 2] = tr_wait_acc;
        a.trace[blockIdx.x * 8 + 3] = tr_wait_ab;
        a.trace[blockIdx.x * 8 + 4] = MLD_PAIR_CLOCK() - tr_start;
      }
#endif
    }
  } else if (warp < 2 + EPI_WARPS) {
    // --------------------------------------------------------------- epilogue
    const int quad = warp & 3;  // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
    const int part = (warp - 2) >> 2;  // this warp's chunks: part, part + EPI_PARTS, ...
    uint32_t acc_phase0 = 0, acc_phase1 = 0;
    int local = 0;
    bool ok = true;
    WorkList work = work0;
    Segment sg;
    [[maybe_unused]] long long tr_full = 0, tr_flag = 0;
    [[maybe_unused]] const long long tr_start = MLD_PAIR_CLOCK();
    for (; ok && work.next(sg); ++local) {
      const int acc = local & 1;
      const int mi = sg.tile % a.m_tiles, ni = sg.tile / a.m_tiles;
      [[maybe_unused]] const long long tf0 = MLD_PAIR_CLOCK();
      if (!mbar_wait(&tmem_full[acc], acc ? acc_phase1 : acc_phase0)) {
        atomicExch(a.error, kErrPairBase + 4);
        ok = false;
        break;
      }
      if (acc) acc_phase1 ^= 1; else acc_phase0 ^= 1;
      tc_after();
      tr_full += MLD_PAIR_CLOCK() - tf0;
      // A tile shared with a neighbour: the pair that holds the tile's LAST k-blocks meets it first in its range
      // and leaves its raw accumulators in the slot of the pair before it; the pair that holds the tile's FIRST
      // k-blocks meets it last in its range, adds what it finds in its own slot and writes the outputs.  Each of
      // the eight epilogue warps of a pair hands over its own 32 rows.
      const bool hands_over = sg.kb0 > 0, takes_over = sg.kb1 < a.k_blocks;
      const int slot = hands_over ? pair - 1 : pair;
      uint4* const slot_rows =
          reinterpret_cast<uint4*>(a.split_ws) + ((size_t)(slot * 2 + static_cast<int>(rank)) * 4 + quad) * (8 * 8 * 32) + lane;
      uint32_t* const slot_flag = a.split_flags + ((slot * 2 + static_cast<int>(rank)) * 4 + quad) * 4 + part;
      if (hands_over) {
        for (int c0 = part * 32; c0 < a.tile_n; c0 += 32 * EPI_PARTS) {
          uint32_t r[32];
          tmem_ld32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * 256 + c0), r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            slot_rows[((c0 >> 5) * 8 + j) * 32] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
        }
        __threadfence();
        tc_before();
        __syncwarp();
        if (lane == 0) {
          st_release_gpu(slot_flag, a.epoch);
          arrive_remote(tmem_empty_lead + acc * 8);
        }
        continue;
      }
      if (takes_over) {
        [[maybe_unused]] const long long tg0 = MLD_PAIR_CLOCK();
        uint32_t seen = 0;
        if (lane == 0) {
          const unsigned long long t0 = globaltimer_ns();
          while ((seen = ld_acquire_gpu(slot_flag)) != a.epoch && globaltimer_ns() - t0 <= kWaitLimitNs) __nanosleep(64);
        }
        seen = __shfl_sync(0xffffffffu, seen, 0);
        if (seen != a.epoch) {
          atomicExch(a.error, kErrPairBase + 8);
          ok = false;
          break;
        }
        tr_flag += MLD_PAIR_CLOCK() - tg0;
      }
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
      for (int c0 = part * 32; c0 < a.tile_n; c0 += 32 * EPI_PARTS) {
        uint32_t r[32];
        // int8 route: lane l holds the constants of column c0 + l, handed round by shuffles below
        float col_scale = 0.0f, col_offset = 0.0f;  // w_scale and weights_sum of the column
        if constexpr (I8) {
          const int nl = n0 + c0 + lane;
          if (c0 + lane < a.tile_n && nl < a.N) {
            col_scale = __half2float(a.scale[nl]);
            if (a.w_sum != nullptr) col_offset = static_cast<float>(a.w_sum[nl]);
          }
        }
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(acc * 256 + c0);
        tmem_ld32(taddr, r);
        tmem_ld_wait();
        if (takes_over) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 o = __ldcg(&slot_rows[((c0 >> 5) * 8 + j) * 32]);
            if constexpr (I8) {
              r[4 * j] += o.x, r[4 * j + 1] += o.y, r[4 * j + 2] += o.z, r[4 * j + 3] += o.w;
            } else {
              r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + __uint_as_float(o.x));
              r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + __uint_as_float(o.y));
              r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + __uint_as_float(o.z));
              r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + __uint_as_float(o.w));
            }
          }
        }
        if constexpr (I8) {
          // CreateDequantization (quantize_and_dequantize.cc:867-964):
          //   res = float(acc) * (w_scale * src_scale) + w_scale * src_zero_point * weights_sum
          // (every lane takes part in the shuffles, rows past M included)
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float ws = __shfl_sync(0xffffffffu, col_scale, j), wo = __shfl_sync(0xffffffffu, col_offset, j);
            float v = static_cast<float>(static_cast<int32_t>(r[j])) * (ws * a_scale);
            if (a.w_sum != nullptr) v += ws * a_off * wo;
            r[j] = __float_as_uint(v);
          }
        }
        if (m < a.M) {
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            const int n = n0 + c0 + j;
            if (c0 + j >= a.tile_n || n >= a.N4) break;
            __half2 h01 = __floats2half2_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            __half2 h23 = __floats2half2_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            if (a.bias != nullptr) {  // [N4] halves: the four of this column block in one load
              const uint2 bv = __ldg(reinterpret_cast<const uint2*>(static_cast<const __half*>(a.bias) + n));
              h01 = __hadd2(h01, *reinterpret_cast<const __half2*>(&bv.x));
              h23 = __hadd2(h23, *reinterpret_cast<const __half2*>(&bv.y));
            }
            const __half h[4] = {__low2half(h01), __high2half(h01), __low2half(h23), __high2half(h23)};
            if (a.dst_layout == MLD_LAYOUT_SLICED) {
              uint2 pk;
              pk.x = *reinterpret_cast<const uint32_t*>(&h01);
              pk.y = *reinterpret_cast<const uint32_t*>(&h23);
              const size_t at = ((size_t)(n >> 2) * a.M + m) * 4;
              if (a.outs.world > 1) {
                for (int pr = 0; pr < a.outs.world; ++pr) *reinterpret_cast<uint2*>(static_cast<__half*>(a.outs.y[pr]) + at) = pk;
              } else {
                *reinterpret_cast<uint2*>(static_cast<__half*>(a.y) + at) = pk;
              }
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
#ifdef MLD_TRACE
    if (a.trace != nullptr && PREPARED && warp == 2 && lane == 0) {
      a.trace[blockIdx.x * 8 + 0] = tr_full;
      a.trace[blockIdx.x * 8 + 1] = tr_flag;
      a.trace[blockIdx.x * 8 + 5] = MLD_PAIR_CLOCK() - tr_start;
    }
#endif
    if (a.outs.world > 1) __threadfence_system();  // the peer stores are performed before the kernel ends
  } else if (PREPARED) {
    // nothing to transform: the remaining warps only take part in the barriers at both ends
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
        const int ni = sg.tile / a.m_tiles;
        const int nb0 = (ni * a.tile_n + static_cast<int>(rank) * half_n) / 4 * BLK;  // byte column of the box
        for (int kb = sg.kb0; kb < sg.kb1; ++kb) {
          if (!mbar_wait(&w_empty[ws], wphase ^ 1)) {
            atomicExch(a.error, kErrPairBase + 7);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&full_w[ws], static_cast<uint32_t>(a.w_box_bytes));
          tma_load_2d(sW + (size_t)ws * w_stage, &tmap_w, &full_w[ws], nb0 / 4, kb * SLICES);  // 32-bit elements
          if (++ws == a.w_stages) {
            ws = 0;
            wphase ^= 1;
          }
        }
      }
    }
  } else if (warp >= 22) {
    // -------------------------------------------------------------- forwarders
    if (lane == 0) {
      const int parity_of_mine = warp - 22;  // stages of even / odd iterations
      int stage = 0, iter = 0;
      uint32_t phase = 0;
      bool ok = true;
      const int n_iter = work0.stages_in_all();
      for (; iter < n_iter && ok; ++iter) {
        if ((iter & 1) == parity_of_mine) {
          if (!mbar_wait(&xf_done[stage], phase)) {
            atomicExch(a.error, kErrPairBase + 6);
            ok = false;
            break;
          }
          arrive_remote(full_ab_lead + stage * 8);
        }
        if (++stage == a.stages) {
          stage = 0;
          phase ^= 1;
        }
      }
    }
  } else {
    // -------------------------------------------------------------- transform
    const int group = (warp - 6) >> 3;                // this group takes the iterations of its parity
    const int tt = (threadIdx.x - 6 * 32) & 255;      // 0..255 inside the group
    const int row = tt & 127;                         // weight row of this CTA's half of the tile
    const int half = tt >> 7;                         // which four of the row's eight 16-byte chunks
    const bool active = row < half_n;
    const int col4 = row & 3;                         // column of the row inside its 4x4 blocks
    uint8_t* const b_row = sB + (row >> 3) * 1024 + (row & 7) * 128;
    const int sw = row & 7;                           // 16-byte chunk c of the row sits at chunk c ^ sw
    // prmt selector: byte col4 of two words -> the low bytes of the two 16-bit halves (bytes 1 and 3 are masked
    // off by the user)
    const uint32_t sel8 = static_cast<uint32_t>(col4) | (static_cast<uint32_t>(4 + col4) << 8);
    int stage = 0, ws = 0;       // positions in the operand ring and in the packed-weight ring
    uint32_t phase = 0, wphase = 0;
    auto advance = [&](int n) {
      for (int i = 0; i < n; ++i) {
        if (++stage == a.stages) {
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
    long long tr_wait = 0;
    int xf_iter = 0;  // stages of earlier tiles (parity decides which group starts a tile)
    [[maybe_unused]] long long tr_work = 0, tr_fence = 0, tr_arrive = 0;
    [[maybe_unused]] const long long tr_start = MLD_PAIR_CLOCK();
    WorkList work = work0;
    Segment sg;
    while (ok && work.next(sg)) {
      const int ni = sg.tile / a.m_tiles;
      const int n = ni * a.tile_n + static_cast<int>(rank) * half_n + row;
      const bool has_n = active && n < a.N4;
      // fp16 routes: this row's scale for the group the first k-block's chunks fall in, fetched a k-block ahead
      // (a thread's four chunks are 32 consecutive inputs: one scale group whenever groups are whole
      // multiples of 32 inputs, the usual case; then one load per stage, issued a stage ahead, serves all four.
      // Scalars, not arrays: anything indexed here would end up in local memory.)
      const bool one_group = a.scale_mode != MLD_SCALE_BLOCK || (a.group_slices & 7) == 0;
      auto scale_at = [&](int slice) -> __half {
        if (a.scale == nullptr || !has_n) return __float2half_rn(a.scalar_scale);
        int g = a.scale_mode != MLD_SCALE_BLOCK ? 0 : (a.gs_shift >= 0 ? slice >> a.gs_shift : slice / a.group_slices);
        if (g >= a.G) g = a.G - 1;
        return __ldg(a.scale + (size_t)g * a.N4 + n);
      };
      // the group's first stage of this tile, and from there every second one
      int kb = sg.kb0 + ((xf_iter ^ group) & 1);
      if (kb != sg.kb0) advance(1);  // skip the other group's stage
      __half sc_next = __float2half_rn(0.0f);
      if constexpr (!I8) {
        if (kb < sg.kb1) sc_next = scale_at(kb * SLICES + 8 * half);
      }
      for (; kb < sg.kb1; kb += 2) {
        const __half sc_cur = sc_next;
        if constexpr (!I8) {
          if (kb + 2 < sg.kb1) sc_next = scale_at((kb + 2) * SLICES + 8 * half);
        }
        const long long t0 = MLD_PAIR_CLOCK();
        // the packed box has landed, and the operand stage it is transformed into is free again
        if (!mbar_wait(&full_w[ws], wphase) || !mbar_wait(&empty[stage], phase ^ 1)) {
          atomicExch(a.error, kErrPairBase + 5);
          ok = false;
          break;
        }
        tr_wait += MLD_PAIR_CLOCK() - t0;
        const long long tw0 = MLD_PAIR_CLOCK();
#ifdef MLD_TRACE
        const bool do_work = a.skip_transform == 0;
#else
        constexpr bool do_work = true;
#endif
        if ((active || I8) && do_work) {
          const uint8_t* wp = sW + (size_t)ws * w_stage + (row >> 2) * BLK;
          uint8_t* bp = b_row + (size_t)stage * kBBytes;
          if constexpr (I8) {
            // A thread takes one 4x4-block column of four weight rows and ONE 16-byte chunk of K (four packed
            // rows): four 16-byte blocks in, transposed byte-wise and re-biased u8 -> s8, four 16-byte pieces
            // out (rows 4 blk .. 4 blk + 3, chunk c).  Lane = (blk & 7) + 8 * (chunk & 3): both the loads
            // and the swizzled stores then spread evenly over the banks.
            const int blk_i = ((tt >> 5) & 3) * 8 + (lane & 7);   // 4x4-block column of this CTA's half: rows 4 blk_i ..
            const int c = (tt >> 7) * 4 + (lane >> 3);             // chunk of the 128-byte row
            if (4 * blk_i < half_n) {
              const uint8_t* wq = sW + (size_t)ws * w_stage + blk_i * 16;
              uint32_t t[4][4];  // t[slice][row] = bytes k0..k3 of that packed row for weight row `row`
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 v = *reinterpret_cast<const uint4*>(wq + (size_t)(4 * c + q) * w_pitch);
                const uint32_t p0 = __byte_perm(v.x, v.y, 0x5140), p1 = __byte_perm(v.x, v.y, 0x7362);
                const uint32_t q0 = __byte_perm(v.z, v.w, 0x5140), q1 = __byte_perm(v.z, v.w, 0x7362);
                t[q][0] = __byte_perm(p0, q0, 0x5410) ^ 0x80808080u;
                t[q][1] = __byte_perm(p0, q0, 0x7632) ^ 0x80808080u;
                t[q][2] = __byte_perm(p1, q1, 0x5410) ^ 0x80808080u;
                t[q][3] = __byte_perm(p1, q1, 0x7632) ^ 0x80808080u;
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int r = 4 * blk_i + j;
                uint8_t* dst = sB + (size_t)stage * kBBytes + (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4);
                *reinterpret_cast<uint4*>(dst) = make_uint4(t[0][j], t[1][j], t[2][j], t[3][j]);
              }
            }
          } else {
            // chunk c: K elements 8 c .. 8 c + 7 = packed rows 2 c, 2 c + 1
            const __half shift = __ushort2half_rn(static_cast<unsigned short>(MODE == kModeInt4F16 ? 8 : 128));
            if constexpr (MODE == kModeInt4F16) {
              uint2 blk[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) blk[i] = *reinterpret_cast<const uint2*>(wp + (size_t)(8 * half + i) * w_pitch);
#pragma unroll
              for (int c = 0; c < 4; ++c) {
                const __half scc = one_group ? sc_cur : scale_at(kb * SLICES + 2 * (4 * half + c));
                const __half2 s2 = __half2half2(scc);
                const __half2 b2 = __half2half2(__hmul(__hneg(scc), shift));
                uint32_t o[4];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  // nibble (k % 4) * 4 + col4: k0, k1 in the halves of .x, k2, k3 in those of .y
                  o[2 * q] = dq2(((blk[2 * c + q].x >> (4 * col4)) & 0x000F000Fu) | 0x64006400u, s2, b2);
                  o[2 * q + 1] = dq2(((blk[2 * c + q].y >> (4 * col4)) & 0x000F000Fu) | 0x64006400u, s2, b2);
                }
                *reinterpret_cast<uint4*>(bp + (((4 * half + c) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
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
                uint32_t o[4];
#pragma unroll
                for (int q = 0; q < 2; ++q) {
                  const uint4 v = blk[2 * c + q];
                  // bytes col4 of k0, k1 -> the low bytes of the two halves
                  o[2 * q] = dq2((__byte_perm(v.x, v.y, sel8) & 0x00FF00FFu) | 0x64006400u, s2, b2);
                  o[2 * q + 1] = dq2((__byte_perm(v.z, v.w, sel8) & 0x00FF00FFu) | 0x64006400u, s2, b2);
                }
                *reinterpret_cast<uint4*>(bp + (((4 * half + c) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
              }
            }
          }
        }
        // the tile was written through the generic proxy; the MMA reads it through the async proxy
        const long long tw1 = MLD_PAIR_CLOCK();
        fence_proxy_async();
        const long long tw2 = MLD_PAIR_CLOCK();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&w_empty[ws]);    // the box may be overwritten
          mbar_arrive(&xf_done[stage]);  // local; a forwarder passes it on to the pair's first CTA
        }
        tr_work += tw1 - tw0;
        tr_fence += tw2 - tw1;
        tr_arrive += MLD_PAIR_CLOCK() - tw2;
        // on to this group's next stage: past its own and, unless the tile ends first, the other group's
        advance(kb + 1 < sg.kb1 ? 2 : 1);
      }
      xf_iter += sg.kb1 - sg.kb0;
    }
#ifdef MLD_TRACE
    if (a.trace != nullptr && tt == 0 && group == 0) {
      a.trace[blockIdx.x * 8 + 5] = tr_wait;
      a.trace[blockIdx.x * 8 + 6] = MLD_PAIR_CLOCK() - tr_start;
      a.trace[blockIdx.x * 8 + 7] = tr_work;
      a.trace[blockIdx.x * 8 + 0] = tr_fence;     // (overwrites the producer's slots: the transform split is what is wanted now)
      a.trace[blockIdx.x * 8 + 1] = tr_arrive;
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
static long long* g_pair_trace = nullptr;
extern "C" __attribute__((visibility("default"))) void mld_debug_set_pair_trace(void* p) {
  g_pair_trace = static_cast<long long*>(p);
}
#endif

PairGeometry pair_geometry(int M, int N, int K, int mode, int sms, bool may_share) {
  PairGeometry g;
  const int N4 = align_n(N, 4);
  const bool i8 = mode == kModeInt8I8 || mode == kModePreparedI8;
  g.kp = align_n(K, i8 ? 16 : 8);
  g.m_tiles = div_up(M, 2 * kRowsPerCta);
  const int k_per_stage = i8 ? 128 : 64;
  g.k_blocks = div_up(g.kp, k_per_stage);
  const int pairs = sms / 2 > 0 ? sms / 2 : 1;
  // UMMA N of the pair.  Measured: a stage takes the same time for every width up to 256 (each MMA re-reads its
  // 128 x 16 activation fragment from shared memory, which takes as long as the arithmetic of 256 columns), so
  // what counts is the number of stages the busiest SM pair runs: whole tile waves, or, when neighbouring pairs
  // may share a tile along K, an even share of all stages.  Among the widths with the fewest stages the
  // narrowest with the same tile count wastes least on columns past N.
  auto stages_of_busiest = [&](int tn) -> long {
    const long tiles = (long)g.m_tiles * div_up(N4, tn);
    const long whole = tiles / pairs, rest = tiles % pairs;
    if (may_share && whole >= 1 && rest != 0)
      return (whole - 1) * g.k_blocks + ((pairs + rest) * (long)g.k_blocks + pairs - 1) / pairs;
    return (tiles + pairs - 1) / pairs * g.k_blocks;
  };
  int best_n = 256;
  long best_cost = -1;
  for (int tn = 256; tn >= 128; tn -= 16) {
    const long cost = stages_of_busiest(tn);
    if (best_cost < 0 || cost < best_cost || (cost == best_cost && div_up(N4, tn) == div_up(N4, best_n))) {
      best_cost = cost;
      best_n = tn;
    }
  }
  if (N4 < 128) best_n = align_n(N4, 16);  // one narrow tile
  g.tile_n = best_n;
#ifdef MLD_TRACE
  if (const char* e = getenv("MLD_PAIR_TN")) g.tile_n = atoi(e);
#endif
  g.n_tiles = div_up(N4, g.tile_n);
  const int blk = mode == kModeInt4F16 ? 8 : 16;
  g.w_box_bytes = (k_per_stage / 4) * (g.tile_n / 2 / 4) * blk;
  const int w_stage = (g.w_box_bytes + 127) & ~127;
  const int fixed = 1024 + (5 * 16 + 4) * 8 + 64;
  // operand stages of 32 KB, as many as leave room for a packed-weight ring at least one stage deeper
  const int budget = 226 * 1024 - fixed;
  int stages = 2, w_stages = 3;
  for (int st = 6; st >= 2; --st) {
    int ws = (budget - st * (kABytes + kBBytes)) / w_stage;
    if (ws > 2 * st) ws = 2 * st;
    if (ws > 16) ws = 16;
    if (ws >= st + 1) {
      stages = st;
      w_stages = ws;
      break;
    }
  }
#ifdef MLD_TRACE
  if (const char* e = getenv("MLD_PAIR_STAGES")) stages = atoi(e) < stages ? atoi(e) : stages;
#endif
  g.stages = stages;
  g.w_stages = w_stages;
  g.smem_bytes = (size_t)stages * (kABytes + kBBytes) + (size_t)w_stages * w_stage + fixed;
  const long tiles = (long)g.m_tiles * g.n_tiles;
  // Tiles that do not fill a last wave: the last whole wave and the remainder are cut along K and dealt out
  // evenly (between one and two tiles' worth of k-blocks per pair); the waves before it go out as whole tiles.
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
  return g;
}

int launch_gemm_pair(int mode, const void* a_mat, const void* packed, const PairGeometry& g, int M, int N, int K,
                     const void* scale, int scale_mode, int G, int group_slices, float scalar_scale, const void* bias,
                     const float* a_params, const int32_t* w_sum, void* y, int dst_layout, int* error,
                     cudaStream_t stream, const PeerOutputs* outs, const PairSplit* split) {
  if (g.shares_tiles && (split == nullptr || split->ws == nullptr || split->flags == nullptr || split->epoch == 0)) {
    set_last_error_text("this GEMM geometry shares tiles between SM pairs and needs a split workspace");
    return MLD_INVALID_ARGUMENT;
  }
  const int N4 = align_n(N, 4);
  const bool i8 = mode == kModeInt8I8 || mode == kModePreparedI8;
  const bool prepared = mode >= kModePreparedF16;
  const int esz = i8 ? 1 : 2;
  const int blk = mode == kModeInt4F16 ? 8 : 16;
  const int SS = div_up(K, 4), DS = N4 / 4;
  CUtensorMap ta, tw;
  int rc = make_tmap_2d(&ta, a_mat, (uint64_t)g.kp * esz, M, (uint64_t)g.kp * esz, kKBytes, kRowsPerCta, esz,
                        CU_TENSOR_MAP_SWIZZLE_128B, i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                        true);
  if (rc != MLD_OK) return rc;
  // packed weights: [K/4] rows of N4/4 blocks; the box is one stage's rows of the CTA's half of the tile
  if (prepared)  // K-major rows [N4][kp], boxes of one swizzle atom of K x the CTA's half of the tile's rows
    rc = make_tmap_2d(&tw, packed, (uint64_t)g.kp * esz, N4, (uint64_t)g.kp * esz, kKBytes, g.tile_n / 2, esz,
                      CU_TENSOR_MAP_SWIZZLE_128B,
                      i8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, true);
  else
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
  a.w_stages = g.w_stages;
  a.w_box_bytes = g.w_box_bytes;
  a.src_slices = SS;
  a.scale = scale_mode == MLD_SCALE_SCALAR ? nullptr : static_cast<const __half*>(scale);
  a.scale_mode = scale_mode;
  a.G = G;
  a.group_slices = group_slices;
  a.gs_shift = -1;
  for (int sh = 0; sh < 24; ++sh)
    if ((1 << sh) == group_slices) a.gs_shift = sh;
  a.scalar_scale = scalar_scale;
  a.bias = bias;
  a.a_params = a_params;
  a.w_sum = w_sum;
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
#ifdef MLD_TRACE
  a.trace = g_pair_trace;
  a.skip_transform = getenv("MLD_PAIR_SKIP_XF") != nullptr ? 1 : 0;
#endif
  void (*kern)(CUtensorMap, CUtensorMap, PairArgs) = nullptr;
  switch (mode) {
    case kModeInt4F16: kern = gemm_pair_kernel<kModeInt4F16>; break;
    case kModeInt8F16: kern = gemm_pair_kernel<kModeInt8F16>; break;
    case kModeInt8I8: kern = gemm_pair_kernel<kModeInt8I8>; break;
    case kModePreparedF16: kern = gemm_pair_kernel<kModePreparedF16>; break;
    case kModePreparedI8: kern = gemm_pair_kernel<kModePreparedI8>; break;
    default: set_last_error_text("bad GEMM mode"); return MLD_INVALID_ARGUMENT;
  }
  static bool configured[5][kMaxDevices];
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
  MLD_CUDA_CHECK(cudaLaunchKernelEx(&cfg, kern, ta, tw, a));
  count_launch();
  return MLD_OK;
}

}  // namespace mld
