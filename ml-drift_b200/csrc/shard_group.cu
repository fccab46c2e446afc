// A FullyConnected node split by output channels over the GPUs of one node,
// with the gather of the shard outputs.
//
// Output channels are independent dot products
// (ml_drift/common/task/testing_ref_ops.cc:961-988), so rank r computes the
// rows [r N/G, (r+1) N/G) from its own packed sub-matrix.  In the reference's
// sliced output layout [N/4][tokens][4] a rank's block is one contiguous range,
// so the gathered tensor is the concatenation of the blocks in rank order.  Two
// ways to assemble it on every rank:
//   NCCL         every rank computes into its own range, then one in-place
//                ncclAllGather;
//   peer stores  the prefill GEMM's epilogue stores each output tile into
//                every rank's tensor as it leaves tensor memory (plain stores
//                over NVLink), so the transfer runs under the remaining tiles'
//                math; a small kernel then tells the peers "my block is
//                complete" and waits (bounded) for theirs.
// The reference is single-device; this file has no counterpart there.
#include <cuda_fp16.h>

#include <cstring>

#include "common.cuh"
#include "kernels.h"
#include "nccl_lazy.h"

namespace mld {
namespace {

// Block -> every peer's tensor, for the routes whose kernels do not store remotely themselves.
__global__ void __launch_bounds__(256) scatter_block_kernel(const uint2* __restrict__ src, PeerOutputs outs, int rank,
                                                            size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    const uint2 v = src[i];
    for (int pr = 0; pr < outs.world; ++pr)
      if (pr != rank) static_cast<uint2*>(outs.y[pr])[i] = v;
  }
  __threadfence_system();
}

// Tells every rank "I have reached this point of step s" and waits until every rank has said so.  Used twice
// per run: before the remote stores ("I am done reading the previous gathered tensor: you may overwrite my
// copy") and after them ("my block has been delivered everywhere").  One warp; lane r watches rank r.  The
// step number comes from a device counter, so a replayed CUDA graph produces fresh values.
struct SignalArgs {
  int world, rank;
  unsigned* step;            // local counter
  unsigned* flag_peers[8];   // this rank's flag in every rank's block
  const unsigned* flags;     // local flags, one per rank
  int* error;
  unsigned long long limit_ns;
};
__global__ void __launch_bounds__(32) signal_and_wait_kernel(SignalArgs a) {
  unsigned seq = 0;
  if (threadIdx.x == 0) {
    seq = *a.step + 1;
    *a.step = seq;
    __threadfence_system();  // everything this GPU wrote before (the kernels ahead in the stream) is performed
  }
  seq = __shfl_sync(0xffffffffu, seq, 0);
  if (static_cast<int>(threadIdx.x) < a.world) st_release_sys(a.flag_peers[threadIdx.x], seq);
  if (static_cast<int>(threadIdx.x) < a.world) {
    const unsigned long long t0 = globaltimer_ns();
    while (static_cast<int>(ld_acquire_sys(a.flags + threadIdx.x) - seq) < 0) {
      if (globaltimer_ns() - t0 > a.limit_ns) {
        atomicExch(a.error, kErrPeerWait);
        break;
      }
    }
  }
}

}  // namespace
}  // namespace mld

using namespace mld;

struct mld_shard_group {
  int rank, world, device;
  size_t output_bytes, block_bytes;   // block = output + flags + counters
  uint8_t* block;                     // [output | flags (8 x u32) | step | error]
  uint8_t* peers[8];
  bool peers_ready;
  ncclComm_t comm;
  unsigned long long limit_ns;
  size_t off_flags, off_step, off_error;   // flags: [2 rounds][8 ranks] u32; step: [2] u32
};

static int handshake(mld_shard_group* g, int round, cudaStream_t stream) {
  SignalArgs sa;
  memset(&sa, 0, sizeof sa);
  sa.world = g->world;
  sa.rank = g->rank;
  sa.step = reinterpret_cast<unsigned*>(g->block + g->off_step) + round;
  for (int r = 0; r < g->world; ++r)
    sa.flag_peers[r] = reinterpret_cast<unsigned*>(g->peers[r] + g->off_flags) + round * 8 + g->rank;
  sa.flags = reinterpret_cast<const unsigned*>(g->block + g->off_flags) + round * 8;
  sa.error = reinterpret_cast<int*>(g->block + g->off_error);
  sa.limit_ns = g->limit_ns;
  signal_and_wait_kernel<<<1, 32, 0, stream>>>(sa);
  MLD_LAUNCH_CHECK();
  return MLD_OK;
}

extern "C" {

int mld_shard_group_create(int32_t rank, int32_t world, int32_t device, size_t output_bytes, const void* nccl_id128,
                           mld_shard_group** out) {
  MLD_REQUIRE(out != nullptr, "null argument");
  *out = nullptr;
  MLD_REQUIRE(world >= 1 && world <= 8 && rank >= 0 && rank < world, "bad rank/world");
  MLD_REQUIRE(output_bytes > 0 && output_bytes % 16 == 0, "output_bytes must be a positive multiple of 16");
  if (device < 0) MLD_CUDA_CHECK(cudaGetDevice(&device));
  MLD_CUDA_CHECK(cudaSetDevice(device));
  mld_shard_group* g = new mld_shard_group();
  g->rank = rank;
  g->world = world;
  g->device = device;
  g->output_bytes = output_bytes;
  g->off_flags = (output_bytes + 255) & ~size_t(255);
  g->off_step = g->off_flags + 64;
  g->off_error = g->off_flags + 128;
  g->block_bytes = g->off_flags + 256;
  g->block = nullptr;
  for (int r = 0; r < 8; ++r) g->peers[r] = nullptr;
  g->peers_ready = world == 1;
  g->comm = nullptr;
  g->limit_ns = 2000ull * 1000ull * 1000ull;
  if (cudaMalloc(&g->block, g->block_bytes) != cudaSuccess) {
    set_last_error_text("shard group: device allocation failed");
    delete g;
    return MLD_CUDA_ERROR;
  }
  cudaMemset(g->block + g->off_flags, 0, 256);
  g->peers[rank] = g->block;
  if (world > 1 && nccl_id128 != nullptr) {
    if (!nccl().load()) {
      set_last_error_text("libnccl.so.2 could not be loaded");
      mld_shard_group_destroy(g);
      return MLD_NCCL_ERROR;
    }
    ncclUniqueId id;
    memcpy(&id, nccl_id128, sizeof id);
    const int nrc = nccl().CommInitRank(&g->comm, world, id, rank);
    if (nrc != 0) {
      set_last_error_text(nccl().GetErrorString ? nccl().GetErrorString(nrc) : "ncclCommInitRank failed");
      g->comm = nullptr;
      mld_shard_group_destroy(g);
      return MLD_NCCL_ERROR;
    }
  }
  *out = g;
  return MLD_OK;
}

int mld_shard_group_destroy(mld_shard_group* g) {
  if (g == nullptr) return MLD_OK;
  if (g->comm != nullptr && nccl().CommDestroy) nccl().CommDestroy(g->comm);
  for (int r = 0; r < 8; ++r)
    if (g->peers[r] != nullptr && g->peers[r] != g->block) cudaIpcCloseMemHandle(g->peers[r]);
  if (g->block != nullptr) cudaFree(g->block);
  delete g;
  return MLD_OK;
}

int mld_shard_group_ipc_export(mld_shard_group* g, void* handle64) {
  MLD_REQUIRE(g != nullptr && handle64 != nullptr, "null argument");
  cudaIpcMemHandle_t h;
  MLD_CUDA_CHECK(cudaIpcGetMemHandle(&h, g->block));
  memcpy(handle64, &h, sizeof h);
  return MLD_OK;
}

int mld_shard_group_ipc_import(mld_shard_group* g, const void* handles) {
  MLD_REQUIRE(g != nullptr && handles != nullptr, "null argument");
  MLD_CUDA_CHECK(cudaSetDevice(g->device));
  for (int r = 0; r < g->world; ++r) {
    if (r == g->rank) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, static_cast<const uint8_t*>(handles) + (size_t)r * 64, sizeof h);
    void* p = nullptr;
    MLD_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    g->peers[r] = static_cast<uint8_t*>(p);
  }
  g->peers_ready = true;
  return MLD_OK;
}

void* mld_shard_group_output(mld_shard_group* g) { return g != nullptr ? g->block : nullptr; }

int mld_shard_group_device_status(mld_shard_group* g, int32_t* code) {
  MLD_REQUIRE(g != nullptr && code != nullptr, "null argument");
  int c = 0;
  MLD_CUDA_CHECK(cudaMemcpy(&c, g->block + g->off_error, sizeof(int), cudaMemcpyDeviceToHost));
  *code = c;
  if (c != 0) {
    MLD_CUDA_CHECK(cudaMemset(g->block + g->off_error, 0, sizeof(int)));
    set_last_error_text("a rank's block did not arrive within the wait limit");
    return MLD_TIMEOUT;
  }
  return MLD_OK;
}

int mld_fc_run_sharded(mld_fc_plan* plan, mld_shard_group* g, const void* src, const void* weights, const void* scale,
                       const void* zero_point, const void* bias, int32_t tokens, int32_t gather, void* stream_v) {
  MLD_REQUIRE(plan != nullptr && g != nullptr, "null argument");
  MLD_REQUIRE(gather == MLD_GATHER_NCCL || gather == MLD_GATHER_PEER_STORES, "bad gather mode");
  int n = 0, dst_layout = 0, max_tokens = 0, device = 0;
  fc_plan_shape(plan, &n, &dst_layout, &max_tokens, &device);
  MLD_REQUIRE(device == g->device, "plan and shard group live on different devices");
  MLD_REQUIRE(dst_layout == MLD_LAYOUT_SLICED, "a sharded operator writes the sliced layout (its block is contiguous there)");
  MLD_REQUIRE(n % 4 == 0, "the shard's output channels must be a multiple of 4");
  MLD_REQUIRE(tokens >= 0 && tokens <= max_tokens, "tokens exceeds the plan's max_tokens");
  if (tokens == 0) return MLD_OK;
  const size_t block_bytes = (size_t)n * tokens * sizeof(__half);
  MLD_REQUIRE(block_bytes * g->world <= g->output_bytes, "the gathered tensor does not fit the group's output buffer");
  cudaStream_t stream = static_cast<cudaStream_t>(stream_v);
  uint8_t* mine = g->block + (size_t)g->rank * block_bytes;
  if (g->world == 1) return fc_run_internal(plan, src, weights, scale, zero_point, bias, mine, tokens, stream_v, nullptr, nullptr);
  if (gather == MLD_GATHER_NCCL) {
    MLD_REQUIRE(g->comm != nullptr, "this shard group was created without an NCCL id");
    int rc = fc_run_internal(plan, src, weights, scale, zero_point, bias, mine, tokens, stream_v, nullptr, nullptr);
    if (rc != MLD_OK) return rc;
    const int nrc = nccl().AllGather(mine, g->block, block_bytes / sizeof(__half), kNcclHalf, g->comm, stream);
    if (nrc != 0) {
      set_last_error_text(nccl().GetErrorString ? nccl().GetErrorString(nrc) : "ncclAllGather failed");
      return MLD_NCCL_ERROR;
    }
    return MLD_OK;
  }
  MLD_REQUIRE(g->peers_ready, "exchange blocks not imported yet (mld_shard_group_ipc_import)");
  PeerOutputs outs;
  memset(&outs, 0, sizeof outs);
  outs.world = g->world;
  for (int r = 0; r < g->world; ++r) outs.y[r] = g->peers[r] + (size_t)g->rank * block_bytes;
  // nobody's tensor is overwritten before its owner has reached this run (its stream is past whatever read
  // the previous gathered tensor)
  int rc = handshake(g, 0, stream);
  if (rc != MLD_OK) return rc;
  bool stored_remotely = false;
  rc = fc_run_internal(plan, src, weights, scale, zero_point, bias, mine, tokens, stream_v, nullptr, nullptr, &outs,
                           &stored_remotely);
  if (rc != MLD_OK) return rc;
  if (!stored_remotely) {
    const size_t n8 = block_bytes / 8;
    const int blocks = static_cast<int>(n8 / 256 < 1184 ? (n8 + 255) / 256 : 1184);
    scatter_block_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const uint2*>(mine), outs, g->rank, n8);
    MLD_LAUNCH_CHECK();
  }
  return handshake(g, 1, stream);
}

}  // extern "C"
