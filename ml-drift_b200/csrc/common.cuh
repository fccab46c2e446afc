// Shared helpers for the mldfc CUDA sources: status plumbing, launch
// accounting, and thin wrappers over the sm_100a PTX this library uses
// (mbarrier, TMA bulk-tensor copies, tcgen05).
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mldfc.h"

namespace mld {

// ---------------------------------------------------------------- host side
void set_last_error(const char* what, cudaError_t err);
void set_last_error_text(const char* what);
void count_launch(int n = 1);

#define MLD_CUDA_CHECK(expr)                         \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) {                         \
      ::mld::set_last_error(#expr, _e);              \
      return MLD_CUDA_ERROR;                         \
    }                                                \
  } while (0)

// Checks the launch that has just been enqueued.
#define MLD_LAUNCH_CHECK()                           \
  do {                                               \
    ::mld::count_launch();                           \
    MLD_CUDA_CHECK(cudaGetLastError());              \
  } while (0)

#define MLD_REQUIRE(cond, msg)                       \
  do {                                               \
    if (!(cond)) {                                   \
      ::mld::set_last_error_text(msg);               \
      return MLD_INVALID_ARGUMENT;                   \
    }                                                \
  } while (0)

static inline int div_up(int a, int b) { return (a + b - 1) / b; }
static inline int64_t div_up64(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline int align_n(int a, int n) { return div_up(a, n) * n; }

int sm_count(int device);

// Function attributes such as the dynamic shared-memory limit are per device: a kernel is configured
// once on every device it is launched on.  `done` is a zero-initialised table owned by the caller (one
// per kernel instantiation); returns true when the current device still needs the attribute set.
constexpr int kMaxDevices = 64;
inline bool needs_configure(bool (&done)[kMaxDevices], int* device_out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
    *device_out = -1;
    return true;  // unknown device: set the attribute every time
  }
  *device_out = dev;
  return !done[dev];
}

// cuTensorMapEncodeTiled fetched through the runtime (no libcuda link).
typedef CUresult (*encode_tiled_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_tiled_fn get_encode_tiled();

// 2-D tiled tensor map over a row-major byte matrix: `rows` rows of
// `row_bytes` bytes with pitch `pitch_bytes`; box = box_rows x box_bytes.
// elem_bytes selects the element type used to express the inner dimension
// (1, 2 or 4); swizzle is a CUtensorMapSwizzle value.
int make_tmap_2d(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows,
                 uint64_t pitch_bytes, uint32_t box_bytes, uint32_t box_rows, int elem_bytes,
                 CUtensorMapSwizzle swizzle, CUtensorMapDataType dtype_override = CU_TENSOR_MAP_DATA_TYPE_UINT8,
                 bool use_override = false);

// -------------------------------------------------------------- device side
#ifdef __CUDACC__

// Upper bound on any device-side wait.  A wait that runs out records an error
// code and the kernel drains and returns; nothing spins forever.
constexpr unsigned long long kWaitLimitNs = 2000ull * 1000ull * 1000ull;

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint64_t* bar) {
  asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the time limit ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i) {
      if (mbar_try_wait(bar, parity)) return true;
    }
    if (globaltimer_ns() - t0 > kWaitLimitNs) return false;
  }
}

// TMA: 2-D tiled load global -> shared, completion on an mbarrier.
// c0 = inner coordinate (elements of the map's type), c1 = row.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
// Same with an L2 cache-policy operand (used to mark streamed weights evict-first).
__device__ __forceinline__ void tma_load_2d_hint(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0,
                                                 int c1, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
      "[%0], [%1, {%3, %4}], [%2], %5;"
      ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
      "l"(policy)
      : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// Untiled bulk copy global -> shared (both 16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_load_1d(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}
// Fire-and-forget request to bring [gsrc, gsrc + bytes) into L2 (16-byte aligned, size % 16 == 0).
__device__ __forceinline__ void bulk_prefetch_l2(const void* gsrc, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(gsrc), "r"(bytes) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until every rank's flag has reached `seq`; false when the time limit ran out.
__device__ __forceinline__ bool wait_peer_flags(const unsigned* flags, int world, unsigned seq,
                                                unsigned long long limit_ns) {
  const unsigned long long t0 = globaltimer_ns();
  for (int r = 0; r < world; ++r) {
    while (static_cast<int>(ld_acquire_sys(flags + r) - seq) < 0) {
      if (globaltimer_ns() - t0 > limit_ns) return false;
    }
  }
  return true;
}

// Programmatic dependent launch: wait for the preceding kernel's memory, and
// allow the following kernel to start its prologue.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Host side of the same: launches `kern` so that it may become resident while the kernel before it on the stream
// is still running.  Every kernel launched this way calls pdl_wait() before its first access to global memory.
template <typename... Params, typename... Args>
inline cudaError_t launch_overlapped(void (*kern)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<Params>(args)...);
}

#endif  // __CUDACC__

}  // namespace mld
