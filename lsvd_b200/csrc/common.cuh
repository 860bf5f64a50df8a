// Shared device/host helpers for the sm_100a kernels: status plumbing, mbarrier and bulk-copy
// (TMA) wrappers with bounded waits, warp reductions.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <utility>

#include "../../include/lsvd_b200.h"

namespace lsvd {

// ---- host side -------------------------------------------------------------------------------
void set_last_cuda_error(cudaError_t e);

#define LSVD_CUDA_TRY(expr)                      \
  do {                                           \
    cudaError_t _e = (expr);                     \
    if (_e != cudaSuccess) {                     \
      ::lsvd::set_last_cuda_error(_e);           \
      return LSVD_ERR_CUDA;                      \
    }                                            \
  } while (0)

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

int device_sm_count();           // SM count of the current device (cached per device)
int device_max_smem_optin();     // opt-in shared memory per block of the current device
// Raise a kernel's dynamic shared memory limit on the current device (remembered, so repeated calls are free).
cudaError_t ensure_dynamic_smem(const void* kernel, int bytes);

// Kernels of one decode step run back to back on a stream, each a few microseconds long.  They are launched
// with programmatic stream serialisation: the next kernel's blocks may become resident while the previous
// kernel drains, and wait in grid_dependency_sync() (first statement of every such kernel) until the previous
// grid has completed and its writes are visible.  LSVD_CHAINED_LAUNCH=0 in the environment turns it off.
// The attention kernels use it.  On the FFN side only the mixffn quantisers and the products that ask for a weight
// prefetch do (LSVD_CHAIN_FFN=0 turns those off): for the other quantisers and products it measured faster at 1..32
// tokens (FFN block 52.5 / 56.8 instead of 56.9 / 59.2 us at 1 / 16 tokens) but slower at 64 tokens (143 instead of
// 117 us) and behind the attention kernels (167 instead of 153 us for attention + FFN).
bool chained_launch_enabled();
bool ffn_chain_enabled();

#ifdef __CUDACC__
template <typename... KArgs, typename... Args>
inline cudaError_t launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                  int cluster_x, bool chain, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (chain && chained_launch_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = static_cast<unsigned>(cluster_x);
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}
#endif

// ---- device side -----------------------------------------------------------------------------
#ifdef __CUDACC__

// Let the next kernel of the stream start becoming resident, then wait for the previous one to have completed
// (both are no-ops for a kernel launched without programmatic serialisation).
__device__ __forceinline__ void grid_dependency_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dependency_sync() {
  grid_dependency_release();
  grid_dependency_wait();
}

// Record the first error code seen by a kernel; later codes do not overwrite it.
__device__ __forceinline__ void report_status(int32_t* status_word, int code) {
  if (status_word != nullptr) atomicCAS(status_word, 0, code);
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// Wait for a phase of an mbarrier for at most kMbarTimeoutNs of wall time (and a hard cap on polls, in
// case the timer does not advance).  Returns false when the limit ran out; the caller must then stop
// using the pipeline and report LSVD_ERR_TIMEOUT.
constexpr uint64_t kMbarTimeoutNs = 2000000000ull;   // 2 s
constexpr uint32_t kMbarMaxPolls = 1u << 26;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = global_timer_ns();
  for (uint32_t i = 0; i < kMbarMaxPolls; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (global_timer_ns() - t0 > kMbarTimeoutNs) return false;
    __nanosleep(40);      // keep the issue slots for the warps that have work
  }
  return false;
}

// One-dimensional bulk copy global -> shared (TMA, no tensor map): 16-byte aligned addresses,
// size a multiple of 16; completion is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Named barrier `id` of `count` threads that also ORs a flag over them: every participant gets the same answer, so a
// decision to stop (a bounded wait that gave up somewhere) is taken by all of them or by none -- nobody is left
// waiting alone at the next barrier.
__device__ __forceinline__ bool named_barrier_or(int id, int count, bool flag) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\t"
      "barrier.red.or.pred q, %2, %3, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"(flag ? 1u : 0u), "r"(id), "r"(count)
      : "memory");
  return r != 0u;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Warp maximum of finite-or-minus-infinity floats through the integer redux unit: the key is
// monotonic in the float value.
__device__ __forceinline__ float warp_max_redux(float v) {
  int i = __float_as_int(v);
  int key = i ^ ((i >> 31) & 0x7fffffff);
  key = __reduce_max_sync(0xffffffffu, key);
  return __int_as_float(key ^ ((key >> 31) & 0x7fffffff));
}

// Sign-extended byte `idx` of a 32-bit word as a float, without the narrow integer conversions:
// one byte-permute with sign replication, one int32 -> fp32 conversion.
template <int kIdx>
__device__ __forceinline__ float s8_to_f32(uint32_t w) {
  constexpr uint32_t sel = (kIdx) | ((8u | kIdx) << 4) | ((8u | kIdx) << 8) | ((8u | kIdx) << 12);
  int v;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(v) : "r"(w), "r"(0u), "r"(sel));   // selector bit 3: replicate the sign
  return __int2float_rn(v);
}

#endif  // __CUDACC__

}  // namespace lsvd
