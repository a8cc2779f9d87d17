// Shared device/host helpers for the llb200 C-ABI library (sm_100a only).
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "../../include/llb200.h"

namespace llb {

// ------------------------------------------------------------------ host error plumbing
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);

#define LL_CHECK_ARG(cond, ...)                    \
  do {                                             \
    if (!(cond)) {                                 \
      llb::set_error(__VA_ARGS__);                 \
      return LL_ERR_ARG;                           \
    }                                              \
  } while (0)

#define LL_CUDA(expr)                              \
  do {                                             \
    cudaError_t _e = (expr);                       \
    if (_e != cudaSuccess) return llb::cuda_fail(_e, #expr); \
  } while (0)

#define LL_LAUNCH_OK(name)                         \
  do {                                             \
    cudaError_t _e = cudaGetLastError();           \
    if (_e != cudaSuccess) return llb::cuda_fail(_e, name); \
  } while (0)

int sm_count();

// ------------------------------------------------------------------ small device helpers
__device__ __forceinline__ float bf16_bits_to_f32(uint32_t b) { return __uint_as_float(b << 16); }
__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float x) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(x));
}

template <typename T> struct dt;
template <> struct dt<float> {
  static __device__ __forceinline__ float ld(const float* p, size_t i) { return p[i]; }
  static __device__ __forceinline__ void st(float* p, size_t i, float v) { p[i] = v; }
  static __device__ __forceinline__ float rd(float v) { return v; }
};
template <> struct dt<__nv_bfloat16> {
  static __device__ __forceinline__ float ld(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }
  static __device__ __forceinline__ void st(__nv_bfloat16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float rd(float v) { return bf16r(v); }
};
template <> struct dt<__half> {
  static __device__ __forceinline__ float ld(const __half* p, size_t i) { return __half2float(p[i]); }
  static __device__ __forceinline__ void st(__half* p, size_t i, float v) { p[i] = __float2half_rn(v); }
  static __device__ __forceinline__ float rd(float v) { return __half2float(__float2half_rn(v)); }
};

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

// Row tile `t` of a grouped problem whose groups are the segments offsets[g] .. offsets[g + 1] of a sorted row space, every
// group cut into tiles of `bm` rows: which group, its first row, and how many of the tile's rows belong to the group.
// Called by one whole warp; 32 groups are examined per pass (two loads per lane in flight, a shuffle scan of the tile
// counts), so the lookup costs a couple of memory round trips instead of one per group.  Lane 0 writes out[0..2] =
// (group or -1 when t is past the last tile, first row, rows).
__device__ __forceinline__ void grouped_tile_lookup(const int32_t* __restrict__ offsets, int n_groups, int t, int bm, int* out) {
  const int lane = threadIdx.x & 31;
  int before = 0;
  bool found = false;
  for (int g0 = 0; g0 < n_groups && !found; g0 += 32) {
    const int g = g0 + lane;
    const int o0 = g < n_groups ? offsets[g] : 0, o1 = g < n_groups ? offsets[g + 1] : 0;
    const int tiles = (o1 - o0 + bm - 1) / bm;
    int incl = tiles;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, d);
      if (lane >= d) incl += v;
    }
    const int excl = before + incl - tiles;
    const bool mine = g < n_groups && t >= excl && t < excl + tiles;
    const unsigned ball = __ballot_sync(0xffffffffu, mine);
    if (ball != 0u) {
      found = true;
      if (mine) {
        const int r0 = o0 + (t - excl) * bm;
        out[0] = g;
        out[1] = r0;
        out[2] = min(bm, o1 - r0);
      }
    }
    before += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (!found && lane == 0) out[0] = -1;
}

// ------------------------------------------------------------------ PTX: mbarrier / TMA / PDL
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ void mbar_wait(uint64_t* bar, uint32_t parity) {
  while (!mbar_try_wait(bar, parity)) {
  }
}
// 2-D tiled TMA load (global -> shared), completion on an mbarrier, with an L2 cache hint.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar,
                                            uint64_t cache_hint) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(dst)),
      "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(cache_hint)
      : "memory");
}
// 1-D bulk copy (global -> shared), size multiple of 16 B, 16 B aligned both sides.
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// L2 eviction policies for streamed-once data (weights) and reused data.
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
// Programmatic dependent launch: let the next kernel in the stream start its prologue /
// wait until every kernel this one depends on has completed and flushed.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}

// D(16x8,f32) += A(16x16,bf16,row) * B(16x8,bf16,col)
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Every kernel of the decode chain asks for the maximum shared-memory carve-out: an SM cannot change its
// L1/shared split while a CTA is resident, so under programmatic dependent launch a kernel that prefers
// a different split than its (co-resident) predecessor waits for the SM to drain - measured: +12 us per
// c_proj -> fc edge, +25 us per block, when the chain started on a small-smem kernel.
template <typename F>
inline void prefer_max_smem(F* kernel) {
  cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// Launch helper: optional programmatic-stream-serialization attribute (PDL).
template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool pdl,
                          Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

}  // namespace llb
