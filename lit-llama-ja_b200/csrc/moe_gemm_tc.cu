// Grouped expert GEMM of the mixture-of-experts feed-forward on the 5th-generation tensor cores
// (tcgen05 + TMEM + TMA), for steps with many rows per expert (prefill).
//
// The (token, choice) pairs are sorted by expert (ll_moe_route) and the rows of the activations are
// gathered into that order once (ll_moe_gather_rows), so every operand is a plain row-major matrix
// that TMA can tile:
//   mode 1 (GLU) : h[r][n] = glu(xs[r] . gate_e[n], xs[r] . up_e[n])     w [X][2N][K] = [gate; up]
//   mode 0 (down): y[perm[r]][n] = h[r] . down_e[n]                       w [X][N][K]
// for the sorted rows r of expert e.  A CTA owns 128 sorted rows of ONE expert (found from the device-side
// offsets, as in the mma.sync form: no host synchronisation) x 256 accumulator columns in TMEM:
//   GLU : columns 0..127 = gate tile, 128..255 = up tile of the same 128 outputs; the clamped gated unit is
//         the epilogue, applied to the two accumulators as they are read back from TMEM;
//   down: columns 0..255 = 256 outputs, scattered to (token, choice) order by the epilogue.
// A row tile may run past its expert's last row: those rows (the next expert's, or zero fill) are
// computed and never stored.
//   warp 0   : TMA producer (A box 128 x 64, two B boxes 128 x 64, 128-byte swizzle) into a 2-stage ring; two CTAs
//              share an SM (2 x 256 TMEM columns), so one CTA's first loads and epilogue run under the other's MMAs
//   warp 1   : TMEM allocation, one thread issues tcgen05.mma 128 x 256 x 16 (bf16 in, fp32 accumulate)
//   warps 2-5: epilogue, one accumulator row per thread
// Every wait on an mbarrier is bounded; a wait that runs out records a code in g_moe_tc_error, the roles
// stop, the CTA waits for its copies in flight (bounded), frees its TMEM and returns.
#include "tcgen05.cuh"

namespace llb {
namespace {

constexpr int MT_BN = 128;                 // rows of one B box
constexpr int MT_STAGES = 2;                 // two CTAs per SM: one CTA's prologue and epilogue run under the other's main loop
constexpr int MT_A_BYTES = BM * BK * 2, MT_B_BYTES = 2 * MT_BN * BK * 2;
constexpr int MT_TMEM_COLS = 256;
constexpr uint32_t MT_WAIT_LIMIT = 1u << 22;

__device__ int g_moe_tc_error = 0;

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int code) {
  for (uint32_t i = 0; i < MT_WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  atomicCAS(&g_moe_tc_error, 0, code);
  return false;
}

// 2-D tiled TMA load, default L2 policy (both operands are re-read by other CTAs through L2)
__device__ __forceinline__ void tma_box(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(dst)),
               "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}

template <int MODE>
__global__ void __launch_bounds__(192, 2) moe_gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a,
                                                             const __grid_constant__ CUtensorMap map_b,
                                                             const int32_t* __restrict__ offsets, const int32_t* __restrict__ perm,
                                                             int X, int N, int K, float limit, float alpha, float shift,
                                                             __nv_bfloat16* __restrict__ c, int ldc) {
  extern __shared__ __align__(1024) uint8_t smem[];
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem) + 1023) & ~(uintptr_t)1023);
  uint8_t* sa = base;                              // [STAGES][128][64] bf16, swizzled
  uint8_t* sb = base + MT_STAGES * MT_A_BYTES;     // [STAGES][256][64]
  uint64_t* full = reinterpret_cast<uint64_t*>(sb + MT_STAGES * MT_B_BYTES);
  uint64_t* empty = full + MT_STAGES;
  uint64_t* tmem_full = empty + MT_STAGES;
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(tmem_full + 1);
  int* s_tile = reinterpret_cast<int*>(tmem_ptr + 1);   // expert, first sorted row, rows of the expert in this tile
  int* s_fail = s_tile + 3;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0) grouped_tile_lookup(offsets, X, blockIdx.y, BM, s_tile);
  if (threadIdx.x == 32) *s_fail = 0;
  __syncthreads();
  if (s_tile[0] < 0) return;                       // before anything is allocated
  const int e = s_tile[0], r0 = s_tile[1], cnt = s_tile[2];
  const int n0 = blockIdx.x * (MODE == 1 ? MT_BN : 2 * MT_BN);
  // rows of the expert's weight matrix under the two B boxes
  const int brow0 = MODE == 1 ? e * 2 * N + n0 : e * N + n0;
  const int brow1 = MODE == 1 ? e * 2 * N + N + n0 : e * N + n0 + MT_BN;
  const int nkb = (K + BK - 1) / BK;

  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&map_a);
    prefetch_tensormap(&map_b);
    for (int i = 0; i < MT_STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(tmem_full, 1);
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(tmem_ptr, MT_TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_d = *tmem_ptr;

  if (warp == 0) {
    if (lane == 0) {
      int s = 0, issued = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait_bounded(&empty[s], phase ^ 1, 1)) { *s_fail = 1; break; }
        mbar_expect_tx(&full[s], MT_A_BYTES + MT_B_BYTES);
        tma_box(sa + s * MT_A_BYTES, &map_a, kb * BK, r0, &full[s]);
        tma_box(sb + s * MT_B_BYTES, &map_b, kb * BK, brow0, &full[s]);
        tma_box(sb + s * MT_B_BYTES + MT_BN * BK * 2, &map_b, kb * BK, brow1, &full[s]);
        ++issued;
        if (++s == MT_STAGES) { s = 0; phase ^= 1u; }
      }
      if (*s_fail && issued > 0) {   // give the copies already issued time to land before the CTA leaves
        for (int w = 0; w < 2048; ++w) __nanosleep(512);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = instr_desc_bf16(BM, 2 * MT_BN);
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait_bounded(&full[s], phase, 2)) { *s_fail = 1; ok = false; break; }
        tc_fence_after();
        const uint64_t adesc = smem_desc_sw128(smem_u32(sa + s * MT_A_BYTES));
        const uint64_t bdesc = smem_desc_sw128(smem_u32(sb + s * MT_B_BYTES));
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_bf16(tmem_d, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k), idesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit(&empty[s]);
        if (++s == MT_STAGES) { s = 0; phase ^= 1u; }
      }
      (void)ok;
      umma_commit(tmem_full);       // also on the failure path: the epilogue's wait ends
    }
  } else {
    const int quarter = warp & 3;   // a warp may only touch TMEM lanes [32 * (warp % 4), +32)
    const int rt = quarter * 32 + lane;
    const bool waited = mbar_wait_bounded(tmem_full, 0, 3);
    tc_fence_after();
    if (waited && *s_fail == 0) {
      const bool row_ok = rt < cnt;
      long long dst_row = 0;
      if (row_ok) dst_row = MODE == 1 ? (long long)(r0 + rt) : (long long)perm[r0 + rt];
      __nv_bfloat16* dst = c + dst_row * ldc;
      const uint32_t trow = tmem_d + ((uint32_t)(quarter * 32) << 16);
      constexpr int NCOL = MODE == 1 ? MT_BN : 2 * MT_BN;
#pragma unroll 1
      for (int c0 = 0; c0 < NCOL; c0 += 32) {
        if (n0 + c0 >= N) break;            // uniform over the CTA
        uint32_t v[32];
        tmem_ld_32x32(trow + (uint32_t)c0, v);
        float f[32];
        if (MODE == 1) {
          uint32_t u[32];
          tmem_ld_32x32(trow + (uint32_t)(MT_BN + c0), u);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float g = fminf(__uint_as_float(v[j]), limit);
            const float up = fminf(fmaxf(__uint_as_float(u[j]), -limit), limit);
            f[j] = g / (1.f + expf(-alpha * g)) * (up + shift);
          }
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
        }
        if (!row_ok) continue;
        const int col = n0 + c0;
        if (col + 32 <= N && (ldc & 7) == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t pk[4];
#pragma unroll
            for (int q = 0; q < 4; ++q)
              pk[q] = (uint32_t)f32_to_bf16_bits(f[j * 8 + 2 * q]) | ((uint32_t)f32_to_bf16_bits(f[j * 8 + 2 * q + 1]) << 16);
            *reinterpret_cast<uint4*>(dst + col + j * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
          }
        } else {
          for (int j = 0; j < 32 && col + j < N; ++j) dst[col + j] = __float2bfloat16_rn(f[j]);
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_d, MT_TMEM_COLS);
  }
}

// xs[r][:] = x[perm[r] / top][:] for the sorted rows r (16-byte pieces)
__global__ void moe_gather_rows_kernel(const uint4* __restrict__ x, long long ldx16, const int32_t* __restrict__ perm, int top,
                                       uint4* __restrict__ out, int k16) {
  const int r = blockIdx.x;
  const uint4* src = x + (long long)(perm[r] / top) * ldx16;
  uint4* dst = out + (long long)r * k16;
  for (int i = threadIdx.x; i < k16; i += blockDim.x) dst[i] = src[i];
}

template <int MODE>
int launch_moe_tc(const CUtensorMap& ma, const CUtensorMap& mb, const int32_t* offsets, const int32_t* perm, int X, int N, int K,
                  float limit, float alpha, float shift, void* c, int ldc, int n_rows, cudaStream_t st) {
  constexpr size_t smem = (size_t)MT_STAGES * (MT_A_BYTES + MT_B_BYTES) + (2 * MT_STAGES + 1) * 8 + 32 + 1024;
  static bool configured = false;
  if (!configured) {
    LL_CUDA(cudaFuncSetAttribute(moe_gemm_tc_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured = true;
  }
  const int ncols = MODE == 1 ? MT_BN : 2 * MT_BN;
  dim3 grid((N + ncols - 1) / ncols, (n_rows + BM - 1) / BM + X);
  moe_gemm_tc_kernel<MODE><<<grid, 192, smem, st>>>(ma, mb, offsets, perm, X, N, K, limit, alpha, shift, (__nv_bfloat16*)c, ldc);
  LL_LAUNCH_OK("moe_gemm_tc_kernel");
  return LL_OK;
}

}  // namespace
}  // namespace llb

using namespace llb;

extern "C" {

int ll_moe_gather_rows(const void* x, int ldx, const int32_t* perm, int top, int n_rows, int K, void* out, ll_stream stream) {
  LL_CHECK_ARG(x && perm && out && top > 0 && n_rows >= 0 && K > 0, "bad moe_gather_rows arguments");
  LL_CHECK_ARG(K % 8 == 0 && ldx % 8 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)out & 15) == 0,
               "moe_gather_rows: rows must be 16-byte aligned bf16");
  if (n_rows == 0) return LL_OK;
  moe_gather_rows_kernel<<<n_rows, K / 8 >= 256 ? 256 : 128, 0, (cudaStream_t)stream>>>((const uint4*)x, ldx / 8, perm, top, (uint4*)out,
                                                                                     K / 8);
  LL_LAUNCH_OK("moe_gather_rows_kernel");
  return LL_OK;
}

int ll_moe_grouped_gemm_tc(const void* a, const void* w, const int32_t* offsets, const int32_t* perm, int mode, int n_rows,
                           int n_experts, int N, int K, float limit, float alpha, void* c, int ldc, ll_stream stream) {
  LL_CHECK_ARG(a && w && offsets && perm && c, "moe_grouped_gemm_tc: null pointer");
  LL_CHECK_ARG(n_rows >= 0 && n_experts > 0 && N > 0 && K > 0 && ldc >= N && mode >= 0 && mode <= 2, "bad moe_grouped_gemm_tc arguments");
  const float shift = mode == 2 ? 0.f : 1.f;     // mode 2: the up branch enters as it is
  if (mode == 2) mode = 1;
  LL_CHECK_ARG(K % 8 == 0 && ((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0 && ((uintptr_t)c & 15) == 0,
               "moe_grouped_gemm_tc: K must be a multiple of 8 and the operands 16-byte aligned (TMA rows)");
  if (n_rows == 0) return LL_OK;
  const long long wrows = (long long)n_experts * (mode == 1 ? 2 : 1) * N;
  LL_CHECK_ARG(wrows < (1ll << 31), "moe_grouped_gemm_tc: weight stack too tall for one tensor map");
  CUtensorMap ma, mb;
  if (int r = make_map(a, n_rows, K, BM, &ma)) return r;
  if (int r = make_map(w, (int)wrows, K, MT_BN, &mb)) return r;
  cudaStream_t st = (cudaStream_t)stream;
  if (mode == 1) return launch_moe_tc<1>(ma, mb, offsets, perm, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st);
  return launch_moe_tc<0>(ma, mb, offsets, perm, n_experts, N, K, limit, alpha, shift, c, ldc, n_rows, st);
}

// 0, or the code of the first bounded wait that ran out in a kernel of this file (1: ring slot, 2: operands, 3: accumulator).
// Synchronises the device.
int ll_moe_tc_error(void) {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_moe_tc_error, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // extern "C"
