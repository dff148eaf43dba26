// Tensor-core GEMM for prompts: C[M, N] = A[M, K] * W[N, K]^T, bfloat16 in, float32 accumulation
// in TMEM, on the 5th-generation tensor cores (tcgen05.mma, cta_group::1).
//
// One block computes a 128 x 128 tile of C. Roles by warp:
//   warp 0      TMA producer: A and W tiles of 128 rows x 64 k (128-byte swizzle) into a ring of
//               kStages stages; a stage's `full` barrier counts the bytes that have landed
//   warp 1      allocates TMEM, then one elected lane issues the MMAs (four K = 16 steps per stage)
//               and commits them to the stage's `empty` barrier, and to `accum_full` at the end
//   warps 2..5  epilogue: tcgen05.ld of the accumulator (warp w owns TMEM lanes 32 * (w % 4) ..),
//               conversion, store
// Every wait is bounded; a wait that gives up records a status, raises the block's abort flag,
// and the block still frees its TMEM and returns.
//
// The reference leaves these products to nn.Linear (src/model.py:17-19,34-37,137).
#include "tcgen05.cuh"

namespace llmie {
using namespace tc;

constexpr int kBM = 128, kBN = 128, kBK = 64, kStages = 4;
constexpr int kTileBytes = kBM * kBK * 2;                    // 16 KB per operand tile
constexpr int kGemmThreads = 192;
constexpr int kGemmSmem = 2 * kStages * kTileBytes + 1024;   // + alignment slack

struct GemmShared {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t accum_full;
  uint32_t tmem_base;
  int abort;
};

template <typename OutT>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w,
               OutT* __restrict__ C, int M, int N, int K, int ldc, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ GemmShared sh;
  uint8_t* tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_tiles = tiles;
  uint8_t* w_tiles = tiles + kStages * kTileBytes;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.y * kBM, n0 = blockIdx.x * kBN;
  const int k_tiles = (K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    mbar_init(&sh.accum_full, 1);
    sh.abort = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, kBN);          // 128 columns of float32 for the 128 x 128 accumulator
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  volatile int* abort = &sh.abort;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&map_a);
      tma_prefetch_desc(&map_w);
      int issued = 0;
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % kStages;
        if (kt >= kStages && !mbar_wait(&sh.empty[s], ((kt / kStages) - 1) & 1, abort)) {
          if (!*abort) { *abort = 1; atomicExch(status, kStatusTimeoutEmpty); }
          break;
        }
        mbar_arrive_expect_tx(&sh.full[s], 2 * kTileBytes);
        tma_load_2d(a_tiles + s * kTileBytes, &map_a, kt * kBK, m0, &sh.full[s]);
        tma_load_2d(w_tiles + s * kTileBytes, &map_w, kt * kBK, n0, &sh.full[s]);
        issued = kt + 1;
      }
      if (*abort) {
        // the block is winding down: let this thread's own copies land (bounded) before the
        // shared memory they write to is given up
        for (int kt = max(0, issued - kStages); kt < issued; ++kt) {
          uint64_t* bar = &sh.full[kt % kStages];
          for (unsigned spin = 0; spin < (1u << 16) && !mbar_test(bar, (kt / kStages) & 1); ++spin) __nanosleep(64);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_instr_desc_bf16(kBM, kBN, 0, 0);
      for (int kt = 0; kt < k_tiles; ++kt) {
        const int s = kt % kStages;
        if (!mbar_wait(&sh.full[s], (kt / kStages) & 1, abort)) {
          if (!*abort) { *abort = 1; atomicExch(status, kStatusTimeoutFull); }
          break;
        }
        tc_fence_after_sync();
        const uint32_t a_addr = smem_u32(a_tiles + s * kTileBytes);
        const uint32_t w_addr = smem_u32(w_tiles + s * kTileBytes);
#pragma unroll
        for (int kk = 0; kk < kBK / 16; ++kk) {
          const uint64_t da = make_smem_desc(a_addr + kk * 32, 16, 1024);
          const uint64_t dw = make_smem_desc(w_addr + kk * 32, 16, 1024);
          mma_bf16_ss(tmem, da, dw, idesc, (kt > 0 || kk > 0) ? 1u : 0u);
        }
        mma_commit(&sh.empty[s]);              // the stage is free once these MMAs have read it
      }
      mma_commit(&sh.accum_full);
    }
  } else {
    const int quarter = warp & 3;               // TMEM lanes this warp may read
    // the whole warp decides together: tcgen05.ld is a warp-wide instruction
    const bool ok = __all_sync(0xffffffffu, mbar_wait(&sh.accum_full, 0, abort));
    if (!ok && !*abort) { *abort = 1; atomicExch(status, kStatusTimeoutMma); }
    tc_fence_after_sync();
    const int row = m0 + quarter * 32 + lane;
    if (ok) {
#pragma unroll 1
      for (int c0 = 0; c0 < kBN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, r);
        tmem_ld_wait();
        if (row < M) {
          OutT* dst = C + (size_t)row * ldc + n0 + c0;
          if (n0 + c0 + 32 <= N) {
            if (sizeof(OutT) == 2) {
#pragma unroll
              for (int i = 0; i < 32; i += 8) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __uint_as_float(r[i + e]);
                store8(reinterpret_cast<__nv_bfloat16*>(dst) + i, v);
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; i += 4)
                *reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + i) =
                    make_float4(__uint_as_float(r[i]), __uint_as_float(r[i + 1]), __uint_as_float(r[i + 2]),
                                __uint_as_float(r[i + 3]));
            }
          } else {
            for (int i = 0; i < 32 && n0 + c0 + i < N; ++i) dst[i] = from_f32<OutT>(__uint_as_float(r[i]));
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, kBN);
  }
}

// The give-up path of the bounded waits, on its own: one block sets up what the GEMM block sets up (an
// mbarrier, a TMEM allocation), then one thread waits, for at most `limit` polls, on a barrier at which
// nothing ever arrives. The wait returns false, the thread records kStatusTimeoutFull and raises the abort
// flag as the GEMM's roles do, and the block frees its TMEM and returns. It ends within microseconds.
__global__ void __launch_bounds__(64, 1) wait_probe_kernel(int* __restrict__ status, unsigned limit) {
  __shared__ GemmShared sh;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    mbar_init(&sh.full[0], 1);
    sh.abort = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, 32);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  volatile int* abort = &sh.abort;
  if (warp == 0 && elect_one()) {
    if (!mbar_wait(&sh.full[0], 0, abort, limit)) {
      if (!*abort) { *abort = 1; atomicExch(status, kStatusTimeoutFull); }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(sh.tmem_base, 32);
  }
}

}  // namespace llmie

using namespace llmie;

// Runs the give-up path of a bounded wait once (see wait_probe_kernel): afterwards *status holds the code of
// a load that did not arrive. limit: polls before the wait gives up, 1 .. 2^20.
extern "C" int llmie_tc_wait_probe(int* status, int limit, cudaStream_t stream) {
  if (!status || limit < 1 || limit > (1 << 20)) return LLMIE_ERR_BAD_ARG;
  wait_probe_kernel<<<1, 64, 0, stream>>>(status, (unsigned)limit);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// A [M, K] and W [N, K] bfloat16 row-major (K % 8 == 0, 16-byte aligned), C [M, ldc] bfloat16
// (out_dtype 1) or float32 (out_dtype 0) with ldc % 8 == 0 and 16-byte aligned. status: one int in
// device memory that a failed wait sets (0 = fine); the caller zeroes it and reads it back.
extern "C" int llmie_gemm_tc(const void* A, const void* W, void* C, int M, int N, int K, int ldc, int out_dtype,
                             int* status, cudaStream_t stream) {
  if (M < 0 || N <= 0 || K <= 0 || ldc < N) return LLMIE_ERR_BAD_ARG;
  if (K % 8 || ldc % 8) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (!aligned16(A) || !aligned16(W) || !aligned16(C)) return LLMIE_ERR_ALIGNMENT;
  if (M == 0) return LLMIE_OK;
  CUtensorMap map_a, map_w;
  int rc = tc::make_tmap_bf16_2d(&map_a, A, (uint64_t)M, (uint64_t)K, (uint64_t)K, kBM);
  if (rc != LLMIE_OK) return rc;
  rc = tc::make_tmap_bf16_2d(&map_w, W, (uint64_t)N, (uint64_t)K, (uint64_t)K, kBN);
  if (rc != LLMIE_OK) return rc;
  dim3 grid((N + kBN - 1) / kBN, (M + kBM - 1) / kBM);
  if (grid.y > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
  cudaError_t e;
  if (out_dtype == LLMIE_BF16) {
    e = cudaFuncSetAttribute(gemm_tc_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
    if (e != cudaSuccess) return (int)e;
    gemm_tc_kernel<__nv_bfloat16><<<grid, kGemmThreads, kGemmSmem, stream>>>(map_a, map_w, (__nv_bfloat16*)C, M, N, K,
                                                                            ldc, status);
  } else if (out_dtype == LLMIE_F32) {
    e = cudaFuncSetAttribute(gemm_tc_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
    if (e != cudaSuccess) return (int)e;
    gemm_tc_kernel<float><<<grid, kGemmThreads, kGemmSmem, stream>>>(map_a, map_w, (float*)C, M, N, K, ldc, status);
  } else {
    return LLMIE_ERR_DTYPE;
  }
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
