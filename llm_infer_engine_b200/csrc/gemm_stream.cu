// Weight-streaming GEMM for steps of 9 to 64 rows: Y[M, N] = X[M, K] * W[N, K]^T, bfloat16 in, float32
// accumulation in TMEM, on the tcgen05 tensor cores with the operands swapped: a tile of 128 WEIGHT rows is
// the M side of the MMA and the step's rows (padded to 16, 32 or 64) are its N side. The arithmetic is
// negligible; the kernel is a streamer of W, which it reads exactly once.
//
// A tile of 128 weight rows is the work of one thread-block CLUSTER of S blocks (S = 1, 2, 4 or 8): block r
// of the cluster multiplies the r-th slice of K, so that also a matrix of few rows (2,048 x 8,192 is 16 tiles)
// is streamed by most of the SMs. The S partial tiles meet in shared memory: each block leaves its partial
// sums in its own shared memory, and block r adds up rows [r * 128 / S, (r + 1) * 128 / S) of all S partials,
// read from the peers' shared memory, IN SLICE ORDER, and stores them. No workspace in global memory, no
// atomics, and a result that does not depend on timing. Clusters take the tiles j, j + n_clusters, ...
//
// Roles by warp:
//   warp 0      TMA producer: per 64 columns of K one stage of the ring = the W tile (16 KB) and the X tile
//               (MPAD x 64, from L2); the first ring-full of W loads is issued before the wait on the previous
//               kernel, since no kernel writes weights
//   warp 1      allocates TMEM (two accumulators of MPAD columns), one lane issues the MMAs and commits
//   warps 2..5  epilogue: tcgen05.ld of the accumulator (thread = one weight row = one output column, MPAD
//               values), the exchange described above when S > 1, and the final store: bfloat16 Y, float32 Y,
//               or `H += Y` into a float32 residual stream
// Every wait is bounded; a wait that gives up records a status, raises the block's abort flag, and the block
// still frees its TMEM and returns (its peers' waits on it then run out the same way).
//
// The reference leaves these products to nn.Linear (src/model.py:17-19,34-37,137).
#include "tcgen05.cuh"

namespace llmie {
using namespace tc;

constexpr int kSRows = 128, kSBK = 64;
constexpr int kSWBytes = kSRows * kSBK * 2;          // 16 KB of weights per stage
constexpr int kSThreads = 192;
constexpr int kSMaxStages = 12;
constexpr int kSSmemBudget = 220 * 1024;             // dynamic shared memory: the ring and the exchange tile

struct StreamShared {
  uint64_t full[kSMaxStages];
  uint64_t empty[kSMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint64_t peers_ready;      // every epilogue warp of every block of the cluster has left its partial sums
  uint64_t peers_done;       // ... has finished reading the partial sums of this tile
  uint32_t tmem_base;
  int abort;
};

__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

enum { kStoreBf16 = 0, kStoreF32 = 1, kAddF32 = 2 };

__device__ __forceinline__ void final_store(void* out, int mode, size_t idx, float v) {
  if (mode == kStoreBf16) reinterpret_cast<__nv_bfloat16*>(out)[idx] = __float2bfloat16_rn(v);
  else if (mode == kStoreF32) reinterpret_cast<float*>(out)[idx] = v;
  else reinterpret_cast<float*>(out)[idx] += v;
}

template <int MPAD>
__global__ void __launch_bounds__(kSThreads, 1)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                   void* __restrict__ out, int M, int N, int K, int n_splits, int chunks_per_split, int n_tiles,
                   int n_clusters, int n_stages, int mode, int* __restrict__ status) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  __shared__ StreamShared sh;
  constexpr int kXBytes = MPAD * kSBK * 2;
  constexpr int kStageBytes = kSWBytes + kXBytes;
  uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  float* xchg = reinterpret_cast<float*>(ring + (size_t)n_stages * kStageBytes);     // [MPAD][128], when S > 1
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = n_splits > 1 ? (int)cluster_block_rank() : 0;
  const int first_tile = blockIdx.x / n_splits;
  const int total_chunks = (K + kSBK - 1) / kSBK;
  const int c0 = split * chunks_per_split, c1 = min(total_chunks, c0 + chunks_per_split);

  if (threadIdx.x == 0) {
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(&sh.full[s], 1);
      mbar_init(&sh.empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh.acc_full[b], 1);
      mbar_init(&sh.acc_empty[b], 4);          // one arrival per epilogue warp
    }
    mbar_init(&sh.peers_ready, 4 * n_splits);  // one per epilogue warp of every block of the cluster
    mbar_init(&sh.peers_done, 4 * n_splits);
    sh.abort = 0;
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, 128);            // two accumulators of up to 64 columns
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  if (n_splits > 1) cluster_sync_all();        // no block arrives at a peer's barrier before it exists
  const uint32_t tmem = sh.tmem_base;
  volatile int* abort = &sh.abort;

  if (warp == 0) {
    if (elect_one()) {
      tma_prefetch_desc(&map_w);
      tma_prefetch_desc(&map_x);
      // Stages are numbered through all of the block's tiles. The weights of the first ring-full are asked for
      // before the wait on the previous kernel; X, which that kernel may have written, after it.
      int it = 0, early = 0, issued = 0;
      bool waited = false, stop = false;
      auto load_early_x = [&]() {
        pdl_wait();
        waited = true;
        int jt = 0;
        for (int t2 = first_tile; t2 < n_tiles && jt < early; t2 += n_clusters)
          for (int c2 = c0; c2 < c1 && jt < early; ++c2, ++jt)
            tma_load_2d(ring + (size_t)(jt % n_stages) * kStageBytes + kSWBytes, &map_x, c2 * kSBK, 0,
                        &sh.full[jt % n_stages]);
      };
      for (int t = first_tile; t < n_tiles && !stop; t += n_clusters) {
        for (int c = c0; c < c1; ++c, ++it) {
          const int s = it % n_stages;
          uint8_t* stage = ring + (size_t)s * kStageBytes;
          if (it < n_stages) {
            mbar_arrive_expect_tx(&sh.full[s], kStageBytes);
            tma_load_2d(stage, &map_w, c * kSBK, t * kSRows, &sh.full[s]);
            early = issued = it + 1;
            continue;                            // its X follows after the wait on the previous kernel
          }
          if (!waited) load_early_x();
          if (!mbar_wait(&sh.empty[s], ((it / n_stages) - 1) & 1, abort)) {
            if (!*abort) { *abort = 1; atomicExch(status, kStatusTimeoutEmpty); }
            stop = true;
            break;
          }
          mbar_arrive_expect_tx(&sh.full[s], kStageBytes);
          tma_load_2d(stage, &map_w, c * kSBK, t * kSRows, &sh.full[s]);
          tma_load_2d(stage + kSWBytes, &map_x, c * kSBK, 0, &sh.full[s]);
          issued = it + 1;
        }
      }
      if (!waited) load_early_x();               // everything fitted into the first ring-full
      if (*abort) {
        // winding down: let this thread's own copies land (bounded) before the shared memory is given up
        for (int jt = max(0, issued - n_stages); jt < issued; ++jt) {
          uint64_t* bar = &sh.full[jt % n_stages];
          for (unsigned spin = 0; spin < (1u << 16) && !mbar_test(bar, (jt / n_stages) & 1); ++spin) __nanosleep(64);
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_instr_desc_bf16(kSRows, MPAD, 0, 0);
      int it = 0, tile_i = 0;
      bool ok = true;
      for (int t = first_tile; t < n_tiles && ok; t += n_clusters, ++tile_i) {
        const int buf = tile_i & 1;
        if (tile_i >= 2 && !mbar_wait(&sh.acc_empty[buf], ((tile_i >> 1) - 1) & 1, abort)) {
          if (!*abort) { *abort = 1; atomicExch(status, kStatusTimeoutMma); }
          break;
        }
        tc_fence_after_sync();
        const uint32_t acc = tmem + (uint32_t)(buf * 64);
        for (int c = c0; c < c1; ++c, ++it) {
          const int s = it % n_stages;
          if (!mbar_wait(&sh.full[s], (it / n_stages) & 1, abort)) {
            if (!*abort) { *abort = 1; atomicExch(status, kStatusTimeoutFull); }
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t w_addr = smem_u32(ring + (size_t)s * kStageBytes);
          const uint32_t x_addr = w_addr + kSWBytes;
#pragma unroll
          for (int kk = 0; kk < kSBK / 16; ++kk) {
            const uint64_t dw = make_smem_desc(w_addr + kk * 32, 16, 1024);
            const uint64_t dx = make_smem_desc(x_addr + kk * 32, 16, 1024);
            mma_bf16_ss(acc, dw, dx, idesc, (c > c0 || kk > 0) ? 1u : 0u);
          }
          mma_commit(&sh.empty[s]);
        }
        if (ok) mma_commit(&sh.acc_full[buf]);
      }
    }
  } else {
    const int quarter = warp & 3;                 // the TMEM lanes this warp may read
    const int epi_tid = quarter * 32 + lane;      // 0..127: the weight row within the tile
    pdl_wait();                                   // everything below writes global memory
    int tile_i = 0;
    for (int t = first_tile; t < n_tiles; t += n_clusters, ++tile_i) {
      const int buf = tile_i & 1;
      const bool got = __all_sync(0xffffffffu, mbar_wait(&sh.acc_full[buf], (tile_i >> 1) & 1, abort));
      if (!got && !*abort) { *abort = 1; atomicExch(status, kStatusTimeoutMma); }
      epi_sync();                                 // every epilogue warp arrives here, whatever its wait said
      if (*abort) break;                          // the same decision in all four warps
      tc_fence_after_sync();
      float v[MPAD];
      const uint32_t taddr = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * 64);
      if constexpr (MPAD == 16) {
        uint32_t r[16];
        tmem_ld_32x16(taddr, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
      } else {
#pragma unroll
        for (int c = 0; c < MPAD; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + (uint32_t)c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[c + i] = __uint_as_float(r[i]);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.acc_empty[buf]);   // the accumulator may be overwritten
      if (n_splits == 1) {
        const int n = t * kSRows + epi_tid;
        if (n < N) {
#pragma unroll
          for (int m = 0; m < MPAD; ++m)
            if (m < M) final_store(out, mode, (size_t)m * N + n, v[m]);
        }
        continue;
      }
      // ---- S > 1: the partial sums of the S slices meet in shared memory
      if (tile_i > 0) {                           // the peers have read the previous tile out of xchg
        const bool freed = __all_sync(0xffffffffu, mbar_wait_cluster(&sh.peers_done, (tile_i - 1) & 1, abort));
        if (!freed && !*abort) { *abort = 1; atomicExch(status, kStatusTimeoutMma); }
      }
#pragma unroll
      for (int m = 0; m < MPAD; ++m)
        if (m < M) xchg[m * kSRows + epi_tid] = v[m];
      fence_cluster();
      __syncwarp();
      if (lane < n_splits) mbar_arrive_cluster(map_to_block(smem_u32(&sh.peers_ready), (uint32_t)lane));
      const bool ready = __all_sync(0xffffffffu, mbar_wait_cluster(&sh.peers_ready, tile_i & 1, abort));
      if (!ready && !*abort) { *abort = 1; atomicExch(status, kStatusTimeoutMma); }
      if (ready) {
        // this block's share of the tile: rows [split * rows_per, + rows_per), all M; slices added in order
        const int rows_per = kSRows / n_splits;
        const uint32_t base = smem_u32(xchg);
        for (int item = epi_tid; item < rows_per * M; item += 128) {
          const int m = item / rows_per, row = split * rows_per + (item - m * rows_per);
          const uint32_t off = base + (uint32_t)(m * kSRows + row) * 4u;
          float part[8];
#pragma unroll
          for (int sp = 0; sp < 8; ++sp)           // all loads are on their way before the first is used
            part[sp] = sp < n_splits ? ld_cluster_f32(map_to_block(off, (uint32_t)sp)) : 0.f;
          float sum = 0.f;
#pragma unroll
          for (int sp = 0; sp < 8; ++sp) sum += part[sp];      // slice order; absent slices add zero
          const int n = t * kSRows + row;
          if (n < N) final_store(out, mode, (size_t)m * N + n, sum);
        }
      }
      __syncwarp();
      if (lane < n_splits) mbar_arrive_cluster(map_to_block(smem_u32(&sh.peers_done), (uint32_t)lane));
    }
    if (n_splits > 1 && tile_i > 0 && !*abort) {  // no peer still reads this block's shared memory
      const bool freed = __all_sync(0xffffffffu, mbar_wait_cluster(&sh.peers_done, (tile_i - 1) & 1, abort));
      if (!freed && !*abort) { *abort = 1; atomicExch(status, kStatusTimeoutMma); }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, 128);
  }
  if (n_splits > 1) cluster_sync_all();           // shared memory of a block outlives its peers' accesses to it
}

struct StreamPlan {
  int mpad, n_tiles, n_splits, chunks_per_split, n_clusters, n_stages, smem;
};

static StreamPlan stream_plan(int M, int N, int K, int n_sms, int force_splits = 0) {
  StreamPlan p;
  p.mpad = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
  p.n_tiles = (N + kSRows - 1) / kSRows;
  const int chunks = (K + kSBK - 1) / kSBK;
  // slices of K (blocks per cluster): a power of two up to 8, as many as it takes to occupy the SMs with the
  // tiles there are, each slice at least 256 columns (4 chunks) long
  int s = 1;
  while (s < 8 && p.n_tiles * s * 2 <= n_sms && chunks / (s * 2) >= 4) s *= 2;
  if (force_splits == 1 || force_splits == 2 || force_splits == 4 || force_splits == 8) s = force_splits;
  while (s > 1 && chunks < s) s /= 2;
  p.chunks_per_split = (chunks + s - 1) / s;
  p.n_splits = s;
  p.n_clusters = n_sms / s;
  if (p.n_clusters > p.n_tiles) p.n_clusters = p.n_tiles;
  if (p.n_clusters < 1) p.n_clusters = 1;
  const int stage = kSWBytes + p.mpad * kSBK * 2;
  const int xchg = s > 1 ? p.mpad * kSRows * 4 : 0;
  p.n_stages = (kSSmemBudget - xchg) / stage;
  if (p.n_stages > kSMaxStages) p.n_stages = kSMaxStages;
  p.smem = p.n_stages * stage + xchg + 1024;
  return p;
}

}  // namespace llmie

using namespace llmie;

// How many clusters of `splits` blocks of the kernel for `rows` rows the device can hold at once (0 on error).
extern "C" int llmie_gemm_stream_active_clusters(int rows, int N, int K, int n_sms, int splits) {
  const StreamPlan p = stream_plan(rows, N, K, n_sms, splits);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.n_clusters * p.n_splits);
  cfg.blockDim = dim3(kSThreads);
  cfg.dynamicSmemBytes = p.smem;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = p.n_splits;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  cudaError_t e;
  if (p.mpad == 16) {
    cudaFuncSetAttribute(gemm_stream_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem);
    e = cudaOccupancyMaxActiveClusters(&n, gemm_stream_kernel<16>, &cfg);
  } else if (p.mpad == 32) {
    cudaFuncSetAttribute(gemm_stream_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem);
    e = cudaOccupancyMaxActiveClusters(&n, gemm_stream_kernel<32>, &cfg);
  } else {
    cudaFuncSetAttribute(gemm_stream_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem);
    e = cudaOccupancyMaxActiveClusters(&n, gemm_stream_kernel<64>, &cfg);
  }
  return e == cudaSuccess ? n : 0;
}

// X [M <= 64, K] and W [N, K] bfloat16 row-major (K % 8 == 0, 16-byte aligned). mode 0: out bfloat16 [M, N];
// 1: out float32 [M, N]; 2: out float32 [M, N] += the product. n_sms: SMs of the device (sizes the grid).
// splits: 0 lets the launcher choose into how many slices K is cut; 1, 2, 4 or 8 fixes it.
// status: one int in device memory that a failed wait sets (0 = fine).
extern "C" int llmie_gemm_stream(const void* X, const void* W, void* out, int M, int N, int K, int mode, int n_sms,
                                 int splits, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || mode < 0 || mode > 2 || n_sms <= 0) return LLMIE_ERR_BAD_ARG;
  if (M > 64 || K % 8) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (!aligned16(X) || !aligned16(W) || !aligned16(out)) return LLMIE_ERR_ALIGNMENT;
  const StreamPlan p = stream_plan(M, N, K, n_sms, splits);
  CUtensorMap map_w, map_x;
  int rc = tc::make_tmap_bf16_2d(&map_w, W, (uint64_t)N, (uint64_t)K, (uint64_t)K, kSRows);
  if (rc != LLMIE_OK) return rc;
  rc = tc::make_tmap_bf16_2d(&map_x, X, (uint64_t)M, (uint64_t)K, (uint64_t)K, (uint32_t)p.mpad);
  if (rc != LLMIE_OK) return rc;
  const dim3 grid(p.n_clusters * p.n_splits);
  cudaError_t e;
#define LLMIE_STREAM_CASE(MP)                                                                                       \
  case MP:                                                                                                          \
    e = cudaFuncSetAttribute(gemm_stream_kernel<MP>, cudaFuncAttributeMaxDynamicSharedMemorySize, p.smem);          \
    if (e != cudaSuccess) return (int)e;                                                                            \
    if (p.n_splits > 1)                                                                                             \
      launch_k_cluster(gemm_stream_kernel<MP>, grid, dim3(kSThreads), (size_t)p.smem, stream, (unsigned)p.n_splits, \
                       map_w, map_x, out, M, N, K, p.n_splits, p.chunks_per_split, p.n_tiles, p.n_clusters,         \
                       p.n_stages, mode, status);                                                                   \
    else                                                                                                            \
      launch_k(gemm_stream_kernel<MP>, grid, dim3(kSThreads), (size_t)p.smem, stream, map_w, map_x, out, M, N, K,   \
               p.n_splits, p.chunks_per_split, p.n_tiles, p.n_clusters, p.n_stages, mode, status);                  \
    break;
  switch (p.mpad) {
    LLMIE_STREAM_CASE(16)
    LLMIE_STREAM_CASE(32)
    LLMIE_STREAM_CASE(64)
    default:
      return LLMIE_ERR_UNSUPPORTED_SIZE;
  }
#undef LLMIE_STREAM_CASE
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
