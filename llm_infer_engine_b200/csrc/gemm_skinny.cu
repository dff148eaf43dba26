// Weight-streaming matrix product for one-token steps: y[b, n] = sum_k x[b, k] W[n, k] with a
// handful of rows b (the batch) and a large bfloat16 W that must be read from HBM once. The
// time is the weight read; everything here serves that: 16-byte loads of W straight into
// tensor-core fragments (no shared-memory staging of W), the warps of a block split K
// between them so that enough bytes are in flight, and the work after the product (SwiGLU, the
// residual add, float32 logits) happens in the same kernel, so that a decode layer is few
// launches.
//
// Tensor-core shape: mma.sync m16n8k16 with the WEIGHTS as the 16-row operand and the batch as
// the 8-column operand (swap-AB), so a batch of 8 wastes nothing. A thread's 16-byte load of a
// weight row holds k = 8t .. 8t+7 of a 32-wide chunk; it feeds two MMAs, and the matching
// activations x[b][8t .. 8t+7] are loaded with the same k order, so the (harmless) permutation of
// k inside a chunk is the same on both operands.
//
// Row pairing: a block owns 16 weight rows, "low" rows lo+0..7 and "high" rows hi+0..7, which a
// thread sees as the two row halves of its fragment. Plain products use hi = lo + 8. For SwiGLU
// the low rows are gate rows j..j+7 and the high rows the up rows of the same j, so gate and up
// of one output meet in one block and silu(gate) * up is applied before anything is stored
// (src/model.py:23 of the reference does this with three GEMMs and two elementwise kernels).
#include "common.cuh"

namespace llmie {

constexpr int kSkUnroll = 4;     // 32-wide chunks of K a warp has in flight per round

enum SkinnyEpilogue { kStoreBf16 = 0, kStoreF32 = 1, kAddF32 = 2, kSwiGLU = 3 };

__device__ __forceinline__ void mma_bf16_16x8x16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                                 unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
// 16 bytes of a weight row: read-only path, not kept in L1 (every byte is used once), and L2 is asked to
// fetch 256 bytes around a miss (the rest of the run is about to be asked for)
__device__ __forceinline__ uint4 ldg16_stream(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}

// The whole matrix has to be in flight within a memory latency or two, so a block uses many
// warps on its 16 rows: warp w takes the chunks w, w + WARPS, ...; every round it first requests
// the NEXT kSkUnroll chunks of weights, then multiplies the ones that have arrived.
// NB: batch blocks of 8 (batch <= 8 * NB). EPI: what happens to the 16 x batch results.
template <int NB, int EPI, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
skinny_gemm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ W, void* __restrict__ out,
                   int batch, int K, int ldo, int tile_stride, int hi_delta) {
  pdl_launch_dependents();
  __shared__ float red[WARPS][NB][16][8 + 1];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int lo = blockIdx.x * tile_stride, hi = lo + hi_delta;
  // the 16 weight rows of this block are asked into L2 at once, before anything else
  if (threadIdx.x < 16) {
    const int row = threadIdx.x < 8 ? lo + threadIdx.x : hi + threadIdx.x - 8;
    l2_prefetch(W + (size_t)row * K, (unsigned)K * 2u);
  }
  const uint4* w_lo = reinterpret_cast<const uint4*>(W + (size_t)(lo + g) * K) + t;
  const uint4* w_hi = reinterpret_cast<const uint4*>(W + (size_t)(hi + g) * K) + t;
  const uint4* xr[NB];
  bool xok[NB];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    const int b = nb * 8 + g;
    xok[nb] = b < batch;
    xr[nb] = reinterpret_cast<const uint4*>(x + (size_t)(xok[nb] ? b : 0) * K) + t;
  }
  float acc[NB][4];
#pragma unroll
  for (int nb = 0; nb < NB; ++nb)
#pragma unroll
    for (int i = 0; i < 4; ++i) acc[nb][i] = 0.f;

  const int n_chunks = K >> 5;                      // chunks of 32 k; 4 uint4 per row per chunk
  // each warp takes a contiguous run of K, so that a row is read in long pieces
  const int per_warp = (n_chunks + WARPS - 1) / WARPS;
  const int c_begin = warp * per_warp, c_end = min(n_chunks, c_begin + per_warp);
  uint4 wa[kSkUnroll], wb[kSkUnroll], na[kSkUnroll], nbuf[kSkUnroll];
#pragma unroll
  for (int u = 0; u < kSkUnroll; ++u) {
    const int c = c_begin + u;
    if (c < c_end) {
      wa[u] = ldg16_stream(w_lo + c * 4);
      wb[u] = ldg16_stream(w_hi + c * 4);
    }
  }
  // The weights are written by no kernel, so their first loads are already on their way while
  // the kernel before this one finishes; x (and out, for the add) are its results: wait for it here.
  pdl_wait();
  // the activations of a round are requested a round ahead too, with the weights of that round, so
  // that no round waits for an L2 round trip of its own (one batch block; more would not fit the registers)
  constexpr bool kAhead = NB == 1;
  uint4 xcur[kSkUnroll][NB], xnext[kSkUnroll][NB];
  if (kAhead) {
#pragma unroll
    for (int u = 0; u < kSkUnroll; ++u) {
      const int c = c_begin + u;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        xcur[u][nb] = make_uint4(0u, 0u, 0u, 0u);
        if (c < c_end && xok[nb]) xcur[u][nb] = ldg16(xr[nb] + c * 4);
      }
    }
  }
  for (int c0 = c_begin; c0 < c_end; c0 += kSkUnroll) {
#pragma unroll
    for (int u = 0; u < kSkUnroll; ++u) {           // request the next round
      const int c = c0 + kSkUnroll + u;
      if (c < c_end) {
        na[u] = ldg16_stream(w_lo + c * 4);
        nbuf[u] = ldg16_stream(w_hi + c * 4);
      }
      if (kAhead) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          xnext[u][nb] = make_uint4(0u, 0u, 0u, 0u);
          if (c < c_end && xok[nb]) xnext[u][nb] = ldg16(xr[nb] + c * 4);
        }
      }
    }
    if (!kAhead) {
#pragma unroll
      for (int u = 0; u < kSkUnroll; ++u) {
        const int c = c0 + u;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          xcur[u][nb] = make_uint4(0u, 0u, 0u, 0u);
          if (c < c_end && xok[nb]) xcur[u][nb] = ldg16(xr[nb] + c * 4);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kSkUnroll; ++u) {
      const int c = c0 + u;
      if (c < c_end) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          mma_bf16_16x8x16(acc[nb], wa[u].x, wb[u].x, wa[u].y, wb[u].y, xcur[u][nb].x, xcur[u][nb].y);
          mma_bf16_16x8x16(acc[nb], wa[u].z, wb[u].z, wa[u].w, wb[u].w, xcur[u][nb].z, xcur[u][nb].w);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < kSkUnroll; ++u) {
      wa[u] = na[u];
      wb[u] = nbuf[u];
      if (kAhead) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) xcur[u][nb] = xnext[u][nb];
      }
    }
  }
  // this warp's share of K: rows g / g+8 of the tile, batch columns 2t, 2t+1 of each block
#pragma unroll
  for (int nb = 0; nb < NB; ++nb) {
    red[warp][nb][g][2 * t] = acc[nb][0];
    red[warp][nb][g][2 * t + 1] = acc[nb][1];
    red[warp][nb][g + 8][2 * t] = acc[nb][2];
    red[warp][nb][g + 8][2 * t + 1] = acc[nb][3];
  }
  __syncthreads();

  if (EPI == kSwiGLU) {
    // rows 0..7 gate, 8..15 up of outputs lo .. lo+7; out is [batch, ldo] bfloat16
    for (int idx = threadIdx.x; idx < NB * 64; idx += WARPS * 32) {
      const int j = idx & 7, col = (idx >> 3) & 7, nb = idx >> 6;
      const int b = nb * 8 + col;
      if (b >= batch) continue;
      float gate = 0.f, up = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        gate += red[w][nb][j][col];
        up += red[w][nb][j + 8][col];
      }
      const float act = gate / (1.f + expf(-gate)) * up;
      reinterpret_cast<__nv_bfloat16*>(out)[(size_t)b * ldo + lo + j] = __float2bfloat16_rn(act);
    }
  } else {
    for (int idx = threadIdx.x; idx < NB * 128; idx += WARPS * 32) {
      const int r = idx & 15, col = (idx >> 4) & 7, nb = idx >> 7;
      const int b = nb * 8 + col;
      if (b >= batch) continue;
      float v = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) v += red[w][nb][r][col];
      const int n = (r < 8 ? lo + r : hi + r - 8);
      const size_t o = (size_t)b * ldo + n;
      if (EPI == kStoreBf16) reinterpret_cast<__nv_bfloat16*>(out)[o] = __float2bfloat16_rn(v);
      if (EPI == kStoreF32) reinterpret_cast<float*>(out)[o] = v;
      if (EPI == kAddF32) reinterpret_cast<float*>(out)[o] += v;
    }
  }
}

template <int NB, int WARPS>
static int launch_epi(int epi, const void* x, const void* W, void* out, int batch, int K, int ldo, int tiles,
                      int tile_stride, int hi_delta, cudaStream_t stream) {
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)W;
  switch (epi) {
    case kStoreBf16:
      launch_k(skinny_gemm_kernel<NB, kStoreBf16, WARPS>, dim3(tiles), dim3(WARPS * 32), 0, stream, xp, wp, out, batch, K, ldo, tile_stride, hi_delta);
      break;
    case kStoreF32:
      launch_k(skinny_gemm_kernel<NB, kStoreF32, WARPS>, dim3(tiles), dim3(WARPS * 32), 0, stream, xp, wp, out, batch, K, ldo, tile_stride, hi_delta);
      break;
    case kAddF32:
      launch_k(skinny_gemm_kernel<NB, kAddF32, WARPS>, dim3(tiles), dim3(WARPS * 32), 0, stream, xp, wp, out, batch, K, ldo, tile_stride, hi_delta);
      break;
    case kSwiGLU:
      launch_k(skinny_gemm_kernel<NB, kSwiGLU, WARPS>, dim3(tiles), dim3(WARPS * 32), 0, stream, xp, wp, out, batch, K, ldo, tile_stride, hi_delta);
      break;
    default:
      return LLMIE_ERR_BAD_ARG;
  }
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// Warps per block. Few tiles (a small N): many warps per tile, so that the whole matrix is
// requested at once. Many tiles: small blocks, several per SM, whose start-up and reduction
// overlap with their neighbours' loads.
template <int NB>
static int launch_nb(int epi, const void* x, const void* W, void* out, int batch, int K, int ldo, int tiles,
                     int tile_stride, int hi_delta, cudaStream_t stream) {
  const int chunks = K / 32;
  // An SM holds about 16 of these warps (registers). Doubling the warps of a block must leave every block
  // resident at once: 192 tiles of 16 warps would run as 148 blocks and then 44.
  int warps = 4;
  while (warps < 16 && tiles * warps * 2 <= 148 * 16 && chunks >= warps * 2 * kSkUnroll) warps *= 2;
  if (warps >= 16) return launch_epi<NB, 16>(epi, x, W, out, batch, K, ldo, tiles, tile_stride, hi_delta, stream);
  if (warps >= 8) return launch_epi<NB, 8>(epi, x, W, out, batch, K, ldo, tiles, tile_stride, hi_delta, stream);
  return launch_epi<NB, 4>(epi, x, W, out, batch, K, ldo, tiles, tile_stride, hi_delta, stream);
}

}  // namespace llmie

using namespace llmie;

// Largest batch the kernel takes; above it the caller uses a tiled GEMM.
extern "C" int llmie_gemm_skinny_max_batch(void) { return 32; }

// x [batch, K] bfloat16, W [N, K] bfloat16 (for epilogue 3: W = [gate rows; up rows], N = 2 * ff).
// epilogue 0: out bfloat16 [batch, ldo] = y      1: out float32 [batch, ldo] = y
//          2: out float32 [batch, ldo] += y      3: out bfloat16 [batch, ldo] = silu(gate) * up, ff columns
// Needs K % 32 == 0, N % 16 == 0 (epilogue 3: ff % 8 == 0), 16-byte aligned x and W.
extern "C" int llmie_gemm_skinny(const void* x, const void* W, void* out, int batch, int N, int K, int ldo,
                                 int epilogue, cudaStream_t stream) {
  if (batch < 0 || N <= 0 || K <= 0) return LLMIE_ERR_BAD_ARG;
  if (batch > 32) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (K % 32) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (!aligned16(x) || !aligned16(W)) return LLMIE_ERR_ALIGNMENT;
  int tiles, tile_stride, hi_delta;
  if (epilogue == kSwiGLU) {
    if (N % 2 || (N / 2) % 8 || ldo < N / 2) return LLMIE_ERR_UNSUPPORTED_SIZE;
    tiles = N / 16; tile_stride = 8; hi_delta = N / 2;
  } else {
    if (N % 16 || ldo < N) return LLMIE_ERR_UNSUPPORTED_SIZE;
    tiles = N / 16; tile_stride = 16; hi_delta = 8;
  }
  if (batch == 0) return LLMIE_OK;
  if (batch <= 8) return launch_nb<1>(epilogue, x, W, out, batch, K, ldo, tiles, tile_stride, hi_delta, stream);
  if (batch <= 16) return launch_nb<2>(epilogue, x, W, out, batch, K, ldo, tiles, tile_stride, hi_delta, stream);
  return launch_nb<4>(epilogue, x, W, out, batch, K, ldo, tiles, tile_stride, hi_delta, stream);
}
