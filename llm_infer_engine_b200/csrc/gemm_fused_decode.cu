// One-token steps, first product of a branch: RMSNorm -> weight-streaming product -> the
// branch's next elementwise step, in ONE kernel, for up to 8 rows.
//
//   variant "qkv":   x = rmsnorm(h) ; [q k v] = x Wqkv^T ; rotate q and k by position ;
//                    q -> activation buffer, rotated k and v -> the paged KV cache
//   variant "gate":  x = rmsnorm(h) ; act = silu(x Wg^T) * (x Wu^T)
//   variant "f32":   x = rmsnorm(h) ; out = x W^T in float32 (the LM head after the final norm)
//
// In the reference these are 5, 5 and 2 launches (src/model.py:114,54,62,69-74; :127,23; :183).
// In a one-token step every launch costs a few microseconds of latency whatever it computes,
// and the layer is a chain of dependent launches, so fewer launches is what shortens it.
//
// The norm costs no extra pass: with w the norm weight, rmsnorm(h) W^T = rstd * ((h * w) W^T),
// so the block turns h * w into bfloat16 operands while it adds up h^2, multiplies as in
// gemm_skinny.cu (weights as the 16-row MMA operand, 16-byte loads straight into fragments,
// warps splitting K), and applies rstd = rsqrt(mean(h^2) + eps) to the finished sums. The rows
// of h * w are staged in shared memory once per block and reused for every tile of weight rows
// the block owns; the first weights of the first tile are requested before anything else, even
// before the wait for the previous kernel (no kernel writes weights).
#include "common.cuh"
#include <math.h>

namespace llmie {

constexpr int kFdUnroll = 4;
constexpr int kFdPad = 32;          // bfloat16 elements of padding per staged row: 16-byte reads do not collide

enum FusedVariant { kVarQkvRope = 0, kVarGateSwiGLU = 1, kVarF32 = 2 };

struct RopeStoreArgs {
  __nv_bfloat16* q_out;          // [batch, n_q * hd]
  __nv_bfloat16* k_cache;        // [pages, n_kv, page_size, hd]
  __nv_bfloat16* v_cache;
  const float2* table;           // [table_len, hd / 2] of (cos, sin)
  const int* tok_pos;            // [batch]
  const int* tok_seq;            // [batch]
  const int* seq_slot;
  const int* block_table;
  int max_pages, page_size, n_q, n_kv, hd, table_len, write_kv;
};

__device__ __forceinline__ void fd_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// 16 bytes of a weight row: read-only path, not kept in L1 (every byte is used once), and L2 is asked to
// fetch 256 bytes around a miss (the rest of the run is about to be asked for)
__device__ __forceinline__ uint4 fd_ldg16(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::256B.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
__device__ __forceinline__ unsigned fd_pack(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}

// Weight rows of tile `tile`: low rows lo..lo+7 and high rows hi..hi+7.
template <int VAR>
__device__ __forceinline__ void tile_rows(int tile, int hd, int half_n, int& lo, int& hi) {
  if (VAR == kVarQkvRope) {                 // rows i0..i0+7 and i0+hd/2.. of one head: rotation partners
    const int per_head = hd >> 4;
    const int head = tile / per_head, i0 = (tile - head * per_head) << 3;
    lo = head * hd + i0;
    hi = lo + (hd >> 1);
  } else if (VAR == kVarGateSwiGLU) {       // gate rows j..j+7 and the up rows of the same j
    lo = tile << 3;
    hi = half_n + lo;
  } else {
    lo = tile << 4;
    hi = lo + 8;
  }
}

// Fused epilogue of one tile for the lane that holds rows (g, g + 8) and batch columns 2t, 2t + 1.
// What the rotation epilogue looks up by token, fetched ahead by the lanes that will need it: the token's
// position, the cache page it is written to, and (for the lane's first tile) its angle's cosine and sine.
// The chain token -> sequence -> slot -> page is three dependent loads. All of it was written before the
// previous kernel was launched, so it is fetched while that kernel is still running.
struct RopeAhead {
  float2 cs[2];
  int pos[2];
  int page[2];
  int tile;          // the tile that cs belongs to
};

template <int VAR>
__device__ __forceinline__ void rope_ahead(RopeAhead& ra, int tile, int tiles, int t, int g, int batch, int half_n,
                                           const RopeStoreArgs& rope) {
  ra.tile = -1;
  if (VAR != kVarQkvRope) return;
  const int hd = rope.hd;
  int lo = 0, hi = 0;
  if (tile < tiles) tile_rows<VAR>(tile, hd, half_n, lo, hi);
  const int head = lo / hd, i = lo - head * hd + g;
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    const int b = 2 * t + cc;
    ra.pos[cc] = 0;
    ra.page[cc] = 0;
    ra.cs[cc] = make_float2(1.f, 0.f);
    if (b >= batch) continue;
    const int pos = rope.tok_pos[b];
    ra.pos[cc] = pos;
    if (rope.write_kv) {
      const int slot = rope.seq_slot[rope.tok_seq[b]];
      ra.page[cc] = rope.block_table[(size_t)slot * rope.max_pages + pos / rope.page_size];
    }
    if (tile < tiles && head < rope.n_q + rope.n_kv)
      ra.cs[cc] = rope.table[(size_t)min(pos, rope.table_len - 1) * (hd >> 1) + i];
  }
  if (tile < tiles) ra.tile = tile;
}

template <int VAR>
__device__ __forceinline__ void tile_epilogue(const float (&acc)[4], int tile, int lo, int hi, int g, int t, float rs0,
                                              float rs1, int batch, void* out, int ldo, const RopeStoreArgs& rope,
                                              const RopeAhead& ra) {
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    const int b = 2 * t + cc;
    if (b >= batch) continue;
    const float rs = cc ? rs1 : rs0;
    float x1 = acc[cc] * rs, x2 = acc[2 + cc] * rs;
    if (VAR == kVarF32) {
      float* o = reinterpret_cast<float*>(out) + (size_t)b * ldo;
      o[lo + g] = x1;
      o[hi + g] = x2;
    } else if (VAR == kVarGateSwiGLU) {
      const float act = x1 / (1.f + expf(-x1)) * x2;
      reinterpret_cast<__nv_bfloat16*>(out)[(size_t)b * ldo + lo + g] = __float2bfloat16_rn(act);
    } else {
      // rows lo + g and lo + g + hd/2 of one head: elements i and i + hd/2
      const int hd = rope.hd;
      const int head = lo / hd, i = lo - head * hd + g, half = hd >> 1;
      const int pos = ra.pos[cc];
      if (head < rope.n_q + rope.n_kv) {
        const float2 cs = tile == ra.tile ? ra.cs[cc] : rope.table[(size_t)min(pos, rope.table_len - 1) * half + i];
        const float y1 = x1 * cs.x - x2 * cs.y, y2 = x2 * cs.x + x1 * cs.y;
        x1 = y1;
        x2 = y2;
      }
      __nv_bfloat16* dst = nullptr;
      if (head < rope.n_q) {
        dst = rope.q_out + ((size_t)b * rope.n_q + head) * hd;
      } else if (rope.write_kv) {
        const int page = ra.page[cc];
        const bool is_k = head < rope.n_q + rope.n_kv;
        const int hk = head - rope.n_q - (is_k ? 0 : rope.n_kv);
        dst = (is_k ? rope.k_cache : rope.v_cache) +
              (((size_t)page * rope.n_kv + hk) * rope.page_size + (pos % rope.page_size)) * hd;
      }
      if (dst) {
        dst[i] = __float2bfloat16_rn(x1);
        dst[i + half] = __float2bfloat16_rn(x2);
      }
    }
  }
}

__device__ __forceinline__ void fd_team_sync(int team, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(threads) : "memory");
}

// The block's warps form teams of S warps (S a power of two up to WARPS). A team takes a tile of 16
// weight rows at a time (tile numbers go round the blocks first); each of its warps owns a
// contiguous run of K and streams its share of the rows straight into mma.sync fragments. A warp's
// work is a flat sequence of rounds (kFdUnroll chunks of 32 each) that runs on across tile
// boundaries; two register buffers take turns, so the loads of the next round are always in flight
// while the current one is used, and no buffer is ever copied. At the end of a tile the partial sums
// meet in the team's first warp through shared memory (two buffers in turn, one team barrier per
// tile; no block-wide barrier), whose lanes hold whole (row, row + 8) x (column pair) results: the
// rotation pairs, the gate and up rows, or plain outputs. With S = 1 (many tiles: the LM head) a
// warp streams whole rows and nothing is exchanged at all.
template <int VAR, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
norm_gemm_kernel(const float* __restrict__ h, const float* __restrict__ norm_w, float eps,
                 const __nv_bfloat16* __restrict__ W, void* __restrict__ out, int batch, int K, int ldo, int tiles,
                 int half_n, int S, RopeStoreArgs rope) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char fd_smem[];
  const int xs_stride = K + kFdPad;                                        // elements
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(fd_smem);           // [8][K + pad]
  float4* red = reinterpret_cast<float4*>(fd_smem + (size_t)8 * xs_stride * 2);   // [2][WARPS][32]
  float* ssw = reinterpret_cast<float*>(red + 2 * WARPS * 32);             // [WARPS][8]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int team = warp / S, j = warp - team * S;
  const int n_chunks = K >> 5;
  const int per_warp = (n_chunks + S - 1) / S;
  const int c_begin = j * per_warp, c_end = min(n_chunks, c_begin + per_warp);
  const bool has_k = c_begin < c_end;          // a warp beyond the end of K only joins its team's barriers
  const int n_rounds = has_k ? (c_end - c_begin + kFdUnroll - 1) / kFdUnroll : 1;
  const int tile_stride = (WARPS / S) * gridDim.x;
  const int hd = rope.hd;

  int ltile = team * gridDim.x + blockIdx.x, lr = 0;   // where the next loads come from
  const uint4* lw_lo = nullptr;
  const uint4* lw_hi = nullptr;
#define LLMIE_POINT_LOADS()                                                          \
  do {                                                                               \
    if (ltile < tiles) {                                                             \
      int ra_, rb_;                                                                  \
      tile_rows<VAR>(ltile, hd, half_n, ra_, rb_);                                   \
      lw_lo = reinterpret_cast<const uint4*>(W + (size_t)(ra_ + g) * K) + t;         \
      lw_hi = reinterpret_cast<const uint4*>(W + (size_t)(rb_ + g) * K) + t;         \
    }                                                                                \
  } while (0)
#define LLMIE_ISSUE(wa, wb)                                                          \
  do {                                                                               \
    if (ltile < tiles && has_k) {                                                    \
      const int lc0_ = c_begin + lr * kFdUnroll;                                     \
      _Pragma("unroll") for (int u = 0; u < kFdUnroll; ++u) {                        \
        const int c = lc0_ + u;                                                      \
        if (c < c_end) {                                                             \
          wa[u] = fd_ldg16(lw_lo + c * 4);                                           \
          wb[u] = fd_ldg16(lw_hi + c * 4);                                           \
        }                                                                            \
      }                                                                              \
      if (++lr >= n_rounds) {                                                        \
        lr = 0;                                                                      \
        ltile += tile_stride;                                                        \
        LLMIE_POINT_LOADS();                                                         \
      }                                                                              \
    }                                                                                \
  } while (0)
  LLMIE_POINT_LOADS();
  uint4 a0[kFdUnroll], b0[kFdUnroll], a1[kFdUnroll], b1[kFdUnroll];
  LLMIE_ISSUE(a0, b0);     // weights are written by no kernel: two rounds are on their way before the
  LLMIE_ISSUE(a1, b1);     // previous kernel has finished
  RopeAhead ra;
  if (j == 0) rope_ahead<VAR>(ra, team * gridDim.x + blockIdx.x, tiles, t, g, batch, half_n, rope);
  pdl_wait();              // h is the previous kernels' result

  // ---- h * w as bfloat16 rows in shared memory, and the sum of squares of every row
  {
    float ssq[8];
#pragma unroll
    for (int b = 0; b < 8; ++b) ssq[b] = 0.f;
    for (int k = threadIdx.x * 8; k < K; k += WARPS * 32 * 8) {
      float wv[8];
      load8(norm_w + k, wv);
#pragma unroll
      for (int b = 0; b < 8; ++b) {
        float hv[8];
        if (b < batch) {
          load8(h + (size_t)b * K + k, hv);
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) hv[e] = 0.f;
        }
        uint4 packed;
        packed.x = fd_pack(hv[0] * wv[0], hv[1] * wv[1]);
        packed.y = fd_pack(hv[2] * wv[2], hv[3] * wv[3]);
        packed.z = fd_pack(hv[4] * wv[4], hv[5] * wv[5]);
        packed.w = fd_pack(hv[6] * wv[6], hv[7] * wv[7]);
        *reinterpret_cast<uint4*>(xs + (size_t)b * xs_stride + k) = packed;
#pragma unroll
        for (int e = 0; e < 8; ++e) ssq[b] = fmaf(hv[e], hv[e], ssq[b]);
      }
    }
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      const float sq = warp_sum(ssq[b]);
      if (lane == 0) ssw[warp * 8 + b] = sq;
    }
    __syncthreads();
  }
  float rs0, rs1;                     // rstd of the two batch columns this lane holds results of
  {
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      s0 += ssw[w * 8 + 2 * t];
      s1 += ssw[w * 8 + 2 * t + 1];
    }
    rs0 = rsqrtf(s0 / (float)K + eps);
    rs1 = rsqrtf(s1 / (float)K + eps);
  }
  const uint4* x_row = reinterpret_cast<const uint4*>(xs + (size_t)g * xs_stride) + t;   // this lane's batch row

  int tile = team * gridDim.x + blockIdx.x, cr = 0, parity = 0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};     // two chains of products, summed per tile
#define LLMIE_CONSUME(wa, wb)                                                        \
  do {                                                                               \
    const int c0_ = c_begin + cr * kFdUnroll;                                        \
    _Pragma("unroll") for (int u = 0; u < kFdUnroll; ++u) {                          \
      const int c = c0_ + u;                                                         \
      if (c < c_end) {                                                               \
        const uint4 xv = x_row[c * 4];                                               \
        fd_mma(acc, wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);                 \
        fd_mma(acc2, wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);                \
      }                                                                              \
    }                                                                                \
    if (++cr >= n_rounds) {                                                          \
      _Pragma("unroll") for (int i = 0; i < 4; ++i) {                                \
        acc[i] += acc2[i];                                                           \
        acc2[i] = 0.f;                                                               \
      }                                                                              \
      if (S > 1) {                                                                   \
        float4* mine = red + ((parity * WARPS + warp) * 32 + lane);                  \
        if (j != 0) *mine = make_float4(acc[0], acc[1], acc[2], acc[3]);             \
        fd_team_sync(team, S * 32);                                                  \
        if (j == 0) {                                                                \
          for (int o = 1; o < S; ++o) {                                              \
            const float4 v = mine[o * 32];                                           \
            acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;              \
          }                                                                          \
        }                                                                            \
        parity ^= 1;                                                                 \
      }                                                                              \
      if (j == 0) {                                                                  \
        int lo, hi;                                                                  \
        tile_rows<VAR>(tile, hd, half_n, lo, hi);                                    \
        tile_epilogue<VAR>(acc, tile, lo, hi, g, t, rs0, rs1, batch, out, ldo, rope, ra); \
      }                                                                              \
      acc[0] = acc[1] = acc[2] = acc[3] = 0.f;                                       \
      cr = 0;                                                                        \
      tile += tile_stride;                                                           \
    }                                                                                \
  } while (0)
  while (tile < tiles) {
    LLMIE_CONSUME(a0, b0);
    LLMIE_ISSUE(a0, b0);
    if (tile >= tiles) break;
    LLMIE_CONSUME(a1, b1);
    LLMIE_ISSUE(a1, b1);
  }
#undef LLMIE_POINT_LOADS
#undef LLMIE_ISSUE
#undef LLMIE_CONSUME
}

template <int VAR, int WARPS>
static size_t fused_smem(int K) {
  return (size_t)8 * (K + kFdPad) * 2 + (size_t)2 * WARPS * 32 * sizeof(float4) + (size_t)WARPS * 8 * sizeof(float);
}

// Blocks of this instance that one SM holds at once (0 if it cannot run at all with this K).
template <int VAR, int WARPS>
static int fused_blocks_per_sm(int K) {
  static int cached_k = -1, cached = 0;
  if (cached_k != K) {
    const size_t smem = fused_smem<VAR, WARPS>(K);
    int n = 0;
    if (smem <= 200 * 1024) {
      if (smem > 48 * 1024)
        cudaFuncSetAttribute(norm_gemm_kernel<VAR, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, norm_gemm_kernel<VAR, WARPS>, WARPS * 32, smem) != cudaSuccess)
        n = 0;
    }
    cached = n;
    cached_k = K;
  }
  return cached;
}

constexpr int kFdWarps = 8;

// Team size and grid: the largest teams that leave a team at most about two tiles (the second tile's first
// loads are requested while the first is finished, which hides the tile's end; measured on the gate / up
// product of the 1B shape: 4 warps a tile and 1.7 tiles a team beat 2 warps and one tile by 1.7 % of the
// whole step); few tiles make few blocks, spread over the SMs.
template <int VAR>
static int launch_fused_w(const float* h, const float* norm_w, float eps, const void* W, void* out, int batch, int K,
                          int ldo, int tiles, int half_n, const RopeStoreArgs& rope, cudaStream_t stream) {
  const int per_sm = fused_blocks_per_sm<VAR, kFdWarps>(K);
  if (per_sm < 1) return LLMIE_ERR_UNSUPPORTED_SIZE;
  const long long resident_warps = 148LL * per_sm * kFdWarps;
  int S = kFdWarps;
  while (S > 1 && (long long)tiles * S > 2 * resident_warps) S >>= 1;
  const int teams_per_block = kFdWarps / S;
  int blocks = (tiles + teams_per_block - 1) / teams_per_block;
  if (blocks > 148 * per_sm) blocks = 148 * per_sm;
  launch_k(norm_gemm_kernel<VAR, kFdWarps>, dim3(blocks), dim3(kFdWarps * 32), fused_smem<VAR, kFdWarps>(K), stream, h,
           norm_w, eps, (const __nv_bfloat16*)W, out, batch, K, ldo, tiles, half_n, S, rope);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

static int check_common(const float* h, const float* norm_w, const void* W, int batch, int N, int K) {
  if (batch < 0 || N <= 0 || K <= 0) return LLMIE_ERR_BAD_ARG;
  if (batch > 8 || K % 32) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (!aligned16(h) || !aligned16(norm_w) || !aligned16(W)) return LLMIE_ERR_ALIGNMENT;
  return LLMIE_OK;
}

}  // namespace llmie

using namespace llmie;

// 1 when the fused kernels take this (batch, K): up to 8 rows, K a multiple of 32 that fits shared memory.
extern "C" int llmie_norm_gemm_supported(int batch, int K) {
  return (batch >= 1 && batch <= 8 && K % 32 == 0 && (size_t)8 * (K + kFdPad) * 2 + 12 * 1024 <= 200 * 1024) ? 1 : 0;
}

// act[batch, ff] = silu(x Wg^T) * (x Wu^T), x = rmsnorm(h) with weight norm_w; W = [gate rows; up rows] (2 ff rows).
extern "C" int llmie_norm_gate_swiglu(const float* h, const float* norm_w, float eps, const void* W, void* act,
                                      int batch, int ff, int K, cudaStream_t stream) {
  int rc = check_common(h, norm_w, W, batch, ff, K);
  if (rc != LLMIE_OK) return rc;
  if (ff % 8) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (batch == 0) return LLMIE_OK;
  RopeStoreArgs none = {};
  none.hd = 16;
  return launch_fused_w<kVarGateSwiGLU>(h, norm_w, eps, W, act, batch, K, ff, ff / 8, ff, none, stream);
}

// out[batch, N] float32 = rmsnorm(h) W^T.
extern "C" int llmie_norm_gemm_f32(const float* h, const float* norm_w, float eps, const void* W, float* out, int batch,
                                   int N, int K, cudaStream_t stream) {
  int rc = check_common(h, norm_w, W, batch, N, K);
  if (rc != LLMIE_OK) return rc;
  if (N % 16) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (batch == 0) return LLMIE_OK;
  RopeStoreArgs none = {};
  none.hd = 16;
  return launch_fused_w<kVarF32>(h, norm_w, eps, W, out, batch, K, N, N / 16, 0, none, stream);
}

// [q k v] = rmsnorm(h) Wqkv^T, q and k rotated by table[tok_pos]; q -> q_out, k and v -> the paged cache
// (only q when write_kv == 0). Wqkv rows: n_q heads of q, n_kv of k, n_kv of v, each hd wide; full rotation.
extern "C" int llmie_norm_qkv_rope(const float* h, const float* norm_w, float eps, const void* W, void* q_out,
                                   void* k_cache, void* v_cache, const float* table, const int* tok_pos,
                                   const int* tok_seq, const int* seq_slot, const int* block_table, int max_pages,
                                   int page_size, int batch, int n_q, int n_kv, int hd, int K, int table_len,
                                   int write_kv, cudaStream_t stream) {
  int rc = check_common(h, norm_w, W, batch, (n_q + 2 * n_kv) * hd, K);
  if (rc != LLMIE_OK) return rc;
  if (hd % 16 || n_q <= 0 || n_kv <= 0 || page_size <= 0 || max_pages <= 0 || table_len <= 0 || !table)
    return LLMIE_ERR_BAD_ARG;
  if (batch == 0) return LLMIE_OK;
  RopeStoreArgs r;
  r.q_out = (__nv_bfloat16*)q_out;
  r.k_cache = (__nv_bfloat16*)k_cache;
  r.v_cache = (__nv_bfloat16*)v_cache;
  r.table = reinterpret_cast<const float2*>(table);
  r.tok_pos = tok_pos;
  r.tok_seq = tok_seq;
  r.seq_slot = seq_slot;
  r.block_table = block_table;
  r.max_pages = max_pages;
  r.page_size = page_size;
  r.n_q = n_q;
  r.n_kv = n_kv;
  r.hd = hd;
  r.table_len = table_len;
  r.write_kv = write_kv;
  const int tiles = (n_q + 2 * n_kv) * (hd / 16);
  return launch_fused_w<kVarQkvRope>(h, norm_w, eps, W, nullptr, batch, K, 0, tiles, 0, r, stream);
}
