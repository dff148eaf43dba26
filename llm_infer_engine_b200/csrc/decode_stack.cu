// A whole one-token step of a stack of Llama-style layers in ONE persistent kernel.
//
// A one-token step at small batch is a chain of dependent phases (norm + QKV + rotation, attention,
// output projection, norm + gate/up + SwiGLU, down projection, ... final norm + head), each of
// which lasts a few microseconds. Here one block per SM stays resident for the whole step and the
// phases are separated by grid-wide barriers instead of kernel boundaries. The reference runs the
// same chain as ~17 launches per layer (src/model.py:39-127), or one CUDA graph of them for
// batch 1 (src/cuda_graph.py).
//
// Measured on B200 at the Llama 3.2 1B shape, batch 8, 512 cached tokens: 1.27 ms per step, against
// 0.93 ms for the same step as a CUDA graph of the stand-alone kernels. Per layer (us, block 0):
// QKV 8.6, attention 7.4 (+6.5 waiting for the slowest block), output projection 5.0, gate/up 19.6,
// down 15.5, barriers 1.7-3.4 each. With one block of 8 warps per SM a phase streams its weights at
// about 30 GB/s per SM, staging of the activations (two to five microseconds) is not overlapped with
// it, and 5 barriers a layer cost what the launch gaps did. The engine therefore uses this kernel
// only when LLMIE_STACKED_DECODE=1 is set; it is kept, tested, as the base for a version that
// overlaps phases.
//
// The math of every phase is that of the stand-alone kernels, whose code it follows:
//   gemm_fused_decode.cu  h * w staged as bfloat16 rows in shared memory, weights streamed
//                         straight into mma.sync fragments, rstd applied to the sums
//   attention_decode.cu   one cache page per work item, all query heads of a KV head; the group
//                         that finishes a (sequence, KV head) last merges its pages
// Data that another block wrote earlier in the same launch (h, q, attention partials, activations,
// this step's K/V rows) is read with loads that bypass L1, which is not coherent between SMs.
// All phases share one copy of the product code (a loop over phase descriptors): five inlined
// copies made the compiler keep the weight buffers in local memory.
//
// Limits (the caller checks them and otherwise runs the per-kernel path): bfloat16 weights and
// cache, at most 8 sequences, pages of 64, head size 64 or 128 with the whole head rotated, at
// most 8 query heads per KV head, no window, widths that are multiples of 32, and eight rows of
// the widest activation must fit one SM's shared memory.
#include "common.cuh"
#include <cooperative_groups.h>
#include <math.h>

namespace llmie {

constexpr int kStWarps = 8;
constexpr int kStThreads = kStWarps * 32;
constexpr int kStUnroll = 4;
constexpr int kStPad = 32;                 // bfloat16 elements of padding per staged row
constexpr int kStMaxGroups = 4;               // attention work groups per block, at most
constexpr int kStatusBarrierTimeout = 4;

struct StackLayer {                        // one entry of the run order
  const __nv_bfloat16* wqkv;               // [(n_q + 2 n_kv) hd, d]
  const __nv_bfloat16* wo;                 // [d, n_q hd]
  const __nv_bfloat16* wgu;                // [2 ff, d] = [gate rows; up rows]
  const __nv_bfloat16* wdown;              // [d, ff]
  const float* norm1;
  const float* norm2;
  __nv_bfloat16* k_cache;                  // [pages, n_kv, 64, hd]
  __nv_bfloat16* v_cache;
  const float2* rope_table;                // [table_len, hd / 2] (cos, sin)
  float eps1, eps2;
  float scale;                             // of the scores
  int table_len;
  int write_kv;                            // 0: this entry reads an earlier entry's cache
  int pad_;
};

struct StackParams {
  const StackLayer* layers;
  int n_layers;
  const __nv_bfloat16* embedding;          // [vocab, d]
  const float* final_norm;
  float final_eps;
  const __nv_bfloat16* head;               // [vocab, d]
  int vocab, d, ff, n_q, n_kv, hd;
  const int* tokens;                       // [batch]
  const int* slots;                        // [batch]
  int* seq_lens;                           // [slots]: tokens each sequence holds; advanced at the end
  int batch, scratch_slot;
  const int* block_table;
  int max_pages, n_runs;                   // n_runs * 64 covers the longest sequence of this launch
  int red_offset;                          // bytes of shared memory before the reduction scratch
  int s_qkv, s_o, s_gate, s_down, s_head;  // warps per team in each product phase
  int* counters;                           // [8 n_kv], zero between launches
  float* h;                                // [8, d]
  __nv_bfloat16* q;                        // [8, n_q hd]
  __nv_bfloat16* attn;                     // [8, n_q hd]
  __nv_bfloat16* act;                      // [8, ff]
  float* part_m;                           // [8, n_q, n_runs]
  float* part_l;
  float* part_acc;                         // [8, n_q, n_runs, hd]
  float* logits;                           // [8, vocab]
  unsigned long long* bar_counter;         // never reset; see grid_barrier
  unsigned long long* epoch;               // launches so far
  int* status;
  unsigned long long* phase_ns;            // optional [10 n_layers + 2]: block 0's clock at the start and after every phase
};

__device__ __forceinline__ void st_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 st_ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint4 st_ldcg16(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ unsigned st_pack(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}
__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]) {
  const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(hh[i]);
    out[2 * i] = f.x;
    out[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void group_sync(int group, int threads) {      // the threads of one attention work group
  asm volatile("bar.sync %0, %1;" ::"r"(group + 1), "r"(threads) : "memory");
}

// All blocks of the launch meet here. The counter only ever grows: barrier number k of launch
// number e completes when it reaches (e * barriers_per_launch + k + 1) * blocks, so nothing has
// to be reset while some block may still be polling. The wait is bounded; a block that gives up
// sets the status word and the whole launch winds down (every other block gives up at the same
// barrier). Returns false when the launch is to be abandoned.
__device__ __forceinline__ bool grid_barrier(unsigned long long* counter, unsigned long long target, int* status, int* s_abort) {
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    atomicAdd(counter, 1ull);
    unsigned spins = 0;
    while (ld_acquire_u64(counter) < target) {
      if (++spins > (1u << 22)) {
        atomicExch(status, kStatusBarrierTimeout);
        *s_abort = 1;
        break;
      }
    }
    __threadfence();
  }
  __syncthreads();
  return *s_abort == 0;
}

enum StackGemm { kGemmQkvRope = 0, kGemmGateSwiGLU = 1, kGemmF32 = 2, kGemmAddH = 3 };

__device__ __forceinline__ void st_tile_rows(int VAR, int tile, int hd, int half_n, int& lo, int& hi) {
  if (VAR == kGemmQkvRope) {
    const int per_head = hd >> 4;
    const int head = tile / per_head, i0 = (tile - head * per_head) << 3;
    lo = head * hd + i0;
    hi = lo + (hd >> 1);
  } else if (VAR == kGemmGateSwiGLU) {
    lo = tile << 3;
    hi = half_n + lo;
  } else {
    lo = tile << 4;
    hi = lo + 8;
  }
}

struct StackShared {
  int pos[8];
  int slot[8];
  int tok[8];
  float ssw[kStWarps * 8];     // sums of squares of the staged rows, per warp
  int last[kStMaxGroups];
  int abort;
};

__device__ __forceinline__ void team_sync(int team, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(team + 1), "r"(threads) : "memory");
}

// Rows of h * w (or of the embedding row * w at the first layer) as bfloat16 in shared memory, and
// per warp the sums of squares of the rows. A thread takes eight consecutive elements of four rows
// at a time, so those loads are in flight together while few registers are held. With FROM_EMB,
// block b also writes row b of the float32 residual stream. Ends with a block barrier.
__device__ __forceinline__ void stage_normed(bool FROM_EMB, const StackParams& p, const float* norm_w, int K,
                                             __nv_bfloat16* xs, StackShared& sh) {
  const int xs_stride = K + kStPad;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
  for (int b0 = 0; b0 < 8; b0 += 4) {
    float ssq[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = threadIdx.x * 8; k < K; k += kStThreads * 8) {
      float wv[8];
      load8(norm_w + k, wv);
      float hv[4][8];
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int b = b0 + r;
        if (b < p.batch) {
          if (FROM_EMB) {
            unpack8(st_ldg16(p.embedding + (size_t)sh.tok[b] * K + k), hv[r]);
          } else {
            const float4 a = __ldcg(reinterpret_cast<const float4*>(p.h + (size_t)b * K + k));
            const float4 c = __ldcg(reinterpret_cast<const float4*>(p.h + (size_t)b * K + k + 4));
            hv[r][0] = a.x; hv[r][1] = a.y; hv[r][2] = a.z; hv[r][3] = a.w;
            hv[r][4] = c.x; hv[r][5] = c.y; hv[r][6] = c.z; hv[r][7] = c.w;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 8; ++e) hv[r][e] = 0.f;
        }
      }
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        const int b = b0 + r;
        if (FROM_EMB && b < p.batch && (int)blockIdx.x == b) store8(p.h + (size_t)b * K + k, hv[r]);
        uint4 packed;
        packed.x = st_pack(hv[r][0] * wv[0], hv[r][1] * wv[1]);
        packed.y = st_pack(hv[r][2] * wv[2], hv[r][3] * wv[3]);
        packed.z = st_pack(hv[r][4] * wv[4], hv[r][5] * wv[5]);
        packed.w = st_pack(hv[r][6] * wv[6], hv[r][7] * wv[7]);
        *reinterpret_cast<uint4*>(xs + (size_t)b * xs_stride + k) = packed;
#pragma unroll
        for (int e = 0; e < 8; ++e) ssq[r] = fmaf(hv[r][e], hv[r][e], ssq[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < 4; ++r) {
      const float v = warp_sum(ssq[r]);
      if (lane == 0) sh.ssw[warp * 8 + b0 + r] = v;
    }
  }
  __syncthreads();
}

// rows of a bfloat16 activation [batch, K] into shared memory. Ends with a block barrier.
__device__ __forceinline__ void stage_plain(const StackParams& p, const __nv_bfloat16* src, int K, __nv_bfloat16* xs) {
  const int xs_stride = K + kStPad;
  const int per_row = K >> 3;
#pragma unroll 4
  for (int i = threadIdx.x; i < 8 * per_row; i += kStThreads) {
    const int b = i / per_row, k = (i - b * per_row) << 3;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (b < p.batch) v = st_ldcg16(src + (size_t)b * K + k);
    *reinterpret_cast<uint4*>(xs + (size_t)b * xs_stride + k) = v;
  }
  __syncthreads();
}

// Fused epilogue of one tile for the lane that holds rows (g, g + 8) and batch columns 2t, 2t + 1.
__device__ __forceinline__ void tile_epilogue(int VAR, const StackParams& p, const StackLayer* L, const float (&acc)[4], int lo,
                                              int hi, int g, int t, float rs0, float rs1, void* out, int ldo,
                                              const StackShared& sh) {
  const int hd = p.hd;
#pragma unroll
  for (int cc = 0; cc < 2; ++cc) {
    const int b = 2 * t + cc;
    if (b >= p.batch) continue;
    const float rs = cc ? rs1 : rs0;
    float x1 = acc[cc] * rs, x2 = acc[2 + cc] * rs;
    if (VAR == kGemmF32) {
      float* o = reinterpret_cast<float*>(out) + (size_t)b * ldo;
      o[lo + g] = x1;
      o[hi + g] = x2;
    } else if (VAR == kGemmAddH) {
      float* o = reinterpret_cast<float*>(out) + (size_t)b * ldo;
      o[lo + g] = __ldcg(o + lo + g) + x1;
      o[hi + g] = __ldcg(o + hi + g) + x2;
    } else if (VAR == kGemmGateSwiGLU) {
      const float a = x1 / (1.f + expf(-x1)) * x2;
      reinterpret_cast<__nv_bfloat16*>(out)[(size_t)b * ldo + lo + g] = __float2bfloat16_rn(a);
    } else {
      const int head = lo / hd, i = lo - head * hd + g, half = hd >> 1;
      const int pos = sh.pos[b];
      if (head < p.n_q + p.n_kv) {
        const float2 cs = L->rope_table[(size_t)min(pos, L->table_len - 1) * half + i];
        const float y1 = x1 * cs.x - x2 * cs.y, y2 = x2 * cs.x + x1 * cs.y;
        x1 = y1;
        x2 = y2;
      }
      __nv_bfloat16* dst = nullptr;
      if (head < p.n_q) {
        dst = p.q + ((size_t)b * p.n_q + head) * hd;
      } else if (L->write_kv) {
        const int page = p.block_table[(size_t)sh.slot[b] * p.max_pages + pos / 64];
        const bool is_k = head < p.n_q + p.n_kv;
        const int hk = head - p.n_q - (is_k ? 0 : p.n_kv);
        dst = (is_k ? L->k_cache : L->v_cache) + (((size_t)page * p.n_kv + hk) * 64 + (pos & 63)) * hd;
      }
      if (dst) {
        dst[i] = __float2bfloat16_rn(x1);
        dst[i + half] = __float2bfloat16_rn(x2);
      }
    }
  }
}

// End of a tile: the team's partial sums meet in its first warp (two buffers of shared memory in
// turn, one team barrier per tile), whose lanes then run the epilogue; the sums start again at zero.
__device__ __forceinline__ void finish_tile(int VAR, const StackParams& p, const StackLayer* L, float (&acc)[4], int S,
                                            int team, int j, int warp, int lane, int g, int t, int& parity,
                                            float4* red, int tile, int hd, int half_n, float rs0, float rs1,
                                            void* out, int ldo, const StackShared& sh) {
  if (S > 1) {
    float4* mine = red + ((parity * kStWarps + warp) * 32 + lane);
    if (j != 0) *mine = make_float4(acc[0], acc[1], acc[2], acc[3]);
    team_sync(team, S * 32);
    if (j == 0) {
      for (int o = 1; o < S; ++o) {
        const float4 v = mine[o * 32];
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
      }
    }
    parity ^= 1;
  }
  if (j == 0) {
    int lo, hi;
    st_tile_rows(VAR, tile, hd, half_n, lo, hi);
    tile_epilogue(VAR, p, L, acc, lo, hi, g, t, rs0, rs1, out, ldo, sh);
  }
  acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
}

// One product phase: out = x W^T over tiles of 16 weight rows, x being the staged rows.
//
// The block's warps form teams of S warps. A team takes a tile at a time (tile numbers
// go round the SMs first, so few tiles still spread over all of them); each of its warps owns a
// contiguous run of K and streams its share of the 16 rows straight into mma.sync fragments.
// A warp's work is a flat sequence of rounds (kStUnroll chunks of 32 each) that runs on across
// tile boundaries; two register buffers take turns, so that the loads of the next round are
// always issued before the current round is waited for, and a buffer is never copied (a copy
// would wait for its loads). Partial sums meet in the team's first warp through shared memory
// (two buffers in turn, one team barrier per tile), and that warp's lanes hold whole
// (row, row + 8) x (column pair) results, which is what every epilogue needs: rotation pairs,
// gate and up rows, or plain stores. S is chosen by the launcher so that the teams of the grid
// cover the tiles in one pass where that is possible. The first loads are issued before x is staged.
__device__ __forceinline__ void gemm_phase(int VAR, bool NORMED, bool FROM_EMB, const StackParams& p, const StackLayer* L, const __nv_bfloat16* W, int K,
                                        int tiles, int half_n, void* out, int ldo, int S, const float* norm_w,
                                        float eps, const __nv_bfloat16* x_src, __nv_bfloat16* xs, float4* red,
                                        StackShared& sh) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  const int team = warp / S, j = warp - team * S;
  const int n_chunks = K >> 5;
  const int per_warp = (n_chunks + S - 1) / S;
  const int c_begin = j * per_warp, c_end = min(n_chunks, c_begin + per_warp);
  const int hd = p.hd;
  const int xs_stride = K + kStPad;
  const int tile_stride = (kStWarps / S) * gridDim.x;
  const bool has_k = c_begin < c_end;          // a warp beyond the end of K only joins the team's barriers
  // where the next loads come from
  // rounds of a tile are taken in a rotated order that differs from SM to SM, so that the SMs do not
  // all ask for the same offset within their rows at the same time
  const int n_rounds = has_k ? (c_end - c_begin + kStUnroll - 1) / kStUnroll : 1;
  const int rot = (blockIdx.x * 5 + team * 3) % n_rounds;
  int ltile = team * gridDim.x + blockIdx.x, lr = 0;
  const uint4* lw_lo = nullptr;
  const uint4* lw_hi = nullptr;
#define LLMIE_POINT_LOADS()                                                          \
  do {                                                                               \
    if (ltile < tiles) {                                                             \
      int ra_, rb_;                                                                  \
      st_tile_rows(VAR, ltile, hd, half_n, ra_, rb_);                                \
      lw_lo = reinterpret_cast<const uint4*>(W + (size_t)(ra_ + g) * K) + t;         \
      lw_hi = reinterpret_cast<const uint4*>(W + (size_t)(rb_ + g) * K) + t;         \
    }                                                                                \
  } while (0)
  // the loads of the next round into one of the two register buffers
#define LLMIE_ISSUE(wa, wb)                                                          \
  do {                                                                               \
    if (ltile < tiles && has_k) {                                                    \
      int rr_ = lr + rot;                                                            \
      if (rr_ >= n_rounds) rr_ -= n_rounds;                                          \
      const int lc0_ = c_begin + rr_ * kStUnroll;                                    \
      _Pragma("unroll") for (int u = 0; u < kStUnroll; ++u) {                        \
        const int c = lc0_ + u;                                                      \
        if (c < c_end) {                                                             \
          wa[u] = st_ldg16(lw_lo + c * 4);                                           \
          wb[u] = st_ldg16(lw_hi + c * 4);                                           \
        }                                                                            \
      }                                                                              \
      if (++lr >= n_rounds) {                                                        \
        lr = 0;                                                                      \
        ltile += tile_stride;                                                        \
        LLMIE_POINT_LOADS();                                                         \
      }                                                                              \
    }                                                                                \
  } while (0)
  // one round of math from a buffer; at the end of a tile, the team's sums and the epilogue
#define LLMIE_CONSUME(wa, wb)                                                        \
  do {                                                                               \
    int rr_ = cr + rot;                                                              \
    if (rr_ >= n_rounds) rr_ -= n_rounds;                                            \
    const int c0_ = c_begin + rr_ * kStUnroll;                                       \
    _Pragma("unroll") for (int u = 0; u < kStUnroll; ++u) {                          \
      const int c = c0_ + u;                                                         \
      if (c < c_end) {                                                               \
        const uint4 xv = x_row[c * 4];                                               \
        st_mma(acc, wa[u].x, wb[u].x, wa[u].y, wb[u].y, xv.x, xv.y);                 \
        st_mma(acc2, wa[u].z, wb[u].z, wa[u].w, wb[u].w, xv.z, xv.w);                \
      }                                                                              \
    }                                                                                \
    if (++cr >= n_rounds) {                                                          \
      _Pragma("unroll") for (int i = 0; i < 4; ++i) {                                \
        acc[i] += acc2[i];                                                           \
        acc2[i] = 0.f;                                                               \
      }                                                                              \
      finish_tile(VAR, p, L, acc, S, team, j, warp, lane, g, t, parity, red, tile, hd, half_n, rs0, rs1, out, ldo, \
                  sh);                                                               \
      cr = 0;                                                                        \
      tile += tile_stride;                                                           \
    }                                                                                \
  } while (0)

  LLMIE_POINT_LOADS();
  uint4 a0[kStUnroll], b0[kStUnroll], a1[kStUnroll], b1[kStUnroll];
  LLMIE_ISSUE(a0, b0);

  float rs0 = 1.f, rs1 = 1.f;        // rstd of the two batch columns this lane holds
  if (NORMED) {
    stage_normed(FROM_EMB, p, norm_w, K, xs, sh);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int w = 0; w < kStWarps; ++w) {
      s0 += sh.ssw[w * 8 + 2 * t];
      s1 += sh.ssw[w * 8 + 2 * t + 1];
    }
    rs0 = rsqrtf(s0 / (float)K + eps);
    rs1 = rsqrtf(s1 / (float)K + eps);
  } else {
    stage_plain(p, x_src, K, xs);
  }
  const uint4* x_row = reinterpret_cast<const uint4*>(xs + (size_t)g * xs_stride) + t;

  int tile = team * gridDim.x + blockIdx.x, cr = 0, parity = 0;
  float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};   // two chains of products, summed per tile
  while (tile < tiles) {
    LLMIE_ISSUE(a1, b1);
    LLMIE_CONSUME(a0, b0);
    if (tile >= tiles) break;
    LLMIE_ISSUE(a0, b0);
    LLMIE_CONSUME(a1, b1);
  }
#undef LLMIE_POINT_LOADS
#undef LLMIE_ISSUE
#undef LLMIE_CONSUME
}

// Merge of the pages of one (sequence, query head) by one warp (src/flash_decode.py:182-205):
// M = max m_r, w_r = exp(m_r - M), out = sum w_r acc_r / sum w_r l_r over the pages in order.
template <int HD>
__device__ __forceinline__ void merge_head(const StackParams& p, int seq, int head, int r1) {
  const int lane = threadIdx.x & 31;
  const size_t base = ((size_t)seq * p.n_q + head) * p.n_runs;
  float M = -INFINITY;
  for (int r = lane; r <= r1; r += 32) M = fmaxf(M, __ldcg(p.part_m + base + r));
  M = warp_max(M);
  float denom = 0.f;
  float num[HD / 32];
#pragma unroll
  for (int i = 0; i < HD / 32; ++i) num[i] = 0.f;
  for (int r0 = 0; r0 <= r1; r0 += 32) {
    const int r = r0 + lane;
    float w = 0.f;
    if (r <= r1) {
      w = expf(__ldcg(p.part_m + base + r) - M);
      denom = fmaf(w, __ldcg(p.part_l + base + r), denom);
    }
    const int n_here = min(32, r1 - r0 + 1);
#pragma unroll 8
    for (int i = 0; i < n_here; ++i) {
      const float wi = __shfl_sync(0xffffffffu, w, i);
#pragma unroll
      for (int k = 0; k < HD / 32; ++k)
        num[k] = fmaf(wi, __ldcg(p.part_acc + (base + r0 + i) * HD + lane + 32 * k), num[k]);
    }
  }
  denom = warp_sum(denom);
  const float inv = 1.f / denom;
#pragma unroll
  for (int k = 0; k < HD / 32; ++k)
    p.attn[((size_t)seq * p.n_q + head) * HD + lane + 32 * k] = __float2bfloat16_rn(num[k] * inv);
}

// One attention work item: page `run` of KV head `hk` of sequence `seq`, for all G query heads,
// by one group of GW warps (see attention_decode.cu). att_smem: this group's scratch. The page's
// K and V rows are requested up front and stay packed in registers; the query heads are taken
// four at a time to bound the register count.
template <int HD, int GW>
__device__ __forceinline__ void attention_item(const StackParams& p, const StackLayer* L, int seq, int hk, int run, int group,
                               float* att_smem, StackShared& sh) {
  constexpr int E = 8, LPK = HD / E, KPW = 32 / LPK, kRun = 64, kWarps = GW, GC = 4;
  constexpr int kIter = kRun / (kWarps * KPW);
  float(*scores)[kRun] = reinterpret_cast<float(*)[kRun]>(att_smem);                   // [8][kRun]
  float(*red)[GC][HD] = reinterpret_cast<float(*)[GC][HD]>(att_smem + 8 * kRun);       // [kWarps][GC][HD]
  const int G = p.n_q / p.n_kv;
  const float scale = L->scale;
  const int len = sh.pos[seq] + 1;
  const int begin = run * kRun, end = min(len, (run + 1) * kRun);
  if (begin >= end) return;
  const int n_keys = end - begin;
  const int tid = threadIdx.x % (GW * 32), warp = tid >> 5, lane = tid & 31;
  const int sub = lane / LPK, e0 = (lane % LPK) * E;
  const int page = p.block_table[(size_t)sh.slot[seq] * p.max_pages + run];
  const size_t base = ((size_t)page * p.n_kv + hk) * (size_t)kRun * HD;
  uint4 kraw[kIter], vraw[kIter];
#pragma unroll
  for (int it = 0; it < kIter; ++it)
    kraw[it] = st_ldcg16(L->k_cache + base + (size_t)((it * kWarps + warp) * KPW + sub) * HD + e0);
#pragma unroll
  for (int it = 0; it < kIter; ++it)
    vraw[it] = st_ldcg16(L->v_cache + base + (size_t)((it * kWarps + warp) * KPW + sub) * HD + e0);
  for (int g0 = 0; g0 < G; g0 += GC) {
    float qv[GC][E];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      if (g0 + g < G) {
        float tmp[E];
        unpack8(st_ldcg16(p.q + ((size_t)seq * p.n_q + (size_t)hk * G + g0 + g) * HD + e0), tmp);
#pragma unroll
        for (int e = 0; e < E; ++e) qv[g][e] = tmp[e] * scale;
      } else {
#pragma unroll
        for (int e = 0; e < E; ++e) qv[g][e] = 0.f;
      }
    }
#pragma unroll
    for (int it = 0; it < kIter; ++it) {
      const int row = (it * kWarps + warp) * KPW + sub;
      float kf[E];
      unpack8(kraw[it], kf);
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) dot = fmaf(qv[g][e], kf[e], dot);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        if ((lane % LPK) == 0 && g0 + g < G) scores[g0 + g][row] = dot;
      }
    }
  }
  group_sync(group, GW * 32);
  for (int g = warp; g < G; g += kWarps) {
    float* s = scores[g];
    float m = -INFINITY;
    for (int j = lane; j < kRun; j += 32) m = fmaxf(m, j < n_keys ? s[j] : -INFINITY);
    m = warp_max(m);
    float l = 0.f;
    for (int j = lane; j < kRun; j += 32) {
      const float pr = j < n_keys ? expf(s[j] - m) : 0.f;
      s[j] = pr;
      l += pr;
    }
    l = warp_sum(l);
    if (lane == 0) {
      const size_t idx = ((size_t)seq * p.n_q + (size_t)hk * G + g) * p.n_runs + run;
      p.part_m[idx] = m;
      p.part_l[idx] = l;
    }
  }
  group_sync(group, GW * 32);
  for (int g0 = 0; g0 < G; g0 += GC) {
    float acc[GC][E];
#pragma unroll
    for (int g = 0; g < GC; ++g)
#pragma unroll
      for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
#pragma unroll
    for (int it = 0; it < kIter; ++it) {
      const int row = (it * kWarps + warp) * KPW + sub;
      float vf[E];
      unpack8(vraw[it], vf);
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        const float pr = (g0 + g < G) ? scores[g0 + g][row] : 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) acc[g][e] = fmaf(pr, vf[e], acc[g][e]);
      }
    }
#pragma unroll
    for (int g = 0; g < GC; ++g)
#pragma unroll
      for (int e = 0; e < E; ++e)
#pragma unroll
        for (int o = 16; o >= LPK; o >>= 1) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
    if (lane < LPK) {
#pragma unroll
      for (int g = 0; g < GC; ++g)
#pragma unroll
        for (int e = 0; e < E; ++e) red[warp][g][e0 + e] = acc[g][e];
    }
    group_sync(group, GW * 32);
    for (int i = tid; i < GC * HD; i += GW * 32) {
      const int g = i / HD, d = i % HD;
      if (g0 + g >= G) continue;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) sum += red[w][g][d];
      p.part_acc[(((size_t)seq * p.n_q + (size_t)hk * G + g0 + g) * p.n_runs + run) * HD + d] = sum;
    }
    group_sync(group, GW * 32);      // the scratch is reused by the next four heads and by this group's next item
  }
  // ---- the group that finishes a (sequence, KV head) last merges its pages; the counter is left at zero
  const int r1 = (len - 1) / kRun;
  __threadfence();           // this group's partial results are visible before it is counted
  group_sync(group, GW * 32);
  if (tid == 0) {
    int* c = p.counters + seq * p.n_kv + hk;
    const int done = atomicAdd(c, 1) + 1;
    sh.last[group] = (done == r1 + 1);
    if (done == r1 + 1) *c = 0;
  }
  group_sync(group, GW * 32);
  if (!sh.last[group]) return;
  __threadfence();
  for (int g = warp; g < G; g += kWarps) merge_head<HD>(p, seq, hk * G + g, r1);
}

template <int HD>
__global__ void __launch_bounds__(kStThreads, 1) decode_stack_kernel(const __grid_constant__ StackParams p) {
  extern __shared__ __align__(16) unsigned char st_smem[];
  __shared__ StackShared sh;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(st_smem);          // [8][K + pad], K the phase's inner size
  float4* red = reinterpret_cast<float4*>(st_smem + p.red_offset);        // [2][warps][32 lanes]
  float* att_smem = reinterpret_cast<float*>(st_smem);                    // aliases xs during attention
  constexpr int GW = HD == 64 ? 2 : 4;             // warps per attention work group
  constexpr int kGroups = kStWarps / GW;
  constexpr int kAttFloats = 8 * 64 + GW * 4 * HD;

  if (threadIdx.x < 8) {
    const int b = threadIdx.x;
    const int slot = b < p.batch ? p.slots[b] : p.scratch_slot;
    sh.slot[b] = slot;
    sh.pos[b] = p.seq_lens[slot];
    sh.tok[b] = b < p.batch ? p.tokens[b] : 0;
  }
  if (threadIdx.x == 0) sh.abort = 0;
  __syncthreads();
  const unsigned long long per_launch = (unsigned long long)p.n_layers * 5ull;
  unsigned long long target = (*p.epoch) * per_launch * gridDim.x;
  const int group = threadIdx.x / (GW * 32);
  const int n_groups = gridDim.x * kGroups;
  int n_phase = 0;
#define LLMIE_STAMP()                                                                 \
  do {                                                                                 \
    if (p.phase_ns && blockIdx.x == 0 && threadIdx.x == 0) {                           \
      unsigned long long t_;                                                           \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                           \
      p.phase_ns[n_phase] = t_;                                                        \
    }                                                                                  \
    ++n_phase;                                                                         \
  } while (0)
#define LLMIE_BARRIER()                                                        \
  do {                                                                          \
    LLMIE_STAMP();                                                              \
    target += gridDim.x;                                                        \
    if (!grid_barrier(p.bar_counter, target, p.status, &sh.abort)) return;      \
    LLMIE_STAMP();                                                              \
  } while (0)
  LLMIE_STAMP();

  // The phases of the step in order: per layer A (norm, QKV, rotation, cache write), B (attention),
  // C (output projection, h += y), D (norm, gate / up, SwiGLU), E (down projection, h += y); at the
  // end the final norm and the head. One copy of the product code serves all of them.
  const int n_phases = p.n_layers * 5 + 1;
  for (int ph = 0; ph < n_phases; ++ph) {
    const int l = ph / 5;
    const int kind = (ph == n_phases - 1) ? 5 : ph - l * 5;
    const StackLayer* L = p.layers + (l < p.n_layers ? l : p.n_layers - 1);
    if (kind == 1) {
      // one cache page per work item; pages in the outer order, so that the pages that hold keys
      // come first and spread over all groups
      const int per_run = p.batch * p.n_kv;
      const int n_items = per_run * p.n_runs;
      for (int item = blockIdx.x * kGroups + group; item < n_items; item += n_groups) {
        const int run = item / per_run, rest = item - run * per_run;
        attention_item<HD, GW>(p, L, rest / p.n_kv, rest % p.n_kv, run, group, att_smem + group * kAttFloats, sh);
      }
    } else {
      int var, K, tiles, half_n = 0, ldo, S;
      bool normed = false;
      const __nv_bfloat16* W;
      const __nv_bfloat16* x_src = nullptr;
      const float* norm_w = nullptr;
      float eps = 0.f;
      void* out;
      if (kind == 0) {
        var = kGemmQkvRope; normed = true; W = L->wqkv; K = p.d; tiles = (p.n_q + 2 * p.n_kv) * (HD >> 4);
        out = nullptr; ldo = 0; S = p.s_qkv; norm_w = L->norm1; eps = L->eps1;
      } else if (kind == 2) {
        var = kGemmAddH; W = L->wo; K = p.n_q * HD; tiles = p.d >> 4; out = p.h; ldo = p.d; S = p.s_o; x_src = p.attn;
      } else if (kind == 3) {
        var = kGemmGateSwiGLU; normed = true; W = L->wgu; K = p.d; tiles = p.ff >> 3; half_n = p.ff;
        out = p.act; ldo = p.ff; S = p.s_gate; norm_w = L->norm2; eps = L->eps2;
      } else if (kind == 4) {
        var = kGemmAddH; W = L->wdown; K = p.ff; tiles = p.d >> 4; out = p.h; ldo = p.d; S = p.s_down; x_src = p.act;
      } else {
        var = kGemmF32; normed = true; W = p.head; K = p.d; tiles = p.vocab >> 4; out = p.logits; ldo = p.vocab;
        S = p.s_head; norm_w = p.final_norm; eps = p.final_eps;
      }
      gemm_phase(var, normed, ph == 0, p, L, W, K, tiles, half_n, out, ldo, S, norm_w, eps, x_src, xs, red, sh);
    }
    if (ph + 1 < n_phases) LLMIE_BARRIER();
  }
#undef LLMIE_BARRIER
  LLMIE_STAMP();
#undef LLMIE_STAMP
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    for (int b = 0; b < p.batch; ++b)
      if (sh.slot[b] != p.scratch_slot) p.seq_lens[sh.slot[b]] = sh.pos[b] + 1;
    *p.epoch += 1ull;
  }
}

// Shared memory: the staged rows (or the attention scratch of the four work groups, whichever is
// larger), then the reduction scratch.
static size_t stack_staging_bytes(int d, int ff, int n_q, int hd) {
  int kmax = d > ff ? d : ff;
  if (n_q * hd > kmax) kmax = n_q * hd;
  const size_t rows = (size_t)8 * (kmax + kStPad) * 2;
  const size_t att = (size_t)kStMaxGroups * (8 * 64 + 4 * 4 * hd) * sizeof(float);
  return rows > att ? rows : att;
}
static size_t stack_smem_bytes(int d, int ff, int n_q, int hd) {
  return stack_staging_bytes(d, ff, n_q, hd) + (size_t)2 * kStWarps * 32 * sizeof(float4);
}

template <int HD>
static int launch_stack(StackParams& p, cudaStream_t stream) {
  p.red_offset = (int)stack_staging_bytes(p.d, p.ff, p.n_q, HD);
  const size_t smem = stack_smem_bytes(p.d, p.ff, p.n_q, HD);
  if (smem > 220 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  cudaError_t e = cudaFuncSetAttribute(decode_stack_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       (int)smem);
  if (e != cudaSuccess) return (int)e;
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_stack_kernel<HD>, kStThreads, smem);
  if (e != cudaSuccess) return (int)e;
  if (per_sm < 1) return LLMIE_ERR_UNSUPPORTED_SIZE;
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  // warps per team: as many as leave every tile of the phase a team of its own in one pass
  auto team_size = [sms](int tiles) {
    int s = kStWarps;
    while (s > 1 && (long long)tiles * s > (long long)sms * kStWarps) s >>= 1;
    return s;
  };
  p.s_qkv = team_size((p.n_q + 2 * p.n_kv) * (HD >> 4));
  p.s_o = team_size(p.d >> 4);
  p.s_gate = team_size(p.ff >> 3);
  p.s_down = team_size(p.d >> 4);
  p.s_head = team_size(p.vocab >> 4);
  // every block must be resident at once (they wait for one another): a cooperative launch of one block per SM
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(sms);
  cfg.blockDim = dim3(kStThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_stack_kernel<HD>, p);
  if (e != cudaSuccess) return (int)e;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

}  // namespace llmie

using namespace llmie;

extern "C" int llmie_decode_stack_layer_bytes(void) { return (int)sizeof(StackLayer); }

// 1 when decode_stack takes these sizes.
extern "C" int llmie_decode_stack_supported(int batch, int d, int ff, int n_q, int n_kv, int hd, int vocab) {
  if (batch < 1 || batch > 8) return 0;
  if (hd != 64 && hd != 128) return 0;
  if (n_q % n_kv || n_q / n_kv > 8) return 0;
  if (d % 32 || ff % 32 || (n_q * hd) % 32 || vocab % 16) return 0;
  if (stack_smem_bytes(d, ff, n_q, hd) > 220 * 1024) return 0;
  return 1;
}

// layers: device array of n_layers StackLayer records (see llmie_decode_stack_layer_bytes). All other
// pointers as in StackParams. bar_counter and epoch: two 64-bit words in device memory, zero before the
// first launch and never touched by the host again. counters: 8 n_kv int32, zero before the first
// launch (every launch leaves them zero). status: set to 4 if a grid barrier gave up.
// phase_ns: null, or 10 n_layers + 2 words that receive block 0's nanosecond clock at the start of the
// launch and after every phase (a measuring aid).
extern "C" int llmie_decode_stack(const void* layers, int n_layers, const void* embedding, const float* final_norm,
                                  float final_eps, const void* head, int vocab, int d, int ff, int n_q, int n_kv, int hd,
                                  const int* tokens,
                                  const int* slots, int* seq_lens, int batch, int scratch_slot, const int* block_table,
                                  int max_pages, int n_runs, float* h, void* q, void* attn, void* act, float* part_m,
                                  float* part_l, float* part_acc, float* logits, unsigned long long* bar_counter,
                                  unsigned long long* epoch, int* counters, int* status,
                                  unsigned long long* phase_ns, cudaStream_t stream) {
  if (!llmie_decode_stack_supported(batch, d, ff, n_q, n_kv, hd, vocab) || n_layers < 1 || n_runs < 1 ||
      max_pages < n_runs)
    return LLMIE_ERR_UNSUPPORTED_SIZE;
  StackParams p;
  p.layers = (const StackLayer*)layers;
  p.n_layers = n_layers;
  p.embedding = (const __nv_bfloat16*)embedding;
  p.final_norm = final_norm;
  p.final_eps = final_eps;
  p.head = (const __nv_bfloat16*)head;
  p.vocab = vocab; p.d = d; p.ff = ff; p.n_q = n_q; p.n_kv = n_kv; p.hd = hd;
  p.tokens = tokens; p.slots = slots; p.seq_lens = seq_lens;
  p.batch = batch; p.scratch_slot = scratch_slot;
  p.block_table = block_table; p.max_pages = max_pages; p.n_runs = n_runs;
  p.h = h;
  p.q = (__nv_bfloat16*)q; p.attn = (__nv_bfloat16*)attn; p.act = (__nv_bfloat16*)act;
  p.part_m = part_m; p.part_l = part_l; p.part_acc = part_acc; p.logits = logits;
  p.bar_counter = bar_counter; p.epoch = epoch; p.status = status;
  p.phase_ns = phase_ns;
  p.counters = counters;
  return hd == 64 ? launch_stack<64>(p, stream) : launch_stack<128>(p, stream);
}
