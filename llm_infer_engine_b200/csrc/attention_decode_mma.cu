// Attention for one-token steps on the tensor cores: a warp per cache page.
//
// One block serves one (sequence, KV head) - or one run of its pages - for up to 16 of the query
// heads that share the KV head. The 16 x head_dim block of queries is the A operand of
// mma.sync.m16n8k16; a WARP takes whole pages (64 keys), half a page at a time: it copies K and V
// rows into its own two-stage shared-memory tiles (cp.async, the next half page while it works on
// this one), computes S = Q K^T with 4 x head_dim/16 tensor-core products, keeps a running
// maximum and sum per query head in registers (the online softmax of src/flash_attn.py:118-134
// for one query row per head), converts P to bfloat16 in registers (the accumulator layout of two
// neighbouring 8-key tiles is the A layout of one 16-key step) and adds P V. Warps of a block take
// pages in turn and never wait for one another until the end, where their (max, sum, accumulator)
// triples meet in shared memory (src/flash_decode.py:182-205 is the same merge). A sequence whose
// pages all belong to one block is written straight to the output; otherwise each block leaves a
// partial result per run and the block that finishes last merges them, as in attention_decode.cu.
//
// Against the split-KV kernel on CUDA cores (attention_decode.cu): no block-wide barrier per
// page, no shuffle reductions per key, and a sequence is merged inside its block instead of
// through global memory. bfloat16 only (the float32 engine keeps the CUDA-core kernel), pages of
// 64 keys, head size 64 or 128. Scores, softmax statistics and accumulators are float32; the
// probabilities enter the second product as bfloat16, as the reference's do (src/flash_attn.py:131).
// Rows of a page beyond a sequence's length get probability zero; the cache holds finite numbers
// there (it starts as zeros and only ever receives keys and values).
#include "common.cuh"
#include <math.h>

namespace llmie {

constexpr int kMdPage = 64;

__device__ __forceinline__ int md_first_visible(int len, int window) {
  return (window > 0 && len - window > 0) ? len - window : 0;
}
__device__ __forceinline__ void md_mma(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                       unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void md_ldmatrix(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void md_ldmatrix_trans(unsigned (&r)[4], unsigned addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
// 2^x by the special-function unit. Scores are kept in units of log2 (scaled by log2 e once), so every
// exponential of the softmax and of the merges is this one instruction; -inf gives 0.
__device__ __forceinline__ float md_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned md_pack(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<unsigned*>(&v);
}

// Merge of the runs of one (sequence, query head) by one warp.
template <int HD>
__device__ __forceinline__ void md_merge_head(const float* part_m, const float* part_l, const float* part_acc,
                                              __nv_bfloat16* out_row, size_t base, int r0, int r1) {
  const int lane = threadIdx.x & 31;
  float M = -INFINITY;
  for (int r = r0 + lane; r <= r1; r += 32) M = fmaxf(M, __ldcg(part_m + base + r));
  M = warp_max(M);
  float denom = 0.f;
  float num[HD / 32];
#pragma unroll
  for (int i = 0; i < HD / 32; ++i) num[i] = 0.f;
  for (int c0 = r0; c0 <= r1; c0 += 32) {
    const int r = c0 + lane;
    float w = 0.f;
    if (r <= r1) {
      w = md_exp2(__ldcg(part_m + base + r) - M);
      denom = fmaf(w, __ldcg(part_l + base + r), denom);
    }
    const int n_here = min(32, r1 - c0 + 1);
#pragma unroll 4
    for (int i = 0; i < n_here; ++i) {
      const float wi = __shfl_sync(0xffffffffu, w, i);
#pragma unroll
      for (int k = 0; k < HD / 32; ++k) num[k] = fmaf(wi, __ldcg(part_acc + (base + c0 + i) * HD + lane + 32 * k), num[k]);
    }
  }
  denom = warp_sum(denom);
  const float inv = 1.f / denom;
#pragma unroll
  for (int k = 0; k < HD / 32; ++k) out_row[lane + 32 * k] = __float2bfloat16_rn(num[k] * inv);
}

// grid (n_runs, n_kv * chunks, n_seqs), chunks = ceil(G / 16); WARPS warps per block.
// With ROPE the kernel takes the step's raw projections instead of finished queries: `q` is then the packed
// [n_seqs, (n_q + 2 n_kv) * HD] rows of q, k and v heads (row pitch q_ld), `rope` the float32 (cos, sin) table
// [table_len, HD / 2]. Every lane rotates its own query fragments in registers (the rotate-half partner of a
// column lies HD / 2 columns on, which is the same lane's fragment KS / 2 k-steps on), and the one warp whose
// half page holds the sequence's newest position rotates the new key, puts key and value into its staged tile
// and (with write_kv) into the cache. Rotation in float32, one rounding to bfloat16, as the separate kernel.
template <int HD, int WARPS, bool ROPE>
__global__ void __launch_bounds__(WARPS * 32, (HD == 64 && WARPS <= 4) ? 16 / WARPS : 1)
decode_mma_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* k_cache,
                  const __nv_bfloat16* v_cache, float* __restrict__ part_m, float* __restrict__ part_l,
                  float* __restrict__ part_acc, const int* __restrict__ seq_slot, const int* __restrict__ seq_kvlen,
                  const int* __restrict__ block_table, int max_pages, int n_q, int n_kv, float scale, int window,
                  int pages_per_run, int n_runs, int* __restrict__ counters, __nv_bfloat16* __restrict__ out,
                  const float2* __restrict__ rope, int table_len, int q_ld, int write_kv) {
  pdl_launch_dependents();
  constexpr int PITCH = HD + 8;                         // elements; rows 16 bytes apart in the banks
  constexpr int KS = HD / 16;                           // k-steps of Q K^T
  constexpr int NT = HD / 8;                            // n-tiles of P V
  constexpr int kTile = kMdPage * PITCH;                // elements of one staged page of K (or V)
  constexpr int kPieces = HD / 8;                       // 16-byte pieces per row
  constexpr int kHalf = kMdPage / 2;                    // keys a warp works on at a time
  extern __shared__ __align__(16) unsigned char md_smem[];
  __shared__ int is_last;

  const int run = blockIdx.x, seq = blockIdx.z;
  const int G = n_q / n_kv;
  const int chunks = (G + 15) / 16;
  const int hk = blockIdx.y / chunks;
  const int g0 = (blockIdx.y % chunks) * 16;
  const int ng = min(16, G - g0);

  const int len = seq_kvlen[seq];
  const int lo = md_first_visible(len, window);
  const int p_first = max(run * pages_per_run, lo / kMdPage);
  const int p_last = min((run + 1) * pages_per_run - 1, (len - 1) / kMdPage);
  if (len <= 0 || p_first > p_last) return;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  // this warp's shared memory: two stages, each a half page (32 keys) of K and of V
  __nv_bfloat16* k_tile = reinterpret_cast<__nv_bfloat16*>(md_smem) + (size_t)warp * 2 * kTile;
  const unsigned tile_addr = (unsigned)__cvta_generic_to_shared(k_tile);
  constexpr unsigned kHalfBytes = (unsigned)(kHalf * PITCH * 2);          // one half page of K (or V)
  const int* pages = block_table + (size_t)seq_slot[seq] * max_pages;
  const size_t head_off = (size_t)hk * kMdPage * HD;
  const size_t page_stride = (size_t)n_kv * kMdPage * HD;

  // The warp's work is the sequence of half pages (p, h) of its pages that hold a visible key.
  auto visible = [&](int p, int h) {
    const int first = max(lo - p * kMdPage, 0), last = min(len - p * kMdPage, kMdPage);
    return max(first, h * kHalf) < min(last, h * kHalf + kHalf);
  };
  auto advance = [&](int& p, int& h) {
    do {
      if (++h == 2) {
        h = 0;
        p += WARPS;
      }
    } while (p <= p_last && !visible(p, h));
  };
  // K and V rows of half page (p, h) into stage s: one group of asynchronous copies
  auto issue = [&](int p, int h, int s) {
    const size_t src = (size_t)pages[p] * page_stride + head_off + (size_t)h * kHalf * HD;
    const unsigned dst = tile_addr + (unsigned)s * 2u * kHalfBytes;
#pragma unroll
    for (int i = 0; i < kHalf * kPieces / 32; ++i) {
      const int idx = i * 32 + lane;
      const int row = idx / kPieces, piece = idx % kPieces;
      const unsigned off = (unsigned)(row * PITCH + piece * 8) * 2u;
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + off),
                   "l"(k_cache + src + (size_t)row * HD + piece * 8) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + kHalfBytes + off),
                   "l"(v_cache + src + (size_t)row * HD + piece * 8) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  int p = p_first + warp, h = 0;
  if (p <= p_last && !visible(p, h)) advance(p, h);
  int np = p, nh = h;                                    // the unit after (p, h)
  if (p <= p_last) advance(np, nh);
  // The kernel before this one wrote the queries and the newest key and value, which lie in the
  // sequence's last page. Lengths, slots and the page table were written before that kernel was even
  // launched, and every other page long ago: those are read, and their copies requested, while the
  // previous kernel is still running.
  const int p_new = (len - 1) / kMdPage;
  const bool early0 = p <= p_last && p != p_new, early1 = early0 && np <= p_last && np != p_new;
  if (early0) issue(p, h, 0);
  if (early1) issue(np, nh, 1);
  pdl_wait();
  if (p <= p_last && !early0) issue(p, h, 0);
  if (np <= p_last && !early1) issue(np, nh, 1);
  // the queries of this head group as A fragments: rows g and g + 8, all of head_dim
  unsigned qa[KS][4];
  {
    const size_t q_row = ROPE ? (size_t)seq * q_ld : (size_t)seq * n_q * HD;
    const __nv_bfloat16* q_lo = q + q_row + ((size_t)hk * G + g0 + g) * HD;
    const __nv_bfloat16* q_hi = q_lo + (size_t)8 * HD;
    const bool lo_ok = g < ng, hi_ok = g + 8 < ng;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
      const int c = ks * 16 + 2 * t;
      qa[ks][0] = lo_ok ? *reinterpret_cast<const unsigned*>(q_lo + c) : 0u;
      qa[ks][1] = hi_ok ? *reinterpret_cast<const unsigned*>(q_hi + c) : 0u;
      qa[ks][2] = lo_ok ? *reinterpret_cast<const unsigned*>(q_lo + c + 8) : 0u;
      qa[ks][3] = hi_ok ? *reinterpret_cast<const unsigned*>(q_hi + c + 8) : 0u;
    }
    if constexpr (ROPE) {
      const int tpos = min(len - 1, table_len - 1);
      const float2* cs = rope + (size_t)tpos * (HD / 2);
#pragma unroll
      for (int ks = 0; ks < KS / 2; ++ks) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {                    // registers 0, 1: columns c, c + 1; 2, 3: c + 8, c + 9
          const int c = ks * 16 + 2 * t + (r >> 1) * 8;
          const float2 c0 = cs[c], c1 = cs[c + 1];
          const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[ks][r]));
          const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[ks + KS / 2][r]));
          qa[ks][r] = md_pack(x1.x * c0.x - x2.x * c0.y, x1.y * c1.x - x2.y * c1.y);
          qa[ks + KS / 2][r] = md_pack(x2.x * c0.x + x1.x * c0.y, x2.y * c1.x + x1.y * c1.y);
        }
      }
    }
  }
  float o[NT][4];
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) o[nt][0] = o[nt][1] = o[nt][2] = o[nt][3] = 0.f;
  float m_lo = -INFINITY, m_hi = -INFINITY;            // running maxima of rows g and g + 8 (units of log2)
  float l_lo = 0.f, l_hi = 0.f;                        // this lane's share of the running sums

  const float scale2 = scale * 1.4426950408889634f;    // scores in units of log2
  // ldmatrix row addresses: lane i gives row (i & 7) of matrix (i >> 3)
  const int lm_r = lane & 7, lm_m = lane >> 3;
  for (int idx = 0; p <= p_last; ++idx) {
    const int s_ = idx & 1;
    const unsigned k_addr = tile_addr + (unsigned)s_ * 2u * kHalfBytes, v_addr = k_addr + kHalfBytes;
    if (np <= p_last) asm volatile("cp.async.wait_group 1;" ::: "memory");   // this unit has arrived, the next is on its way
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    if constexpr (ROPE) {
      if (p == p_new && h == ((len - 1) % kMdPage) / kHalf) {
        // the sequence's newest position lies in this half page: its key and value come from the step's
        // projections, not from the cache (which holds whatever the page held before at that row)
        const int row = (len - 1) % kHalf;
        const __nv_bfloat16* k_raw = q + (size_t)seq * q_ld + (size_t)(n_q + hk) * HD;
        const __nv_bfloat16* v_raw = k_raw + (size_t)n_kv * HD;
        const int tpos = min(len - 1, table_len - 1);
        const float2* cs = rope + (size_t)tpos * (HD / 2);
        __nv_bfloat16* k_row = k_tile + (size_t)s_ * 2 * (kHalf * PITCH) + (size_t)row * PITCH;
        __nv_bfloat16* v_row = k_row + kHalf * PITCH;
        const bool to_cache = write_kv && g0 == 0;       // one writer per (sequence, KV head)
        const size_t dst = (size_t)pages[p] * page_stride + head_off + (size_t)(h * kHalf + row) * HD;
        for (int d = lane; d < HD / 2; d += 32) {
          const float2 c = cs[d];
          const float x1 = __bfloat162float(k_raw[d]), x2 = __bfloat162float(k_raw[d + HD / 2]);
          const __nv_bfloat16 y1 = __float2bfloat16_rn(x1 * c.x - x2 * c.y);
          const __nv_bfloat16 y2 = __float2bfloat16_rn(x2 * c.x + x1 * c.y);
          const __nv_bfloat16 v1 = v_raw[d], v2 = v_raw[d + HD / 2];
          k_row[d] = y1;
          k_row[d + HD / 2] = y2;
          v_row[d] = v1;
          v_row[d + HD / 2] = v2;
          if (to_cache) {
            __nv_bfloat16* kc = const_cast<__nv_bfloat16*>(k_cache) + dst;
            __nv_bfloat16* vc = const_cast<__nv_bfloat16*>(v_cache) + dst;
            kc[d] = y1;
            kc[d + HD / 2] = y2;
            vc[d] = v1;
            vc[d + HD / 2] = v2;
          }
        }
        __syncwarp();
      }
    }
    // ---- S = Q K^T: 4 tiles of 8 keys
    float s[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ++ks) {
#pragma unroll
      for (int pr = 0; pr < 2; ++pr) {                   // pairs of key tiles
        unsigned b[4];
        const int key = (2 * pr + (lm_m >> 1)) * 8 + lm_r, col = ks * 16 + (lm_m & 1) * 8;
        md_ldmatrix(b, k_addr + (unsigned)(key * PITCH + col) * 2u);
        md_mma(s[2 * pr], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[0], b[1]);
        md_mma(s[2 * pr + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b[2], b[3]);
      }
    }
    // ---- scale, mask, running maximum and sum; probabilities relative to the new maximum
    const int first = max(lo - p * kMdPage, 0) - h * kHalf;
    const int last = min(len - p * kMdPage, kMdPage) - h * kHalf;       // visible keys of the half page: [first, last)
    float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int key = nt * 8 + 2 * t + c;
        const bool vis = key >= first && key < last;
        s[nt][c] = vis ? s[nt][c] * scale2 : -INFINITY;
        s[nt][2 + c] = vis ? s[nt][2 + c] * scale2 : -INFINITY;
        mx_lo = fmaxf(mx_lo, s[nt][c]);
        mx_hi = fmaxf(mx_hi, s[nt][2 + c]);
      }
    }
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
    mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
    mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
    const float n_lo = fmaxf(m_lo, mx_lo), n_hi = fmaxf(m_hi, mx_hi);     // finite: the unit holds a visible key
    const float f_lo = md_exp2(m_lo - n_lo);             // 0 for the first unit (m = -inf)
    const float f_hi = md_exp2(m_hi - n_hi);
    m_lo = n_lo;
    m_hi = n_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
    unsigned pa[2][4];                                   // P as A fragments: 2 steps of 16 keys
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const float p0 = md_exp2(s[nt][0] - n_lo), p1 = md_exp2(s[nt][1] - n_lo);
      const float p2 = md_exp2(s[nt][2] - n_hi), p3 = md_exp2(s[nt][3] - n_hi);
      sum_lo += p0 + p1;
      sum_hi += p2 + p3;
      pa[nt >> 1][(nt & 1) * 2] = md_pack(p0, p1);
      pa[nt >> 1][(nt & 1) * 2 + 1] = md_pack(p2, p3);
    }
    l_lo = l_lo * f_lo + sum_lo;
    l_hi = l_hi * f_hi + sum_hi;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
      o[nt][0] *= f_lo;
      o[nt][1] *= f_lo;
      o[nt][2] *= f_hi;
      o[nt][3] *= f_hi;
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int pr = 0; pr < NT / 2; ++pr) {
        unsigned b[4];
        const int key = kk * 16 + (lm_m & 1) * 8 + lm_r, col = (2 * pr + (lm_m >> 1)) * 8;
        md_ldmatrix_trans(b, v_addr + (unsigned)(key * PITCH + col) * 2u);
        md_mma(o[2 * pr], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[0], b[1]);
        md_mma(o[2 * pr + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b[2], b[3]);
      }
    }
    __syncwarp();                                        // every lane has read this stage: it is free
    p = np;
    h = nh;
    if (np <= p_last) {
      advance(np, nh);
      if (np <= p_last) issue(np, nh, s_);
    }
  }

  // ---- the warps' results meet: each leaves (m, l, O) for its 16 rows in its own K tile
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  constexpr int kRowFloats = HD + 2;                    // O row, then m and l
  float* mine = reinterpret_cast<float*>(k_tile);      // 16 rows of kRowFloats floats: fits a tile
  __syncwarp();
#pragma unroll
  for (int nt = 0; nt < NT; ++nt) {
    mine[g * kRowFloats + nt * 8 + 2 * t] = o[nt][0];
    mine[g * kRowFloats + nt * 8 + 2 * t + 1] = o[nt][1];
    mine[(g + 8) * kRowFloats + nt * 8 + 2 * t] = o[nt][2];
    mine[(g + 8) * kRowFloats + nt * 8 + 2 * t + 1] = o[nt][3];
  }
  if (t == 0) {
    mine[g * kRowFloats + HD] = m_lo;
    mine[g * kRowFloats + HD + 1] = l_lo;
    mine[(g + 8) * kRowFloats + HD] = m_hi;
    mine[(g + 8) * kRowFloats + HD + 1] = l_hi;
  }
  __syncthreads();
  const float* all = reinterpret_cast<const float*>(md_smem);
  constexpr int kWarpFloats = 2 * kTile / 2;            // floats between two warps' tiles (2 tiles of bf16)
  for (int i = threadIdx.x; i < ng * HD; i += WARPS * 32) {
    const int row = i / HD, d = i % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) M = fmaxf(M, all[w * kWarpFloats + row * kRowFloats + HD]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) {
      const float* r = all + w * kWarpFloats + row * kRowFloats;
      const float mw = r[HD];
      const float f = (mw == -INFINITY) ? 0.f : md_exp2(mw - M);
      num = fmaf(f, r[d], num);
      den = fmaf(f, r[HD + 1], den);
    }
    const size_t head = (size_t)seq * n_q + (size_t)hk * G + g0 + row;
    if (n_runs == 1) {
      out[head * HD + d] = __float2bfloat16_rn(num / den);
    } else {
      part_acc[(head * n_runs + run) * HD + d] = num;
      if (d == 0) {
        part_m[head * n_runs + run] = M;
        part_l[head * n_runs + run] = den;
      }
    }
  }
  if (n_runs == 1) return;
  // ---- the block that finishes last for this (sequence, head group) merges the runs
  const int r0 = (lo / kMdPage) / pages_per_run, r1 = ((len - 1) / kMdPage) / pages_per_run;
  __threadfence();                     // this block's partial results are visible before it is counted
  __syncthreads();
  if (threadIdx.x == 0) {
    int* c = counters + (size_t)seq * gridDim.y + blockIdx.y;
    const int done = atomicAdd(c, 1) + 1;
    is_last = (done == r1 - r0 + 1);
    if (is_last) *c = 0;               // left clean for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int row = warp; row < ng; row += WARPS) {
    const size_t head = (size_t)seq * n_q + (size_t)hk * G + g0 + row;
    md_merge_head<HD>(part_m, part_l, part_acc, out + head * HD, head * n_runs, r0, r1);
  }
}

template <int HD, int WARPS, bool ROPE>
static int launch_mma(const void* q, const void* k_cache, const void* v_cache, float* part_m, float* part_l,
                      float* part_acc, const int* seq_slot, const int* seq_kvlen, const int* block_table, int max_pages,
                      int n_seqs, int n_q, int n_kv, float scale, int window, int pages_per_run, int n_runs,
                      int* counters, void* out, const float2* rope, int table_len, int q_ld, int write_kv,
                      cudaStream_t stream) {
  const int G = n_q / n_kv;
  const int chunks = (G + 15) / 16;
  const size_t smem = (size_t)WARPS * 2 * kMdPage * (HD + 8) * sizeof(__nv_bfloat16);
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(decode_mma_kernel<HD, WARPS, ROPE>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch_k(decode_mma_kernel<HD, WARPS, ROPE>, dim3(n_runs, n_kv * chunks, n_seqs), dim3(WARPS * 32), smem, stream,
           (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, part_m, part_l,
           part_acc, seq_slot, seq_kvlen, block_table, max_pages, n_q, n_kv, scale, window, pages_per_run, n_runs,
           counters, (__nv_bfloat16*)out, rope, table_len, q_ld, write_kv);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

}  // namespace llmie

using namespace llmie;

extern "C" int llmie_attention_decode_mma_supported(int head_dim, int dtype, int page_size) {
  return (dtype == LLMIE_BF16 && page_size == 64 && (head_dim == 64 || head_dim == 128)) ? 1 : 0;
}

// Pages per block for a step of n_seqs sequences none longer than max_kv_len. A whole sequence per
// block wherever its warps then take at most four pages each in turn: merging runs through global
// memory costs more than a few pages (measured on B200, 8 sequences of 520 keys: one run 0.858 ms per
// step, two runs 0.900 ms). Longer sequences are halved while the grid stays within max_blocks.
// n_groups = KV heads x chunks of 16 query heads.
extern "C" int llmie_attention_decode_mma_pages(int n_seqs, int n_groups, int max_kv_len, int max_blocks) {
  const int total = max_kv_len > 0 ? (max_kv_len + kMdPage - 1) / kMdPage : 1;
  int pp = total;
  while (pp > 8 && (pp + 7) / 8 > 4) {
    const int half = (pp + 1) / 2;
    if ((long long)n_seqs * n_groups * ((total + half - 1) / half) > max_blocks) break;
    pp = half;
  }
  // A sequence that is split pays for the merge anyway: few sequences are then cut on, down to a page
  // a warp, while the grid stays within one block per SM (measured, one sequence of 3,500 keys: two runs
  // 12.5 us, eight runs 7.1 us; eight such sequences are best left at two runs, 14.1 us).
  if (pp < total) {
    while ((pp + 7) / 8 > 1) {
      const int half = (pp + 1) / 2;
      if ((long long)n_seqs * n_groups * ((total + half - 1) / half) > 148) break;
      pp = half;
    }
  }
  return pp;
}

// q, out bfloat16 [n_seqs, n_q hd]; caches [pages, n_kv, 64, hd]; seq_kvlen: keys each sequence holds
// including this step's. n_runs * pages_per_run * 64 must cover the longest sequence. part_*: float32
// scratch as in llmie_attention_decode (untouched when n_runs == 1); counters: int32 zeros, one per
// (sequence, KV head, chunk of 16 query heads), left zero.
static int decode_mma_entry(const void* q, const void* k_cache, const void* v_cache, void* out, float* part_m,
                            float* part_l, float* part_acc, int* counters, const int* seq_slot, const int* seq_kvlen,
                            const int* block_table, int max_pages, int page_size, int n_seqs, int n_q, int n_kv, int hd,
                            float scale, int window, int pages_per_run, int n_runs, const float2* rope, int table_len,
                            int q_ld, int write_kv, cudaStream_t stream) {
  if (n_seqs < 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || max_pages <= 0 || pages_per_run <= 0 || n_runs <= 0)
    return LLMIE_ERR_BAD_ARG;
  if (!llmie_attention_decode_mma_supported(hd, LLMIE_BF16, page_size)) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (n_runs > 1 && (!part_m || !part_l || !part_acc || !counters)) return LLMIE_ERR_BAD_ARG;
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache)) return LLMIE_ERR_ALIGNMENT;
  if (n_seqs == 0) return LLMIE_OK;
  const int chunks = (n_q / n_kv + 15) / 16;
  // Warps per block. More warps finish a block's pages sooner; fewer let more blocks stay on an SM at once
  // (a block holds two page tiles per warp in shared memory), and a grid that does not fit in one wave
  // takes two. Estimate: waves x (pages a warp takes in turn + a fixed part), smallest wins.
  const long long blocks = (long long)n_seqs * n_kv * chunks * n_runs;
  const int tile_bytes = 2 * kMdPage * (hd + 8) * (int)sizeof(__nv_bfloat16);
  const int options[4] = {8, 4, 3, 2};
  int best_w = 4;
  double best_cost = 1e30;
  for (int i = 0; i < 4; ++i) {
    const int w = options[i];
    if (w * tile_bytes > 200 * 1024) continue;
    int per_sm = (227 * 1024) / (w * tile_bytes + 1024);                      // 1 KB of every block is the system's
    if (hd == 64 && per_sm > 16 / w) per_sm = 16 / w > 0 ? 16 / w : 1;       // registers
    if (per_sm < 1) continue;
    const long long slots = 148LL * per_sm;
    const double waves = (double)((blocks + slots - 1) / slots);
    const double cost = waves * ((pages_per_run + w - 1) / w + 1.5);
    if (cost < best_cost) {
      best_cost = cost;
      best_w = w;
    }
  }
#define LLMIE_MMA(HD, W)                                                                                             \
  return rope ? launch_mma<HD, W, true>(q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen,          \
                                        block_table, max_pages, n_seqs, n_q, n_kv, scale, window, pages_per_run,     \
                                        n_runs, counters, out, rope, table_len, q_ld, write_kv, stream)              \
              : launch_mma<HD, W, false>(q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen,         \
                                         block_table, max_pages, n_seqs, n_q, n_kv, scale, window, pages_per_run,    \
                                         n_runs, counters, out, nullptr, 0, 0, 0, stream)
  if (hd == 64) {
    if (best_w == 8) LLMIE_MMA(64, 8);
    if (best_w == 4) LLMIE_MMA(64, 4);
    if (best_w == 3) LLMIE_MMA(64, 3);
    LLMIE_MMA(64, 2);
  }
  if (best_w >= 4) LLMIE_MMA(128, 4);
  if (best_w == 3) LLMIE_MMA(128, 3);
  LLMIE_MMA(128, 2);
#undef LLMIE_MMA
}

extern "C" int llmie_attention_decode_mma(const void* q, const void* k_cache, const void* v_cache, void* out,
                                          float* part_m, float* part_l, float* part_acc, int* counters,
                                          const int* seq_slot, const int* seq_kvlen, const int* block_table,
                                          int max_pages, int page_size, int n_seqs, int n_q, int n_kv, int hd,
                                          float scale, int window, int pages_per_run, int n_runs,
                                          cudaStream_t stream) {
  return decode_mma_entry(q, k_cache, v_cache, out, part_m, part_l, part_acc, counters, seq_slot, seq_kvlen, block_table,
                          max_pages, page_size, n_seqs, n_q, n_kv, hd, scale, window, pages_per_run, n_runs, nullptr, 0,
                          0, 0, stream);
}

// The same with position encoding and the cache write inside: qkv bfloat16 [n_seqs, (n_q + 2 n_kv) hd] holds the
// step's raw projections (q heads, k heads, v heads), rope float32 [table_len, hd / 2, 2] the (cos, sin) of every
// position for a rotation over the whole head size. The new key (rotated) and value of sequence i are used for
// position seq_kvlen[i] - 1 and, with write_kv, written to the cache there.
extern "C" int llmie_attention_decode_mma_rope(const void* qkv, void* k_cache, void* v_cache, void* out,
                                               const float* rope, int table_len, float* part_m, float* part_l,
                                               float* part_acc, int* counters, const int* seq_slot,
                                               const int* seq_kvlen, const int* block_table, int max_pages,
                                               int page_size, int n_seqs, int n_q, int n_kv, int hd, float scale,
                                               int window, int pages_per_run, int n_runs, int write_kv,
                                               cudaStream_t stream) {
  if (!rope || table_len <= 0) return LLMIE_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(rope) & 7u) != 0) return LLMIE_ERR_ALIGNMENT;
  return decode_mma_entry(qkv, k_cache, v_cache, out, part_m, part_l, part_acc, counters, seq_slot, seq_kvlen,
                          block_table, max_pages, page_size, n_seqs, n_q, n_kv, hd, scale, window, pages_per_run, n_runs,
                          reinterpret_cast<const float2*>(rope), table_len, (n_q + 2 * n_kv) * hd, write_kv ? 1 : 0,
                          stream);
}
