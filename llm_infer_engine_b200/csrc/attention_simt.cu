// Plain attention over the paged KV cache, for any number of new tokens per sequence.
//
// One warp per (token, query head). It is the float32 path's attention for prefill and
// decode alike, and the plain twin that the tensor-core and split-KV kernels are checked
// against. The math is that of the reference's prefill and decode kernels
// (src/flash_attn.py:42-82, src/flash_decode.py:73-113): scores q.k / sqrt(hd) over the keys
// a token may see, online softmax with float32 running max / sum / accumulator, query head
// h reading key/value head h / (Hq / Hkv).
//
// A token at absolute position p of its sequence sees keys lo..p of that sequence's slot,
// lo = max(0, p - window + 1) when window > 0, else 0. Keys of this very step were written to
// the cache by the rotary kernel before this kernel runs, so prefill at any start position,
// decode, and mixtures need no separate code.
#include "common.cuh"
#include <math.h>

namespace llmie {

constexpr int kAttnWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__global__ void __launch_bounds__(kAttnWarps * 32)
attention_paged_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                       T* __restrict__ out, const int* __restrict__ tok_pos, const int* __restrict__ tok_seq,
                       const int* __restrict__ seq_slot, const int* __restrict__ block_table, int max_pages,
                       int page_size, int n_items, int n_q, int n_kv, int hd, float scale, int window) {
  extern __shared__ float q_smem[];  // [kAttnWarps][hd]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int item = blockIdx.x * kAttnWarps + warp;
  if (item >= n_items) return;  // whole warp leaves together; no block-wide barrier below
  const int t = item / n_q, h = item - t * n_q;
  const int hk = h / (n_q / n_kv);
  const int pos = tok_pos[t];
  const int slot = seq_slot[tok_seq[t]];
  const int* pages = block_table + (size_t)slot * max_pages;
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

  float* qs = q_smem + warp * hd;
  const T* qrow = q + ((size_t)t * n_q + h) * hd;
  for (int i = lane; i < hd; i += 32) qs[i] = to_f32(qrow[i]) * scale;
  __syncwarp();

  constexpr int kAcc = kMaxHeadDim / 32;
  float acc[kAcc];
#pragma unroll
  for (int i = 0; i < kAcc; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  for (int base = lo; base <= pos; base += 32) {
    const int j = base + lane;
    const bool valid = j <= pos;
    size_t row = 0;
    float s = -INFINITY;
    if (valid) {
      const int page = pages[j / page_size];
      row = (((size_t)page * n_kv + hk) * page_size + (j % page_size)) * hd;
      const T* kr = k_cache + row;
      float dot = 0.f;
      for (int d0 = 0; d0 < hd; d0 += 8) {
        float kv[8];
        load8(kr + d0, kv);
#pragma unroll
        for (int e = 0; e < 8; ++e) dot = fmaf(qs[d0 + e], kv[e], dot);
      }
      s = dot;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);  // m == -inf on the first chunk gives 0
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < kAcc; ++i) acc[i] *= alpha;
    m = m_new;
    const int n_here = min(32, pos - base + 1);
    for (int jj = 0; jj < n_here; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const unsigned long long rj = __shfl_sync(0xffffffffu, (unsigned long long)row, jj);
      const T* vr = v_cache + rj;
#pragma unroll
      for (int i = 0; i < kAcc; ++i) {
        const int d = lane + 32 * i;
        if (d < hd) acc[i] = fmaf(pj, to_f32(vr[d]), acc[i]);
      }
    }
  }
  const float inv_l = 1.f / l;
  T* orow = out + ((size_t)t * n_q + h) * hd;
#pragma unroll
  for (int i = 0; i < kAcc; ++i) {
    const int d = lane + 32 * i;
    if (d < hd) orow[d] = from_f32<T>(acc[i] * inv_l);
  }
}

}  // namespace llmie

using namespace llmie;

// q, out: [n_tokens, n_q * hd]; caches: [n_pages, n_kv, page_size, hd]; all of `dtype`.
extern "C" int llmie_attention_paged(const void* q, const void* k_cache, const void* v_cache, void* out,
                                     const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                     const int* block_table, int max_pages, int page_size, int n_tokens, int n_q,
                                     int n_kv, int hd, float scale, int window, int dtype, cudaStream_t stream) {
  if (n_tokens < 0 || n_q <= 0 || n_kv <= 0 || hd <= 0 || page_size <= 0 || max_pages <= 0) return LLMIE_ERR_BAD_ARG;
  if (n_q % n_kv) return LLMIE_ERR_BAD_ARG;
  if (hd % 16 || hd > kMaxHeadDim) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (!aligned16(k_cache) || !aligned16(v_cache)) return LLMIE_ERR_ALIGNMENT;
  if (n_tokens == 0) return LLMIE_OK;
  const long long n_items = (long long)n_tokens * n_q;
  if (n_items > 0x7fffffffLL) return LLMIE_ERR_UNSUPPORTED_SIZE;
  const int blocks = (int)((n_items + kAttnWarps - 1) / kAttnWarps);
  const size_t smem = (size_t)kAttnWarps * hd * sizeof(float);
  if (dtype == LLMIE_F32)
    attention_paged_kernel<float><<<blocks, kAttnWarps * 32, smem, stream>>>(
        (const float*)q, (const float*)k_cache, (const float*)v_cache, (float*)out, tok_pos, tok_seq, seq_slot,
        block_table, max_pages, page_size, (int)n_items, n_q, n_kv, hd, scale, window);
  else if (dtype == LLMIE_BF16)
    attention_paged_kernel<__nv_bfloat16><<<blocks, kAttnWarps * 32, smem, stream>>>(
        (const __nv_bfloat16*)q, (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, (__nv_bfloat16*)out,
        tok_pos, tok_seq, seq_slot, block_table, max_pages, page_size, (int)n_items, n_q, n_kv, hd, scale, window);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
