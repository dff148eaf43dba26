// Memory-bound parts of a step: embedding gather, residual add fused with RMSNorm,
// SwiGLU, rotary position encoding fused with the KV-cache write, and the small kernels
// that keep per-sequence lengths on the device. The residual stream is float32 in both
// precisions; activations between GEMMs are T (float or bfloat16).
#include "common.cuh"

namespace llmie {

// ------------------------------------------------------------------------------------------
// h[t, :] = table[token[t], :]         (src/model.py:157 of the reference: a plain row gather)
template <typename W>
__global__ void embedding_kernel(const int* __restrict__ tokens, const W* __restrict__ table,
                                 float* __restrict__ h, int d, int vocab) {
  // The step's index arrays (positions, lengths, slots) come from the kernel before this one. Later
  // kernels read them ahead of their own waits, so nothing after this kernel may be scheduled before
  // those arrays are complete: the dependents are released after the wait, not at the top.
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  int id = tokens[t];
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);  // the host refuses such ids; never read outside
  const W* row = table + (size_t)id * d;
  float* out = h + (size_t)t * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) out[i] = to_f32(row[i]);
}

// ------------------------------------------------------------------------------------------
// Residual add + RMSNorm (src/rms_norm.py:32-39 and src/model.py:113-127 of the reference):
//   r = rows ? rows[b] : b
//   x = h[r] (+ delta[r])                     float32 sum
//   if (!rows && delta) h[r] = x              the residual stream is updated in place
//   y[b] = x * rsqrt(mean(x^2) + eps) * w     one rounding, at the store
// One block per output row; the row is held in shared memory between the two passes.
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                   const float* __restrict__ w, T* __restrict__ y,
                                   const int* __restrict__ rows, int d, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row_buf[];
  __shared__ float red[32];
  const int b = blockIdx.x;
  const int r = rows ? rows[b] : b;
  float* hr = h + (size_t)r * d;
  const T* dr = delta ? delta + (size_t)r * d : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float x = hr[i];
    if (dr) {
      x += to_f32(dr[i]);
      if (!rows) hr[i] = x;
    }
    row_buf[i] = x;
    ss += x * x;
  }
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)d + eps);
  T* yr = y + (size_t)b * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) yr[i] = from_f32<T>(row_buf[i] * rstd * w[i]);
}

// The same for rows of at most 8 * 1024 elements with d % 8 == 0: each thread owns one run of 8
// elements, kept in registers, so the row is read once.
template <typename T>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ h, const T* __restrict__ delta,
                                       const float* __restrict__ w, T* __restrict__ y,
                                       const int* __restrict__ rows, int d, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float red[32];
  const int b = blockIdx.x;
  const int r = rows ? rows[b] : b;
  const int i = threadIdx.x * 8;
  const bool active = i < d;
  float x[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) x[e] = 0.f;
  if (active) {
    float* hr = h + (size_t)r * d + i;
    load8(hr, x);
    if (delta) {
      float dv[8];
      load8(delta + (size_t)r * d + i, dv);
#pragma unroll
      for (int e = 0; e < 8; ++e) x[e] += dv[e];
      if (!rows) store8(hr, x);
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) ss += x[e] * x[e];
  ss = block_sum(ss, red);
  const float rstd = rsqrtf(ss / (float)d + eps);
  if (active) {
    float wv[8], o[8];
    load8(w + i, wv);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = x[e] * rstd * wv[e];
    store8(y + (size_t)b * d + i, o);
  }
}

// h += delta, no norm (used when a block arrangement needs the bare sum)
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ h, const T* __restrict__ delta, size_t n) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < n; i += stride) h[i] += to_f32(delta[i]);
}

// ------------------------------------------------------------------------------------------
// out[t, j] = silu(gate_up[t, j]) * gate_up[t, ff + j]      (src/model.py:23 of the reference)
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int ff, size_t total) {
  pdl_launch_dependents();
  pdl_wait();
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    const size_t t = i / ff;
    const int j = (int)(i - t * ff);
    const float g = to_f32(gate_up[t * 2 * ff + j]);
    const float u = to_f32(gate_up[t * 2 * ff + ff + j]);
    const float s = g / (1.f + expf(-g));
    out[i] = from_f32<T>(s * u);
  }
}

// The same, eight outputs per thread with 16-byte loads (ff % 8 == 0): a block row per token, so that
// no index is divided. bfloat16 results keep 8 bits: their exponential and quotient are the fast ones
// (errors of a few 2^-22); the 32-bit path keeps the exact ones.
template <typename T>
__device__ __forceinline__ float silu_for(float g) {
  return g / (1.f + expf(-g));
}
template <>
__device__ __forceinline__ float silu_for<__nv_bfloat16>(float g) {
  return __fdividef(g, 1.f + __expf(-g));
}

template <typename T>
__global__ void swiglu_vec_kernel(const T* __restrict__ gate_up, T* __restrict__ out, int ff8, int n_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int j8 = blockIdx.x * blockDim.x + threadIdx.x;
  if (j8 >= ff8) return;
  for (int t = blockIdx.y; t < n_tokens; t += gridDim.y) {
    const T* row = gate_up + (size_t)t * ff8 * 16;
    float g[8], u[8], o[8];
    load8(row + (size_t)j8 * 8, g);
    load8(row + (size_t)(ff8 + j8) * 8, u);
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = silu_for<T>(g[e]) * u[e];
    store8(out + ((size_t)t * ff8 + j8) * 8, o);
  }
}

// ------------------------------------------------------------------------------------------
// Rotary position encoding fused with the KV-cache write
// (src/rope.py:74-91 rotate-half, :122-185 the fused K rotation + cache write of the reference).
//   qkv[t] = [ q heads | k heads | v heads ], each head `hd` wide
//   q_out[t, h] = rot(q)          k_cache[page(t), hk, pos % P] = rot(k)       v_cache[...] = v
// rot pairs element i with i + rot_dim/2 for i < rot_dim/2 using table[pos] = (cos, sin);
// elements >= rot_dim pass through. table == nullptr means no rotation at all.
// With write_kv == 0 only q is produced (a layer that reads another layer's cache).
template <typename T>
__global__ void rope_store_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                  T* __restrict__ k_cache, T* __restrict__ v_cache,
                                  const float2* __restrict__ table, const int* __restrict__ tok_pos,
                                  const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                                  const int* __restrict__ block_table, int max_pages, int page_size,
                                  int n_q, int n_kv, int hd, int rot_dim, int table_len, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  int pos = tok_pos[t];
  const int half = rot_dim >> 1;
  const int row_w = (n_q + 2 * n_kv) * hd;
  const T* src = qkv + (size_t)t * row_w;
  const int tpos = pos < table_len ? pos : table_len - 1;  // the host refuses pos >= table_len
  const float2* cs = table ? table + (size_t)tpos * half : nullptr;

  // q heads: items are (head, i) with i < hd; rotated pairs are produced by the thread of i < half
  const int q_items = n_q * hd;
  T* qo = q_out + (size_t)t * q_items;
  for (int it = threadIdx.x; it < q_items; it += blockDim.x) {
    const int i = it % hd;
    const int base = it - i;
    if (cs && i < rot_dim) {
      if (i < half) {
        const float x1 = to_f32(src[base + i]), x2 = to_f32(src[base + i + half]);
        const float2 c = cs[i];
        qo[base + i] = from_f32<T>(x1 * c.x - x2 * c.y);
        qo[base + i + half] = from_f32<T>(x2 * c.x + x1 * c.y);
      }
    } else {
      qo[base + i] = src[base + i];
    }
  }
  if (!write_kv) return;

  const int slot = seq_slot[tok_seq[t]];
  const int page = block_table[(size_t)slot * max_pages + pos / page_size];
  const int in_page = pos % page_size;
  const int kv_items = n_kv * hd;
  const T* ks = src + q_items;
  const T* vs = ks + kv_items;
  for (int it = threadIdx.x; it < kv_items; it += blockDim.x) {
    const int i = it % hd;
    const int hk = it / hd;
    const size_t dst = (((size_t)page * n_kv + hk) * page_size + in_page) * hd;
    v_cache[dst + i] = vs[it];
    if (cs && i < rot_dim) {
      if (i < half) {
        const float x1 = to_f32(ks[it]), x2 = to_f32(ks[it + half]);
        const float2 c = cs[i];
        k_cache[dst + i] = from_f32<T>(x1 * c.x - x2 * c.y);
        k_cache[dst + i + half] = from_f32<T>(x2 * c.x + x1 * c.y);
      }
    } else {
      k_cache[dst + i] = ks[it];
    }
  }
}

// The same for full rotation (rot_dim == hd, hd % 16 == 0): a thread rotates eight pairs at a
// time with 16-byte loads and stores. Items per token: query heads, then key heads (rotated,
// to the cache), then value heads (copied to the cache).
template <typename T>
__global__ void rope_store_vec_kernel(const T* __restrict__ qkv, T* __restrict__ q_out,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache,
                                      const float2* __restrict__ table, const int* __restrict__ tok_pos,
                                      const int* __restrict__ tok_seq, const int* __restrict__ seq_slot,
                                      const int* __restrict__ block_table, int max_pages, int page_size,
                                      int n_q, int n_kv, int hd, int table_len, int write_kv) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = tok_pos[t];
  const int half = hd >> 1;
  const int vec_per_half = half >> 3;
  const T* src = qkv + (size_t)t * (n_q + 2 * n_kv) * hd;
  const int tpos = pos < table_len ? pos : table_len - 1;
  const float2* cs = table + (size_t)tpos * half;
  size_t kv_row = 0;
  if (write_kv) {
    const int slot = seq_slot[tok_seq[t]];
    const int page = block_table[(size_t)slot * max_pages + pos / page_size];
    kv_row = ((size_t)page * n_kv * page_size + (pos % page_size)) * hd;      // head 0; heads are page_size * hd apart
  }
  const int rot_items = (n_q + (write_kv ? n_kv : 0)) * vec_per_half;
  for (int it = threadIdx.x; it < rot_items; it += blockDim.x) {
    const int head = it / vec_per_half;
    const int i = (it - head * vec_per_half) * 8;
    const T* x = src + (size_t)head * hd;                     // k heads follow the q heads in qkv
    float x1[8], x2[8], y1[8], y2[8];
    load8(x + i, x1);
    load8(x + i + half, x2);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float2 c = cs[i + e];
      y1[e] = x1[e] * c.x - x2[e] * c.y;
      y2[e] = x2[e] * c.x + x1[e] * c.y;
    }
    T* dst = head < n_q ? q_out + ((size_t)t * n_q + head) * hd
                        : k_cache + kv_row + (size_t)(head - n_q) * page_size * hd;
    store8(dst + i, y1);
    store8(dst + i + half, y2);
  }
  if (write_kv) {
    const int v_items = n_kv * (hd >> 3);
    const T* vs = src + (size_t)(n_q + n_kv) * hd;
    for (int it = threadIdx.x; it < v_items; it += blockDim.x) {
      const int head = it / (hd >> 3);
      const int i = (it - head * (hd >> 3)) * 8;
      *reinterpret_cast<uint4*>(v_cache + kv_row + (size_t)head * page_size * hd + i) =
          *reinterpret_cast<const uint4*>(vs + (size_t)head * hd + i);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Decode-step metadata from the device-resident lengths, so that a captured step needs no
// host rewrites: lane i continues sequence slots[i] by one token at position len[slot].
__global__ void prepare_decode_kernel(const int* __restrict__ slots, const int* __restrict__ seq_lens,
                                      int* __restrict__ tok_pos, int* __restrict__ tok_seq,
                                      int* __restrict__ cu_q, int* __restrict__ seq_start,
                                      int* __restrict__ seq_kvlen, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int len = seq_lens[slots[i]];
    tok_pos[i] = len;
    tok_seq[i] = i;
    cu_q[i] = i;
    seq_start[i] = len;
    seq_kvlen[i] = len + 1;
  }
  if (i == 0) cu_q[n] = n;
}

// seq_lens[slot] = kv length after the step, except for the scratch slot that padding lanes use.
__global__ void advance_lengths_kernel(const int* __restrict__ slots, const int* __restrict__ seq_kvlen,
                                       int* __restrict__ seq_lens, int n, int scratch_slot) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) {
    const int s = slots[i];
    if (s != scratch_slot) seq_lens[s] = seq_kvlen[i];
  }
}

static inline int norm_threads(int d) {
  int t = (d + 7) / 8;
  t = ((t + 31) / 32) * 32;
  return t < 32 ? 32 : (t > 1024 ? 1024 : t);
}

}  // namespace llmie

using namespace llmie;

extern "C" int llmie_embedding(const int* tokens, const void* table, int table_dtype, float* h, int n_tokens,
                               int d, int vocab, cudaStream_t stream) {
  if (n_tokens < 0 || d <= 0 || vocab <= 0) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  const int threads = norm_threads(d);
  if (table_dtype == LLMIE_F32)
    launch_k(embedding_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const float*)table, h, d, vocab);
  else if (table_dtype == LLMIE_BF16)
    launch_k(embedding_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, tokens, (const __nv_bfloat16*)table, h, d, vocab);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

template <typename T>
static int add_rmsnorm_launch(float* h, const void* delta, const float* w, void* y, const int* rows, int n_out,
                              int d, float eps, cudaStream_t stream) {
  if (d % 8 == 0 && d <= 8 * 1024 && aligned16(h) && aligned16(w) && aligned16(y) && (!delta || aligned16(delta))) {
    const int threads = ((d / 8 + 31) / 32) * 32;
    launch_k(add_rmsnorm_vec_kernel<T>, dim3(n_out), dim3(threads), 0, stream, h, (const T*)delta, w, (T*)y, rows, d, eps);
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  launch_k(add_rmsnorm_kernel<T>, dim3(n_out), dim3(norm_threads(d)), smem, stream, h, (const T*)delta, w, (T*)y, rows, d, eps);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// y[n_out, d] (dtype) from h[*, d] float32; delta (dtype) and rows may be null.
extern "C" int llmie_add_rmsnorm(float* h, const void* delta, const float* w, void* y, const int* rows, int n_out,
                                 int d, float eps, int dtype, cudaStream_t stream) {
  if (n_out < 0 || d <= 0) return LLMIE_ERR_BAD_ARG;
  if (n_out == 0) return LLMIE_OK;
  if (dtype == LLMIE_F32) return add_rmsnorm_launch<float>(h, delta, w, y, rows, n_out, d, eps, stream);
  if (dtype == LLMIE_BF16) return add_rmsnorm_launch<__nv_bfloat16>(h, delta, w, y, rows, n_out, d, eps, stream);
  return LLMIE_ERR_DTYPE;
}

extern "C" int llmie_residual_add(float* h, const void* delta, long long n, int dtype, cudaStream_t stream) {
  if (n < 0) return LLMIE_ERR_BAD_ARG;
  if (n == 0) return LLMIE_OK;
  const int threads = 256;
  long long blocks = (n + threads - 1) / threads;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (dtype == LLMIE_F32)
    launch_k(residual_add_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, h, (const float*)delta, (size_t)n);
  else if (dtype == LLMIE_BF16)
    launch_k(residual_add_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, h, (const __nv_bfloat16*)delta, (size_t)n);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_swiglu(const void* gate_up, void* out, int n_tokens, int ff, int dtype, cudaStream_t stream) {
  if (n_tokens < 0 || ff <= 0) return LLMIE_ERR_BAD_ARG;
  const size_t total = (size_t)n_tokens * ff;
  if (total == 0) return LLMIE_OK;
  if (ff % 8 == 0 && aligned16(gate_up) && aligned16(out)) {
    const int ff8 = ff / 8;
    const int threads = ff8 >= 256 ? 256 : ((ff8 + 31) / 32) * 32;
    const dim3 grid((ff8 + threads - 1) / threads, n_tokens < 32768 ? n_tokens : 32768);
    if (dtype == LLMIE_F32)
      launch_k(swiglu_vec_kernel<float>, grid, dim3(threads), 0, stream, (const float*)gate_up, (float*)out, ff8, n_tokens);
    else if (dtype == LLMIE_BF16)
      launch_k(swiglu_vec_kernel<__nv_bfloat16>, grid, dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up,
               (__nv_bfloat16*)out, ff8, n_tokens);
    else
      return LLMIE_ERR_DTYPE;
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  const int threads = 256;
  size_t blocks = (total + threads - 1) / threads;
  if (blocks > 148 * 32) blocks = 148 * 32;
  if (dtype == LLMIE_F32)
    launch_k(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, stream, (const float*)gate_up, (float*)out, ff, total);
  else if (dtype == LLMIE_BF16)
    launch_k(swiglu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, stream, (const __nv_bfloat16*)gate_up,
                                                                     (__nv_bfloat16*)out, ff, total);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_rope_store(const void* qkv, void* q_out, void* k_cache, void* v_cache, const float* table,
                                const int* tok_pos, const int* tok_seq, const int* seq_slot,
                                const int* block_table, int max_pages, int page_size, int n_tokens, int n_q,
                                int n_kv, int hd, int rot_dim, int table_len, int write_kv, int dtype,
                                cudaStream_t stream) {
  if (n_tokens < 0 || n_q <= 0 || n_kv < 0 || hd <= 0 || page_size <= 0 || max_pages <= 0) return LLMIE_ERR_BAD_ARG;
  if (rot_dim < 0 || rot_dim > hd || (rot_dim & 1)) return LLMIE_ERR_BAD_ARG;
  if (table && table_len <= 0) return LLMIE_ERR_BAD_ARG;
  if (n_tokens == 0) return LLMIE_OK;
  int threads = ((n_q * hd / 2 + 31) / 32) * 32;
  threads = threads < 64 ? 64 : (threads > 512 ? 512 : threads);
  const float2* tab = reinterpret_cast<const float2*>(table);
  if (dtype == LLMIE_BF16 && table && rot_dim == hd && hd % 16 == 0 && aligned16(qkv) && aligned16(q_out) &&
      (!write_kv || (aligned16(k_cache) && aligned16(v_cache)))) {
    int vt = (((n_q + n_kv) * (hd / 16) + 31) / 32) * 32;
    vt = vt < 32 ? 32 : (vt > 256 ? 256 : vt);
    launch_k(rope_store_vec_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(vt), 0, stream, 
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tab, tok_pos,
        tok_seq, seq_slot, block_table, max_pages, page_size, n_q, n_kv, hd, table_len, write_kv);
    LLMIE_LAUNCH_CHECK();
    return LLMIE_OK;
  }
  if (dtype == LLMIE_F32)
    launch_k(rope_store_kernel<float>, dim3(n_tokens), dim3(threads), 0, stream, 
        (const float*)qkv, (float*)q_out, (float*)k_cache, (float*)v_cache, tab, tok_pos, tok_seq, seq_slot,
        block_table, max_pages, page_size, n_q, n_kv, hd, rot_dim, table_len, write_kv);
  else if (dtype == LLMIE_BF16)
    launch_k(rope_store_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(threads), 0, stream, 
        (const __nv_bfloat16*)qkv, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, tab,
        tok_pos, tok_seq, seq_slot, block_table, max_pages, page_size, n_q, n_kv, hd, rot_dim, table_len, write_kv);
  else
    return LLMIE_ERR_DTYPE;
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_prepare_decode(const int* slots, const int* seq_lens, int* tok_pos, int* tok_seq, int* cu_q,
                                    int* seq_start, int* seq_kvlen, int n, cudaStream_t stream) {
  if (n <= 0) return LLMIE_ERR_BAD_ARG;
  launch_k(prepare_decode_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, slots, seq_lens, tok_pos, tok_seq, cu_q, seq_start,
                                                             seq_kvlen, n);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_advance_lengths(const int* slots, const int* seq_kvlen, int* seq_lens, int n, int scratch_slot,
                                     cudaStream_t stream) {
  if (n <= 0) return LLMIE_ERR_BAD_ARG;
  launch_k(advance_lengths_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, slots, seq_kvlen, seq_lens, n, scratch_slot);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

