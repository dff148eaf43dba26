// Split-KV attention for one-token steps over the paged cache.
//
// The reference splits the keys of a sequence into runs of 256 (here: runs of one cache page, 64 keys), computes a partial
// (max, sum, accumulator) per (sequence, query head, run) and merges the runs with a
// log-sum-exp (src/flash_decode.py:8-137 and :140-212); every query head re-reads its KV head.
// Here one block serves ALL query heads of a KV head for its run of keys, so the cache is
// read once per KV head: block (run, kv head, sequence) computes G = Hq / Hkv partials, a
// second kernel merges the runs. Lengths come from the device (`seq_kvlen`), so a captured
// step needs no host rewrites; runs that lie beyond a sequence's length leave at once.
//
// A 16-byte load covers E elements of a key (8 bfloat16 or 4 float); LPK = HD / E lanes share
// one key, 32 / LPK keys are in flight per warp. Scores, softmax and accumulators are float32.
//
// Scratch: part_m, part_l [n_seqs, Hq, n_runs] and part_acc [n_seqs, Hq, n_runs, HD], float32,
// written by the first kernel and read by the second. Entries of runs that hold no visible key
// are never written and never read.
#include "common.cuh"
#include <math.h>

namespace llmie {

constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;

template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> { static constexpr int E = 8; };
template <> struct Vec16<float> { static constexpr int E = 4; };

template <typename T, int E>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[E]);
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16, 8>(const __nv_bfloat16* p, float (&out)[8]) { load8(p, out); }
template <>
__device__ __forceinline__ void load_vec<float, 4>(const float* p, float (&out)[4]) {
  float4 a = *reinterpret_cast<const float4*>(p);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
}

// The visible key range of a sequence that holds `len` tokens after this step: [lo, len).
__device__ __forceinline__ int first_visible(int len, int window) {
  return (window > 0 && len - window > 0) ? len - window : 0;
}

// One block = one cache page (64 keys) of one KV head of one sequence, for all its query heads. A
// page's K and V rows are contiguous in the cache, so the block asks for all of them at once (every
// 16-byte load is issued, straight into registers, before anything is computed): one memory latency
// per block instead of one per key. run_len must be 64.
template <typename T, int HD, int GMAX>
__global__ void __launch_bounds__(kDecThreads)
decode_split_kernel(const T* __restrict__ q, const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                    float* __restrict__ part_m, float* __restrict__ part_l, float* __restrict__ part_acc,
                    const int* __restrict__ seq_slot, const int* __restrict__ seq_kvlen,
                    const int* __restrict__ block_table, int max_pages, int page_size, int n_q, int n_kv,
                    float scale, int window, int run_len, int n_runs, int* __restrict__ counters,
                    T* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int E = Vec16<T>::E;
  constexpr int LPK = HD / E;          // lanes per key
  constexpr int KPW = 32 / LPK;        // keys per warp per iteration
  constexpr int kRun = 64;             // keys per block
  __shared__ int is_last;
  constexpr int kIter = kRun / (kDecWarps * KPW);
  static_assert(LPK >= 1 && LPK <= 32 && 32 % LPK == 0 && kIter >= 1, "head size not supported by this kernel");
  __shared__ float scores[GMAX][kRun];
  __shared__ float red[kDecWarps][GMAX][HD];

  const int run = blockIdx.x, seq = blockIdx.z;
  const int G = n_q / n_kv;
  const int chunks = (G + GMAX - 1) / GMAX;
  const int hk = blockIdx.y / chunks;
  const int g0 = (blockIdx.y % chunks) * GMAX;       // first query head (within the group) of this block
  const int ng = min(GMAX, G - g0);

  const int len = seq_kvlen[seq];
  if (len <= 0) {
    // a sequence without keys: its output rows are zeros (written here only in the one-launch form;
    // the separate merge kernel does the same)
    if (counters != nullptr && run == 0)
      for (int i = threadIdx.x; i < ng * HD; i += kDecThreads)
        out[((size_t)seq * n_q + (size_t)hk * G + g0) * HD + i] = from_f32<T>(0.f);
    return;
  }
  const int lo = first_visible(len, window);
  const int begin = max(run * kRun, lo);
  const int end = min(len, (run + 1) * kRun);
  if (begin >= end) return;
  const int first = begin - run * kRun, n_keys = end - begin;      // keys [first, first + n_keys) of the page

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPK;          // which of the warp's KPW keys
  const int e0 = (lane % LPK) * E;     // first element of this lane's slice
  const int* pages = block_table + (size_t)seq_slot[seq] * max_pages;
  const size_t head_off = (size_t)hk * page_size * HD;
  const size_t page_stride = (size_t)n_kv * page_size * HD;
  const size_t page_base = (size_t)pages[begin / 64] * page_stride + head_off;     // the page
  const T* kp = k_cache + page_base;
  const T* vp = v_cache + page_base;

  // Every byte of this block's K and V page is requested here, before anything is computed. Rows
  // outside [first, first + n_keys) hold other positions of the page (never another sequence's);
  // they get probability zero.
  float kreg[kIter][E], vreg[kIter][E];
#pragma unroll
  for (int it = 0; it < kIter; ++it) {
    const int row = (it * kDecWarps + warp) * KPW + sub;
    load_vec<T, E>(kp + (size_t)row * HD + e0, kreg[it]);
  }
#pragma unroll
  for (int it = 0; it < kIter; ++it) {
    const int row = (it * kDecWarps + warp) * KPW + sub;
    load_vec<T, E>(vp + (size_t)row * HD + e0, vreg[it]);
  }
  // this lane's slice of each query head, pre-scaled
  float qv[GMAX][E];
#pragma unroll
  for (int g = 0; g < GMAX; ++g) {
    if (g < ng) {
      const T* qp = q + ((size_t)seq * n_q + (size_t)hk * G + g0 + g) * HD + e0;
      float tmp[E];
      load_vec<T, E>(qp, tmp);
#pragma unroll
      for (int e = 0; e < E; ++e) qv[g][e] = tmp[e] * scale;
    } else {
#pragma unroll
      for (int e = 0; e < E; ++e) qv[g][e] = 0.f;
    }
  }

  // ---- phase 1: scores of the page's rows
#pragma unroll
  for (int it = 0; it < kIter; ++it) {
    const int row = (it * kDecWarps + warp) * KPW + sub;
    float kv[E];
#pragma unroll
    for (int e = 0; e < E; ++e) kv[e] = kreg[it][e];
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) dot = fmaf(qv[g][e], kv[e], dot);
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      if ((lane % LPK) == 0 && g < ng) scores[g][row] = dot;
    }
  }
  __syncthreads();

  // ---- phase 2: softmax statistics per head over the visible rows; scores become probabilities
  for (int g = warp; g < ng; g += kDecWarps) {
    float* s = scores[g];
    float m = -INFINITY;
    for (int j = lane; j < kRun; j += 32) {
      const bool vis = j >= first && j < first + n_keys;
      m = fmaxf(m, vis ? s[j] : -INFINITY);
    }
    m = warp_max(m);
    float l = 0.f;
    for (int j = lane; j < kRun; j += 32) {
      const bool vis = j >= first && j < first + n_keys;
      const float p = vis ? expf(s[j] - m) : 0.f;
      s[j] = p;
      l += p;
    }
    l = warp_sum(l);
    if (lane == 0) {
      const size_t idx = ((size_t)seq * n_q + (size_t)hk * G + g0 + g) * n_runs + run;
      part_m[idx] = m;
      part_l[idx] = l;
    }
  }
  __syncthreads();

  // ---- phase 3: accumulate p * v
  float acc[GMAX][E];
#pragma unroll
  for (int g = 0; g < GMAX; ++g)
#pragma unroll
    for (int e = 0; e < E; ++e) acc[g][e] = 0.f;
#pragma unroll
  for (int it = 0; it < kIter; ++it) {
    const int row = (it * kDecWarps + warp) * KPW + sub;
    float vv[E];
#pragma unroll
    for (int e = 0; e < E; ++e) vv[e] = vreg[it][e];
#pragma unroll
    for (int g = 0; g < GMAX; ++g) {
      const float p = (g < ng) ? scores[g][row] : 0.f;
#pragma unroll
      for (int e = 0; e < E; ++e) acc[g][e] = fmaf(p, vv[e], acc[g][e]);
    }
  }
  // lanes with the same element slice (same lane % LPK) hold different keys: add them up
#pragma unroll
  for (int g = 0; g < GMAX; ++g)
#pragma unroll
    for (int e = 0; e < E; ++e)
#pragma unroll
      for (int o = 16; o >= LPK; o >>= 1) acc[g][e] += __shfl_xor_sync(0xffffffffu, acc[g][e], o);
  if (lane < LPK) {
#pragma unroll
    for (int g = 0; g < GMAX; ++g)
#pragma unroll
      for (int e = 0; e < E; ++e) red[warp][g][e0 + e] = acc[g][e];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < ng * HD; i += kDecThreads) {
    const int g = i / HD, d = i % HD;
    float sum = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) sum += red[w][g][d];
    part_acc[(((size_t)seq * n_q + (size_t)hk * G + g0 + g) * n_runs + run) * HD + d] = sum;
  }
  if (counters == nullptr) return;     // a separate kernel merges the runs

  // ---- the block that finishes last for this (sequence, head group) merges the runs
  // (src/flash_decode.py:182-205): M = max m_r, w_r = exp(m_r - M), out = sum w_r acc_r / sum w_r l_r,
  // over the runs that hold a visible key, in run order, whichever block does it.
  const int r0 = lo / kRun, r1 = (len - 1) / kRun;
  __threadfence();                     // this block's partials are visible before it is counted
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
  // The other blocks' partial results are read from L2 (__ldcg), never through this SM's L1: an earlier
  // block on this SM may have read a neighbouring entry of the same 128-byte line before this one was written.
  // weights of the runs, 64 runs at a time (they sit where the scores were), then every thread
  // owns output elements and walks the runs with independent loads
  __shared__ float head_max[GMAX], head_inv[GMAX];
  for (int g = warp; g < ng; g += kDecWarps) {
    const size_t base = ((size_t)seq * n_q + (size_t)hk * G + g0 + g) * n_runs;
    float M = -INFINITY;
    for (int r = r0 + lane; r <= r1; r += 32) M = fmaxf(M, __ldcg(part_m + base + r));
    M = warp_max(M);
    float denom = 0.f;
    for (int r = r0 + lane; r <= r1; r += 32) denom += expf(__ldcg(part_m + base + r) - M) * __ldcg(part_l + base + r);
    denom = warp_sum(denom);
    if (lane == 0) {
      head_max[g] = M;
      head_inv[g] = 1.f / denom;
    }
  }
  constexpr int kItems = (GMAX * HD + kDecThreads - 1) / kDecThreads;
  float num[kItems];
#pragma unroll
  for (int i = 0; i < kItems; ++i) num[i] = 0.f;
  for (int c0 = r0; c0 <= r1; c0 += kRun) {
    const int n_here = min(kRun, r1 - c0 + 1);
    __syncthreads();
    for (int i = threadIdx.x; i < ng * n_here; i += kDecThreads) {
      const int g = i / n_here, r = i - g * n_here;
      const size_t base = ((size_t)seq * n_q + (size_t)hk * G + g0 + g) * n_runs;
      scores[g][r] = expf(__ldcg(part_m + base + c0 + r) - head_max[g]);
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < kItems; ++i) {
      const int item = threadIdx.x + i * kDecThreads;
      if (item < ng * HD) {
        const int g = item / HD, d = item - g * HD;
        const float* pa = part_acc + (((size_t)seq * n_q + (size_t)hk * G + g0 + g) * n_runs + c0) * HD + d;
        float a = num[i];
#pragma unroll 8
        for (int r = 0; r < n_here; ++r) a = fmaf(scores[g][r], __ldcg(pa + (size_t)r * HD), a);
        num[i] = a;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < kItems; ++i) {
    const int item = threadIdx.x + i * kDecThreads;
    if (item < ng * HD) {
      const int g = item / HD, d = item - g * HD;
      out[((size_t)seq * n_q + (size_t)hk * G + g0 + g) * HD + d] = from_f32<T>(num[i] * head_inv[g]);
    }
  }
}

// Merge of the runs (src/flash_decode.py:182-205): M = max m_r, w_r = exp(m_r - M),
// out = sum w_r acc_r / sum w_r l_r, over the runs that hold a visible key, in run order.
template <typename T>
__global__ void decode_merge_kernel(const float* __restrict__ part_m, const float* __restrict__ part_l,
                                    const float* __restrict__ part_acc, T* __restrict__ out,
                                    const int* __restrict__ seq_kvlen, int n_q, int hd, int window, int run_len,
                                    int n_runs) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.y, h = blockIdx.x;
  const int len = seq_kvlen[seq];
  if (len <= 0) {        // no keys: no block wrote partial results for this sequence; its output is zeros
    for (int d = threadIdx.x; d < hd; d += blockDim.x) out[((size_t)seq * n_q + h) * hd + d] = from_f32<T>(0.f);
    return;
  }
  const int lo = first_visible(len, window);
  const int r0 = lo / run_len, r1 = (len - 1) / run_len;
  const size_t base = ((size_t)seq * n_q + h) * n_runs;
  float M = -INFINITY;
  for (int r = r0; r <= r1; ++r) M = fmaxf(M, part_m[base + r]);
  float denom = 0.f;
  for (int r = r0; r <= r1; ++r) denom += expf(part_m[base + r] - M) * part_l[base + r];
  const float inv = 1.f / denom;
  for (int d = threadIdx.x; d < hd; d += blockDim.x) {
    float num = 0.f;
    for (int r = r0; r <= r1; ++r) num += expf(part_m[base + r] - M) * part_acc[(base + r) * hd + d];
    out[((size_t)seq * n_q + h) * hd + d] = from_f32<T>(num * inv);
  }
}

template <typename T, int HD, int GMAX>
static int launch_split(const void* q, const void* k_cache, const void* v_cache, float* part_m, float* part_l,
                        float* part_acc, const int* seq_slot, const int* seq_kvlen, const int* block_table,
                        int max_pages, int page_size, int n_seqs, int n_q, int n_kv, float scale, int window,
                        int run_len, int n_runs, int* counters, void* out, cudaStream_t stream) {
  const int G = n_q / n_kv;
  const int chunks = (G + GMAX - 1) / GMAX;
  dim3 grid(n_runs, n_kv * chunks, n_seqs);
  if (run_len != 64) return LLMIE_ERR_UNSUPPORTED_SIZE;
  launch_k(decode_split_kernel<T, HD, GMAX>, dim3(grid), dim3(kDecThreads), 0, stream, (const T*)q, (const T*)k_cache,
           (const T*)v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen, block_table, max_pages, page_size, n_q,
           n_kv, scale, window, run_len, n_runs, counters, (T*)out);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

template <typename T, int HD>
static int launch_split_g(int G, const void* q, const void* k_cache, const void* v_cache, float* part_m,
                          float* part_l, float* part_acc, const int* seq_slot, const int* seq_kvlen,
                          const int* block_table, int max_pages, int page_size, int n_seqs, int n_q, int n_kv,
                          float scale, int window, int run_len, int n_runs, int* counters, void* out,
                          cudaStream_t stream) {
  if (G <= 4)
    return launch_split<T, HD, 4>(q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen, block_table,
                                  max_pages, page_size, n_seqs, n_q, n_kv, scale, window, run_len, n_runs, counters,
                                  out, stream);
  return launch_split<T, HD, 8>(q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen, block_table,
                                max_pages, page_size, n_seqs, n_q, n_kv, scale, window, run_len, n_runs, counters, out,
                                stream);
}

template <typename T>
static int launch_split_hd(int hd, int G, const void* q, const void* k_cache, const void* v_cache, float* part_m,
                           float* part_l, float* part_acc, const int* seq_slot, const int* seq_kvlen,
                           const int* block_table, int max_pages, int page_size, int n_seqs, int n_q, int n_kv,
                           float scale, int window, int run_len, int n_runs, int* counters, void* out,
                           cudaStream_t stream) {
#define LLMIE_CASE(HD)                                                                                          \
  case HD:                                                                                                      \
    return launch_split_g<T, HD>(G, q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen,          \
                                 block_table, max_pages, page_size, n_seqs, n_q, n_kv, scale, window, run_len,  \
                                 n_runs, counters, out, stream);
  switch (hd) {
    LLMIE_CASE(16)
    LLMIE_CASE(32)
    LLMIE_CASE(64)
    LLMIE_CASE(128)
    default:
      return LLMIE_ERR_UNSUPPORTED_SIZE;
  }
#undef LLMIE_CASE
}

}  // namespace llmie

using namespace llmie;

// 1 when attention_decode takes this head size and dtype, else 0 (the caller then uses the plain kernel).
extern "C" int llmie_attention_decode_supported(int hd, int dtype) {
  if (dtype != LLMIE_F32 && dtype != LLMIE_BF16) return 0;
  return (hd == 16 || hd == 32 || hd == 64 || hd == 128) ? 1 : 0;
}

// Keys per block (`run_len`) that the kernels use: one cache page.
extern "C" int llmie_attention_decode_run_len(int n_seqs, int hd, int dtype) {
  (void)n_seqs; (void)hd; (void)dtype;
  return 64;
}

// q, out: [n_seqs, n_q * hd] (one token per sequence); caches [n_pages, n_kv, page_size, hd].
// part_m, part_l: float32 [n_seqs * n_q * n_runs]; part_acc: float32 [n_seqs * n_q * n_runs * hd].
// n_runs * run_len must cover the longest sequence the lengths on the device can name.
extern "C" int llmie_attention_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                                      float* part_m, float* part_l, float* part_acc, const int* seq_slot,
                                      const int* seq_kvlen, const int* block_table, int max_pages, int page_size,
                                      int n_seqs, int n_q, int n_kv, int hd, float scale, int window, int run_len,
                                      int n_runs, int dtype, cudaStream_t stream) {
  if (n_seqs < 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || page_size <= 0 || max_pages <= 0) return LLMIE_ERR_BAD_ARG;
  if (n_runs <= 0) return LLMIE_ERR_BAD_ARG;
  if (page_size != 64 || run_len != 64) return LLMIE_ERR_UNSUPPORTED_SIZE;    // a run is one cache page of 64 keys
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache)) return LLMIE_ERR_ALIGNMENT;
  if (n_seqs == 0) return LLMIE_OK;
  if (n_seqs > 65535 || n_runs > 0x7fffffff / 1) return LLMIE_ERR_UNSUPPORTED_SIZE;
  const int G = n_q / n_kv;
  int rc;
  if (dtype == LLMIE_F32)
    rc = launch_split_hd<float>(hd, G, q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen,
                                block_table, max_pages, page_size, n_seqs, n_q, n_kv, scale, window, run_len, n_runs,
                                nullptr, nullptr, stream);
  else if (dtype == LLMIE_BF16)
    rc = launch_split_hd<__nv_bfloat16>(hd, G, q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen,
                                        block_table, max_pages, page_size, n_seqs, n_q, n_kv, scale, window, run_len,
                                        n_runs, nullptr, nullptr, stream);
  else
    return LLMIE_ERR_DTYPE;
  if (rc != LLMIE_OK) return rc;
  dim3 grid(n_q, n_seqs);
  const int threads = hd < 32 ? 32 : (hd > 256 ? 256 : ((hd + 31) / 32) * 32);
  if (dtype == LLMIE_F32)
    launch_k(decode_merge_kernel<float>, dim3(grid), dim3(threads), 0, stream, part_m, part_l, part_acc, (float*)out, seq_kvlen, n_q, hd,
                                                             window, run_len, n_runs);
  else
    launch_k(decode_merge_kernel<__nv_bfloat16>, dim3(grid), dim3(threads), 0, stream, part_m, part_l, part_acc, (__nv_bfloat16*)out,
                                                                     seq_kvlen, n_q, hd, window, run_len, n_runs);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// The same in ONE launch: the block that finishes last for a (sequence, KV head) merges its runs.
// counters: int32 [n_seqs * n_kv * ceil(G / 4 or 8)], all zero before the first call; every launch
// leaves them zero again. Launches that share `counters` must not overlap on the GPU.
extern "C" int llmie_attention_decode_fused(const void* q, const void* k_cache, const void* v_cache, void* out,
                                            float* part_m, float* part_l, float* part_acc, int* counters,
                                            const int* seq_slot, const int* seq_kvlen, const int* block_table,
                                            int max_pages, int page_size, int n_seqs, int n_q, int n_kv, int hd,
                                            float scale, int window, int run_len, int n_runs, int dtype,
                                            cudaStream_t stream) {
  if (n_seqs < 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || page_size <= 0 || max_pages <= 0 || !counters)
    return LLMIE_ERR_BAD_ARG;
  if (n_runs <= 0) return LLMIE_ERR_BAD_ARG;
  if (page_size != 64 || run_len != 64) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (!aligned16(q) || !aligned16(k_cache) || !aligned16(v_cache)) return LLMIE_ERR_ALIGNMENT;
  if (n_seqs == 0) return LLMIE_OK;
  if (n_seqs > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
  const int G = n_q / n_kv;
  if (dtype == LLMIE_F32)
    return launch_split_hd<float>(hd, G, q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen,
                                  block_table, max_pages, page_size, n_seqs, n_q, n_kv, scale, window, run_len, n_runs,
                                  counters, out, stream);
  if (dtype == LLMIE_BF16)
    return launch_split_hd<__nv_bfloat16>(hd, G, q, k_cache, v_cache, part_m, part_l, part_acc, seq_slot, seq_kvlen,
                                          block_table, max_pages, page_size, n_seqs, n_q, n_kv, scale, window, run_len,
                                          n_runs, counters, out, stream);
  return LLMIE_ERR_DTYPE;
}

// ------------------------------------------------------------------------------------------
// The same attention for callers that must not allocate: scratch lives in the device image.
// See attention_decode_noalloc.h for who needs this, the limit and the sharing rules.
#include "attention_decode_noalloc.h"
#include <mutex>

namespace llmie {
constexpr size_t kNoAllocFloats = LLMIE_NOALLOC_SCRATCH_BYTES / sizeof(float);
// Device code could name this array directly. Host code cannot: on the host the name is only a
// stand-in for the symbol, not a device address, so the launcher below asks the runtime for the
// address once per device and hands THAT to the kernels.
static __device__ __align__(256) float g_noalloc_scratch[kNoAllocFloats];

constexpr int kMaxDevices = 64;
static float* g_noalloc_addr[kMaxDevices] = {nullptr};
static std::mutex g_noalloc_mutex;

// Device address of the array on the CURRENT device; looked up on first use per device.
static int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return LLMIE_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (!g_noalloc_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!p) return LLMIE_ERR_BAD_ARG;
    g_noalloc_addr[dev] = p;
  }
  *out = g_noalloc_addr[dev];
  return LLMIE_OK;
}
}  // namespace llmie

extern "C" unsigned long long llmie_attention_decode_noalloc_capacity(void) { return LLMIE_NOALLOC_SCRATCH_BYTES; }

extern "C" int llmie_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                              const int* seq_slot, const int* seq_kvlen, const int* block_table,
                                              int max_pages, int page_size, int n_seqs, int n_q, int n_kv, int hd,
                                              float scale, int window, int run_len, int n_runs, int dtype,
                                              cudaStream_t stream) {
  if (n_seqs < 0 || n_q <= 0 || n_runs <= 0 || hd <= 0) return LLMIE_ERR_BAD_ARG;
  const unsigned long long n_ml = (unsigned long long)n_seqs * (unsigned long long)n_q * (unsigned long long)n_runs;
  const unsigned long long need = n_ml * (unsigned long long)(hd + 2);
  if (need > kNoAllocFloats) return LLMIE_ERR_SCRATCH_TOO_SMALL;
  float* scratch = nullptr;
  const int rc = noalloc_scratch(&scratch);
  if (rc != LLMIE_OK) return rc;
  // [part_m | part_l | part_acc]; every entry that the merge kernel reads is written by the split
  // kernel of this same call, so what an earlier call left behind is never seen.
  return llmie_attention_decode(q, k_cache, v_cache, out, scratch, scratch + n_ml, scratch + 2 * n_ml, seq_slot,
                                seq_kvlen, block_table, max_pages, page_size, n_seqs, n_q, n_kv, hd, scale, window,
                                run_len, n_runs, dtype, stream);
}
