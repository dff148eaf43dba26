// Token choice on the device: argmax, and temperature sampling with a top-p cut.
//
// The reference samples with torch ops on the logits (src/sampler.py:4-33): temperature <= 0
// is argmax; otherwise softmax(logits / T), tokens sorted by falling probability are dropped
// once the mass BEFORE them exceeds top_p (the first is always kept), the rest is renormalised
// and one token is drawn. Here one block per row does the same in float32 without a sort:
//   w_i = exp((x_i - max) / T),  Z = sum w
//   S(t) = sum of w_i > t;  kept = { i : S(w_i) <= top_p * Z }, found by bisection on the bits of t
//   draw: inverse CDF over token ids among the kept, at u * (kept mass)
// u is a counter-based uniform number from (seed, sequence id, how many tokens that sequence
// has drawn), so a sequence's draws do not depend on what else is in the batch.
#include "common.cuh"
#include <math.h>

namespace llmie {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
  z ^= z >> 30; z *= 0xbf58476d1ce4e5b9ULL;
  z ^= z >> 27; z *= 0x94d049bb133111ebULL;
  z ^= z >> 31;
  return z;
}
// 24 random bits scaled into [0, 1): exact in float32.
__device__ __forceinline__ float uniform24(unsigned long long seed, int seq_id, int counter) {
  unsigned long long x = mix64(seed + 0x9E3779B97F4A7C15ULL * (unsigned long long)(seq_id + 1));
  x = mix64(x + 0x9E3779B97F4A7C15ULL * (unsigned long long)(counter + 1));
  return (float)(x >> 40) * (1.0f / 16777216.0f);
}

struct MaxIdx { float v; int i; };
__device__ __forceinline__ MaxIdx better(MaxIdx a, MaxIdx b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

// argmax over a row with 1024 threads; ties go to the lowest index. NaN never wins.
__device__ MaxIdx block_argmax(const float* row, int V, MaxIdx* scratch) {
  MaxIdx best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x) best = better(best, MaxIdx{row[i], i});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  MaxIdx r = (lane < (blockDim.x >> 5)) ? scratch[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, r.v, o), __shfl_xor_sync(0xffffffffu, r.i, o)};
    r = better(r, other);
  }
  if (r.i == 0x7fffffff) r.i = 0;  // a row of NaN or -inf: still a valid token id
  return r;
}

__global__ void __launch_bounds__(kSampleThreads)
sample_kernel(const float* __restrict__ logits, int ld, int V, float temperature, float top_p,
              unsigned long long seed, const unsigned* __restrict__ dev_params, const int* __restrict__ seq_ids,
              int* __restrict__ counters, int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  if (dev_params) {
    // settings kept in device memory: a captured launch then serves every temperature, top_p and seed
    temperature = __uint_as_float(dev_params[0]);
    top_p = __uint_as_float(dev_params[1]);
    seed = (unsigned long long)dev_params[2] | ((unsigned long long)dev_params[3] << 32);
  }
  __shared__ MaxIdx arg_scratch[32];
  __shared__ float red[32];
  __shared__ float chunk_sum[kSampleThreads];
  __shared__ int chosen;
  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * ld;
  const MaxIdx top = block_argmax(row, V, arg_scratch);
  if (temperature <= 0.f) {
    if (threadIdx.x == 0) out[r] = top.i;
    return;
  }
  const float inv_t = 1.f / temperature;
  const float mx = top.v;

  // contiguous chunk per thread, so that the inverse CDF runs in token-id order
  const int chunk = (V + blockDim.x - 1) / blockDim.x;
  const int begin = min(V, (int)threadIdx.x * chunk), end = min(V, begin + chunk);

  float z = 0.f;
  for (int i = begin; i < end; ++i) z += expf((row[i] - mx) * inv_t);
  const float Z = block_sum(z, red);

  float thresh = 0.f;  // keep w >= thresh
  if (top_p < 1.f) {
    const float target = fmaxf(top_p, 0.f) * Z;
    unsigned lo = 0u, hi = 0x3f800000u;  // bits of 0.0 .. 1.0; S(bits(1.0)) = 0 always qualifies
    while (lo < hi) {
      const unsigned mid = lo + ((hi - lo) >> 1);
      const float t = __uint_as_float(mid);
      float s = 0.f;
      for (int i = begin; i < end; ++i) {
        const float w = expf((row[i] - mx) * inv_t);
        if (w > t) s += w;
      }
      s = block_sum(s, red);
      if (s <= target) hi = mid; else lo = mid + 1;
    }
    thresh = __uint_as_float(lo);
  }

  float mine = 0.f;
  for (int i = begin; i < end; ++i) {
    const float w = expf((row[i] - mx) * inv_t);
    if (w >= thresh) mine += w;
  }
  chunk_sum[threadIdx.x] = mine;
  if (threadIdx.x == 0) chosen = -1;
  __syncthreads();
  if (threadIdx.x == 0) {
    // serial scan over 1024 partial sums: cheap, and the order is fixed
    float total = 0.f;
    for (int i = 0; i < kSampleThreads; ++i) total += chunk_sum[i];
    const int counter = counters[r];
    const float u = uniform24(seed, seq_ids[r], counter);
    counters[r] = counter + 1;
    const float target = u * total;
    float run = 0.f;
    int owner = -1;
    for (int i = 0; i < kSampleThreads; ++i) {
      if (chunk_sum[i] > 0.f) {
        if (target < run + chunk_sum[i]) { owner = i; break; }
        run += chunk_sum[i];
      }
    }
    int pick = top.i;  // falls back to the most likely token if rounding ran past the end
    if (owner >= 0) {
      const int b = min(V, owner * chunk), e = min(V, b + chunk);
      int last_kept = -1;
      bool found = false;
      for (int i = b; i < e; ++i) {
        const float w = expf((row[i] - mx) * inv_t);
        if (w >= thresh) {
          last_kept = i;
          run += w;
          if (target < run) { pick = i; found = true; break; }
        }
      }
      if (!found && last_kept >= 0) pick = last_kept;
    }
    chosen = pick;
  }
  __syncthreads();
  if (threadIdx.x == 0) out[r] = chosen;
}

// Greedy choice with many blocks per row, for large vocabularies: block (s, r) scans one slice
// of row r, a second kernel merges the slices. Ties go to the lowest index in both stages.
__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float* __restrict__ logits, int ld, int V, int slices, float* __restrict__ part_val,
                      int* __restrict__ part_idx) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ MaxIdx scratch[32];
  const int s = blockIdx.x, r = blockIdx.y;
  const int chunk = ((V + slices - 1) / slices + 3) & ~3;      // whole groups of four, so that slices stay aligned
  const int begin = min(V, s * chunk), end = min(V, begin + chunk);
  const float* row = logits + (size_t)r * ld;
  MaxIdx best{-INFINITY, 0x7fffffff};
  if ((ld & 3) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15u) == 0) {
    // 16-byte loads; within a thread and between threads the lowest index still wins a tie
    const int end4 = begin + ((end - begin) & ~3);
    for (int i = begin + 4 * threadIdx.x; i < end4; i += 4 * blockDim.x) {
      const float4 q = *reinterpret_cast<const float4*>(row + i);
      best = better(best, MaxIdx{q.x, i});
      best = better(best, MaxIdx{q.y, i + 1});
      best = better(best, MaxIdx{q.z, i + 2});
      best = better(best, MaxIdx{q.w, i + 3});
    }
    for (int i = end4 + threadIdx.x; i < end; i += blockDim.x) best = better(best, MaxIdx{row[i], i});
  } else {
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best = better(best, MaxIdx{row[i], i});
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) scratch[warp] = best;
  __syncthreads();
  if (warp == 0) {
    MaxIdx m = (lane < (blockDim.x >> 5)) ? scratch[lane] : MaxIdx{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      MaxIdx other{__shfl_xor_sync(0xffffffffu, m.v, o), __shfl_xor_sync(0xffffffffu, m.i, o)};
      m = better(m, other);
    }
    if (lane == 0) {
      part_val[r * slices + s] = m.v;
      part_idx[r * slices + s] = m.i;
    }
  }
}

__global__ void argmax_merge_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx, int slices,
                                    int* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  const int r = blockIdx.x, lane = threadIdx.x;
  MaxIdx best{-INFINITY, 0x7fffffff};
  for (int s = lane; s < slices; s += 32) best = better(best, MaxIdx{part_val[r * slices + s], part_idx[r * slices + s]});
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    MaxIdx other{__shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o)};
    best = better(best, other);
  }
  if (lane == 0) out[r] = best.i == 0x7fffffff ? 0 : best.i;
}

// tokens[i] = sampled[i] for the lanes of a decode step (feeds the next step on the device)
__global__ void copy_int_kernel(const int* __restrict__ src, int* __restrict__ dst, int n) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = src[i];
}

}  // namespace llmie

using namespace llmie;

// logits: [n_rows, ld] float32 with V <= ld valid columns. seq_ids / counters: [n_rows] (unused when
// temperature <= 0, may then be null). out: [n_rows] int32. dev_params: null, or four 32-bit words in device
// memory [bits of temperature, bits of top_p, low and high half of the seed] that stand for the three
// arguments; seq_ids and counters are then always required.
extern "C" int llmie_sample(const float* logits, int n_rows, int V, int ld, float temperature, float top_p,
                            unsigned long long seed, const unsigned* dev_params, const int* seq_ids, int* counters,
                            int* out, cudaStream_t stream) {
  if (n_rows < 0 || V <= 0 || ld < V) return LLMIE_ERR_BAD_ARG;
  if ((temperature > 0.f || dev_params) && (!seq_ids || !counters)) return LLMIE_ERR_BAD_ARG;
  if (n_rows == 0) return LLMIE_OK;
  launch_k(sample_kernel, dim3(n_rows), dim3(kSampleThreads), 0, stream, logits, ld, V, temperature, top_p, seed,
           dev_params, seq_ids, counters, out);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

extern "C" int llmie_copy_int(const int* src, int* dst, int n, cudaStream_t stream) {
  if (n < 0) return LLMIE_ERR_BAD_ARG;
  if (n == 0) return LLMIE_OK;
  launch_k(copy_int_kernel, dim3((n + 255) / 256), dim3(256), 0, stream, src, dst, n);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

// Greedy tokens with `slices` blocks per row. part_val / part_idx: scratch of n_rows * slices elements.
extern "C" int llmie_argmax(const float* logits, int n_rows, int V, int ld, int slices, float* part_val, int* part_idx,
                            int* out, cudaStream_t stream) {
  if (n_rows < 0 || V <= 0 || ld < V || slices <= 0 || slices > 1024) return LLMIE_ERR_BAD_ARG;
  if (n_rows == 0) return LLMIE_OK;
  if (n_rows > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
  launch_k(argmax_partial_kernel, dim3(dim3(slices, n_rows)), dim3(256), 0, stream, logits, ld, V, slices, part_val, part_idx);
  LLMIE_LAUNCH_CHECK();
  launch_k(argmax_merge_kernel, dim3(n_rows), dim3(32), 0, stream, part_val, part_idx, slices, out);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}
