// A whole one-token step of a stack of Llama-style layers in ONE persistent kernel.
//
// A one-token step at small batch is a chain of dependent phases (norm + QKV + rotation, attention,
// output projection, norm + gate/up + SwiGLU, down projection, ... final norm + head), each of
// which lasts a few microseconds. Here one block per SM stays resident for the whole step and the
// phases are separated by grid-wide barriers instead of kernel boundaries. The reference runs the
// same chain as ~17 launches per layer (src/model.py:39-127), or one CUDA graph of them for
// batch 1 (src/cuda_graph.py).
//
// Weights never depend on data, so their stream is decoupled from the phases: four producer warps
// per block request every 16-row tile segment of every phase, in order, into a ring of
// shared-memory slots with bulk asynchronous copies (cp.async.bulk, completion counted by an
// mbarrier per slot), as far ahead as the ring has room - through barriers, staging and attention.
// Eight consumer warps stage the activations of a phase in shared memory, multiply slot by slot
// with mma.sync (16-byte fragment reads from the slot), and release slots through a second
// mbarrier. Every wait (slot barriers, grid barriers) is bounded and ends the launch with a status.
//
// Measured on B200 at the Llama 3.2 1B shape, batch 8, 512 cached tokens: 1.21 ms per step, against
// 0.77 ms for the same step as a CUDA graph of the stand-alone kernels. Per layer (us, block 0):
// QKV 8.5, attention 8.9 (+6.7 waiting for the slowest block), output projection 5.2, gate/up 16.2,
// down 15.7, other barriers about 2 each. The ring is full most of the time (the producers wait
// 75 % of the launch): the consumer warps are the limit. They spend per layer about 12 us staging
// activations, 11 us in the products, 10 us in reductions and epilogues, 16 us in attention and
// 10 us at barriers, and only the ring's 128 KB per SM (3 us of streaming) can run ahead of that;
// a bound of about 43 us a layer follows, no better than the stand-alone kernels. The engine
// therefore uses this kernel only when LLMIE_STACKED_DECODE=1 is set; it is kept, tested.
//
// The math of every phase is that of the stand-alone kernels:
//   gemm_fused_decode.cu  h * w staged as bfloat16 rows in shared memory, rstd applied to the sums
//   attention_decode.cu   one cache page per work item, all query heads of a KV head; the group
//                         that finishes a (sequence, KV head) last merges its pages
// Data that another block wrote earlier in the same launch (h, q, attention partials, activations,
// this step's K/V rows) is read with loads that bypass L1, which is not coherent between SMs.
//
// Limits (the caller checks them and otherwise runs the per-kernel path): bfloat16 weights and
// cache, at most 8 sequences, pages of 64, head size 64 or 128 with the whole head rotated, at
// most 8 query heads per KV head, no window, widths that are multiples of 32, a model width of at
// most 4096 (wider feed-forward inputs are taken in passes of 4096 columns).
#include "common.cuh"
#include "tcgen05.cuh"
#include <math.h>

namespace llmie {

using namespace tc;      // mbarriers with bounded waits

constexpr int kStWarps = 8;                  // warps that compute (the "consumers")
constexpr int kStCThreads = kStWarps * 32;
constexpr int kStPWarps = 4;                  // warps that only request weights (the "producers"), a segment each in turn
constexpr int kStThreads = kStCThreads + kStPWarps * 32;
constexpr int kStPad = 32;                   // bfloat16 elements of padding per staged row
constexpr int kStMaxGroups = 4;               // attention work groups per block, at most
constexpr int kStatusBarrierTimeout = 4;
constexpr int kStatusRingTimeout = 5;
// The ring of weight slots in shared memory: a slot holds kSegChunks chunks of 32 k (1 KB) of each of a
// tile's 16 rows; rows are 64 bytes further apart than their data, so that the 16-byte fragment reads of a
// quarter warp (two rows) fall into different banks.
constexpr int kSegChunks = 16;
constexpr int kSegK = kSegChunks * 32;
constexpr int kSlotPitch = kSegK * 2 + 64;    // bytes between rows of a slot
constexpr int kSlotBytes = 16 * kSlotPitch;
constexpr int kMaxSlots = 24;
constexpr int kXsK = 4096;                    // columns of the staged activations at most; wider inputs go in passes

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
  int ring_offset, n_slots;                // the ring of weight slots
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
// named barriers: 1 = the consumer warps, 2.. = attention work groups
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kStCThreads) : "memory"); }
// the consumers' barrier with a vote: true for everyone when any thread brings true
__device__ __forceinline__ bool consumer_sync_any(bool mine) {
  unsigned any;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.or.pred p, 1, %2, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(any) : "r"((unsigned)mine), "n"(kStCThreads) : "memory");
  return any != 0;
}
__device__ __forceinline__ void group_sync(int group, int threads) {      // the threads of one attention work group
  asm volatile("bar.sync %0, %1;" ::"r"(group + 2), "r"(threads) : "memory");
}

// All blocks of the launch meet here (their consumer warps; the producer warp runs ahead: weights
// depend on nothing). The counter only ever grows: barrier number k of launch number e completes
// when it reaches (e * barriers_per_launch + k + 1) * blocks, so nothing has to be reset while
// some block may still be polling. The wait is bounded; a block that gives up sets the status word
// and the whole launch winds down (every other block gives up at the same barrier). Returns false
// when the launch is to be abandoned.
__device__ __forceinline__ bool grid_barrier(unsigned long long* counter, unsigned long long target, int* status,
                                             volatile int* s_abort) {
  __threadfence();
  consumer_sync();
  if (threadIdx.x == 0) {
    atomicAdd(counter, 1ull);
    unsigned spins = 0;
    while (ld_acquire_u64(counter) < target) {
      if (++spins > (1u << 22) || *s_abort) {
        atomicExch(status, kStatusBarrierTimeout);
        *s_abort = 1;
        break;
      }
    }
    __threadfence();
  }
  consumer_sync();
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
  uint64_t full[kMaxSlots];    // a slot's weights have arrived
  uint64_t empty[kMaxSlots];   // every consumer warp is done with the slot
};

// Rows of h * w (or of the embedding row * w at the first layer) as bfloat16 in shared memory, and
// per warp the sums of squares of the rows. A thread takes eight consecutive elements of four rows
// at a time, so those loads are in flight together while few registers are held. With FROM_EMB,
// block b also writes row b of the float32 residual stream. Consumer threads only; ends with
// their barrier.
__device__ __forceinline__ void stage_normed(bool FROM_EMB, const StackParams& p, const float* norm_w, int K,
                                             __nv_bfloat16* xs, StackShared& sh) {
  const int xs_stride = K + kStPad;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
#pragma unroll 1
  for (int b0 = 0; b0 < 8; b0 += 4) {
    float ssq[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = threadIdx.x * 8; k < K; k += kStCThreads * 8) {
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
  consumer_sync();
}

// Columns [k0, k0 + K) of a bfloat16 activation [batch, ld] into shared memory. Consumer threads
// only; ends with their barrier.
__device__ __forceinline__ void stage_plain(const StackParams& p, const __nv_bfloat16* src, int ld, int k0, int K,
                                            __nv_bfloat16* xs) {
  const int xs_stride = K + kStPad;
  const int per_row = K >> 3;
#pragma unroll 4
  for (int i = threadIdx.x; i < 8 * per_row; i += kStCThreads) {
    const int b = i / per_row, k = (i - b * per_row) << 3;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (b < p.batch) v = st_ldcg16(src + (size_t)b * ld + k0 + k);
    *reinterpret_cast<uint4*>(xs + (size_t)b * xs_stride + k) = v;
  }
  consumer_sync();
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

// ------------------------------------------------------------------------------------------ schedule
// The step as a list of passes that the producer warp and the consumer warps walk in the same
// order. Per layer: A (norm, QKV, rotation, cache write), B (attention), C (output projection,
// h += y; in passes of kXsK input columns), D (norm, gate / up, SwiGLU), E (down projection, h += y;
// in passes); at the end the final norm and the head. A pass of a product streams, for every tile
// of 16 weight rows that the block owns (tile numbers go round the blocks), the columns
// [k0, k0 + klen) of those rows in segments of kSegK.
struct Pass {
  int kind;                    // 0 product, 1 attention
  int var;
  bool normed, from_emb, barrier_after;
  const StackLayer* L;
  const __nv_bfloat16* W;      // [rows, ldw]
  int ldw, k0, klen, tiles, half_n;
  void* out;
  int ldo;
  const float* norm_w;
  float eps;
  const __nv_bfloat16* x_src;  // for the passes that are not normed: [batch, ldw]
};

template <int HD>
__device__ __forceinline__ int passes_per_layer(const StackParams& p, int& n_c, int& n_e) {
  n_c = (p.n_q * HD + kXsK - 1) / kXsK;
  n_e = (p.ff + kXsK - 1) / kXsK;
  return 3 + n_c + n_e;
}

template <int HD>
__device__ __forceinline__ void get_pass(const StackParams& p, int idx, int per_layer, int n_c, int n_e, Pass& q) {
  const int l = idx / per_layer;
  q.kind = 0;
  q.normed = false;
  q.from_emb = false;
  q.barrier_after = true;
  q.half_n = 0;
  q.k0 = 0;
  q.norm_w = nullptr;
  q.eps = 0.f;
  q.x_src = nullptr;
  if (l >= p.n_layers) {        // the head
    q.L = p.layers + (p.n_layers - 1);
    q.var = kGemmF32; q.normed = true; q.W = p.head; q.ldw = p.d; q.klen = p.d; q.tiles = p.vocab >> 4;
    q.out = p.logits; q.ldo = p.vocab; q.norm_w = p.final_norm; q.eps = p.final_eps; q.barrier_after = false;
    return;
  }
  const StackLayer* L = p.layers + l;
  q.L = L;
  int r = idx - l * per_layer;
  if (r == 0) {
    q.var = kGemmQkvRope; q.normed = true; q.from_emb = l == 0; q.W = L->wqkv; q.ldw = p.d; q.klen = p.d;
    q.tiles = (p.n_q + 2 * p.n_kv) * (HD >> 4); q.out = nullptr; q.ldo = 0; q.norm_w = L->norm1; q.eps = L->eps1;
    return;
  }
  if (r == 1) {
    q.kind = 1;
    q.tiles = 0;
    return;
  }
  r -= 2;
  if (r < n_c) {
    const int K = p.n_q * HD;
    q.var = kGemmAddH; q.W = L->wo; q.ldw = K; q.k0 = r * kXsK; q.klen = min(kXsK, K - q.k0); q.tiles = p.d >> 4;
    q.out = p.h; q.ldo = p.d; q.x_src = p.attn; q.barrier_after = r == n_c - 1;
    return;
  }
  r -= n_c;
  if (r == 0) {
    q.var = kGemmGateSwiGLU; q.normed = true; q.W = L->wgu; q.ldw = p.d; q.klen = p.d; q.tiles = p.ff >> 3;
    q.half_n = p.ff; q.out = p.act; q.ldo = p.ff; q.norm_w = L->norm2; q.eps = L->eps2;
    return;
  }
  r -= 1;
  q.var = kGemmAddH; q.W = L->wdown; q.ldw = p.ff; q.k0 = r * kXsK; q.klen = min(kXsK, p.ff - q.k0);
  q.tiles = p.d >> 4; q.out = p.h; q.ldo = p.d; q.x_src = p.act; q.barrier_after = r == n_e - 1;
}

__device__ __forceinline__ void bulk_g2s(unsigned dst, const void* src, unsigned bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// The producer warp: requests every segment of every tile of every pass into the ring, as far
// ahead as the ring has room - across passes and grid barriers, since weights depend on nothing.
// So the memory system stays busy while the consumers wait for one another, stage activations
// or do attention. Lane r copies row r of the tile (a bulk asynchronous copy that reports its
// bytes to the slot's barrier).
template <int HD>
__device__ __forceinline__ void produce(const StackParams& p, StackShared& sh, unsigned ring_addr) {
  const int lane = threadIdx.x & 31;
  const int pw = (threadIdx.x - kStCThreads) >> 5;     // which producer warp: it takes every kStPWarps-th segment
  int n_c, n_e;
  const int per_layer = passes_per_layer<HD>(p, n_c, n_e);
  const int n_passes = p.n_layers * per_layer + 1;
  unsigned count = 0;                                  // segments of the block so far
  for (int idx = 0; idx < n_passes; ++idx) {
    Pass q;
    get_pass<HD>(p, idx, per_layer, n_c, n_e, q);
    if (q.kind != 0) continue;
    const int n_seg = (q.klen + kSegK - 1) / kSegK;
    for (int tile = blockIdx.x; tile < q.tiles; tile += gridDim.x) {
      int lo, hi;
      st_tile_rows(q.var, tile, HD, q.half_n, lo, hi);
      const int row = lane < 8 ? lo + lane : hi + lane - 8;
      const __nv_bfloat16* src_row = q.W + (size_t)row * q.ldw + q.k0;
      for (int seg = 0; seg < n_seg; ++seg, ++count) {
        if ((int)(count % kStPWarps) != pw) continue;
        const int slot = count % p.n_slots;
        const unsigned use = count / p.n_slots;
        // (the whole warp decides together: the lanes meet again at the warp barrier below)
        if (!__all_sync(0xffffffffu, mbar_wait(&sh.empty[slot], (use & 1u) ^ 1u, &sh.abort))) {     // the slot's previous use is over
          if (lane == 0 && !sh.abort) {
            atomicExch(p.status, kStatusRingTimeout);
            sh.abort = 1;
          }
          return;
        }
        const int cols = min(kSegK, q.klen - seg * kSegK);
        if (lane == 0) mbar_arrive_expect_tx(&sh.full[slot], 16u * (unsigned)cols * 2u);
        __syncwarp();
        if (lane < 16)
          bulk_g2s(ring_addr + (unsigned)slot * kSlotBytes + (unsigned)lane * kSlotPitch, src_row + seg * kSegK,
                   (unsigned)cols * 2u, &sh.full[slot]);
      }
    }
  }
}

// One product pass on the consumer side: stage the activations, then for every tile of the block
// take its segments from the ring. Warp w multiplies chunk w of a segment (16-byte fragment reads
// from the slot, the matching activations from the staged rows), then lets the slot go. At the end
// of a tile the eight partial sums meet in warp 0 through shared memory (two buffers in turn, one
// consumer barrier per tile), whose lanes hold whole (row, row + 8) x (column pair) results and
// run the epilogue while the others go on with the next tile.
template <int HD>
__device__ __forceinline__ bool consume_pass(const StackParams& p, const Pass& q, StackShared& sh, __nv_bfloat16* xs,
                                             float4* red, const unsigned char* ring, unsigned& count, int& parity) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, t = lane & 3;
  float rs0 = 1.f, rs1 = 1.f;        // rstd of the two batch columns this lane holds
  if (q.normed) {
    stage_normed(q.from_emb, p, q.norm_w, q.klen, xs, sh);
    float s0 = 0.f, s1 = 0.f;
#pragma unroll
    for (int w = 0; w < kStWarps; ++w) {
      s0 += sh.ssw[w * 8 + 2 * t];
      s1 += sh.ssw[w * 8 + 2 * t + 1];
    }
    rs0 = rsqrtf(s0 / (float)q.klen + q.eps);
    rs1 = rsqrtf(s1 / (float)q.klen + q.eps);
  } else {
    stage_plain(p, q.x_src, q.ldw, q.k0, q.klen, xs);
  }
  const int xs_stride = q.klen + kStPad;
  const uint4* x_row = reinterpret_cast<const uint4*>(xs + (size_t)g * xs_stride) + t;
  const int n_seg = (q.klen + kSegK - 1) / kSegK;
  const int n_chunks = q.klen >> 5;
  for (int tile = blockIdx.x; tile < q.tiles; tile += gridDim.x) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    bool failed = false;             // a warp whose wait ran out skips to the tile's barrier and says so there
    for (int seg = 0; seg < n_seg && !failed; ++seg, ++count) {
      const int slot = count % p.n_slots;
      const unsigned use = count / p.n_slots;
      // (the whole warp decides together: mma.sync and the warp barrier below are warp-wide)
      if (!__all_sync(0xffffffffu, mbar_wait(&sh.full[slot], use & 1u, &sh.abort))) {
        if (lane == 0 && !sh.abort) {
          atomicExch(p.status, kStatusRingTimeout);
          sh.abort = 1;
        }
        failed = true;
        break;
      }
#pragma unroll
      for (int i = 0; i < kSegChunks / kStWarps; ++i) {
        const int cs = warp * (kSegChunks / kStWarps) + i;     // this warp's chunks of 32 k within the segment
        const int c = seg * kSegChunks + cs;
        if (c < n_chunks) {
          const unsigned char* base = ring + (size_t)slot * kSlotBytes + cs * 64 + t * 16;
          const uint4 wa = *reinterpret_cast<const uint4*>(base + g * kSlotPitch);
          const uint4 wb = *reinterpret_cast<const uint4*>(base + (g + 8) * kSlotPitch);
          const uint4 xv = x_row[c * 4];
          st_mma(acc, wa.x, wb.x, wa.y, wb.y, xv.x, xv.y);
          st_mma(acc, wa.z, wb.z, wa.w, wb.w, xv.z, xv.w);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sh.empty[slot]);
    }
    float4* mine = red + ((parity * kStWarps + warp) * 32 + lane);
    if (warp != 0) *mine = make_float4(acc[0], acc[1], acc[2], acc[3]);
    // every consumer warp reaches this barrier, whatever happened to its waits: nobody is left behind at it
    if (consumer_sync_any(failed)) return false;
    if (warp == 0) {
#pragma unroll
      for (int o = 1; o < kStWarps; ++o) {
        const float4 v = mine[o * 32];
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
      }
      int lo, hi;
      st_tile_rows(q.var, tile, HD, q.half_n, lo, hi);
      tile_epilogue(q.var, p, q.L, acc, lo, hi, g, t, rs0, rs1, q.out, q.ldo, sh);
    }
    parity ^= 1;
  }
  return true;
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
  extern __shared__ __align__(128) unsigned char st_smem[];
  __shared__ StackShared sh;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(st_smem);          // [8][K + pad], K the pass's inner size
  float4* red = reinterpret_cast<float4*>(st_smem + p.red_offset);        // [2][warps][32 lanes]
  float* att_smem = reinterpret_cast<float*>(st_smem);                    // aliases xs during attention
  const unsigned char* ring = st_smem + p.ring_offset;
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
  if (threadIdx.x == 0) {
    sh.abort = 0;
    for (int i = 0; i < p.n_slots; ++i) {
      mbar_init(&sh.full[i], 1);                   // the producer's expect_tx arrival; the copies report bytes
      mbar_init(&sh.empty[i], kStWarps);           // one arrival per consumer warp
    }
    fence_mbar_init();
  }
  __syncthreads();

  if (threadIdx.x >= kStCThreads) {
    // ---- the producer warps
    produce<HD>(p, sh, smem_u32(ring));
  } else {
    // ---- the consumer warps
    int n_c, n_e;
    const int per_layer = passes_per_layer<HD>(p, n_c, n_e);
    const int n_passes = p.n_layers * per_layer + 1;
    const unsigned long long per_launch = (unsigned long long)p.n_layers * 5ull;
    unsigned long long target = (*p.epoch) * per_launch * gridDim.x;
    const int group = threadIdx.x / (GW * 32);
    const int n_groups = gridDim.x * kGroups;
    int n_phase = 0;
    unsigned count = 0;                            // segments taken from the ring so far
    int parity = 0;
#define LLMIE_STAMP()                                                                 \
  do {                                                                                 \
    if (p.phase_ns && blockIdx.x == 0 && threadIdx.x == 0) {                           \
      unsigned long long t_;                                                           \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                           \
      p.phase_ns[n_phase] = t_;                                                        \
    }                                                                                  \
    ++n_phase;                                                                         \
  } while (0)
    LLMIE_STAMP();
    bool ok = true;
    for (int idx = 0; idx < n_passes && ok; ++idx) {
      Pass q;
      get_pass<HD>(p, idx, per_layer, n_c, n_e, q);
      if (q.kind == 1) {
        // one cache page per work item; pages in the outer order, so that the pages that hold keys
        // come first and spread over all groups
        const int per_run = p.batch * p.n_kv;
        const int n_items = per_run * p.n_runs;
        for (int item = blockIdx.x * kGroups + group; item < n_items; item += n_groups) {
          const int run = item / per_run, rest = item - run * per_run;
          attention_item<HD, GW>(p, q.L, rest / p.n_kv, rest % p.n_kv, run, group, att_smem + group * kAttFloats, sh);
        }
      } else {
        ok = consume_pass<HD>(p, q, sh, xs, red, ring, count, parity);
      }
      if (ok && q.barrier_after) {
        LLMIE_STAMP();
        target += gridDim.x;
        ok = grid_barrier(p.bar_counter, target, p.status, &sh.abort);
        LLMIE_STAMP();
      }
    }
    LLMIE_STAMP();
#undef LLMIE_STAMP
    if (ok && blockIdx.x == 0 && threadIdx.x == 0) {
      for (int b = 0; b < p.batch; ++b)
        if (sh.slot[b] != p.scratch_slot) p.seq_lens[sh.slot[b]] = sh.pos[b] + 1;
      *p.epoch += 1ull;
    }
  }
  // Both roles meet before the block leaves. After a failure, copies may still be on their way into
  // this block's shared memory: give each slot's barrier a bounded time to report them.
  __syncthreads();
  if (sh.abort && threadIdx.x == kStCThreads) {
    for (int i = 0; i < p.n_slots; ++i) {
      for (unsigned spin = 0; spin < (1u << 16); ++spin) {
        if (mbar_test(&sh.full[i], 0) || mbar_test(&sh.full[i], 1)) break;
        __nanosleep(64);
      }
    }
  }
}

// Shared memory: the staged rows (at most kXsK columns; or the attention scratch of the work groups,
// whichever is larger), the reduction scratch, then the ring of weight slots with what is left.
static size_t stack_staging_bytes(int d, int ff, int n_q, int hd) {
  int kmax = d;
  const int wide = ff > n_q * hd ? ff : n_q * hd;
  const int pass = wide > kXsK ? kXsK : wide;
  if (pass > kmax) kmax = pass;
  const size_t rows = (size_t)8 * (kmax + kStPad) * 2;
  const size_t att = (size_t)kStMaxGroups * (8 * 64 + 4 * 4 * hd) * sizeof(float);
  const size_t bytes = rows > att ? rows : att;
  return (bytes + 127) / 128 * 128;
}
static size_t stack_red_bytes() { return (size_t)2 * kStWarps * 32 * sizeof(float4); }
static int stack_slots(int d, int ff, int n_q, int hd) {
  const long long left = 226LL * 1024 - (long long)stack_staging_bytes(d, ff, n_q, hd) - (long long)stack_red_bytes();
  long long n = left / kSlotBytes;
  if (n > kMaxSlots) n = kMaxSlots;
  return (int)n;
}

template <int HD>
static int launch_stack(StackParams& p, cudaStream_t stream) {
  if (p.d > kXsK) return LLMIE_ERR_UNSUPPORTED_SIZE;
  p.red_offset = (int)stack_staging_bytes(p.d, p.ff, p.n_q, HD);
  p.ring_offset = p.red_offset + (int)stack_red_bytes();
  p.n_slots = stack_slots(p.d, p.ff, p.n_q, HD);
  if (p.n_slots < 4) return LLMIE_ERR_UNSUPPORTED_SIZE;
  const size_t smem = (size_t)p.ring_offset + (size_t)p.n_slots * kSlotBytes;
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
  if (d > kXsK || stack_slots(d, ff, n_q, hd) < 4) return 0;
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
