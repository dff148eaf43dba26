// Causal attention for prompts on the 5th-generation tensor cores: tcgen05.mma with TMEM
// accumulators, operands brought in by TMA straight from the paged KV cache.
//
// The math is the reference's prefill kernel (src/flash_attn.py:42-82): scores q.k / sqrt(hd),
// causal mask, online softmax with float32 running max / sum, probabilities rounded to bfloat16
// for the product with V (:72), output accumulated in float32 and divided by the sum at the end
// (:82). Unlike the reference, K and V are never expanded to the query heads (:92-94): query head
// h simply reads key/value head h / (Hq / Hkv) from the cache, and a sequence may start at any
// position (the reference's mask is only right at position 0).
//
// One block = 128 consecutive query tokens of one sequence and one query head, 320 threads:
//   warp 0      TMA producer: the Q tile once, then for every tile of 128 keys the two cache pages
//               of K and of V ([64 keys, hd] each) into their stages
//   warp 1      owns TMEM (two score buffers of 128 columns); one lane issues S = Q K^T two key
//               tiles ahead, as soon as a buffer is free, and O_j = P_j V_j when P_j is there
//   warps 2..9  softmax, two threads per query row (each half of a key tile's columns and half of
//               the output's): read S from TMEM (tcgen05.ld), mask, running max and sum, write P
//               as bfloat16 into shared memory in the tensor core's swizzled operand layout; the
//               P.V tile of the PREVIOUS key tile is added to the output kept in registers in the
//               middle of this work, so that no thread ever waits for the second product
// V is used as an MN-major B operand (rows of the cache are keys, i.e. the K dimension of P.V),
// so nothing is transposed. Every barrier wait is bounded (tcgen05.cuh).
//
// Registers: a block has 10 warps, which the SM deals to its four schedulers in turn, so a scheduler
// may get three warps of each of two blocks. With more than 85 registers a thread (16,384 a scheduler
// / 6 warps / 32) a new block then finds no room beside a running one although half the SM is free,
// and the SM is refilled only when both of its blocks have ended: the head-size-64 kernel, which
// wants two blocks an SM, is therefore held at 80.
#include "tcgen05.cuh"
#include <math.h>

namespace llmie {
using namespace tc;

constexpr int kQTile = 128;       // query rows per block
constexpr int kKTile = 128;       // keys per step (two cache pages of 64)
constexpr int kSoftmaxThreads = 256;   // two per query row: each takes half of a key tile's columns
constexpr int kAttnThreads = 64 + kSoftmaxThreads;
constexpr int kSubTileBytes = 128 * 128;   // [128 rows x 64 bf16], 16 KB

template <int HD> struct AttnCfg {
  static constexpr int kSub = HD / 64;                       // 64-wide blocks of the head dimension
  // Two score buffers: S of the next key tile is computed while the softmax of the current one runs.
  // head size 64: two blocks share an SM (each 256 TMEM columns, 97 KB). The two score buffers fill the 256
  // columns, so the P.V tile of key tile j is written over S_j, which nobody reads any more once P_j is
  // complete; the buffer is free for S_j+2 when the P.V tile has been read out.
  // head size 128: one block per SM, 512 columns: the P.V tile has columns of its own.
  static constexpr int kSBufs = 2;
  static constexpr bool kPvAlias = HD == 64;
  static constexpr int kKStages = 2;
  static constexpr int kVStages = HD == 64 ? 1 : 2;
  static constexpr int kTmemCols = HD == 64 ? 256 : 512;
  static constexpr int kPvCol = 256;                         // TMEM column of the P.V tile if it has its own
  static constexpr int kMaxRegs = HD == 64 ? 80 : 168;   // 168: three warps of a block on one scheduler
  static constexpr int kQBytes = kSub * kSubTileBytes;
  static constexpr int kKvBytes = kSub * kSubTileBytes;      // one K (or V) tile of 128 keys
  static constexpr int kPBytes = 2 * kSubTileBytes;          // P: [128 rows x 128 keys] bf16
  static constexpr int kSmem = kQBytes + (kKStages + kVStages) * kKvBytes + kPBytes + 1024;
};

struct AttnShared {
  uint64_t q_full;
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2], s_free[2];
  uint64_t p_ready, pv_full;
  uint32_t tmem_base;
  int abort;
  // the two threads of a query row tell each other their maxima (and, at the end, their sums) through
  // shared memory; the two warps that share a quarter of the rows meet at an mbarrier of their own
  // (a bounded wait that sleeps in hardware, so a waiting warp does not take issue slots from its partner
  // on the same scheduler). Two value buffers in turn: a thread is never more than one exchange ahead.
  float row_val[2][2][128];
  uint64_t pair_bar[4];
};

// 2^x by the special-function unit (about 2 units in the last place; the probabilities are then
// rounded to bfloat16, whose last place is 2^16 times coarser)
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two float32 operations in one instruction (the packed forms of sm_100): what limits the softmax threads is
// the number of instructions they issue as much as the exponentials.
__device__ __forceinline__ uint64_t pair_of(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void split_pair(uint64_t p, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(p));
}
// (y0, y1) = (x0, x1) * b + c, each still one rounding
__device__ __forceinline__ void fma_pair(float& y0, float& y1, float x0, float x1, uint64_t b, uint64_t c) {
  uint64_t y;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(y) : "l"(pair_of(x0, x1)), "l"(b), "l"(c));
  split_pair(y, y0, y1);
}
__device__ __forceinline__ uint64_t add_pair(uint64_t a, float x0, float x1) {
  uint64_t y;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(y) : "l"(a), "l"(pair_of(x0, x1)));
  return y;
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int HD>
__global__ void __maxnreg__(AttnCfg<HD>::kMaxRegs)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ out,
                            const int* __restrict__ cu_q, const int* __restrict__ seq_slot,
                            const int* __restrict__ seq_start, const int* __restrict__ block_table, int max_pages,
                            int scratch_page, int n_q, int n_kv, float scale, int window, int* __restrict__ status) {
  using Cfg = AttnCfg<HD>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ AttnShared sh;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_smem = base;
  uint8_t* k_smem = q_smem + Cfg::kQBytes;
  uint8_t* v_smem = k_smem + Cfg::kKStages * Cfg::kKvBytes;
  uint8_t* p_smem = v_smem + Cfg::kVStages * Cfg::kKvBytes;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z, head = blockIdx.x;
  const int q_begin = cu_q[seq], q_len = cu_q[seq + 1] - q_begin;
  // Late query tiles see the most keys. Blocks are handed out in the order of blockIdx.x, then y: with
  // the head as x and the query tile (latest first) as y, every head's longest block starts first and
  // the short ones fill the end (longest-processing-time-first), instead of one head after another.
  const int t0 = (gridDim.y - 1 - blockIdx.y) * kQTile;
  if (t0 >= q_len) return;                         // uniform for the block: nothing was set up yet
  const int start = seq_start[seq];                // tokens the sequence held before this step
  const int hk = head / (n_q / n_kv);
  const int rows_here = min(kQTile, q_len - t0);
  // keys this tile of queries may see: [first_key, last_key]
  const int last_key = start + t0 + rows_here - 1;
  const int first_key = (window > 0 && start + t0 - window + 1 > 0) ? start + t0 - window + 1 : 0;
  const int tile_lo = first_key / kKTile, tile_hi = last_key / kKTile;
  const int n_tiles = tile_hi - tile_lo + 1;

  // One thread is the TMA producer. K and V of a key tile are the two cache pages that hold its 128 keys.
  const int* pages = block_table + (size_t)seq_slot[seq] * max_pages;
  auto load_k = [&](int jt) {
    const int ks = jt % Cfg::kKStages;
    const int lp = (tile_lo + jt) * 2;           // logical pages of this key tile
    const int last_page = last_key / 64;         // pages beyond the sequence's last key are not mapped
    const int pg0 = pages[lp];
    const int pg1 = (lp + 1 <= last_page && lp + 1 < max_pages) ? pages[lp + 1] : scratch_page;
    uint8_t* kd = k_smem + ks * Cfg::kKvBytes;
    mbar_arrive_expect_tx(&sh.k_full[ks], Cfg::kKvBytes);
    for (int sub = 0; sub < Cfg::kSub; ++sub) {
      tma_load_2d(kd + sub * kSubTileBytes, &map_k, sub * 64, (pg0 * n_kv + hk) * 64, &sh.k_full[ks]);
      tma_load_2d(kd + sub * kSubTileBytes + 8192, &map_k, sub * 64, (pg1 * n_kv + hk) * 64, &sh.k_full[ks]);
    }
  };
  auto load_v = [&](int jt) {
    const int vs = jt % Cfg::kVStages;
    const int lp = (tile_lo + jt) * 2;
    const int last_page = last_key / 64;
    const int pg0 = pages[lp];
    const int pg1 = (lp + 1 <= last_page && lp + 1 < max_pages) ? pages[lp + 1] : scratch_page;
    uint8_t* vd = v_smem + vs * Cfg::kKvBytes;
    mbar_arrive_expect_tx(&sh.v_full[vs], Cfg::kKvBytes);
    for (int sub = 0; sub < Cfg::kSub; ++sub) {
      tma_load_2d(vd + sub * kSubTileBytes, &map_v, sub * 64, (pg0 * n_kv + hk) * 64, &sh.v_full[vs]);
      tma_load_2d(vd + sub * kSubTileBytes + 8192, &map_v, sub * 64, (pg1 * n_kv + hk) * 64, &sh.v_full[vs]);
    }
  };

  if (threadIdx.x == 0) {
    mbar_init(&sh.q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sh.k_full[s], 1);
      mbar_init(&sh.k_empty[s], 1);
      mbar_init(&sh.v_full[s], 1);
      mbar_init(&sh.v_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&sh.s_full[b], 1);
      mbar_init(&sh.s_free[b], kSoftmaxThreads);
    }
    mbar_init(&sh.p_ready, kSoftmaxThreads);
    mbar_init(&sh.pv_full, 1);
    for (int i = 0; i < 4; ++i) mbar_init(&sh.pair_bar[i], 64);
    sh.abort = 0;
    fence_mbar_init();
    // The first loads leave at once, while warp 1 still asks for tensor memory: only this thread touches the
    // barriers they complete on until the block has met below.
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    mbar_arrive_expect_tx(&sh.q_full, Cfg::kQBytes);
    for (int sub = 0; sub < Cfg::kSub; ++sub)
      tma_load_2d(q_smem + sub * kSubTileBytes, &map_q, head * HD + sub * 64, q_begin + t0, &sh.q_full);
    load_k(0);
    load_v(0);
  }
  if (warp == 1) {
    tmem_alloc(&sh.tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = sh.tmem_base;
  volatile int* abort = &sh.abort;
#define LLMIE_FAIL(code) do { if (!*abort) { *abort = 1; atomicExch(status, (code)); } } while (0)

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (tile 0 is on its way)
    if (lane == 0) {
      int issued = 1;
      for (int jt = 1; jt < n_tiles; ++jt) {
        const int ks = jt % Cfg::kKStages, vs = jt % Cfg::kVStages;
        if (jt >= Cfg::kKStages && !mbar_wait(&sh.k_empty[ks], ((jt / Cfg::kKStages) - 1) & 1, abort)) {
          LLMIE_FAIL(kStatusTimeoutEmpty);
          break;
        }
        load_k(jt);
        if (jt >= Cfg::kVStages && !mbar_wait(&sh.v_empty[vs], ((jt / Cfg::kVStages) - 1) & 1, abort)) {
          LLMIE_FAIL(kStatusTimeoutEmpty);
          issued = jt + 1;                         // K of this tile is in flight
          break;
        }
        load_v(jt);
        issued = jt + 1;
      }
      if (*abort) {   // let copies that are still in flight land before the block gives its memory up
        for (unsigned spin = 0; spin < (1u << 16) && !mbar_test(&sh.q_full, 0); ++spin) __nanosleep(64);
        for (int jt = max(0, issued - 2); jt < issued; ++jt) {
          uint64_t* kb = &sh.k_full[jt % Cfg::kKStages];
          uint64_t* vb = &sh.v_full[jt % Cfg::kVStages];
          const uint32_t kp = (jt / Cfg::kKStages) & 1, vp = (jt / Cfg::kVStages) & 1;
          for (unsigned spin = 0; spin < (1u << 16) && !(mbar_test(kb, kp) && mbar_test(vb, vp)); ++spin) __nanosleep(64);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc_s = make_instr_desc_bf16(kQTile, kKTile, 0, 0);
      constexpr uint32_t idesc_pv = make_instr_desc_bf16(kQTile, HD, 0, 1);     // V is MN-major
      const uint32_t q_addr = smem_u32(q_smem), p_addr = smem_u32(p_smem);
      bool ok = mbar_wait(&sh.q_full, 0, abort);
      if (!ok) LLMIE_FAIL(kStatusTimeoutFull);
      auto issue_scores = [&](int jt) -> bool {
        const int ks = jt % Cfg::kKStages, b = jt % Cfg::kSBufs, use = jt / Cfg::kSBufs;
        if (!mbar_wait(&sh.k_full[ks], (jt / Cfg::kKStages) & 1, abort)) { LLMIE_FAIL(kStatusTimeoutFull); return false; }
        if (use >= 1 && !mbar_wait(&sh.s_free[b], (use - 1) & 1, abort)) { LLMIE_FAIL(kStatusTimeoutMma); return false; }
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(k_smem + ks * Cfg::kKvBytes);
#pragma unroll
        for (int kk = 0; kk < HD / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kSubTileBytes + (kk & 3) * 32;
          mma_bf16_ss(tmem + b * 128, make_smem_desc(q_addr + off, 16, 1024), make_smem_desc(k_addr + off, 16, 1024),
                      idesc_s, kk > 0 ? 1u : 0u);
        }
        mma_commit(&sh.s_full[b]);
        mma_commit(&sh.k_empty[ks]);             // this K tile is free once the scores are computed
        return true;
      };
      if (ok) ok = issue_scores(0);
      if (ok && n_tiles > 1) ok = issue_scores(1);
      for (int jt = 0; ok && jt < n_tiles; ++jt) {
        const int vs = jt % Cfg::kVStages;
        const uint32_t pv_col = Cfg::kPvAlias ? (uint32_t)(jt & 1) * 128 : (uint32_t)Cfg::kPvCol;
        if (!mbar_wait(&sh.p_ready, jt & 1, abort)) { LLMIE_FAIL(kStatusTimeoutMma); break; }
        if (!mbar_wait(&sh.v_full[vs], (jt / Cfg::kVStages) & 1, abort)) { LLMIE_FAIL(kStatusTimeoutFull); break; }
        tc_fence_after_sync();
        const uint32_t v_addr = smem_u32(v_smem + vs * Cfg::kKvBytes);
#pragma unroll
        for (int kk = 0; kk < kKTile / 16; ++kk) {
          // A = P, K-major: 16 keys = 32 bytes inside a 64-key sub-tile. B = V, MN-major: 16 keys = 16 rows.
          const uint64_t dp = make_smem_desc(p_addr + (kk >> 2) * kSubTileBytes + (kk & 3) * 32, 16, 1024);
          const uint64_t dv = make_smem_desc(v_addr + kk * 2048, kSubTileBytes, 1024);
          mma_bf16_ss(tmem + pv_col, dp, dv, idesc_pv, kk > 0 ? 1u : 0u);
        }
        mma_commit(&sh.pv_full);
        mma_commit(&sh.v_empty[vs]);
        // the scores two tiles ahead go into the buffer of this tile, once the softmax threads have let go of it
        if (jt + 2 < n_tiles && !issue_scores(jt + 2)) break;
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax, two threads per query row
    // Warps 2..5 take the first 64 key columns of a tile (and the first half of the head dimension of
    // the output), warps 6..9 the second; a warp reads the TMEM lanes of its quarter (warp % 4).
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;                   // row of the tile = TMEM lane
    const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16);
    const int qpos = start + t0 + r;                     // absolute position of this query
    const int lo = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
    const float sl2 = scale * 1.4426950408889634f;       // exp(x * scale) = exp2(x * scale * log2 e)
    constexpr int kCols = kKTile / 2;                    // key columns of a tile this thread handles
    constexpr int kOut = HD / 2;                         // output columns this thread keeps
    float o[kOut];
#pragma unroll
    for (int d = 0; d < kOut; ++d) o[d] = 0.f;
    float m_run = -INFINITY, l_run = 0.f;                // l_run: the sum over this thread's columns only
    bool ok = true;
    // hands `mine` to the row's other thread and takes its value; n counts the exchanges of this block
    int n_exchanges = 0;
    auto exchange = [&](float mine, float& theirs) -> bool {
      const int buf = n_exchanges & 1;
      sh.row_val[buf][half][r] = mine;
      mbar_arrive(&sh.pair_bar[quarter]);                // release: the value is written before the arrival counts
      const bool ok_ = mbar_wait(&sh.pair_bar[quarter], n_exchanges & 1, abort);
      theirs = sh.row_val[buf][half ^ 1][r];
      ++n_exchanges;
      return ok_;
    };
    // Adds the P.V tile of key tile j to the output, which is first brought to that tile's maximum by alpha_j.
    // The whole warp calls it together, after it has seen pv_full for this tile.
    auto add_pv = [&](int j, float alpha_j) {
      tc_fence_after_sync();
      const uint32_t col = Cfg::kPvAlias ? (uint32_t)(j & 1) * 128 : (uint32_t)Cfg::kPvCol;
      const uint64_t alpha_pair = pair_of(alpha_j, alpha_j);
#pragma unroll
      for (int c0 = 0; c0 < kOut; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + col + half * kOut + c0, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2)
          fma_pair(o[c0 + i], o[c0 + i + 1], o[c0 + i], o[c0 + i + 1], alpha_pair,
                   pair_of(__uint_as_float(v[i]), __uint_as_float(v[i + 1])));
      }
      tc_fence_before_sync();                  // our TMEM reads are done before the arrival below counts
      if (Cfg::kPvAlias) mbar_arrive(&sh.s_free[j & 1]);     // the buffer may take the scores of tile j + 2
    };
    float alpha_prev = 1.f;                    // alpha of the tile whose P.V tile has not been added yet
    for (int jt = 0; jt < n_tiles; ++jt) {
      const int b = jt % Cfg::kSBufs;
      // every decision to give up is taken by the whole warp: the tensor-memory reads below are warp-wide
      // instructions, a warp must never reach them with some of its lanes gone
      if (!__all_sync(0xffffffffu, mbar_wait(&sh.s_full[b], (jt / Cfg::kSBufs) & 1, abort))) { LLMIE_FAIL(kStatusTimeoutMma); ok = false; break; }
      tc_fence_after_sync();
      const int kbase = (tile_lo + jt) * kKTile + half * kCols;
      const bool edge = ((tile_lo + jt) * kKTile + kKTile - 1 > start + t0) ||
                        (window > 0 && (tile_lo + jt) * kKTile < start + t0 + kQTile - window);
      // pass 1: the row's maximum over the keys it may see
      // (four running maxima and, below, four running sums: one chain of 64 dependent operations would be
      // what a row's time consists of)
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
      const int lo_rel = lo - kbase;
#pragma unroll
      for (int c0 = 0; c0 < kCols; c0 += 32) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + b * 128 + half * kCols + c0, v);
        tmem_ld_wait();
        if (edge) {
          // A tile that the causal line or the window's far end crosses: the scores this row may not see become
          // -inf here, in tensor memory too, so that the second pass is the same for every tile (2^-inf = 0).
          // Column c of this thread's half is seen if lo <= kbase + c <= qpos: one unsigned comparison.
          const unsigned span = (unsigned)(qpos - lo);
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if ((unsigned)(c0 + i - lo_rel) > span) v[i] = 0xff800000u;
            mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v[i]));
          }
          tmem_st_32x32(lane_addr + b * 128 + half * kCols + c0, v);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v[i]));
        }
      }
      if (edge) tmem_st_wait();
      float m_tile = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      float other;
      if (!__all_sync(0xffffffffu, exchange(m_tile, other))) { LLMIE_FAIL(kStatusTimeoutMma); ok = false; break; }
      m_tile = fmaxf(m_tile, other);
      const float m_new = fmaxf(m_run, m_tile);
      const float m_use = (m_new == -INFINITY) ? 0.f : m_new;      // a row that has seen no key yet
      const float alpha = exp2_approx((m_run - m_use) * sl2);      // 0 while m_run is -inf
      const float m_scaled = m_use * sl2;
      // pass 2: probabilities, their sum, and P in bfloat16 into the swizzled operand tile
      uint64_t ls[2] = {0ull, 0ull};             // four running sums, as two pairs
      const uint64_t sl2_pair = pair_of(sl2, sl2), m_pair = pair_of(-m_scaled, -m_scaled);
      // 32 keys from column c0 of this thread's half: probabilities, summed and packed two to a word
      auto probabilities = [&](int c0, uint32_t (&w)[16]) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + b * 128 + half * kCols + c0, v);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0, x1;
          fma_pair(x0, x1, __uint_as_float(v[i]), __uint_as_float(v[i + 1]), sl2_pair, m_pair);
          p[i] = exp2_approx(x0);
          p[i + 1] = exp2_approx(x1);
        }
#pragma unroll
        for (int i = 0; i < 32; i += 2) ls[(i >> 1) & 1] = add_pair(ls[(i >> 1) & 1], p[i], p[i + 1]);
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = pack_bf16(p[2 * i], p[2 * i + 1]);
      };
      auto store_p = [&](int c0, const uint32_t (&w)[16]) {
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {                 // four 16-byte chunks of 8 keys
          const int chunk = ((half * kCols + c0) >> 3) + ch;       // 0..15 within the 128 keys
          const uint4 q4 = make_uint4(w[ch * 4 + 0], w[ch * 4 + 1], w[ch * 4 + 2], w[ch * 4 + 3]);
          *reinterpret_cast<uint4*>(p_smem + (chunk >> 3) * kSubTileBytes + swizzle128_offset(r, chunk & 7)) = q4;
        }
      };
      static_assert(kCols == 64, "two chunks of 32 keys a thread");
      {
        // The first 32 probabilities are worked out while the tensor core may still be reading the previous P
        // for its P.V product; they go to shared memory once that product is done. Its tile is then added to
        // the output here, in the middle of this tile's work, where it is long complete: no thread waits for it.
        uint32_t w[16];
        probabilities(0, w);
        if (jt > 0 && !__all_sync(0xffffffffu, mbar_wait(&sh.pv_full, (jt - 1) & 1, abort))) { LLMIE_FAIL(kStatusTimeoutMma); ok = false; break; }
        store_p(0, w);
        if (jt > 0) add_pv(jt - 1, alpha_prev);
        probabilities(32, w);
        store_p(32, w);
      }
      tc_fence_before_sync();                  // our TMEM reads of S are done before the barriers are passed
      if (!Cfg::kPvAlias) mbar_arrive(&sh.s_free[b]);
      fence_proxy_async_smem();                // P is visible to the tensor core's reads
      mbar_arrive(&sh.p_ready);
      float l0, l1, l2, l3;
      split_pair(ls[0], l0, l1);
      split_pair(ls[1], l2, l3);
      l_run = fmaf(l_run, alpha, (l0 + l1) + (l2 + l3));
      m_run = m_new;
      alpha_prev = alpha;
    }
    if (ok) {
      if (__all_sync(0xffffffffu, mbar_wait(&sh.pv_full, (n_tiles - 1) & 1, abort))) add_pv(n_tiles - 1, alpha_prev);
      else { LLMIE_FAIL(kStatusTimeoutMma); ok = false; }
    }
    // the row's sum is the two halves' sums (both were kept relative to the same running maximum)
    if (ok) {
      float other;
      if (exchange(l_run, other)) l_run += other;
      else { LLMIE_FAIL(kStatusTimeoutMma); ok = false; }
    }
    if (ok && r < rows_here) {
      const float inv = 1.f / l_run;
      __nv_bfloat16* dst = out + ((size_t)(q_begin + t0 + r) * n_q + head) * HD + half * kOut;
#pragma unroll
      for (int d = 0; d < kOut; d += 8) {
        float v8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) v8[e] = o[d + e] * inv;
        store8(dst + d, v8);
      }
    }
  }
#undef LLMIE_FAIL
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem, Cfg::kTmemCols);
  }
}

template <int HD>
static int launch_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const int* cu_q,
                          const int* seq_slot, const int* seq_start, const int* block_table, int max_pages,
                          int n_pages_total, int n_tokens, int n_seqs, int max_q_len, int n_q, int n_kv, float scale,
                          int window, int* status, cudaStream_t stream) {
  using Cfg = AttnCfg<HD>;
  CUtensorMap map_q, map_k, map_v;
  int rc = tc::make_tmap_bf16_2d(&map_q, q, (uint64_t)n_tokens, (uint64_t)n_q * HD, (uint64_t)n_q * HD, kQTile);
  if (rc != LLMIE_OK) return rc;
  const uint64_t kv_rows = (uint64_t)n_pages_total * n_kv * 64;
  rc = tc::make_tmap_bf16_2d(&map_k, k_cache, kv_rows, HD, HD, 64);
  if (rc != LLMIE_OK) return rc;
  rc = tc::make_tmap_bf16_2d(&map_v, v_cache, kv_rows, HD, HD, 64);
  if (rc != LLMIE_OK) return rc;
  cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       Cfg::kSmem);
  if (e != cudaSuccess) return (int)e;
  dim3 grid(n_q, (max_q_len + kQTile - 1) / kQTile, n_seqs);
  attention_prefill_tc_kernel<HD><<<grid, kAttnThreads, Cfg::kSmem, stream>>>(
      map_q, map_k, map_v, (__nv_bfloat16*)out, cu_q, seq_slot, seq_start, block_table, max_pages, n_pages_total - 1,
      n_q, n_kv, scale, window, status);
  LLMIE_LAUNCH_CHECK();
  return LLMIE_OK;
}

}  // namespace llmie

using namespace llmie;

extern "C" int llmie_attention_prefill_tc_supported(int hd, int page_size) {
  return ((hd == 64 || hd == 128) && page_size == 64) ? 1 : 0;
}

// q, out: bfloat16 [n_tokens, n_q * hd], sequences packed one after another (cu_q [n_seqs + 1]).
// caches: bfloat16 [n_pages_total, n_kv, 64, hd]; the LAST page (n_pages_total - 1) is a scratch
// page that may be read for key positions nobody holds. seq_start[i]: tokens sequence i held
// before this step (its new keys are already in the cache). max_q_len: longest new run, for the grid.
// scale must be positive.
extern "C" int llmie_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                          const int* cu_q, const int* seq_slot, const int* seq_start,
                                          const int* block_table, int max_pages, int n_pages_total, int n_tokens,
                                          int n_seqs, int max_q_len, int n_q, int n_kv, int hd, float scale, int window,
                                          int* status, cudaStream_t stream) {
  if (n_tokens < 0 || n_seqs < 0 || n_q <= 0 || n_kv <= 0 || n_q % n_kv || max_pages <= 0 || n_pages_total <= 0)
    return LLMIE_ERR_BAD_ARG;
  if (!(scale > 0.f)) return LLMIE_ERR_BAD_ARG;   // the running maximum is taken before the scores are scaled
  if (!aligned16(q) || !aligned16(out) || !aligned16(k_cache) || !aligned16(v_cache)) return LLMIE_ERR_ALIGNMENT;
  if (n_tokens == 0 || n_seqs == 0 || max_q_len <= 0) return LLMIE_OK;
  if (n_seqs > 65535 || n_q > 65535) return LLMIE_ERR_UNSUPPORTED_SIZE;
  if (hd == 64)
    return launch_prefill<64>(q, k_cache, v_cache, out, cu_q, seq_slot, seq_start, block_table, max_pages,
                              n_pages_total, n_tokens, n_seqs, max_q_len, n_q, n_kv, scale, window, status, stream);
  if (hd == 128)
    return launch_prefill<128>(q, k_cache, v_cache, out, cu_q, seq_slot, seq_start, block_table, max_pages,
                               n_pages_total, n_tokens, n_seqs, max_q_len, n_q, n_kv, scale, window, status, stream);
  return LLMIE_ERR_UNSUPPORTED_SIZE;
}
