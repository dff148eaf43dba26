// Split-KV decode attention for callers that must not allocate device memory.
//
// This entry point has no counterpart in the reference; it is an addition of this library.
//
// Who needs it: a host program that has already handed every byte of device memory to a pool
// of its own, a loop with a latency budget in which a cudaMalloc (which can stall the whole
// device, or fail late) is not acceptable, or a plain C caller that has no tensor library to
// allocate on its behalf. `llmie_attention_decode` makes such callers bring three scratch
// buffers; this variant brings its own: a fixed array that lives in the library's device image.
//
// What it does: exactly what `llmie_attention_decode` does (same kernels, same arguments for
// inputs and outputs, same return codes), with the per-run partial results kept in a
// file-scope `static __device__` array of LLMIE_NOALLOC_SCRATCH_BYTES. It calls no cudaMalloc,
// no cudaFree and no routine that allocates.
//
// Cost and limits:
//   * Every GPU on which this library is loaded holds LLMIE_NOALLOC_SCRATCH_BYTES (16 MiB) of
//     device memory from load until the process exits, whether or not this function is called.
//   * page_size and run_len must both be 64 (a run is one cache page); anything else is refused with
//     LLMIE_ERR_UNSUPPORTED_SIZE (-2). n_runs * 64 must cover the longest length in seq_kvlen.
//   * A sequence whose seq_kvlen is 0 (or negative) has no keys: its rows of `out` are set to zero.
//   * n_seqs * n_q * n_runs * (hd + 2) floats must fit in the array; a larger problem is refused
//     with LLMIE_ERR_SCRATCH_TOO_SMALL (-5) and nothing is launched.
//   * The FIRST call on each device looks the array's device address up
//     (cudaGetSymbolAddress, with that device current) and remembers it. Make that first call
//     ahead of any stream capture on that device.
//   * All calls share the one array and it keeps what the last call left in it. Nothing in
//     it has to start at zero: each call writes every entry it later reads. Two calls whose
//     kernels overlap on the GPU (different streams, no ordering between them) race on it;
//     order them, or use `llmie_attention_decode` with separate scratch for one of them.
#pragma once
#include <cuda_runtime.h>

#define LLMIE_NOALLOC_SCRATCH_BYTES (16u * 1024u * 1024u)
#define LLMIE_ERR_SCRATCH_TOO_SMALL (-5)

#ifdef __cplusplus
extern "C" {
#endif

// q, out: [n_seqs, n_q * hd]; caches: [n_pages, n_kv, page_size, hd]; dtype 0 = float32, 1 = bfloat16.
// seq_kvlen[i] counts the keys sequence i holds including this step's token. Returns 0, a negative
// LLMIE_ERR_* code, or a positive cudaError_t.
int llmie_attention_decode_noalloc(const void* q, const void* k_cache, const void* v_cache, void* out,
                                   const int* seq_slot, const int* seq_kvlen, const int* block_table, int max_pages,
                                   int page_size, int n_seqs, int n_q, int n_kv, int hd, float scale, int window,
                                   int run_len, int n_runs, int dtype, cudaStream_t stream);

// Bytes of the built-in scratch array (the value of LLMIE_NOALLOC_SCRATCH_BYTES the library was built with).
unsigned long long llmie_attention_decode_noalloc_capacity(void);

#ifdef __cplusplus
}
#endif
