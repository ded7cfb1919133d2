// An entry point for callers that cannot allocate device memory.
//
// This function has no counterpart in the reference project (xmiksay/rocml allocates all of its
// scratch buffers up front through its own runtime binding); it exists for hosts of this library
// that are not allowed to call cudaMalloc at all: a serving process that hands the whole GPU to
// its own memory pool at start-up, so that any later cudaMalloc fails or fragments that pool; or a
// latency-critical loop that cannot afford the device-wide synchronisation cudaMalloc and cudaFree
// imply.  Such a caller owns its inputs and outputs already; what it lacks is the kernel's work
// space.
//
// rb_attention_decode_static is rb_attention_decode (split-KV decode attention over the paged
// cache, bfloat16, one query token per sequence: see attention_decode.cu) with the work space taken
// from a fixed array that is part of the library's device image instead of from the caller:
//
//   * partial results   4 Mi floats (16 MiB):  n_seqs * nq * n_chunks * hd      must not exceed it
//   * partial max/sum   256 Ki floats (1 MiB): n_seqs * nq * n_chunks * 2       must not exceed it
//   * arrival counters  16 Ki ints (64 KiB):   n_seqs * nkv * ceil(nq/nkv / 16) must not exceed it
//
// Every GPU that loads the library holds these 17 MiB until the process exits.  A call whose sizes
// exceed a limit is refused with RB_ERR_SCRATCH_LIMIT (10006) and one line on stderr naming the
// limit; nothing is launched.  The function calls no cudaMalloc, cudaFree or other allocating
// routine.
//
// The work space is indexed by a sequence's place in the batch (0 .. n_seqs - 1), never by the
// token indices in cu_q, so the limits above hold whatever cu_q contains (the queries may be rows
// taken from a larger packed buffer).
//
// Set-up: the first call on a device looks up the array's device address
// (cudaGetSymbolAddress, with that device current) and remembers it; make that first call before
// any stream capture begins on the device.  The address is looked up for the device that is
// CURRENT in the calling thread (cudaGetDevice), so `stream` must belong to that device.
//
// Sharing: there is ONE array per device and every call uses it.  It keeps whatever the last call
// left; the counters this call will use are cleared (cudaMemsetAsync on `stream`) before the kernel
// runs, the partial results are overwritten before they are read.  Two calls that can overlap on
// the GPU (different streams without an ordering between them) race on the array and give wrong
// results: order them.
//
// Arguments and return value are those of rb_attention_decode without part_acc, part_ml and
// counters: q [n_seqs tokens, >= nq*hd] with row stride q_stride (elements), the cache tensors
// [pages, nkv, 64, hd], block_table [slots, max_pages], seq_slot / cu_q / kv_len per sequence,
// out [tokens, >= nq*hd] with row stride o_stride.  n_chunks = ceil(longest sequence / 64).
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

#define RB_ERR_SCRATCH_LIMIT 10006

int rb_attention_decode_static(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                               const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                               const int* kv_len, int n_seqs, int nq, int nkv, int hd, float scale, int window,
                               int n_chunks, void* out, int o_stride, void* stream);

#ifdef __cplusplus
}
#endif
