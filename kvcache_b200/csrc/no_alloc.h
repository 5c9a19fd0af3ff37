// kvb_flash_decode_static: decode attention over cache pages that allocates nothing.
//
// This entry point has no counterpart in the reference (its split-over-keys launcher calls
// cudaMalloc for its scratch on every call, src/flash_decode.cu:109-112).
//
// Who it is for.  The engine sizes its key/value pool to fill the device, and a host program
// that embeds these kernels may likewise have handed every free byte to a pool or an allocator
// of its own; such a caller has no memory left to ask cudaMalloc for, or is not allowed to ask
// (one memory plan, fixed at start-up, owned by someone else).  The regular entry point,
// kvb_flash_decode, leaves the scratch to the caller: partial results of the splits over the
// keys and one ticket counter per (item, kv head).  This variant brings its own: a fixed array
// in the library's device image, KVB_STATIC_SCRATCH_BYTES long, which every GPU that loads the
// library holds until the process exits.  Inputs and outputs are still the caller's.
// The library is built once per head size (kvb200_attention_flash-d64, -d128, ...): each of
// those modules carries an array of its own, so a process that loads two of them holds two.
// Calls into different modules neither share an array nor race with each other; calls into the
// same module do both.
//
// Contract.
//  * Arguments are those of kvb_flash_decode without `scratch` and `tickets`; the result is the same.
//  * Each item is a segment whose rows fit one tile: seg_q_len * (Hq / Hkv) <= 16 (the engine lists
//    segments of one token, with at most 16 query heads per kv head).  Rows beyond 16 are not
//    computed by either entry point; nothing is read or written outside the item's share.
//  * What the regular entry point refuses (Hq no multiple of Hkv, more than 16 query heads per kv
//    head, a page size that is no power of two, more than 32 splits) is refused before anything is
//    queued on the stream.
//  * It calls no cudaMalloc, cudaFree or other allocating routine.  The first call on a device
//    (with that device current) looks the array's device address up once; make that first call
//    before any stream capture begins.  Host threads that make their first calls at the same time
//    look the same address up twice, which is harmless.
//  * A call needs items * Hkv * nsplit * 16 * (head_dim + 2) floats of partial results plus
//    items * Hkv tickets.  If that exceeds the array the call launches nothing and returns
//    KVB_ERR_STATIC_SCRATCH; use fewer splits, fewer items per call, or the regular entry point.
//  * All calls share the one array, and it keeps what the last call left.  The tickets, which must
//    start at zero, are cleared on the stream before each launch.  Two calls that overlap on the
//    GPU (different streams) race on the array: keep calls on one stream, or order them.
#pragma once
#include <cuda_runtime.h>

#define KVB_STATIC_SCRATCH_BYTES (8u << 20)   /* 8 MiB: partial results and tickets together */
#define KVB_STATIC_TICKET_BYTES (16u << 10)   /* the last 16 KiB hold the tickets: at most 4096 (item, kv head) pairs */
#define KVB_ERR_STATIC_SCRATCH (-5)

#ifdef __cplusplus
extern "C"
#endif
__attribute__((visibility("default")))
int kvb_flash_decode_static(const void* q, void* out, const void* k_pages, const void* v_pages, const int* block_table,
                            int table_stride, const int* items, int n_items, const int* seg_q_start,
                            const int* seg_q_len, const int* seg_kv_len, int Hq, int Hkv, int page_size, int window,
                            int nsplit, float scale, cudaStream_t stream);
