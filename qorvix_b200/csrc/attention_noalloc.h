// Split-KV decode attention for callers that may not allocate device memory.
//
// This entry point has no counterpart in the reference engine; it exists for hosts of this
// library that cannot call cudaMalloc themselves and must not have it called on their behalf:
// an application that handed all device memory to its own pool at start-up, a real-time loop in
// which an allocation (which may synchronise the device or fail) is not acceptable, or a plugin
// whose host owns the allocator.  The regular entry point, qv_attn_decode_bf16, needs a float
// workspace for the partial results of the key slices and expects the caller to provide it;
// this one keeps that workspace inside the library instead.
//
// Where the workspace lives: a file-scope `static __device__` array of QV_ATTN_STATIC_SCRATCH_FLOATS
// floats (8 MiB) in attention_bf16.cu.  Every GPU on which the library is loaded holds those
// 8 MiB until the process exits, whether or not this function is ever called.
//
// Limit: T * H * splits * (hd + 2) must not exceed QV_ATTN_STATIC_SCRATCH_FLOATS (for example 64
// tokens x 32 heads x 7 slices at head size 128).  A larger request is refused with
// QV_ERR_STATIC_SCRATCH_TOO_SMALL and nothing is launched; qv_attn_decode_static_strerror turns
// the code into words.  All other refusals and return codes are those of qv_attn_decode_bf16.
//
// First call: the first call on each device looks up the array's device address (once per
// device, with that device current) and remembers it.  Make that first call outside any
// stream capture.
//
// Sharing: there is one array per device and every call uses it from its start.  Nothing in it
// has to be zero beforehand (each slice's record is written before it is read), and a call
// leaves its partial results behind.  Two calls that may run on the GPU at the same time (on
// different streams, or from different threads) would overwrite each other's partial results:
// keep calls on one stream, or order them with events.
//
// One device per process: the workspace's address is kept per device, but the kernels' launch
// configuration, the word their bounded waits report into and the choice between the two decode
// kernels (qv_attn_set_error_word, qv_attn_set_decode_variant, shared with qv_attn_decode_bf16) are
// kept once per process.  A process that drives several GPUs through this library is not served.
//
// The function allocates nothing: no cudaMalloc, cudaFree or allocating library routine.
#pragma once

#define QV_ATTN_STATIC_SCRATCH_FLOATS (2 * 1024 * 1024)
#define QV_ERR_STATIC_SCRATCH_TOO_SMALL (-4)

#ifdef __cplusplus
extern "C" {
#endif

// Same arguments and meaning as qv_attn_decode_bf16 without the `partial` pointer.
int qv_attn_decode_bf16_static(void* out, int ld_out, const void* q, int ld_q, const void* cache, const int* tok_pos,
                               const int* tok_seg, const int* block_table, int max_blocks, int T, int H, int Hkv, int hd,
                               int page, int window, float scale, int splits, void* stream);

// Words for a code returned by qv_attn_decode_bf16_static.
const char* qv_attn_decode_static_strerror(int code);

#ifdef __cplusplus
}
#endif
