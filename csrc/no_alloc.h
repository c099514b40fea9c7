// Allocation-free C entry point of the native library.
//
// This entry point has no counterpart in the reference implementation; it exists for hosts of
// this library that must not allocate device memory when they call into it: a serving loop that
// has handed the whole device heap to its own arena, a caller running under a memory budget it
// has already spent, a plugin invoked from inside another framework's allocator lock.  Such
// callers cannot pass through torch's caching allocator or cudaMalloc, so the usual
// split-KV decode attention (whose partial results need a workspace) is closed to them.
//
// ferrl_decode_attn_static_ws is the same kernel pair as the regular decode attention
// (csrc/kernels/decode_attn.cu), but its split-KV workspace is a fixed array that lives in the
// library image itself, so the call performs no cudaMalloc / cudaFree and uses no allocating
// library routine.  Inputs and outputs are still the caller's buffers.
//
// Limits and rules
//  * The workspace holds FERRL_STATIC_WS_FLOATS floats (16 MiB). Every GPU that loads this
//    library carries that array until the process exits.  A call whose
//    B * Hq * n_splits * (D + 2) exceeds it is rejected with FERRL_NOALLOC_TOO_LARGE and launches
//    nothing (n_splits <= 1 needs no workspace and is always accepted).
//  * The first call on each device resolves the array's device address (cudaGetSymbolAddress,
//    with that device current) and caches it.  Make that first call outside of any stream
//    capture.
//  * All calls on a device share the one array and it keeps whatever the previous call left in
//    it.  The kernels overwrite every slot they later read, so nothing has to be cleared between
//    calls - but two calls that overlap on the GPU (different streams, no ordering between them)
//    race on it.  Order them on one stream or with events.
//  * The address cache is indexed by device ordinal and holds FERRL_NOALLOC_MAX_DEVICES entries; a
//    call made with a higher ordinal current returns FERRL_NOALLOC_CUDA_ERROR.  Host threads may
//    make their first calls concurrently.
//  * Rejected with FERRL_NOALLOC_BAD_ARGS: a negative `window` or `seq_stride`, and a
//    `tok_stride` smaller than Hkv * D (tokens would overlap).
//  * Shapes follow the regular op: q [B,Hq,D] bf16 contiguous; k_cache / v_cache bf16 with
//    `seq_stride` elements between sequences and `tok_stride` between tokens, heads packed
//    [Hkv,D]; kv_len int32 [B]; out [B,Hq,D] bf16.  D % 8 == 0, D <= 256, Hq/Hkv <= 8.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define FERRL_STATIC_WS_FLOATS (4u * 1024u * 1024u)
#define FERRL_NOALLOC_MAX_DEVICES 64

enum {
  FERRL_NOALLOC_OK = 0,
  FERRL_NOALLOC_TOO_LARGE = 1,   /* workspace need exceeds FERRL_STATIC_WS_FLOATS */
  FERRL_NOALLOC_BAD_ARGS = 2,    /* null pointer, bad head geometry or strides, negative window, n_splits out of [1,16] */
  FERRL_NOALLOC_CUDA_ERROR = 3,  /* cudaGetDevice / cudaGetSymbolAddress / launch failed, or device ordinal >= 64 */
};

/* `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream). */
int ferrl_decode_attn_static_ws(const void* q, const void* k_cache, const void* v_cache, const int* kv_len, void* out,
                                int B, int Hq, int Hkv, int D, long long seq_stride, long long tok_stride, float scale,
                                int window, int n_splits, void* stream);

/* Human-readable text for a return code of the function above. */
const char* ferrl_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
