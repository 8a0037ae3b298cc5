// gl_attention_decode_static: decode attention that allocates nothing.
//
// This entry point has no counterpart in SimonWaldherr/GopherLLM; it exists for
// callers of this library that cannot ask the CUDA runtime for device memory while
// they run.  Examples: a serving process that handed its whole memory budget to its
// own pools at start-up, so that a later cudaMalloc fails or fragments them; a
// latency-bound loop that cannot afford the device-wide synchronisation an
// allocation may cause; a C or C++ host that links this library without PyTorch and
// therefore has no caching allocator to borrow scratch from.
//
// gl_attention_decode splits each sequence's keys over several blocks and needs
// B * heads * splits * (head_dim + 2) floats of scratch for their partial results.
// The caller of gl_attention_decode passes that scratch in DecodeArgs.part_o /
// part_ml.  gl_attention_decode_static ignores those two fields and uses an array
// built into the library instead (GL_DECODE_STATIC_SCRATCH_FLOATS floats = 4 MiB
// of device memory, held by every GPU that loads the library until the process
// ends).  Inputs and outputs (q, out, the cache, seq_ctx, pages) are still the
// caller's.
//
// Rules:
//  * A call whose scratch need exceeds the array returns GL_ERR_SCRATCH (-7) and
//    launches nothing; lower `splits` or the batch.  gl_attention_decode_static_capacity()
//    returns the array's size in floats, gl_attention_decode_scratch(B, heads, splits)
//    the need of a call.
//  * The first call on each device looks up the array's device address
//    (cudaGetSymbolAddress, with that device current).  Make that first call before
//    any stream capture begins.
//  * It calls no cudaMalloc, cudaFree or other allocating routine.
//  * All calls share the one array and it keeps what the last call left.  Nothing in
//    it has to start at zero: each call writes every cell it later reads.  Two calls
//    that overlap on the GPU (different streams, or the same library used from two
//    threads without ordering) race on it; order them on one stream or with events.
//  * The per-device address is looked up by whichever thread calls first on that device and
//    kept in a plain array.  Two threads that both make a device's first call both look it
//    up and store the same value; no lock is taken and none is needed.
//
// The header stands alone: a C host includes it, fills in a DecodeArgs and calls.
#pragma once

#include <cuda_runtime.h>

#define GL_DECODE_STATIC_SCRATCH_FLOATS (1 << 20)

#ifndef GL_DECODE_ARGS_DEFINED
#define GL_DECODE_ARGS_DEFINED
// The argument record of decode attention as a C host sees it (the library's own source
// declares the same layout with typed pointers).  bfloat16 values are 16-bit words.
struct DecodeArgs {
    const void* q;        // [B, nH*hd] bfloat16 queries, already rotated and scaled
    void* out;            // [B, nH*hd] bfloat16
    const void* k_cache;  // [pages, nKV, 64, hd] bfloat16
    const void* v_cache;  // the same shape
    const int* seq_ctx;   // [B] positions cached before this step (the new token's key sits at seq_ctx[b])
    const int* pages;     // [B, max_pages] page numbers of each sequence
    float* part_o;        // ignored by gl_attention_decode_static
    float* part_ml;       // ignored by gl_attention_decode_static
    int B, nH, nKV, max_pages, window, splits;
};
#endif

#ifdef __cplusplus
extern "C" {
#endif
int gl_attention_decode_static(const struct DecodeArgs* args, cudaStream_t stream);
long long gl_attention_decode_static_capacity(void);
long long gl_attention_decode_scratch(int B, int nH, int splits);
#ifdef __cplusplus
}
#endif
