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
#pragma once

#define GL_DECODE_STATIC_SCRATCH_FLOATS (1 << 20)

#ifdef __cplusplus
extern "C" {
#endif
struct DecodeArgs;
int gl_attention_decode_static(const struct DecodeArgs* args, cudaStream_t stream);
long long gl_attention_decode_static_capacity(void);
#ifdef __cplusplus
}
#endif
