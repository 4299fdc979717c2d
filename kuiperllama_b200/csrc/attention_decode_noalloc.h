// kl_attention_decode_noalloc: decode attention for callers that must not allocate.
//
// This entry point has no counterpart in ExiledOfCode/KuiperLLama; it exists for users of this
// library only.
//
// Who needs it.  Some programs that embed these kernels cannot call cudaMalloc at the moment
// they need attention: a serving process that has handed all device memory to its own pool at
// start-up, a latency-critical loop where an allocation's implicit synchronisation is not
// acceptable, or a host without torch's caching allocator.  The regular entry point,
// kl_attention_decode, cuts every sequence's keys over several CTAs and needs scratch memory
// for the pieces' partial results, which its caller has to allocate.  This variant brings its
// own: a fixed array in the library's device image.
//
// What it costs.  The array holds KL_DECODE_NOALLOC_FLOATS float32 values (4 MiB).  Every
// GPU on which a process loads the library holds that memory until the process exits, whether
// or not the entry point is ever called.
//
// Limits.  rows * H * splits * (hd + 2) must not exceed KL_DECODE_NOALLOC_FLOATS; a larger
// call is refused with KL_ERR_BAD_SIZE (-2) and a line on stderr, and nothing is launched.
//
// Set-up.  The first call on each device looks the array's device address up
// (cudaGetSymbolAddress, with that device current) and keeps it.  Make that first call
// before any stream capture begins on the device.
//
// Sharing.  All calls on a device use the same array, and it keeps what the last call left
// there.  Nothing in it has to start at zero: within one call the first kernel writes every
// entry that the second kernel reads.  Two calls whose kernels overlap on the GPU (different
// streams, no ordering between them) race on the array and give wrong results; order them.
//
// Arguments are those of kl_attention_decode without the two scratch pointers.  The entry
// point calls no cudaMalloc, cudaFree or any other allocating routine.
#pragma once
#include <cuda_runtime.h>

#define KL_DECODE_NOALLOC_FLOATS (1 << 20)

extern "C" int kl_attention_decode_noalloc(const void* q, int q_stride, void* out, const void* k_cache,
                                           const void* v_cache, const int* block_table, int blocks_per_seq,
                                           const int* positions, const int* token_slot, int rows, int H, int KV,
                                           int hd, float scale, int window, int splits, cudaStream_t stream);
