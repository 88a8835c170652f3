// cpi_attention_decode_noalloc: decode attention with its split scratch inside the library.
//
// This entry point has no counterpart in the reference (kurulav1/cpi); it is an addition of this
// library for embedders that cannot give the kernel a scratch buffer.
//
// Who needs it.  The ordinary entry point, cpi_attention_decode, wants two float32 buffers for the
// partial results of the key splits, and the Python bindings get them from torch's allocator.  Some
// hosts cannot do that: a program that loads this library as a plain C library and has no allocator
// of its own at hand; a serving process whose start-up code hands all free device memory to another
// component's pool, so that a later cudaMalloc fails; code that runs at a point where a device
// allocation is not allowed to happen because it may block on, or be refused by, the driver.  Such a
// caller still passes its inputs and its output, and nothing else.
//
// What it does.  The partials are kept in one file-scope `static __device__` array of
// cpi_attention_decode_noalloc_capacity() floats (2 Mi floats = 8 MiB).  Every GPU on which the
// library is loaded holds that array until the process exits.  The call allocates nothing: no
// cudaMalloc, no cudaFree, no allocating library routine.
//
// Rules of use.
//   * Sizes: n_tokens * n_heads * n_splits * (head_dim + 2) must not exceed the capacity when
//     n_splits > 1; a larger request is refused with an error (cpi_last_error() names the numbers).
//     With n_splits == 1 no scratch is used.
//   * First call on a device: it asks the CUDA runtime for the array's device address
//     (cudaGetSymbolAddress, with that device current) and remembers it.  Make this first call before
//     any stream capture begins on that device.
//   * All calls share the one array, and it keeps the previous call's contents.  Nothing in it has to
//     start at zero: each call writes every partial it later reads.  Two calls whose kernels may run
//     at the same time on one GPU (different streams, or different host threads) race on the array;
//     keep such calls in one stream or order them yourself.
//   * Shapes: the same as cpi_attention_decode (bfloat16, head size 64 or 128, pages of 64 positions,
//     at most 16 query heads per key/value head).  `n_pages` is the number of pages that k_cache and
//     v_cache hold ([n_pages, n_kv_heads, 64, head_dim] each): the copy engine's descriptors of the two
//     tensors are made from it, on the host, without touching device memory.
//
// Returns 0 after launching on `stream`, non-zero with a message in cpi_last_error() otherwise.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

long cpi_attention_decode_noalloc_capacity(void);

int cpi_attention_decode_noalloc(const void* q, void* out, const void* k_cache, const void* v_cache,
                                 long n_pages, const int* page_table, int max_blocks, int page_size, const int* token_seq,
                                 const int* token_pos, const int* seq_slot, int n_tokens, int n_heads,
                                 int n_kv_heads, int head_dim, int window_kind, int window_size, float scale,
                                 int n_splits, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
