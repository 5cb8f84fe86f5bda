// mf_attention_decode_static — decode attention that needs no memory from its caller beyond inputs
// and outputs.
//
// This entry point has no counterpart in hvasconcelos/mlxforge (whose attention is an MLX library
// call that allocates as it pleases); it exists for users of this library who cannot allocate.
//
// Who that is.  The ordinary entry point, mf_attention_decode, wants two scratch buffers for the
// partial results of its key splits; inside this package torch's caching allocator hands them out.
// A caller outside the package may have nothing to hand out: a C or C++ host that links the library
// without torch and owns no device allocator; a service that was given its device memory once at
// start-up and may not ask for more; code on a path where cudaMalloc is off limits because it
// synchronises the whole device and would stall every other stream.  For them the partial results
// go into an array that is part of the library's own image.
//
// What it costs and where it stops.  The array is MF_DECODE_STATIC_SCRATCH_BYTES (8 MiB) of device
// memory on every GPU that loads the library, from load until the process ends, whether or not this
// entry point is ever called.  A call needs
//     n_tokens * n_heads * ceil(max_ctx / split) * (head_dim + 2) * 4 bytes
// (mf_attention_decode_static_bytes computes it; split = mf_attention_decode_split(head_dim)).  A
// call that needs more is refused with MF_ERR_SCRATCH_LIMIT and a message in `err`; nothing is
// launched.  With splits of 512 keys, 8 MiB covers, for 32 heads of size 64, 8 sequences at a
// context of 63,000 tokens or 64 sequences at 7,600.
//
// Set-up.  The first call on each device looks up the array's device address (cudaGetSymbolAddress,
// with that device current) and remembers it.  Make that first call before any stream capture
// begins on the device; later calls only launch the two kernels.
//
// Sharing.  All calls on a device use the same array and it keeps whatever the last call left.
// Nothing in it has to start at zero: every partial result that the merge kernel reads was written
// by the first kernel of the same call.  Two calls that can run on the GPU at the same time
// (different streams with no ordering between them) race on the array and both results are then
// undefined: order them on one stream or with events.  For head size 64 the same holds between
// this entry point and the ordinary mf_attention_decode, even when that one has scratch of its
// own: the kernel that both launch counts the finished splits of every (token, head group) in a
// table of tickets that is one per device (g_tickets, attention_decode_tma.cu), so ALL decode
// attention calls of head size 64 on a device must be ordered one after the other.
//
// It calls no cudaMalloc, cudaFree or allocating library routine.  Arguments are those of
// mf_attention_decode without the two scratch pointers, plus `err`/`err_len`, an optional buffer
// for a message when the return value is not 0.
#pragma once
#include <cuda_runtime.h>

#define MF_DECODE_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
#define MF_ERR_SCRATCH_LIMIT 10003

#ifdef __cplusplus
extern "C" {
#endif

long long mf_attention_decode_static_bytes(int n_tokens, int n_heads, int hd, int max_ctx);

int mf_attention_decode_static(const void* q, const void* k_pool, const void* v_pool, void* out, int n_tokens,
                               int n_heads, int n_kv, int hd, const int* positions, const int* seq_of_token,
                               const int* block_table, int bt_stride, int page_size, float scale, int window,
                               int max_ctx, cudaStream_t stream, char* err, int err_len);

#ifdef __cplusplus
}
#endif
