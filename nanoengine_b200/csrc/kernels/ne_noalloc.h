// Entry points of libne_kernels.so that allocate nothing.  (No counterpart in the reference: its kernels are reached
// through PyTorch, whose allocator is always at hand.)
//
// For callers that cannot hand the library scratch memory - a plain C/C++ host that links the library without a tensor
// allocator, or code running where cudaMalloc is off limits (a stream capture in progress, a process whose device memory
// was handed out up front) - the scratch sits in a fixed device array inside the library.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

// Absorbed MLA attention over the paged fp8 latent cache with `splits` key slices per query token and the merge of the
// slices, as ne_mla_fp8 + ne_attn_merge, but with the slice scratch taken from a library-owned device array.
//   q8     e4m3 [T*H, 576]            cache  e4m3 [num_blocks, 64, 576]            out  bf16 [T, H, 512]
// Limit: splits * T * H <= 4096 (8 MiB + 16 KiB of scratch per GPU, held from library load to process exit); beyond it
// the call returns 1101 and launches nothing.  The first call on each device looks up the scratch address and must not
// be made during stream capture.  Calls on one device share the scratch: keep them ordered on the GPU.
int ne_mla_fp8_noalloc(const void* q8, const void* cache, int num_blocks, const int* block_tables, int bt_stride,
                       const int* cu_seqlens_q, const int* context_lens, int num_seqs, int T, int H, int splits, float scale,
                       void* out, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
