// Host <-> device KV page copy by index lists (preemption swap, host tier): block src[i] of one side goes to block dst[i]
// of the other, for every layer, in one launch.  The host tier is pinned memory mapped into the device's address space,
// so the SMs read / write it directly over PCIe / C2C; no staging copy and no host synchronisation.
//
// Layout on both sides: [planes][blocks][block_bytes] with their own plane strides (a plane is one layer of one cache
// family; K and V of a GQA cache are separate planes).  One CTA copies one (plane, i) block with 16-byte accesses.
//
// Replaces in the reference: kernel/jit/nano/kvcacheio/hicache.cuh:139-503 (swap in / out by index lists).
#include <cuda_runtime.h>
#include <stdint.h>

namespace ne {

__global__ void __launch_bounds__(256) kv_swap_kernel(uint8_t* __restrict__ dst_base, const uint8_t* __restrict__ src_base,
                                                     const int* __restrict__ src_idx, const int* __restrict__ dst_idx,
                                                     long long block_bytes, long long dst_plane_stride, long long src_plane_stride) {
  const int i = blockIdx.x, plane = blockIdx.y;
  const uint4* s = reinterpret_cast<const uint4*>(src_base + plane * src_plane_stride + (long long)src_idx[i] * block_bytes);
  uint4* d = reinterpret_cast<uint4*>(dst_base + plane * dst_plane_stride + (long long)dst_idx[i] * block_bytes);
  const long long n16 = block_bytes / 16;
  // four loads in flight per thread: host reads are long-latency
  long long k = threadIdx.x;
  for (; k + 3 * blockDim.x < n16; k += 4 * blockDim.x) {
    const uint4 a = s[k], b = s[k + blockDim.x], c = s[k + 2 * blockDim.x], e = s[k + 3 * blockDim.x];
    d[k] = a; d[k + blockDim.x] = b; d[k + 2 * blockDim.x] = c; d[k + 3 * blockDim.x] = e;
  }
  for (; k < n16; k += blockDim.x) d[k] = s[k];
}

}  // namespace ne

// src_idx / dst_idx: device int32 [n].  Both bases must be 16-byte aligned, block_bytes and the plane strides multiples of 16.
extern "C" int ne_kv_swap(void* dst_base, const void* src_base, const int* src_idx, const int* dst_idx, int n, int planes,
                          long long block_bytes, long long dst_plane_stride, long long src_plane_stride, cudaStream_t st) {
  if (n <= 0 || planes <= 0) return 0;
  if (block_bytes % 16 || dst_plane_stride % 16 || src_plane_stride % 16 || ((uintptr_t)dst_base & 15) || ((uintptr_t)src_base & 15)) return 1001;
  if (planes > 65535) return 1001;
  ne::kv_swap_kernel<<<dim3((unsigned)n, (unsigned)planes), 256, 0, st>>>((uint8_t*)dst_base, (const uint8_t*)src_base, src_idx, dst_idx, block_bytes,
                                                                         dst_plane_stride, src_plane_stride);
  return (int)cudaGetLastError();
}
