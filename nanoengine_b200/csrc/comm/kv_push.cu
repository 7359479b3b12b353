// PD disaggregation data path: the prefill GPU pushes the KV pages of finished prompts straight into the decode GPU's
// paged pool with peer stores, translating page ids on the way (prefill page ids differ from decode page ids), then raises
// a per-request completion flag the decode side polls.  One CTA copies one (plane, page) pair - a plane is one layer's
// array of pages in a cache family (MLA latent rows, K or V of a GQA layer, indexer keys) - and the last CTA to finish
// publishes the flags after a system-scope fence, so a flag never overtakes its data.  A request whose pages live in
// several families is several launches on one stream; only the last one carries the flag.
//
// Replaces in the reference: the decode-side pull of runtime/disagg/p2p/cache_transfer.py:648-1142 (coalesced one-sided
// reads followed by a device synchronise) and the byte-stride bookkeeping of disagg/p2p/cache_layout.py:14-240.
#include <cuda.h>

#include <cstring>

#include "ptx.cuh"

namespace ne {

struct KvPushArgs {
  const uint8_t* src; uint8_t* dst;                 // cache bases: [layers, blocks, page_bytes] on each side
  long long src_layer_stride, dst_layer_stride;     // bytes
  int page_bytes;                                   // bytes of one page of one layer (multiple of 16)
  const int* src_blocks; const int* dst_blocks;     // [n_pairs]
  int n_pairs, layers;
  int* flags; const int* flag_index; int n_flags; int flag_value;   // dst-side flag words (peer memory), one per request
  int* cta_counter;
};

__global__ void __launch_bounds__(256) kv_push_kernel(const KvPushArgs a) {
  const int pair = blockIdx.x, layer = blockIdx.y;
  const uint4* s = reinterpret_cast<const uint4*>(a.src + (long long)layer * a.src_layer_stride + (long long)a.src_blocks[pair] * a.page_bytes);
  uint4* d = reinterpret_cast<uint4*>(a.dst + (long long)layer * a.dst_layer_stride + (long long)a.dst_blocks[pair] * a.page_bytes);
  const int n = a.page_bytes / 16;
  for (int i = threadIdx.x; i < n; i += blockDim.x) d[i] = s[i];
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(a.cta_counter, 1) == (int)(gridDim.x * gridDim.y) - 1);
  __syncthreads();
  if (s_last) {
    if (threadIdx.x == 0) *a.cta_counter = 0;
    __threadfence_system();
    for (int f = threadIdx.x; f < a.n_flags; f += blockDim.x) st_release_sys(a.flags + a.flag_index[f], a.flag_value);
  }
}

// Bounded wait for completion flags (decode side): out[i] = 1 if flags[idx[i]] >= want within the budget, else 0.
__global__ void kv_wait_kernel(const int* flags, const int* idx, int n, int want, int* out, int spin_limit) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out[i] = wait_flag_ge(flags + idx[i], want, 4, i, (uint32_t)spin_limit) ? 1 : 0;
}

// The same wait with one expected value per flag, for tickets issued at different times.  A flag that never arrives is an
// answer here (out[i] = 0: that request's push did not happen), not a fault of this GPU, so nothing goes to the status words.
__global__ void kv_wait_each_kernel(const int* flags, const int* idx, const int* want, int n, int* out, int spin_limit) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int* p = flags + idx[i];
  const int w = want[i];
  int ok = 0;
  for (int it = 0; it < spin_limit; ++it) {
    if (ld_acquire_sys(p) >= w) { ok = 1; break; }
    if (it > 16) __nanosleep(it > 1024 ? 512 : 64);
  }
  out[i] = ok;
}

}  // namespace ne

using namespace ne;

extern "C" int ne_kv_push(const void* src, void* dst, long long src_layer_stride, long long dst_layer_stride, int page_bytes,
                          const int* src_blocks, const int* dst_blocks, int n_pairs, int layers, int* flags, const int* flag_index,
                          int n_flags, int flag_value, int* cta_counter, cudaStream_t st) {
  if (n_pairs <= 0 || layers <= 0) return 0;
  if (page_bytes % 16) return 1001;
  KvPushArgs a{(const uint8_t*)src, (uint8_t*)dst, src_layer_stride, dst_layer_stride, page_bytes, src_blocks, dst_blocks, n_pairs, layers,
               flags, flag_index, n_flags, flag_value, cta_counter};
  kv_push_kernel<<<dim3(n_pairs, layers), 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}

extern "C" int ne_kv_wait(const int* flags, const int* idx, int n, int want, int* out, int spin_limit, cudaStream_t st) {
  if (n <= 0) return 0;
  kv_wait_kernel<<<(n + 127) / 128, 128, 0, st>>>(flags, idx, n, want, out, spin_limit);
  return (int)cudaGetLastError();
}

extern "C" int ne_kv_wait_each(const int* flags, const int* idx, const int* want, int n, int* out, int spin_limit, cudaStream_t st) {
  if (n <= 0) return 0;
  kv_wait_each_kernel<<<(n + 127) / 128, 128, 0, st>>>(flags, idx, want, n, out, spin_limit);
  return (int)cudaGetLastError();
}

// ---- mapping another process' device memory ------------------------------------------------------------------------
// A decode worker publishes (handle of the allocation that holds a buffer, byte offset of the buffer inside it); a prefill
// worker on the same machine opens the handle WITH ITS OWN DEVICE CURRENT, which is what makes the mapping reachable from
// kernels running on that device (the runtime enables peer access between the opening device and the exporting one).  An
// allocation can be opened once per process: callers keep the returned base and reuse it for every buffer inside it.
typedef CUresult (*AddrRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

extern "C" int ne_ipc_export(const void* ptr, void* handle64, long long* offset, long long* alloc_bytes) {
  static AddrRangeFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return 1201;
    fn = (AddrRangeFn)p;
  }
  CUdeviceptr base = 0; size_t size = 0;
  if (fn(&base, &size, (CUdeviceptr)(uintptr_t)ptr) != CUDA_SUCCESS) return 1202;
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, (void*)(uintptr_t)base);
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handles are 64 bytes");
  memcpy(handle64, &h, 64);
  *offset = (long long)((uintptr_t)ptr - (uintptr_t)base);
  *alloc_bytes = (long long)size;
  return 0;
}

extern "C" int ne_ipc_open(const void* handle64, void** base_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(base_out, h, cudaIpcMemLazyEnablePeerAccess);
}

extern "C" int ne_ipc_close(void* base) { return (int)cudaIpcCloseMemHandle(base); }
