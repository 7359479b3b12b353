// In-switch (NVLS) tensor-parallel collectives: all-reduce, reduce-scatter and all-gather of bf16 rows through an NVLink
// multicast mapping of a symmetric buffer.  `multimem.ld_reduce` reads one address on every GPU of the group and returns the
// sum (added inside the NVSwitch), `multimem.st` writes one value to every GPU, `multimem.red` bumps a counter on every GPU -
// so an all-reduce moves each row over this GPU's links twice (once in, once out) whatever the group size, and hand-shakes
// are one instruction per rank.
//
// Symmetric region per rank (same offsets everywhere; `mc` = its multicast alias):
//   buf    bf16 [rows_cap][H]   inputs of reduce / all-reduce (each rank's partial rows), or the gathered rows of all-gather
//   outb   bf16 [rows_cap][H]   all-reduce results (written by multimem.st from the rank that reduced the rows)
//   flags  u32  [2]             arrival counters: every rank adds 1 to BOTH copies... of every rank through `mc`
// One kernel per call, at most one CTA per SM (all CTAs of a rank are resident, so they can wait for each other's phases):
//   phase 0  copy the caller's rows into buf (all-gather: multimem.st them into every rank's buf)
//   sync A   the last CTA to finish adds 1 to flags[0] everywhere; every CTA waits until its local flags[0] shows all ranks
//   phase 1  all-reduce: rank r reduces rows [r * n / world, ...) with multimem.ld_reduce and multimem.st's the sums into
//            outb everywhere; reduce-scatter: the sums go straight to the caller's output; all-gather: buf -> output
//   sync B   same hand-shake on flags[1]: nobody's buffers are overwritten by a later call while a peer still reads them
//   phase 2  all-reduce: outb -> output
// The call counter lives in device memory (a captured CUDA graph replays with fresh targets); waits are bounded and report
// through the status words.  Used only when the group's symmetric heap is bound to a multicast object (an opt-in: a rank
// that dies while bound disturbs its peers' GPUs, so the failure tests and the default configuration keep to peer stores).
//
// Replaces in the reference: kernel/jit/sgl/csrc/kimi_k3/comm/sp_collective.cuh:177,229 (multimem.st all-gather with
// multimem.red semaphores), :268 (multimem.ld_reduce pull reduce-scatter), csrc/distributed/custom_all_reduce.cuh:169-216,517.
#include "ptx.cuh"

namespace ne {

constexpr int kKernelNvls = 6;

struct NvlsLayout {
  unsigned long long mc_base, local_base;      // multicast alias and this rank's own mapping of the region
  long long off_buf, off_out, off_flags;
  int rank, world, rows_cap, H;
};

__device__ __forceinline__ void mm_red_add_release(unsigned* mc_p, unsigned v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const void* mc_p) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(mc_p) : "memory");
  return r;
}
__device__ __forceinline__ void mm_st_bf16x8(void* mc_p, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};" ::"l"(mc_p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// All CTAs of this rank have finished a phase (counted by `cta_counter`) -> tell every rank; then wait until every rank told us.
__device__ __forceinline__ bool nvls_sync(const NvlsLayout& L, int which, unsigned target, int* cta_counter, int spin_limit) {
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(cta_counter, 1) == (int)gridDim.x - 1) {
      *cta_counter = 0;
      __threadfence_system();
      mm_red_add_release(reinterpret_cast<unsigned*>(L.mc_base + L.off_flags) + which, 1u);
    }
  }
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    const int* f = reinterpret_cast<const int*>(L.local_base + L.off_flags) + which;
    s_ok = wait_flag_ge(f, (int)target, kKernelNvls, 100 + which, (uint32_t)spin_limit) ? 1 : 0;
  }
  __syncthreads();
  return s_ok != 0;
}

// mode 0: all-reduce of x [rows, H] -> out [rows, H]; 1: reduce-scatter, out [rows / world, H] = this rank's rows of the sum
// (rows must be a multiple of world); 2: all-gather, x [rows, H] is this rank's slice, out [rows * world, H].
__global__ void __launch_bounds__(512, 1) nvls_collective_kernel(const NvlsLayout L, const __nv_bfloat16* __restrict__ x,
                                                                __nv_bfloat16* __restrict__ out, int rows, int mode, int* __restrict__ state,
                                                                int spin_limit) {
  // state: [0] calls made so far (every call uses two hand-shakes), [1] / [2] CTA counters of the two syncs, [3] exit counter
  const unsigned call = (unsigned)state[0];
  const unsigned target = (call + 1u) * (unsigned)L.world;
  const int chunks = L.H / 8;
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x, nthr = (long long)gridDim.x * blockDim.x;
  uint8_t* buf_l = reinterpret_cast<uint8_t*>(L.local_base + L.off_buf);
  uint8_t* buf_m = reinterpret_cast<uint8_t*>(L.mc_base + L.off_buf);
  uint8_t* out_l = reinterpret_cast<uint8_t*>(L.local_base + L.off_out);
  uint8_t* out_m = reinterpret_cast<uint8_t*>(L.mc_base + L.off_out);
  // phase 0
  if (mode == 2) {
    const long long base = (long long)L.rank * rows * chunks;
    for (long long i = tid; i < (long long)rows * chunks; i += nthr) mm_st_bf16x8(buf_m + (base + i) * 16, reinterpret_cast<const uint4*>(x)[i]);
  } else {
    for (long long i = tid; i < (long long)rows * chunks; i += nthr) reinterpret_cast<uint4*>(buf_l)[i] = reinterpret_cast<const uint4*>(x)[i];
  }
  bool ok = nvls_sync(L, 0, target, state + 1, spin_limit);
  // phase 1
  if (ok) {
    if (mode == 2) {
      for (long long i = tid; i < (long long)rows * L.world * chunks; i += nthr) reinterpret_cast<uint4*>(out)[i] = reinterpret_cast<const uint4*>(buf_l)[i];
    } else {
      const int per = (rows + L.world - 1) / L.world;
      const int r0 = L.rank * per, r1 = min(rows, r0 + per);
      for (long long i = tid; i < (long long)max(0, r1 - r0) * chunks; i += nthr) {
        const long long off = ((long long)r0 * chunks + i) * 16;
        const uint4 s = mm_ld_reduce_bf16x8(buf_m + off);
        if (mode == 0) mm_st_bf16x8(out_m + off, s);
        else reinterpret_cast<uint4*>(out)[i] = s;
      }
    }
  }
  ok = nvls_sync(L, 1, target, state + 2, spin_limit) && ok;
  // phase 2
  if (mode == 0) {
    for (long long i = tid; i < (long long)rows * chunks; i += nthr)
      reinterpret_cast<uint4*>(out)[i] = ok ? reinterpret_cast<const uint4*>(out_l)[i] : make_uint4(0, 0, 0, 0);
  }
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(state + 3, 1) == (int)gridDim.x - 1) { state[3] = 0; state[0] = (int)(call + 1u); }
}

}  // namespace ne

using namespace ne;

extern "C" int ne_nvls_layout_size() { return (int)sizeof(NvlsLayout); }

// `state`: 4 zero-initialised device ints owned by the caller.  rows are the caller's rows (see the modes above).
extern "C" int ne_nvls_collective(const NvlsLayout* L, const void* x, void* out, int rows, int mode, int* state, int spin_limit, cudaStream_t st) {
  if (!L->mc_base || L->H % 8 || mode < 0 || mode > 2 || rows < 1) return 1001;
  if ((mode == 2 ? (long long)rows * L->world : (long long)rows) > L->rows_cap) return 1002;
  if (mode == 1 && rows % L->world) return 1003;
  int sms = 0, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  long long items = (long long)rows * (mode == 2 ? L->world : 1) * (L->H / 8);
  int blocks = (int)((items + 511) / 512);
  blocks = blocks < 1 ? 1 : (blocks > sms ? sms : blocks);          // every CTA must be resident: they wait for each other
  nvls_collective_kernel<<<blocks, 512, 0, st>>>(*L, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, rows, mode, state, spin_limit);
  return (int)cudaGetLastError();
}
