// Tensor-parallel collectives over NVLink peer memory, shaped to sit directly behind / in front of the GEMMs they serve.
//
// Every rank of a TP group owns one symmetric region (same offsets everywhere):
//   stage  bf16 [2][world][rows_per_rank][H]   partial sums arriving from every source rank, double-buffered by call parity
//   gather bf16 [2][world * rows_per_rank][H]  rows arriving from their owners, double-buffered by call parity
//   flags  int32 [2][world]                    epoch-tagged: [0] = "my partials are in your stage", [1] = "my rows are in your gather"
//
// GEMM -> reduce-scatter (row-parallel o_proj / down_proj), two launches: the GEMM's scatter epilogue (GemmComm mode 3 of
// ne_gemm_comm) stores every output row of the local partial product straight into the stage slot of the rank that owns the
// row, tile by tile while the other tiles are still being computed, and the GEMM's last CTA raises the flag at every peer;
// tp_reduce, on the owner, waits (bounded) for all sources, adds the `world` partials in rank order and advances the epoch.
// all-gather -> GEMM (column-parallel qkv / gate_up), two launches: tp_push stores this rank's rows into every peer's gather
// buffer and raises the flag from its last CTA; the consuming GEMM reads the gather buffer through its gated A operand (its
// producer warp waits, bounded, for the source ranks of the row block it is about to load, own rows first) and its last CTA
// advances the epoch.  The stand-alone all-gather (tp_wait_copy) copies the gathered rows out of the double buffer, so its
// result does not depend on which half a call used.
// tp_push also serves the plain reduce-scatter (mode 1: row i goes to its owner's stage slot), so an all-reduce is
// push + reduce + push + wait_copy.  Two calls may be in flight on different ranks, never three: a rank cannot pass the wait
// of call n+1 before every peer has finished call n, which is why two buffers per kind are enough.  The epoch lives in
// device memory so captured CUDA graphs replay with fresh tags.  All remote traffic is plain stores; no multicast loads.
//
// Replaces in the reference: the NCCL all_reduce after row-parallel linears (layers/backends/linear/deep_gemm.py:491-499,
// linear/generic.py:314-319), reduce_scatter / all_gather of layers/parallelism_transition.py:67-200, and the push / pull
// kernels of kernel/jit/sgl/csrc/kimi_k3/comm/sp_collective.cuh:115-268 and csrc/distributed/custom_all_reduce.cuh.
#include "ptx.cuh"

namespace ne {

constexpr int kTpMaxWorld = 16;
constexpr int kKernelTp = 5;

struct TpLayout {
  unsigned long long peer_base[kTpMaxWorld];
  long long off_stage, off_gather, off_flags;
  int rank, world, rows_per_rank, H;         // rows_per_rank = capacity of one slot (rows), H = row width in elements
};

__device__ __forceinline__ uint8_t* tp_ptr(const TpLayout& L, int r, long long off) { return reinterpret_cast<uint8_t*>(L.peer_base[r]) + off; }
__device__ __forceinline__ long long stage_off(const TpLayout& L, int parity, int src, long long row) {
  return L.off_stage + (((long long)parity * L.world + src) * L.rows_per_rank + row) * L.H * 2;
}
__device__ __forceinline__ long long gather_off(const TpLayout& L, int parity, long long row) {
  return L.off_gather + ((long long)parity * L.world * L.rows_per_rank + row) * L.H * 2;
}

__global__ void tp_signal_kernel(const TpLayout L, int which, const int* __restrict__ epoch_ptr) {
  const int epoch = *epoch_ptr + 1;
  __threadfence_system();
  if ((int)threadIdx.x < L.world)
    st_release_sys(reinterpret_cast<int*>(tp_ptr(L, threadIdx.x, L.off_flags)) + which * L.world + L.rank, epoch);
}

// mode 0 (all-gather): row i of x -> gather[rank * rpr + i] of EVERY rank.  mode 1 (reduce-scatter): row i of x (i over all
// world * rpr rows) -> stage slot [rank] of owner i / rpr.  mode 2 (one-shot all-reduce of few rows): row i of x -> stage
// slot [rank] of EVERY rank, which then adds all slots itself.  The last CTA to finish raises the flag at every peer.
__global__ void __launch_bounds__(256) tp_push_kernel(const TpLayout L, const __nv_bfloat16* __restrict__ x, int rows, int rpr, int mode,
                                                     const int* __restrict__ epoch_ptr, int* __restrict__ cta_counter) {
  const int epoch = *epoch_ptr + 1, parity = epoch & 1;
  const int chunks = L.H / 8;                               // 16-byte chunks per row
  const long long total = (long long)rows * chunks;
  for (long long it = (long long)blockIdx.x * blockDim.x + threadIdx.x; it < total; it += (long long)gridDim.x * blockDim.x) {
    const int row = (int)(it / chunks), c = (int)(it % chunks);
    const uint4 v = *reinterpret_cast<const uint4*>(x + (long long)row * L.H + c * 8);
    if (mode == 0) {
      const long long off = gather_off(L, parity, (long long)L.rank * rpr + row) + c * 16;
      for (int p = 0; p < L.world; p++) {
        const int r = (L.rank + p) % L.world;              // start with the own copy, stagger the peers
        *reinterpret_cast<uint4*>(tp_ptr(L, r, off)) = v;
      }
    } else if (mode == 1) {
      const int owner = row / rpr;
      *reinterpret_cast<uint4*>(tp_ptr(L, owner, stage_off(L, parity, L.rank, row % rpr) + c * 16)) = v;
    } else {
      const long long off = stage_off(L, parity, L.rank, row) + c * 16;
      for (int p = 0; p < L.world; p++) *reinterpret_cast<uint4*>(tp_ptr(L, (L.rank + p) % L.world, off)) = v;
    }
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(cta_counter, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    if ((int)threadIdx.x < L.world)
      st_release_sys(reinterpret_cast<int*>(tp_ptr(L, threadIdx.x, L.off_flags)) + (mode == 0 ? 1 : 0) * L.world + L.rank, epoch);
    if (threadIdx.x == 0) *cta_counter = 0;
  }
}

// Stand-alone all-gather, receiving side: wait (bounded) for every source, then copy the `rows` gathered rows of the half
// this call used into `out`.  The last CTA advances the epoch.
__global__ void __launch_bounds__(256) tp_wait_copy_kernel(const TpLayout L, __nv_bfloat16* __restrict__ out, int rows, int* __restrict__ epoch_ptr,
                                                          int spin_limit, int* __restrict__ cta_counter) {
  __shared__ int s_ok;
  const int epoch = *epoch_ptr + 1, parity = epoch & 1;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < L.world) {
    const int* f = reinterpret_cast<const int*>(tp_ptr(L, L.rank, L.off_flags)) + L.world + threadIdx.x;
    if (!wait_flag_ge(f, epoch, kKernelTp, 200 + threadIdx.x, (uint32_t)spin_limit)) s_ok = 0;
  }
  __syncthreads();
  const uint4* src = reinterpret_cast<const uint4*>(tp_ptr(L, L.rank, gather_off(L, parity, 0)));
  uint4* dst = reinterpret_cast<uint4*>(out);
  const long long total = (long long)rows * (L.H / 8);
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    dst[i] = s_ok ? src[i] : make_uint4(0, 0, 0, 0);
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(cta_counter, 1) == (int)gridDim.x - 1) { *cta_counter = 0; *epoch_ptr = epoch; }
}

// out[row] = sum over sources (rank order, fp32) of stage[src][row]  (+ add_in[row]); one CTA per row.
__global__ void __launch_bounds__(256) tp_reduce_kernel(const TpLayout L, const __nv_bfloat16* __restrict__ add_in, __nv_bfloat16* __restrict__ out,
                                                       int rows, int* __restrict__ epoch_ptr, int spin_limit, int* __restrict__ cta_counter) {
  __shared__ int s_ok;
  const int epoch = *epoch_ptr + 1, parity = epoch & 1;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < L.world) {
    const int* f = reinterpret_cast<const int*>(tp_ptr(L, L.rank, L.off_flags)) + threadIdx.x;
    if (!wait_flag_ge(f, epoch, kKernelTp, 300 + threadIdx.x, (uint32_t)spin_limit)) s_ok = 0;
  }
  __syncthreads();
  const int row = blockIdx.x;
  for (int c = threadIdx.x * 8; row < rows && c < L.H; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (s_ok) {
      // the partials of eight sources are fetched before any is added: independent loads, latency-bound kernel
      for (int s0 = 0; s0 < L.world; s0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int q = 0; q < 8; q++)
          v[q] = s0 + q < L.world ? *reinterpret_cast<const uint4*>(tp_ptr(L, L.rank, stage_off(L, parity, s0 + q, row) + (long long)c * 2))
                                  : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int q = 0; q < 8; q++) {
          const uint32_t u[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
          for (int j = 0; j < 4; j++) { const float2 f = unpack_bf16x2(u[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
        }
      }
    }
    if (add_in) {
      const uint4 v = *reinterpret_cast<const uint4*>(add_in + (long long)row * L.H + c);
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; j++) { const float2 f = unpack_bf16x2(u[j]); acc[2 * j] += f.x; acc[2 * j + 1] += f.y; }
    }
    *reinterpret_cast<uint4*>(out + (long long)row * L.H + c) = make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]),
                                                                         pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
  // every CTA has read the epoch and its row by now: the last one to get here closes the call
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(cta_counter, 1) == (int)gridDim.x - 1) { *cta_counter = 0; *epoch_ptr = epoch; }
}

__global__ void tp_advance_kernel(int* epoch_ptr) { *epoch_ptr += 1; }

}  // namespace ne

using namespace ne;

extern "C" int ne_tp_layout_size() { return (int)sizeof(TpLayout); }

static int tp_check(const TpLayout* L, int rpr) {
  if (L->world > kTpMaxWorld || L->world < 1 || L->H % 8 || rpr < 1 || rpr > L->rows_per_rank) return 1001;
  return 0;
}

// which: 0 = partials delivered (after a scatter-epilogue GEMM), 1 = rows delivered
extern "C" int ne_tp_signal(const TpLayout* L, int which, const int* epoch_ptr, cudaStream_t st) {
  tp_signal_kernel<<<1, 32, 0, st>>>(*L, which, epoch_ptr);
  return (int)cudaGetLastError();
}

extern "C" int ne_tp_push(const TpLayout* L, const void* x, int rows, int rpr, int mode, const int* epoch_ptr, int* cta_counter, cudaStream_t st) {
  if (int rc = tp_check(L, rpr)) return rc;
  if (rows < 0 || mode < 0 || mode > 2 || (mode != 1 && rows > rpr) || (mode == 1 && rows > L->world * rpr)) return 1001;
  if (rows == 0) return ne_tp_signal(L, mode == 0 ? 1 : 0, epoch_ptr, st);
  long long items = (long long)rows * (L->H / 8);
  int blocks = (int)((items + 255) / 256);
  if (blocks > 592) blocks = 592;
  tp_push_kernel<<<blocks, 256, 0, st>>>(*L, (const __nv_bfloat16*)x, rows, rpr, mode, epoch_ptr, cta_counter);
  return (int)cudaGetLastError();
}

// `cta_counter`: a zeroed device int owned by the caller (left zero).  `rows` = gathered rows (world * rows per rank).
extern "C" int ne_tp_wait_copy(const TpLayout* L, void* out, int rows, int* epoch_ptr, int spin_limit, int* cta_counter, cudaStream_t st) {
  if (rows < 0 || rows > L->world * L->rows_per_rank) return 1001;
  long long items = (long long)rows * (L->H / 8);
  int blocks = (int)((items + 255) / 256);
  blocks = blocks < 1 ? 1 : (blocks > 592 ? 592 : blocks);
  tp_wait_copy_kernel<<<blocks, 256, 0, st>>>(*L, (__nv_bfloat16*)out, rows, epoch_ptr, spin_limit, cta_counter);
  return (int)cudaGetLastError();
}

extern "C" int ne_tp_reduce(const TpLayout* L, const void* add_in, void* out, int rows, int* epoch_ptr, int spin_limit, int* cta_counter,
                            cudaStream_t st) {
  if (int rc = tp_check(L, rows > 0 ? rows : 1)) return rc;
  tp_reduce_kernel<<<rows > 0 ? rows : 1, 256, 0, st>>>(*L, (const __nv_bfloat16*)add_in, (__nv_bfloat16*)out, rows, epoch_ptr, spin_limit, cta_counter);
  return (int)cudaGetLastError();
}

extern "C" int ne_tp_advance(int* epoch_ptr, cudaStream_t st) {
  tp_advance_kernel<<<1, 1, 0, st>>>(epoch_ptr);
  return (int)cudaGetLastError();
}
