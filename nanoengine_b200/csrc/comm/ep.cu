// Expert-parallel dispatch and combine over NVLink peer memory, fused with the grouped expert GEMMs.
//
// Every rank owns one symmetric region (same offsets on all ranks):
//   cnt   int32 [E_local]                     rows arrived per local expert (target of remote atomics)
//   aq    e4m3  [E_local, cap, H]             expert-major activations, written by the SENDERS (quantised 1x128 on the way)
//   as    fp32  [E_local, H/128, cap]         their scales, in the layout the block-scaled GEMM reads
//   abf   bf16  [E_local, cap, H]             (bf16 models instead of aq/as)
//   info  int64 [E_local, cap]                (source rank << 32 | token*K + k) of every row
//   ret   bf16  [T_max*K, H]                  expert outputs coming back, written by the down-proj GEMM EPILOGUE of the owners
//   arrive/done flags int32 [world] each, epoch-tagged
//
// One MoE layer is five launches in stream order:
//   ep_dispatch   (sender)   slot = remote atomicAdd(cnt[e]); quantise + peer-store row, scales, info; last CTA raises `arrive` at all peers
//   grouped GEMM gate_up     (owner) every CTA's prologue waits (bounded) for all peers' `arrive`, then takes `cnt` as the per-expert row counts
//   SwiGLU + requant
//   grouped GEMM down        its epilogue stores each output row straight into the source GPU's `ret` buffer, addressed from the row's
//                            `info` record (the combine "send" costs no extra pass); the last CTA to finish zeroes `cnt` and raises
//                            `done` at all peers
//   ep_reduce     (sender)   bounded wait for every peer's `done`; out[t] = sum_k w[t,k] * ret[t*K+k] (+ shared expert output); the last
//                            CTA advances the epoch
// (the wait, the address table and the two signals used to be kernels of their own: ep_wait_build, ep_signal, ep_advance)
// The epoch lives in device memory so a captured CUDA graph replays with fresh tags.  Nothing here uses multicast loads;
// all remote traffic is plain stores, one atomic per routed pair and flag words.
//
// Replaces in the reference: deep_ep.Buffer.low_latency_dispatch / low_latency_combine and dispatch / combine
// (layers/backends/experts/token_dispatcher.py:91-378) together with the scatter/gather kernels around them
// (triton/hopper/fused_moe_v3.py:214-453); the fused library counterpart is deep_gemm.fp8_fp4_mega_moe.
#include "ptx.cuh"

namespace ne {

constexpr int kMaxWorld = 16;
constexpr int kKernelEp = 3;

struct EpLayout {
  unsigned long long peer_base[kMaxWorld];   // base address of every rank's symmetric region (index = rank)
  long long off_cnt, off_aq, off_as, off_abf, off_info, off_ret, off_arrive, off_done;
  int rank, world, E_local, cap, H, top_k, fp8;
};

__device__ __forceinline__ uint8_t* peer_ptr(const EpLayout& L, int r, long long off) { return reinterpret_cast<uint8_t*>(L.peer_base[r]) + off; }

// one warp per (token, k) pair
__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpLayout L, const __nv_bfloat16* __restrict__ x, const int* __restrict__ idx,
                                                         int* __restrict__ pair_ok, int n_pairs, const int* __restrict__ epoch_ptr,
                                                         int* __restrict__ cta_counter) {
  const int warps = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  const int H = L.H, cap = L.cap;
  for (int i = blockIdx.x * warps + (threadIdx.x >> 5); i < n_pairs; i += gridDim.x * warps) {
    const int e = idx[i];
    if (e < 0) { if (lane == 0) pair_ok[i] = 0; continue; }
    const int dst = e / L.E_local, el = e % L.E_local;
    int slot = 0;
    if (lane == 0) slot = atomicAdd_system(reinterpret_cast<int*>(peer_ptr(L, dst, L.off_cnt)) + el, 1);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (slot >= cap) {                      // receive buffer full: drop the pair and say so
      if (lane == 0) { pair_ok[i] = 0; report(ST_BAD_ARG, kKernelEp, e, slot); }
      continue;
    }
    const long long row = (long long)el * cap + slot;
    const __nv_bfloat16* xr = x + (long long)(i / L.top_k) * H;
    if (L.fp8) {
      uint8_t* aq = peer_ptr(L, dst, L.off_aq) + row * H;
      float* as = reinterpret_cast<float*>(peer_ptr(L, dst, L.off_as)) + (long long)el * (H / 128) * cap + slot;
#pragma unroll 4
      for (int g = 0; g < H / 128; g++) {
        uint2 v = *reinterpret_cast<const uint2*>(xr + g * 128 + lane * 4);
        float2 a = unpack_bf16x2(v.x), b = unpack_bf16x2(v.y);
        float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
        amax = fmaxf(warp_max(amax), 1e-10f);
        float is; const float sg = fp8_group_scale(amax, L.fp8 == 2, &is);
        *reinterpret_cast<uint32_t*>(aq + g * 128 + lane * 4) = pack_e4m3x4(a.x * is, a.y * is, b.x * is, b.y * is);
        if (lane == 0) as[(long long)g * cap] = sg;
      }
    } else {
      __nv_bfloat16* ab = reinterpret_cast<__nv_bfloat16*>(peer_ptr(L, dst, L.off_abf)) + row * H;
      for (int c = lane * 8; c < H; c += 256) *reinterpret_cast<uint4*>(ab + c) = *reinterpret_cast<const uint4*>(xr + c);
    }
    if (lane == 0) {
      reinterpret_cast<long long*>(peer_ptr(L, dst, L.off_info))[row] = ((long long)L.rank << 32) | (long long)i;
      pair_ok[i] = 1;
    }
  }
  // every store of this CTA is ordered before the flag the last CTA raises
  __threadfence_system();
  __syncthreads();
  __shared__ int s_last;
  if (threadIdx.x == 0) s_last = (atomicAdd(cta_counter, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (s_last) {
    const int epoch = *epoch_ptr + 1;
    if (threadIdx.x == 0) *cta_counter = 0;
    __threadfence_system();
    if ((int)threadIdx.x < L.world)
      st_release_sys(reinterpret_cast<int*>(peer_ptr(L, threadIdx.x, L.off_arrive)) + L.rank, epoch);
  }
}

// one CTA per token
__global__ void __launch_bounds__(256) ep_reduce_kernel(const EpLayout L, const int* __restrict__ pair_ok, const float* __restrict__ w,
                                                       const __nv_bfloat16* __restrict__ add_in, __nv_bfloat16* __restrict__ out,
                                                       int* __restrict__ epoch_ptr, int spin_limit, int* __restrict__ cta_counter) {
  __shared__ int s_ok; __shared__ int s_use[64]; __shared__ float s_w[64];
  const int epoch = *epoch_ptr + 1;
  const int t = blockIdx.x, K = L.top_k, H = L.H;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if ((int)threadIdx.x < L.world) {
    const int* f = reinterpret_cast<const int*>(peer_ptr(L, L.rank, L.off_done)) + threadIdx.x;
    if (!wait_flag_ge(f, epoch, kKernelEp, 200 + threadIdx.x, (uint32_t)spin_limit)) s_ok = 0;
  }
  if ((int)threadIdx.x < K) { s_use[threadIdx.x] = pair_ok[(long long)t * K + threadIdx.x]; s_w[threadIdx.x] = w[(long long)t * K + threadIdx.x]; }
  __syncthreads();
  const __nv_bfloat16* ret = reinterpret_cast<const __nv_bfloat16*>(peer_ptr(L, L.rank, L.off_ret));
  // blockIdx.y splits the row into column slices so a decode batch fills the SMs (one CTA per token would leave some idle and
  // keep too few loads in flight on the others)
  const int slice = (((H + 7) / 8 + gridDim.y - 1) / gridDim.y) * 8;
  const int c_end = min(H, ((int)blockIdx.y + 1) * slice);
  for (int c = blockIdx.y * slice + threadIdx.x * 8; c < c_end; c += blockDim.x * 8) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (s_ok) {
      // eight returned rows are fetched before any is used: the loads are independent and the kernel is latency-bound
      for (int k0 = 0; k0 < K; k0 += 8) {
        uint4 v[8];
#pragma unroll
        for (int q = 0; q < 8; q++)
          v[q] = (k0 + q < K && s_use[k0 + q]) ? *reinterpret_cast<const uint4*>(ret + ((long long)t * K + k0 + q) * H + c) : make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int q = 0; q < 8; q++) {
          const float wk = (k0 + q < K && s_use[k0 + q]) ? s_w[k0 + q] : 0.f;
          const uint32_t u[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
#pragma unroll
          for (int j = 0; j < 4; j++) { float2 f = unpack_bf16x2(u[j]); acc[2 * j] += wk * f.x; acc[2 * j + 1] += wk * f.y; }
        }
      }
    }
    if (add_in) {
      uint4 v = *reinterpret_cast<const uint4*>(add_in + (long long)t * H + c);
      uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; j++) {
        float2 f = unpack_bf16x2(u[j]); float2 r = unpack_bf16x2(pack_bf16x2(acc[2 * j], acc[2 * j + 1]));
        acc[2 * j] = r.x + f.x; acc[2 * j + 1] = r.y + f.y;
      }
    }
    *reinterpret_cast<uint4*>(out + (long long)t * H + c) =
        make_uint4(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]), pack_bf16x2(acc[4], acc[5]), pack_bf16x2(acc[6], acc[7]));
  }
  // the layer is over for this rank once every CTA has read the epoch and its rows: the last one moves the epoch on
  __syncthreads();
  if (threadIdx.x == 0 && atomicAdd(cta_counter, 1) == (int)(gridDim.x * gridDim.y) - 1) {
    *cta_counter = 0;
    *epoch_ptr = epoch;
  }
}

__global__ void ep_advance_kernel(int* epoch_ptr) { *epoch_ptr += 1; }

// A rank with no tokens still owes its peers the `arrive` flag.
__global__ void ep_arrive_only_kernel(const EpLayout L, const int* __restrict__ epoch_ptr) {
  const int epoch = *epoch_ptr + 1;
  if ((int)threadIdx.x < L.world) st_release_sys(reinterpret_cast<int*>(peer_ptr(L, threadIdx.x, L.off_arrive)) + L.rank, epoch);
}

}  // namespace ne

using namespace ne;

extern "C" int ne_ep_dispatch(const EpLayout* L, const void* x, const int* idx, int* pair_ok, int n_pairs, const int* epoch_ptr,
                              int* cta_counter, cudaStream_t st) {
  if (L->world > kMaxWorld || L->H % 128) return 1001;
  if (n_pairs <= 0) { ep_arrive_only_kernel<<<1, 32, 0, st>>>(*L, epoch_ptr); return (int)cudaGetLastError(); }
  int blocks = (n_pairs + 7) / 8;
  if (blocks > 1184) blocks = 1184;
  EpLayout Lq = *L;
  if (Lq.fp8 && g_scale_pow2) Lq.fp8 = 2;               // fp8 == 2: group scales rounded up to powers of two
  ep_dispatch_kernel<<<blocks, 256, 0, st>>>(Lq, (const __nv_bfloat16*)x, idx, pair_ok, n_pairs, epoch_ptr, cta_counter);
  return (int)cudaGetLastError();
}

// `cta_counter`: a zeroed device int owned by the caller (the kernel leaves it zero).  With no tokens the epoch still advances.
extern "C" int ne_ep_reduce(const EpLayout* L, const int* pair_ok, const float* w, const void* add_in, void* out, int T, int* epoch_ptr,
                            int spin_limit, int* cta_counter, cudaStream_t st) {
  if (T > 0) {
    if (L->top_k > 64 || L->H % 8) return 1001;
    const int slices = T >= 2048 ? 1 : (T >= 512 ? 2 : 4);
    ep_reduce_kernel<<<dim3(T, slices), 256, 0, st>>>(*L, pair_ok, w, (const __nv_bfloat16*)add_in, (__nv_bfloat16*)out, epoch_ptr, spin_limit,
                                                      cta_counter);
  } else {
    ep_advance_kernel<<<1, 1, 0, st>>>(epoch_ptr);
  }
  return (int)cudaGetLastError();
}

extern "C" int ne_ep_advance(int* epoch_ptr, cudaStream_t st) {
  ep_advance_kernel<<<1, 1, 0, st>>>(epoch_ptr);
  return (int)cudaGetLastError();
}

extern "C" int ne_ep_layout_size() { return (int)sizeof(EpLayout); }
