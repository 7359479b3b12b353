// Thin wrappers over the sm_100a PTX this library is built from: mbarrier, TMA (per-CTA loads only, no
// cluster-multicast form anywhere), tcgen05 (TMEM allocation, UMMA issue/commit, TMEM loads), descriptor
// builders, system-scope loads/stores for peer memory, and multimem.  Every wait is bounded: when the
// budget runs out the waiter records where it gave up in a status buffer and returns false, so a kernel
// can unwind (release TMEM, return) instead of hanging the GPU.
//
// The reference vendors comparable helpers (sgl_kernel/ptx/{tcgen05,tma,mbarrier,sync}.cuh) but none of
// its kernels issues tcgen05.mma; these are written for the kernels in this directory.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ne {
// host-side switch of the library: 1 = every fp8 activation quantiser rounds its group scales up to powers of two
extern int g_scale_pow2;

// ---- status buffer -----------------------------------------------------------------------------
// word 0: first error code (0 = ok); 1: kernel id; 2: block; 3: detail a; 4: detail b.
enum StatusCode : int { ST_OK = 0, ST_MBAR_TIMEOUT = 1, ST_FLAG_TIMEOUT = 2, ST_BAD_ARG = 3, ST_BAD_INDEX = 4 };
extern __device__ int g_status[8];

__device__ __forceinline__ void report(int code, int kernel_id, int a, int b) {
  if (atomicCAS(&g_status[0], 0, code) == 0) {
    g_status[1] = kernel_id; g_status[2] = (int)blockIdx.x; g_status[3] = a; g_status[4] = b;
  }
}

// ---- debug build: bounds on the indices the kernels take from tables ------------------------------------------------------
// Compiled with -DNE_DEBUG_BOUNDS (python -m nanoengine_b200.build_native --debug-bounds; loaded with NE_DEBUG_BOUNDS=1), the
// kernels that turn a table entry into an address (cache rows from a slot mapping, pages from a block table, state slots,
// expert ids) compare it with the bound the host registered (ne_debug_set_bounds) before they use it; a bad entry is recorded in
// the status words (ST_BAD_INDEX, kernel, site, value) and the access is skipped.  In the ordinary build the macro is `true`.
enum BoundKind : int { BK_CACHE_ROWS = 0, BK_CACHE_PAGES = 1, BK_STATE_SLOTS = 2, BK_EXPERTS = 3, BK_COUNT = 4 };
#ifdef NE_DEBUG_BOUNDS
extern __device__ long long g_bounds[BK_COUNT];
__device__ __forceinline__ bool ne_index_ok(long long idx, int kind, int kernel_id, int site) {
  const long long n = g_bounds[kind];
  if (n <= 0 || (idx >= 0 && idx < n)) return true;        // no bound registered: nothing to compare with
  report(ST_BAD_INDEX, kernel_id, site, (int)idx);
  return false;
}
#define NE_INDEX_OK(idx, kind, kernel_id, site) ne_index_ok((long long)(idx), kind, kernel_id, site)
#else
#define NE_INDEX_OK(idx, kind, kernel_id, site) true
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n .reg .pred p;\n elect.sync _|p, 0xffffffff;\n selp.u32 %0, 1, 0, p;\n}\n" : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// arrival on a barrier of another CTA of the cluster (`bar` = its shared::cluster address, see mapa_shared)
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Two tests for the price of one: both are in flight before either result is consumed.
__device__ __forceinline__ void mbar_test2(uint32_t barA, uint32_t parA, uint32_t barB, uint32_t parB, bool& okA, bool& okB) {
  uint32_t a, b;
  asm volatile("{\n .reg .pred pa, pb;\n mbarrier.test_wait.parity.shared::cta.b64 pa, [%2], %3;\n"
               " mbarrier.test_wait.parity.shared::cta.b64 pb, [%4], %5;\n selp.u32 %0, 1, 0, pa;\n selp.u32 %1, 1, 0, pb;\n}\n"
               : "=r"(a), "=r"(b) : "r"(barA), "r"(parA), "r"(barB), "r"(parB) : "memory");
  okA = a != 0; okB = b != 0;
}
// Hardware-suspended wait: the thread sleeps inside the barrier unit until the phase completes or `hint_ns` elapses.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
  uint32_t ok;
  asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
               : "=r"(ok) : "r"(bar), "r"(parity), "r"(hint_ns) : "memory");
  return ok != 0;
}
// Bounded wait (a couple of seconds at most): a short poll for the common case, then hardware-suspended waits of 20 us
// each.  `abort_flag` is a shared-memory word all roles of a CTA watch: once one of them gives up, the others stop too.
constexpr uint32_t kSpinLimit = 1u << 22;          // iteration budget of flag polls on global memory
constexpr uint32_t kMbarTries = 100000;            // x 20 us
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int kernel_id, int where, int polls = 16) {
#pragma unroll 1
  for (int i = 0; i < polls; ++i) if (mbar_test(bar, parity)) return true;
#pragma unroll 1
  for (uint32_t i = 0; i < kMbarTries; ++i) {
    if (mbar_try_wait(bar, parity, 20000u)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  report(ST_MBAR_TIMEOUT, kernel_id, where, (int)parity);
  return false;
}

// ---- thread-block clusters and distributed shared memory ----
__device__ __forceinline__ uint32_t cluster_ctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_nctarank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
// every thread of every CTA of the cluster must call this (no thread may have exited)
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared-memory address of the same offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank)); return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

// ---- TMA -----------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
               ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
               ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
// CTA-pair form: the data lands in this CTA's shared memory, the bytes are counted on `bar`, which may belong to the other CTA of
// the pair (its shared::cluster address).  Each CTA fetches its own tile.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const void* tmap, uint32_t bar, int x, int y, int z, int w) {
  asm volatile("cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
               ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w) : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const void* tmap, uint32_t bar, int x, int y, int z, int w, int v) {
  asm volatile("cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
               ::"r"(dst), "l"(tmap), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w), "r"(v) : "memory");
}
// generic-proxy writes to smem -> visible to the async proxy (UMMA / TMA reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// generic-proxy observations (a flag acquired from a peer GPU) ordered before later async-proxy (TMA) reads of global memory
__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;" ::: "memory"); }

// ---- tcgen05 ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {  // whole warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {   // whole warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// CTA-pair forms (cta_group::2): the same warp of both CTAs allocates / frees; MMAs and commits are issued by the pair's first CTA
__device__ __forceinline__ void tmem_alloc_pair(uint32_t dst_smem, uint32_t ncols) {  // whole warp, in both CTAs
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {   // whole warp, in both CTAs
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// `bar`: shared::cluster address of a barrier in either CTA of the pair
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; kind f16 covers fp16/bf16 inputs, f8f6f4 covers e4m3/e5m2.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n}\n"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// e4m3 operands with UE8M0 block scales read from TMEM (one byte per row and per 32 elements of K; the byte of a 32-bit
// scale-factor word is picked by the scale-factor id fields of the instruction descriptor).
__device__ __forceinline__ void umma_f8_block_scaled(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                                     uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// The same across a CTA pair: M = 256 (128 rows per CTA, each CTA's A tile and its half of B's rows in its own shared memory at the
// same offsets, accumulator and scale factors in each CTA's own TMEM at the same columns).
__device__ __forceinline__ void umma_f8_block_scaled_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                                          uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// Packed e2m1 operands (two per byte, K-major), one UE4M3 scale per 16 elements: K = 64 per instruction, four scale bytes per
// operand row = one 32-bit TMEM word (NVFP4).
__device__ __forceinline__ void umma_nvfp4_block_scaled(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate,
                                                        uint32_t sfa_tmem, uint32_t sfb_tmem) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n}\n"
               ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem) : "memory");
}
// A operand from TMEM (e.g. softmax probabilities), B from smem.
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
               ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// 32 lanes x 32 bit, N consecutive columns: thread i of the warp receives row (lane base + i).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
        "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
        "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x4(uint32_t taddr, const uint32_t (&r)[4]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1, %2, %3, %4};" ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]) : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
               ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}

// ---- asynchronous 16-byte copies global -> shared (src_bytes < 16 zero-fills the rest) ----
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// barrier among `count` threads of a CTA (a multiple of 32), ids 1..15
__device__ __forceinline__ void named_bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }

// ---- descriptors -----------------------------------------------------------------------------------
enum UmmaFmt : uint32_t { FMT_F16 = 0, FMT_BF16 = 1, FMT_E4M3 = 0, FMT_E5M2 = 1 };
// 32-bit instruction descriptor: fp32 accumulate, dense, no negate.  a_mn / b_mn = 1 selects an MN-major operand.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t a_fmt, uint32_t b_fmt, uint32_t M, uint32_t N, uint32_t a_mn = 0, uint32_t b_mn = 0) {
  return (1u << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn << 15) | (b_mn << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}
// Descriptor of the block-scaled kinds: no accumulator-format field (always fp32); bit 23 = UE8M0 scale factors; the
// scale-factor ids (which byte of the 32-bit scale word) sit at bits [4,6) for B and [29,31) for A.
__host__ __device__ constexpr uint32_t make_idesc_block_scaled(uint32_t a_fmt, uint32_t b_fmt, uint32_t M, uint32_t N, uint32_t ue8m0 = 1) {
  return (a_fmt << 7) | (b_fmt << 10) | ((N >> 3) << 17) | (ue8m0 << 23) | ((M >> 4) << 24);
}
constexpr uint32_t FMT_E2M1_MXF4 = 1;      // operand format code of the packed-fp4 kinds
enum SwizzleMode : uint64_t { SW_NONE = 0, SW_128B = 2, SW_64B = 4, SW_32B = 6 };
// 64-bit shared-memory matrix descriptor (Blackwell version field = 1).  Offsets are given in bytes.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t swizzle) {
  return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32) | (1ull << 46) | (swizzle << 61);
}

// ---- memory helpers ---------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(int* p, int v) { asm volatile("st.release.sys.global.b32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v; asm volatile("ld.acquire.sys.global.b32 %0, [%1];" : "=r"(v) : "l"(p) : "memory"); return v;
}
__device__ __forceinline__ void red_add_release_sys(int* p, int v) { asm volatile("red.release.sys.global.add.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory"); }
__device__ __forceinline__ int4 ld_nc_v4(const void* p) {
  int4 v; asm volatile("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p)); return v;
}
// Bounded poll on a flag another GPU (or CTA) sets: waits until *p >= want.
__device__ __forceinline__ bool wait_flag_ge(const int* p, int want, int kernel_id, int where, uint32_t limit = kSpinLimit) {
  for (uint32_t i = 0; i < limit; ++i) {
    if (ld_acquire_sys(p) >= want) return true;
    if (i > 16) __nanosleep(i > 1024 ? 512 : 64);
  }
  report(ST_FLAG_TIMEOUT, kernel_id, where, want);
  return false;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ uint8_t to_e4m3(float x) {
  return (uint8_t)__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
  uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
  return lo | (hi << 16);
}
// Scale of a 128-element group whose absolute maximum is amax: amax / 448, or (pow2) the next power of two at or above
// it, the form the tensor cores' own block scaling takes.  *inv receives the factor that maps the group onto e4m3.
__device__ __forceinline__ float fp8_group_scale(float amax, int pow2, float* inv) {
  float s = amax / 448.f;
  if (!pow2) { *inv = 448.f / amax; return s; }
  const uint32_t b = (__float_as_uint(s) + 0x7fffffu) & 0x7f800000u;
  *inv = __uint_as_float(0x7f000000u - b);
  return __uint_as_float(b);
}
__device__ __forceinline__ float e4m3_to_float(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(v, __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// ---- programmatic dependent launch ---------------------------------------------------------------
// A kernel launched with `launch_pdl` may be scheduled while the kernel before it in the stream is still draining; it runs its
// own set-up (barrier init, TMEM allocation, descriptor prefetch: nothing that touches global memory), then `pdl_wait()`
// blocks until the previous kernel has completed and its writes are visible, and `pdl_trigger()` right after lets the next
// kernel do the same behind this one.  Triggering only after the wait keeps at most one waiting grid resident.  Both are
// no-ops in a kernel launched the ordinary way, and an ordinary launch next in the stream still waits for full completion.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace ne

#include <cstdlib>
namespace ne {
inline bool pdl_enabled() {
  static int v = -1;
  if (v < 0) { const char* e = getenv("NE_PDL"); v = (e && e[0] == '0') ? 0 : 1; }
  return v != 0;
}
// extra launch attributes (a cluster dimension) go first in `attrs`, which must have room for one more entry
inline void pdl_attr(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attrs, unsigned n_before) {
  if (pdl_enabled()) {
    attrs[n_before].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[n_before].val.programmaticStreamSerializationAllowed = 1;
    n_before++;
  }
  cfg.attrs = attrs; cfg.numAttrs = n_before;
}
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
  cudaLaunchAttribute attrs[1];
  pdl_attr(cfg, attrs, 0);
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
}  // namespace ne
