// tcgen05 GEMM family for sm_100a:  D[g, m, n] = sum_k A[g, m, k] * B[g, n, k]   (both operands K-major).
//
//  * bf16 x bf16 -> fp32 accumulation in TMEM, bf16 or fp32 output
//  * fp8 e4m3 x e4m3 with DeepSeek block scales (activations 1x128, weights 128x128): each 128-deep K block is
//    multiplied on the tensor cores into a fresh TMEM accumulator and promoted into fp32 registers with
//    scale_a[m, kb] * scale_b[n/128, kb] by the epilogue warps while the next K block is being multiplied
//  * dense (one group, M rows) or grouped-masked (E groups of up to max_m rows, masked_m[e] valid), the layout
//    the MoE path uses for prefill and decode alike
//
// Structure (one CTA per SM, persistent over tiles): warp 0 issues TMA loads into a multi-stage 128B-swizzled
// shared-memory ring, warp 1 issues tcgen05.mma from one elected thread and owns the TMEM allocation, warps 2-5
// drain TMEM (tcgen05.ld), apply scales, convert and store.  Two TMEM accumulators let the epilogue of one tile
// (or K block) overlap the MMAs of the next.  All mbarrier waits are bounded.
//
// Replaces in the reference: deep_gemm.fp8_gemm_nt / m_grouped_fp8_gemm_nt_masked call sites
// (layers/backends/linear/deep_gemm.py, layers/backends/experts/deep_gemm.py:498-837), the CuTe-DSL small-M bf16
// GEMM (kernel/cutedsl_bf16_gemm.py) and cuBLAS F.linear (layers/backends/linear/generic.py:103-315).
#include <cstring>
#include <mutex>
#include <unordered_map>

#include "ptx.cuh"
#include "tma_host.h"

namespace ne {

int g_scale_pow2 = 0;
__device__ int g_status[8];
#ifdef NE_DEBUG_BOUNDS
__device__ long long g_bounds[BK_COUNT];
#endif

constexpr int kBlockM = 128;
constexpr int kKBytes = 128;            // bytes of K per K block row: one 128B swizzle atom
// One pipeline stage holds kG consecutive K blocks of both operands, fetched by ONE TMA instruction per operand: the
// tensor maps carry the 128-byte K chunk index as their outermost dimension, so a box {128 B, rows, ..., kG} lands as kG
// consecutive swizzled [rows x 128 B] tiles.  An SM retires roughly one TMA instruction per 0.2 us whatever its size, so
// two instructions per K block cap a 128-wide tile well below both the tensor pipe and HBM; two per kG blocks do not.
template <int BLOCK_N, bool kFp4 = false> struct KGroup { static constexpr int value = (BLOCK_N >= 192 || kFp4) ? 1 : 2; };   // the wide tiles keep 4 single-block stages
constexpr int kGemmThreads = 192;
constexpr int kKernelGemm = 1;

// Communication fused into a GEMM launch.  Every pointer is optional; epochs live in device memory so a captured CUDA
// graph replays with fresh tags, and every wait is bounded (status word + no tiles run on expiry).
struct GemmComm {
  // (1) wait prologue (EP dispatch -> grouped GEMM): no tile starts before wait_flags[0 .. wait_world) >= *wait_epoch + 1.
  const int* wait_epoch; const int* wait_flags; int wait_world; unsigned wait_spin;
  // (2) gated A operand (all-gather -> GEMM): rows [s * gate_rpr, (s + 1) * gate_rpr) of A are delivered by source rank s,
  //     which then raises gate_flags[s] to *gate_epoch + 1; the producer warp waits for the sources of the tile it is about
  //     to load, so tiles of rows that have arrived (this rank's own first: mb_rot) run while others are in flight.  The
  //     double-buffered gather area is one tensor map; the half in use is (epoch + 1) & 1, gate_parity_rows rows apart.
  const int* gate_epoch; const int* gate_flags; int gate_rpr, gate_world, gate_parity_rows, mb_rot; unsigned gate_spin;
  // (3) scatter epilogue without an address table.  mode 2 (MoE combine): row r of group g goes to
  //     scatter_base[info >> 32] + (info & 0xffffffff) * ldd * 2 with info = row_info[g * rd_group_stride + r].
  //     mode 3 (GEMM -> reduce-scatter): row r goes to scatter_base[r / scatter_rpr] + parity * scatter_parity_bytes +
  //     (r % scatter_rpr) * ldd * 2, parity = (*scatter_epoch + 1) & 1.
  int scatter_mode; const long long* row_info; unsigned long long scatter_base[16]; int scatter_rpr; long long scatter_parity_bytes;
  const int* scatter_epoch;
  // (4) tail: the last CTA of the grid to finish zeroes tail_clear[0 .. tail_clear_n), stores *tail_epoch + 1 (release, system
  //     scope) to tail_flag[0 .. tail_world) and, if tail_advance is set, increments *tail_advance.
  int* tail_counter; const int* tail_epoch; unsigned long long tail_flag[16]; int tail_world; int* tail_clear; int tail_clear_n;
  int* tail_advance;
};

struct GemmArgs {
  int M, N, K, groups;
  const int* masked_m;                  // [groups] valid rows per group, or nullptr (all M rows valid)
  const int* row_start;                 // contiguous mode: group g owns rows [row_start[g], row_start[g] + masked_m[g]) of one
                                        // flat [M, K] activation matrix (starts are multiples of 128); nullptr = [groups, M, K]
  int a_group_inner;                    // A is stored [rows, groups, K]: TMA coordinates are (k, group, row)
  int k_flat;                           // K in bytes is not a multiple of 128: K stays the maps' innermost dimension (zero-filled tail), one TMA per K block
  void* D; long long ldd; long long d_group_stride;   // in elements
  const float* sa; int sa_ld; long long sa_group_stride;   // activation scales [groups][K/128][sa_ld]
  const float* sb; long long sb_group_stride;              // weight scales [groups][ceil(N/128)][K/128]
  const float* alpha;                   // optional [groups]: the accumulator is multiplied by alpha[group] (plain and NVFP4 GEMMs)
  int out_fp32;                         // 0: bf16 output, 1: fp32, 2: e4m3 (clamped cast, no scale; plain bf16 GEMMs only)
  const long long* row_dst;             // optional scatter epilogue: absolute address of every output row (bf16, may be peer memory),
  long long rd_group_stride;            // indexed [group * rd_group_stride + row]; used by the MoE combine
  GemmComm comm;                        // hooks that fuse a collective into this GEMM (all null / zero for a plain GEMM)
};

constexpr int kFp4SfSlots = 8;          // NVFP4: shared-memory ring of scale-factor tiles (one K block each, 4 KB), 6 in flight
template <int BLOCK_N, bool kFp4 = false, bool kPair = false> struct Smem {
  static constexpr int kABytes = kBlockM * kKBytes;
  static constexpr int kBBytes = (kPair ? BLOCK_N / 2 : BLOCK_N) * kKBytes;      // a CTA of a pair holds half of B's rows
  static constexpr int kG = kPair ? 2 : KGroup<BLOCK_N, kFp4>::value;
  static constexpr int kSfRing = kFp4 ? kFp4SfSlots * 4096 : 0;
  static constexpr int kStageBytes = kG * (kABytes + kBBytes);
  static constexpr int kStaging = 8 * 32 * 80;      // per-warp epilogue staging for up to 8 epilogue warps
  static constexpr int kStaticTables = 6400;       // the kernel's static shared memory: three per-group tables of kSchedCache ints + small
  static constexpr int kBudget = 232448 - 1024 - 256 - kStaging - kStaticTables - kSfRing;
  static constexpr int kStages = (kBudget / kStageBytes) > 10 ? 10 : (kBudget / kStageBytes);
  static constexpr int kBytes = kStages * kStageBytes + kSfRing + kStaging + 1024 /*align*/ + 256 /*barriers*/;
};

constexpr int kSchedCache = 512;        // group tables up to this many groups are staged in shared memory

// Maps a linear tile index to (group, row block, column block).  Three roles of a CTA (producer, MMA issuer, epilogue) each walk
// their own copy, and the lookup sits on the producer's critical path at every tile switch, so it must not scan: a step of a
// linear walk over the groups costs ~300 cycles in one thread (measured: 20k cycles to reach group 94 of a 128-head batched
// GEMM, most of that kernel's run time).  Uniform groups use a division; ragged groups use the table of first-tile indices
// that the CTA builds once in shared memory (`base`, groups + 1 entries) and a binary search.  Only group counts beyond the
// shared-memory table fall back to the incremental walk.
struct TileSched {
  int groups, M, n_blocks;
  const int* masked_m;                  // global or shared memory
  const int* row_start;
  const int* base;                      // shared memory: first tile of every group, total at [groups]; null = none built
  int g = 0, walked = 0;
  int mb_rot = 0;                       // dense single-group GEMMs only: row blocks are visited starting at this one
  int bm = kBlockM, sub = 0;            // CTA pairs: tiles are 256 rows tall, `sub` (0 / 1) is this CTA's 128-row block of the tile
  __device__ TileSched(int groups_, int M_, int nb, const int* mm, const int* rs, const int* base_, int rot = 0, int bm_ = kBlockM, int sub_ = 0)
      : groups(groups_), M(M_), n_blocks(nb), masked_m(mm), row_start(rs), base(base_), mb_rot(rot), bm(bm_), sub(sub_) {}
  // the caller's row block index counts 128-row blocks
  __device__ int blk(int mb) const { return bm == kBlockM ? mb : mb * 2 + sub; }
  __device__ int row0(int grp) const { return row_start ? row_start[grp] : 0; }
  __device__ int rows(int grp) const {
    int r = masked_m ? masked_m[grp] : M;
    int cap = row_start ? M - row_start[grp] : M;      // never step outside the buffer, whatever the counts say
    return r < cap ? r : (cap > 0 ? cap : 0);
  }
  __device__ int tiles_of(int grp) const { return ((rows(grp) + bm - 1) / bm) * n_blocks; }
  __device__ bool get(int tile, int& grp, int& mb, int& nb) {
    if (!masked_m && !row_start) {                      // every group has the same shape
      const int per = ((M + bm - 1) / bm) * n_blocks;
      if (tile >= per * groups) return false;
      grp = tile / per;
      const int l = tile - grp * per;
      mb = l / n_blocks; nb = l - mb * n_blocks;
      if (mb_rot) { const int mbs = (M + bm - 1) / bm; mb += mb_rot; if (mb >= mbs) mb -= mbs; }
      mb = blk(mb);
      return true;
    }
    if (base) {
      if (tile >= base[groups]) return false;
      int lo = g, hi = groups - 1;                      // tiles only move forward: the answer is never before the last one
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (base[mid] <= tile) lo = mid; else hi = mid - 1; }
      g = grp = lo;
      const int l = tile - base[lo];
      mb = blk(l / n_blocks); nb = l % n_blocks;
      return true;
    }
    while (g < groups) {
      const int cnt = tiles_of(g);
      if (tile < walked + cnt) { const int l = tile - walked; grp = g; mb = blk(l / n_blocks); nb = l % n_blocks; return true; }
      walked += cnt; g++;
    }
    return false;
  }
};

// bf16 output goes through a small per-warp staging buffer: each thread parks 32 columns of its row (64 bytes), then the
// warp writes eight rows per instruction with four lanes covering each row's 64 contiguous bytes.  Compared with every
// thread writing 16 bytes of a different row this quadruples the contiguous run per row - what matters most when the rows
// are scattered to peer GPUs by the MoE combine.
constexpr int kStgPitch = 80;                       // 64 bytes of data + 16 of padding: conflict-free for 16-byte accesses
constexpr int kStgWarpBytes = 32 * kStgPitch;
// Which rows a lane serves in the four store rounds of a 32-column chunk, fetched from their owner lanes once per tile
// (the shuffles cost as much as the stores when repeated per chunk).
struct EpiRows { unsigned long long dp[4]; bool ok[4]; };
__device__ __forceinline__ EpiRows epi_rows(bool row_ok, __nv_bfloat16* drow) {
  EpiRows r;
  const int lane = (int)lane_id();
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int rr = i * 8 + (lane >> 2);
    r.ok[i] = __shfl_sync(0xffffffffu, (int)row_ok, rr) != 0;
    r.dp[i] = __shfl_sync(0xffffffffu, (unsigned long long)reinterpret_cast<uintptr_t>(drow), rr);
  }
  return r;
}
// `col` = first column of the chunk relative to the row pointers in `rows`.
__device__ __forceinline__ void epi_store32_bf16(uint8_t* stg, const float (&v)[32], const EpiRows& rows, int col, int ncols_left) {
  const int lane = (int)lane_id();
  uint8_t* mine = stg + lane * kStgPitch;
#pragma unroll
  for (int q = 0; q < 4; q++)
    *reinterpret_cast<uint4*>(mine + q * 16) = make_uint4(pack_bf16x2(v[q * 8], v[q * 8 + 1]), pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]),
                                                          pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]));
  __syncwarp();
  const int ch = lane & 3;
#pragma unroll
  for (int i = 0; i < 4; i++) {
    const int rr = i * 8 + (lane >> 2);
    if (rows.ok[i] && ch * 8 < ncols_left)
      *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(rows.dp[i]) + col + ch * 8) = *reinterpret_cast<const uint4*>(stg + rr * kStgPitch + ch * 16);
  }
  __syncwarp();
}

// First element of an output row: the plain [group, row] position, or where the fused collective wants the row (GemmComm (3)).
__device__ __forceinline__ __nv_bfloat16* scatter_row(const GemmArgs& a, int grp, int row, bool row_ok, int parity, __nv_bfloat16* plain) {
  if (!row_ok) return plain;
  if (a.row_dst) return reinterpret_cast<__nv_bfloat16*>(a.row_dst[(long long)grp * a.rd_group_stride + row]);
  const GemmComm& cm = a.comm;
  if (cm.scatter_mode == 2) {
    const long long info = cm.row_info[(long long)grp * a.rd_group_stride + row];
    return reinterpret_cast<__nv_bfloat16*>(cm.scatter_base[(int)(info >> 32) & 15]) + (info & 0xffffffffll) * a.ldd;
  }
  if (cm.scatter_mode == 3) {
    const int owner = row / cm.scatter_rpr;
    return reinterpret_cast<__nv_bfloat16*>(cm.scatter_base[owner & 15] + (long long)parity * cm.scatter_parity_bytes) + (long long)(row - owner * cm.scatter_rpr) * a.ldd;
  }
  return plain;
}

// Block-scaled tiles at least 64 wide use two epilogue warpgroups that split the tile's columns, halving the
// promotion work per thread and per K block.
template <int BLOCK_N, bool kBlockScaled, bool kHw = false> struct EpiCfg {
  static constexpr int kGroups = (kBlockScaled && BLOCK_N >= 64) ? 2 : 1;
  static constexpr int kThreads = 64 + 128 * kGroups + (kHw ? 128 : 0);      // kHw: four scale-factor warps after the epilogue warps
};

// kHw: fp8 operands whose block scales are powers of two, applied by the tensor cores themselves
// (tcgen05.mma.kind::mxf8f6f4.block_scale, UE8M0 scale factors read from TMEM).  One accumulator per tile, as in a plain
// GEMM: no promotion on the CUDA cores.  The instruction takes one scale byte per operand row and per 32 elements of K;
// the DeepSeek granularity (one per 128 of K, and per 128 x 128 weight block) maps onto it as follows:
//  * the scale factors of A for 4 consecutive K blocks of a 128-row tile are one TMEM word per row: byte j belongs to K
//    block j, selected by the scale-factor id of the instruction descriptor, and all four K = 32 instructions of a K block
//    use the same byte.  Row r + 32 g of the tile is held by lane r (of every 32-lane quarter) in column g.
//  * a tile is at most 128 columns wide and never straddles a weight block, so the weight scale of a K block is one
//    number per tile; it is folded into A's byte (exponents add) and B's scale factors are the constant 1.
// Four extra warps, one per TMEM lane quarter, compute the bytes from the fp32 scale arrays and store them into TMEM
// (tcgen05.st) a few chunks ahead of the MMA issuer.
// A tile wider than a weight block (BLOCK_N = 224: two accumulators and the scale factors just fit the 512 TMEM columns, and
// 7168 = 32 x 224) cannot fold: B gets its own scale bytes, one per tile column and K block (column c + 32 g of the tile: lane
// c, word g, byte = K block of the chunk), written next to A's in every ring entry.  The wide tile moves a fifth fewer operand
// bytes per FLOP through the SM's fill path, which is what bounds these GEMMs.
constexpr int kSfBufsMax = 8;

// kSplit: split-K across a thread-block cluster.  The CTAs of a cluster work on the same output tile, each over its own
// slice of K; every CTA parks its fp32 partial tile in its shared memory and, after a cluster barrier, CTA r adds up rows
// [r * R, (r + 1) * R) of all partials through distributed shared memory and writes them out.  This is what lets a
// 128-token decode GEMM keep every SM pulling weights while using the 128-wide tile (a narrow tile re-reads the
// activation operand once per tile and is bound by the SM's L2 read rate instead of HBM).  One tile per cluster,
// dense operands only (groups = 1, no row tables).
// kMode: 0 = scales (if any) on the CUDA cores, 1 = kHw (fp8, UE8M0 scales on the tensor cores), 2 = NVFP4: packed e2m1 operands
// (kFP8's byte-wide plumbing: a 128-byte K block row holds 256 elements), one UE4M3 scale per 16 elements of either operand
// ([rows, K / 16] bytes, row-major, as ModelOpt checkpoints and the activation quantiser write them), applied by
// tcgen05.mma.kind::mxf4nvf4.block_scale, fp32 accumulator times alpha[group] in the epilogue.  A K block needs 16 scale bytes per
// row of A and B: the four scale warps bring them in with 16-byte cp.async copies, six K blocks ahead, through a ring in shared
// memory (each warp a quarter of the rows), and store them to TMEM as 16 + 16 columns per K block (column 4 i + g: instruction i of
// the K block, rows 32 g .. 32 g + 31 of the tile).
// kPair (with kMode 1): two CTAs of a cluster work on one 256-row tile with tcgen05.mma.cta_group::2.  Each holds its 128 rows of A
// and half of B's rows in its own shared memory (a third less operand traffic per SM than two separate 128 x BLOCK_N tiles), its
// 128 accumulator rows and scale factors in its own TMEM.  The pair's first CTA issues the MMAs once both CTAs' loads have landed
// (both count their bytes on its "full" barrier), and commits to the barriers of both; the second CTA's epilogue and scale warps
// report to the first CTA's barriers.
template <int BLOCK_N, bool kFP8, bool kBlockScaled, bool kSplit, int kMode = 0, bool kPair = false>
__global__ void __launch_bounds__((EpiCfg<BLOCK_N, kBlockScaled, kMode != 0>::kThreads), 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_a64, const __grid_constant__ CUtensorMap tmap_a32,
            const __grid_constant__ CUtensorMap tmap_b, const GemmArgs args) {
  constexpr bool kHw = kMode != 0, kFp4 = kMode == 2;
  static_assert(!kPair || (kMode == 1 && !kSplit), "CTA pairs: the tensor-core-scaled fp8 GEMM");
  using S = Smem<BLOCK_N, kFp4, kPair>;
  constexpr int kTileM = kPair ? 2 * kBlockM : kBlockM;
  constexpr int kStages = S::kStages;
  constexpr int kG = S::kG;
  constexpr int kElemsPerStageK = kFP8 ? 128 : 64;
  constexpr int kUmmaK = kFP8 ? 32 : 16;
  constexpr int kMmasPerStage = kElemsPerStageK / kUmmaK;     // 4
  // TMEM accumulator ring: block-scaled GEMMs hand one accumulator per K block to the epilogue, so they use the
  // deepest ring 512 columns allow (up to 4); plain GEMMs hand over one per tile and need two.
  constexpr int kAcc = kBlockScaled ? ((512 / BLOCK_N) > 4 ? 4 : (512 / BLOCK_N)) : 2;
  static_assert(!kHw || (kFP8 && !kBlockScaled && BLOCK_N <= 224), "hardware block scaling: fp8 operands, one accumulator per tile");
  static_assert(!kFp4 || BLOCK_N == 128, "NVFP4: 128-wide tiles");
  // kHw: the scale factors follow the accumulators.  Folded form: 4 columns of B's constant, then a ring of 4-column entries
  // for A.  Wide form: a ring of 12-column entries, 4 for A and 8 for B.
  constexpr bool kFold = BLOCK_N <= 128 && !kFp4;
  constexpr int kSfBufs = kFp4 ? 4 : (kFold ? 8 : 5);  // ring entries (one chunk of 4 K blocks each; NVFP4: a pair of K blocks each)
  constexpr int kSfGroup = kFold ? 4 : 2;              // chunks whose scales are fetched together
  constexpr uint32_t kSfEntry = kFp4 ? 64 : (kFold ? 4 : 12);
  constexpr uint32_t kSfbCol = kAcc * BLOCK_N, kSfaCol = kSfbCol + (kFold ? 4 : 0);
  constexpr uint32_t kColsUsed = kAcc * BLOCK_N + (kHw ? (kFold ? 4 : 0) + kSfEntry * kSfBufs : 0);
  static_assert(kColsUsed <= 512 && kSfBufs <= kSfBufsMax, "TMEM holds 512 columns");
  constexpr uint32_t kTmemCols = kColsUsed <= 32 ? 32 : (kColsUsed <= 64 ? 64 : (kColsUsed <= 128 ? 128 : (kColsUsed <= 256 ? 256 : 512)));
  constexpr uint32_t kIdesc = kFp4 ? make_idesc_block_scaled(FMT_E2M1_MXF4, FMT_E2M1_MXF4, kBlockM, BLOCK_N, 0)
                              : kHw ? make_idesc_block_scaled(FMT_E4M3, FMT_E4M3, kTileM, BLOCK_N)
                                  : make_idesc(kFP8 ? FMT_E4M3 : FMT_BF16, kFP8 ? FMT_E4M3 : FMT_BF16, kBlockM, BLOCK_N);
  constexpr int kEpi = EpiCfg<BLOCK_N, kBlockScaled>::kGroups;
  constexpr int kCols = BLOCK_N / kEpi;          // columns of the tile each epilogue thread owns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sf_ring = smem + kStages * S::kStageBytes;       // NVFP4 only (S::kSfRing bytes)
  uint8_t* staging = sf_ring + S::kSfRing;
  uint64_t* bars = reinterpret_cast<uint64_t*>(staging + S::kStaging);
  // bars: full[kStages], empty[kStages], tmem_full[kAcc], tmem_empty[kAcc]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 2 * kAcc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + kStages);
  const uint32_t tfull0 = smem_u32(bars + 2 * kStages), tempty0 = smem_u32(bars + 2 * kStages + kAcc);
  const uint32_t smem_base = smem_u32(smem);
  __shared__ uint64_t s_sfbar[2 * kSfBufsMax];            // kHw: scale-factor buffer filled (4 warps arrive) / drained (MMAs retired)
  const uint32_t sffull0 = smem_u32(s_sfbar), sfempty0 = smem_u32(s_sfbar + kSfBufs);

  const int warp = threadIdx.x >> 5;
  const int total_kb = (args.K + kElemsPerStageK - 1) / kElemsPerStageK;
  const int n_blocks = (args.N + BLOCK_N - 1) / BLOCK_N;
  const int split = kSplit ? (int)cluster_nctarank() : 1;
  const int srank = kSplit ? (int)cluster_ctarank() : 0;
  const int num_kb = total_kb / split;                 // the host picks a split that divides the K blocks
  const int num_st = (num_kb + kG - 1) / kG;           // pipeline stages' worth of K blocks per tile
  const int kb_begin = srank * num_kb;
  const int prank = kPair ? (int)cluster_ctarank() : 0;     // 0: the CTA of a pair that issues the MMAs
  const int tile0 = kSplit ? (int)blockIdx.x / split : (kPair ? (int)blockIdx.x / 2 : (int)blockIdx.x);
  const int tile_stride = kSplit ? (int)gridDim.x / split : (kPair ? (int)gridDim.x / 2 : (int)gridDim.x);
  // a barrier of the pair's first CTA, as seen from this one; arrivals there from either CTA
  auto lead = [&](uint32_t bar) { return kPair ? mapa_shared(bar, 0u) : bar; };
  auto arrive_lead = [&](uint32_t bar) { if (kPair && prank != 0) mbar_arrive_cluster(mapa_shared(bar, 0u)); else mbar_arrive(bar); };
  // completion of the MMAs issued so far, signalled to the same barrier of both CTAs
  auto commit = [&](uint32_t bar) { if (kPair) { tc_commit_pair(bar); tc_commit_pair(mapa_shared(bar, 1u)); } else tc_commit(bar); };

  // set-up that touches no global memory comes first: under a programmatic dependent launch it overlaps the previous kernel's tail
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; i++) { mbar_init(full0 + 8 * i, 1); mbar_init(empty0 + 8 * i, 1); }
    for (int i = 0; i < kAcc; i++) { mbar_init(tfull0 + 8 * i, 1); mbar_init(tempty0 + 8 * i, 4 * kEpi * (kPair ? 2 : 1)); }
    if (kHw) for (int i = 0; i < kSfBufs; i++) { mbar_init(sffull0 + 8 * i, kPair ? 8 : 4); mbar_init(sfempty0 + 8 * i, 1); }
    *abort_flag = 0;
    mbar_fence_init();
    tma_prefetch_desc(&tmap_a); tma_prefetch_desc(&tmap_a64); tma_prefetch_desc(&tmap_a32); tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    if (kPair) { tmem_alloc_pair(smem_u32(tmem_slot), kTmemCols); tmem_relinquish_pair(); }
    else { tmem_alloc(smem_u32(tmem_slot), kTmemCols); tmem_relinquish(); }
  }
  pdl_wait();                                          // from here on the previous kernel's results may be read, and ours written
  pdl_trigger();
  const GemmComm& cm = args.comm;
  // wait prologue: the operands of this GEMM (and its row counts) are being written by peer GPUs; their arrival flags are
  // local memory, polled by one thread each.  On expiry the status word is set and the row counts read as zero.
  __shared__ int s_wait_failed;
  if (cm.wait_flags) {
    if (threadIdx.x == 0) s_wait_failed = 0;
    __syncthreads();
    if ((int)threadIdx.x < cm.wait_world &&
        !wait_flag_ge(cm.wait_flags + threadIdx.x, *cm.wait_epoch + 1, kKernelGemm, 600 + (int)threadIdx.x, cm.wait_spin))
      s_wait_failed = 1;
    __syncthreads();
  }
  const bool wait_failed = cm.wait_flags && s_wait_failed;
  const int sc_parity = cm.scatter_epoch ? ((*cm.scatter_epoch + 1) & 1) : 0;
  // the per-group row tables are read once per tile by three roles: keep them in shared memory, a global load per
  // lookup sits on the producer's critical path at every tile switch
  __shared__ int s_mm[kSchedCache], s_rs[kSchedCache];
  const bool cache_tables = args.groups <= kSchedCache;
  if (cache_tables) {
    for (int i = threadIdx.x; i < args.groups; i += blockDim.x) {
      if (args.masked_m) s_mm[i] = wait_failed ? 0 : args.masked_m[i];
      if (args.row_start) s_rs[i] = args.row_start[i];
    }
  }
  const int* mm_tab = args.masked_m ? (cache_tables ? s_mm : args.masked_m) : nullptr;
  const int* rs_tab = args.row_start ? (cache_tables ? s_rs : args.row_start) : nullptr;
  // first tile of every ragged group: counts by all threads, then one warp turns them into running sums
  __shared__ int s_base[kSchedCache + 1];
  static_assert((3 * kSchedCache + 4) * (int)sizeof(int) + 16 * kSfBufsMax + 64 <= S::kStaticTables, "the stage budget must leave room for the static tables");
  const bool ragged = args.masked_m || args.row_start;
  const int* base_tab = (ragged && cache_tables) ? s_base : nullptr;
  if (base_tab) {
    __syncthreads();                                   // the row tables above are complete
    TileSched cnt(args.groups, args.M, n_blocks, mm_tab, rs_tab, nullptr, 0, kTileM, 0);
    for (int i = threadIdx.x; i < args.groups; i += blockDim.x) s_base[i + 1] = cnt.tiles_of(i);
    __syncthreads();
    if (warp == 2) {
      const int lane = (int)lane_id();
      const int per = (args.groups + 31) / 32, lo = lane * per, hi = min(lo + per, args.groups);
      int sum = 0;
      for (int i = lo; i < hi; i++) sum += s_base[i + 1];
      int incl = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) { const int v = __shfl_up_sync(0xffffffffu, incl, o); if (lane >= o) incl += v; }
      int run = incl - sum;                            // tiles before this lane's first group
      if (lane == 0) s_base[0] = 0;
      for (int i = lo; i < hi; i++) { run += s_base[i + 1]; s_base[i + 1] = run; }
    }
    // the __syncthreads that ends the prologue publishes the table
  }
  tc_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();          // the peer's barriers are initialised before anything is signalled to them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      TileSched sched(args.groups, args.M, n_blocks, mm_tab, rs_tab, base_tab, cm.mb_rot, kTileM, prank);
      int stage = 0; uint32_t phase = 0; int grp, mb, nb;
      bool ok = true;
      const int gate_ep = cm.gate_flags ? *cm.gate_epoch + 1 : 0;
      const int a_row_off = cm.gate_flags ? (gate_ep & 1) * cm.gate_parity_rows : 0;
      unsigned gate_seen = 0;
      if (cm.wait_flags) fence_proxy_async_all();      // peers' stores, observed through the flags, before the first TMA read
      for (int tile = tile0; ok && sched.get(tile, grp, mb, nb); tile += tile_stride) {
        if (cm.gate_flags) {
          // sources whose rows this tile reads; each is waited for once per CTA
          const int r_lo = mb * kBlockM, r_hi = min(r_lo + kBlockM, args.M) - 1;
          for (int sr = r_lo / cm.gate_rpr; sr <= r_hi / cm.gate_rpr && sr < cm.gate_world && ok; sr++) {
            if (gate_seen >> sr & 1u) continue;
            if (!wait_flag_ge(cm.gate_flags + sr, gate_ep, kKernelGemm, 700 + sr, cm.gate_spin)) { *abort_flag = 1; ok = false; break; }
            gate_seen |= 1u << sr;
            fence_proxy_async_all();
          }
          if (!ok) break;
        }
        // a tile with few valid rows (decode: a handful of tokens per expert) fetches only the first 32 or 64 rows of
        // the activation block; the MMA still spans 128 rows, whose stale remainder lands in output rows nobody stores
        const int rows_here = sched.rows(grp) - mb * kBlockM;
        const CUtensorMap* ta = kPair ? &tmap_a : (rows_here <= 32 ? &tmap_a32 : (rows_here <= 64 ? &tmap_a64 : &tmap_a));
        const uint32_t a_bytes = kPair ? S::kABytes : (rows_here <= 32 ? 32 * kKBytes : (rows_here <= 64 ? 64 * kKBytes : S::kABytes));
        for (int st = 0; st < num_st; st++) {
          if (!mbar_wait(empty0 + 8 * stage, phase ^ 1, abort_flag, kKernelGemm, 100 + stage)) { ok = false; break; }
          uint32_t a_dst = smem_base + stage * S::kStageBytes, b_dst = a_dst + kG * S::kABytes;
          const int kc = kb_begin + st * kG;
          if (kPair) {
            // both CTAs' bytes are counted on the first CTA's barrier, which alone announces them
            if (prank == 0) mbar_expect_tx(full0 + 8 * stage, 2 * kG * (S::kABytes + S::kBBytes));
            const uint32_t fb = lead(full0 + 8 * stage);
            tma_load_4d_pair(a_dst, ta, fb, 0, a_row_off + sched.row0(grp) + mb * kBlockM, args.row_start ? 0 : grp, kc);
            tma_load_4d_pair(b_dst, &tmap_b, fb, 0, nb * BLOCK_N + prank * (BLOCK_N / 2), grp, kc);
            if (++stage == kStages) { stage = 0; phase ^= 1; }
            continue;
          }
          mbar_expect_tx(full0 + 8 * stage, kG * (a_bytes + S::kBBytes));      // chunks past the end of K arrive as zeros
          if (!args.k_flat) {
            if (args.a_group_inner) tma_load_4d(a_dst, ta, full0 + 8 * stage, 0, grp, mb * kBlockM, kc);
            else tma_load_4d(a_dst, ta, full0 + 8 * stage, 0, a_row_off + sched.row0(grp) + mb * kBlockM, args.row_start ? 0 : grp, kc);
            tma_load_4d(b_dst, &tmap_b, full0 + 8 * stage, 0, nb * BLOCK_N, grp, kc);
          } else {
#pragma unroll
            for (int g = 0; g < kG; g++) {
              const int kx = (kc + g) * kElemsPerStageK;           // past the end of K: the whole box is zero-filled
              if (args.a_group_inner) tma_load_4d(a_dst + g * a_bytes, ta, full0 + 8 * stage, kx, grp, mb * kBlockM, 0);
              else tma_load_4d(a_dst + g * a_bytes, ta, full0 + 8 * stage, kx, a_row_off + sched.row0(grp) + mb * kBlockM, args.row_start ? 0 : grp, 0);
              tma_load_4d(b_dst + g * S::kBBytes, &tmap_b, full0 + 8 * stage, kx, nb * BLOCK_N, grp, 0);
            }
          }
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if ((!kPair || prank == 0) && elect_one()) {
      TileSched sched(args.groups, args.M, n_blocks, mm_tab, rs_tab, base_tab, cm.mb_rot, kTileM, prank);
      int stage = 0; uint32_t phase = 0; int buf = 0; uint32_t bphase = 0; int grp, mb, nb;
      bool ok = true;
      // A test of an mbarrier costs ~150 cycles even when the phase has long completed, and this thread is the serial
      // resource of the CTA.  So the barriers of the NEXT K block are tested before the MMAs of the current one are issued
      // (the issue blocks for about as long as the MMAs run, which hides the test); only a failed test falls back to waiting.
      bool pre_full = mbar_test(full0 + 8 * stage, phase);
      bool pre_te = mbar_test(tempty0 + 8 * buf, bphase ^ 1);
      int sfb = 0; uint32_t sfphase = 0;                // kHw: scale-factor buffer in use and its phase
      bool pre_sf = false;
      for (int tile = tile0; ok && sched.get(tile, grp, mb, nb); tile += tile_stride) {
        if (!kBlockScaled) {
          if (!pre_te && !mbar_wait(tempty0 + 8 * buf, bphase ^ 1, abort_flag, kKernelGemm, 200 + buf)) { ok = false; break; }
          tc_fence_after();
        }
        // the activation box of this tile (see the producer): its K blocks sit a_kstride apart inside the stage
        const int rows_here = sched.rows(grp) - mb * kBlockM;
        const uint32_t a_kstride = kPair ? S::kABytes : (rows_here <= 32 ? 32 * kKBytes : (rows_here <= 64 ? 64 * kKBytes : S::kABytes));
        for (int st = 0; st < num_st && ok; st++) {
          if (!pre_full && !mbar_wait(full0 + 8 * stage, phase, abort_flag, kKernelGemm, 300 + stage)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_base + stage * S::kStageBytes, b_base = a_base + kG * S::kABytes;
          const int nstage = stage + 1 == kStages ? 0 : stage + 1;
          const uint32_t nphase = stage + 1 == kStages ? phase ^ 1 : phase;
#pragma unroll
          for (int g = 0; g < kG; g++) {
            const int kb = st * kG + g;
            if (kb >= num_kb) break;
            if (kBlockScaled) {
              if (!pre_te && !mbar_wait(tempty0 + 8 * buf, bphase ^ 1, abort_flag, kKernelGemm, 210 + buf)) { ok = false; break; }
              tc_fence_after();
            }
            // tests for what comes next, issued ahead of this K block's MMAs
            if (kBlockScaled) {
              const int nbuf = buf + 1 == kAcc ? 0 : buf + 1;
              pre_te = mbar_test(tempty0 + 8 * nbuf, (buf + 1 == kAcc ? bphase ^ 1 : bphase) ^ 1);
            }
            if (g == kG - 1 || kb + 1 >= num_kb) pre_full = mbar_test(full0 + 8 * nstage, nphase);
            if (kHw && (kFp4 ? (kb & 1) == 0 : (kb & 3) == 0)) {
              // a new chunk of four K blocks: its scale factors must be in TMEM
              if (!pre_sf && !mbar_wait(sffull0 + 8 * sfb, sfphase, abort_flag, kKernelGemm, 500 + sfb)) { ok = false; break; }
              tc_fence_after();
            }
            const bool chunk_end = kHw && ((kFp4 ? (kb & 1) == 1 : (kb & 3) == 3) || kb + 1 >= num_kb);
            if (chunk_end) {
              const int nsf = sfb + 1 == kSfBufs ? 0 : sfb + 1;
              pre_sf = mbar_test(sffull0 + 8 * nsf, sfb + 1 == kSfBufs ? sfphase ^ 1 : sfphase);
            }
            uint64_t adesc = make_smem_desc(a_base + g * a_kstride, 16, 1024, SW_128B);
            uint64_t bdesc = make_smem_desc(b_base + g * S::kBBytes, 16, 1024, SW_128B);
            uint32_t d = tmem_base + buf * BLOCK_N;
#pragma unroll
            for (int k = 0; k < kMmasPerStage; k++) {
              uint32_t acc = kBlockScaled ? (k != 0) : ((kb | k) != 0);
              // advancing 32 bytes along K inside the 128B swizzle atom = +2 in the descriptor's 16-byte address units
              if (kFp4) umma_nvfp4_block_scaled(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc, tmem_base + kSfaCol + kSfEntry * sfb + 32 * (kb & 1) + 4 * k,
                                                tmem_base + kSfaCol + kSfEntry * sfb + 32 * (kb & 1) + 16 + 4 * k);
              else if (kPair) umma_f8_block_scaled_pair(d, adesc + 2 * k, bdesc + 2 * k,
                                            kIdesc | ((uint32_t)(kb & 3) << 29) | (kFold ? 0u : (uint32_t)(kb & 3) << 4), acc,
                                            tmem_base + kSfaCol + kSfEntry * sfb, tmem_base + (kFold ? kSfbCol : kSfaCol + kSfEntry * sfb + 4));
              else if (kHw) umma_f8_block_scaled(d, adesc + 2 * k, bdesc + 2 * k,
                                            kIdesc | ((uint32_t)(kb & 3) << 29) | (kFold ? 0u : (uint32_t)(kb & 3) << 4), acc,
                                            tmem_base + kSfaCol + kSfEntry * sfb, tmem_base + (kFold ? kSfbCol : kSfaCol + kSfEntry * sfb + 4));
              else if (kFP8) umma_f8(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
              else umma_f16(d, adesc + 2 * k, bdesc + 2 * k, kIdesc, acc);
            }
            if (chunk_end) { commit(sfempty0 + 8 * sfb); if (++sfb == kSfBufs) { sfb = 0; sfphase ^= 1; } }
            if (kBlockScaled) { tc_commit(tfull0 + 8 * buf); if (++buf == kAcc) { buf = 0; bphase ^= 1; } }
          }
          commit(empty0 + 8 * stage);                   // smem slot reusable once these MMAs retire
          if (++stage == kStages) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        if (!kBlockScaled) {
          commit(tfull0 + 8 * buf);
          if (++buf == kAcc) { buf = 0; bphase ^= 1; }
          pre_te = mbar_test(tempty0 + 8 * buf, bphase ^ 1);
        }
      }
    }
  } else if (kFp4 && warp >= 2 + 4 * kEpi) {
    // ---------------- NVFP4 scale-factor warps ----------------
    const int lane = (int)lane_id(), wq = warp & 3;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const uint32_t ring0 = smem_u32(sf_ring);
    const long long sf_ld = args.K / 8;                 // scale bytes per operand row (args.K counts bytes of packed e2m1)
    const uint8_t* sfa_all = reinterpret_cast<const uint8_t*>(args.sa);
    const uint8_t* sfb_all = reinterpret_cast<const uint8_t*>(args.sb);
    // The copies run kAhead K blocks ahead of the stores, across tile boundaries (a second tile walker); the stores go pair by
    // pair of K blocks (one barrier among the four warps, one TMEM ring entry, one arrival per pair).  The ring has two slots
    // more than are in flight: the slots a pair's copies take were read one barrier earlier by every warp.
    constexpr int kAhead = kFp4SfSlots - 2;
    TileSched sched(args.groups, args.M, n_blocks, mm_tab, rs_tab, base_tab, cm.mb_rot, kTileM, prank);
    TileSched sched_i(args.groups, args.M, n_blocks, mm_tab, rs_tab, base_tab, cm.mb_rot, kTileM, prank);
    int sfb = 0; uint32_t sfphase = 0; int grp, mb, nb;
    bool ok = true;                                      // a wait that ran out clears it; the warp keeps walking (its peers count on it at the barrier)
    int slot_w = 0, slot_r = 0;                          // ring slots written (copies issued) / read
    int tile_i = tile0, kb_i = 0, grp_i, mb_i, nb_i;
    bool live_i = sched_i.get(tile_i, grp_i, mb_i, nb_i);
    const uint8_t *pa_i = nullptr, *pb_i = nullptr;
    auto point = [&]() {
      // this warp copies rows / columns 32 wq + lane of the tile; rows past the end read the tile's first row, columns past N the last
      const int rows_here = sched_i.rows(grp_i) - mb_i * kBlockM;
      const int ar = 32 * wq + lane < rows_here ? 32 * wq + lane : 0;
      const int bc = min(nb_i * BLOCK_N + 32 * wq + lane, args.N - 1);
      pa_i = sfa_all + ((long long)grp_i * args.sa_group_stride + sched_i.row0(grp_i) + mb_i * kBlockM + ar) * sf_ld + (long long)kb_begin * 16;
      pb_i = sfb_all + ((long long)grp_i * args.N + bc) * sf_ld + (long long)kb_begin * 16;
    };
    if (live_i) point();
    auto issue = [&]() {
      if (live_i) {
        const uint32_t dst = ring0 + slot_w * 4096 + (wq * 32 + lane) * 16;
        cp_async16(dst, pa_i + (long long)kb_i * 16, 16u);
        cp_async16(dst + 2048, pb_i + (long long)kb_i * 16, 16u);
        if (++slot_w == kFp4SfSlots) slot_w = 0;
        if (++kb_i == num_kb) {
          kb_i = 0; tile_i += tile_stride;
          live_i = sched_i.get(tile_i, grp_i, mb_i, nb_i);
          if (live_i) point();
        }
      }
      cp_async_commit();                               // one group per K block, empty past the last tile: the waits below count groups
    };
    for (int i = 0; i < kAhead; i++) issue();
    for (int tile = tile0; sched.get(tile, grp, mb, nb); tile += tile_stride) {
      for (int kb0 = 0; kb0 < num_kb; kb0 += 2) {
        const bool two = kb0 + 1 < num_kb;
        if (two) cp_async_wait<kAhead - 2>(); else cp_async_wait<kAhead - 1>();      // this warp's copies of the pair have landed
        named_bar_sync(1, 128);                        // ... and the other three warps'
        uint32_t w0a[16], w0b[16], w1a[16], w1b[16];
        {
          const uint4* src = reinterpret_cast<const uint4*>(sf_ring + slot_r * 4096) + lane;
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const uint4 va = src[g * 32], vb = src[128 + g * 32];
            w0a[g] = va.x; w0a[4 + g] = va.y; w0a[8 + g] = va.z; w0a[12 + g] = va.w;
            w0b[g] = vb.x; w0b[4 + g] = vb.y; w0b[8 + g] = vb.z; w0b[12 + g] = vb.w;
          }
          if (++slot_r == kFp4SfSlots) slot_r = 0;
        }
        if (two) {
          const uint4* src = reinterpret_cast<const uint4*>(sf_ring + slot_r * 4096) + lane;
#pragma unroll
          for (int g = 0; g < 4; g++) {
            const uint4 va = src[g * 32], vb = src[128 + g * 32];
            w1a[g] = va.x; w1a[4 + g] = va.y; w1a[8 + g] = va.z; w1a[12 + g] = va.w;
            w1b[g] = vb.x; w1b[4 + g] = vb.y; w1b[8 + g] = vb.z; w1b[12 + g] = vb.w;
          }
          if (++slot_r == kFp4SfSlots) slot_r = 0;
        }
        issue();
        if (two) issue();
        if (ok && mbar_wait(sfempty0 + 8 * sfb, sfphase ^ 1, abort_flag, kKernelGemm, 520 + sfb)) {
          tc_fence_after();
          const uint32_t ent = tmem_base + lane_addr + kSfaCol + kSfEntry * sfb;
          tmem_st_32x32b_x16(ent, w0a);
          tmem_st_32x32b_x16(ent + 16, w0b);
          if (two) {
            tmem_st_32x32b_x16(ent + 32, w1a);
            tmem_st_32x32b_x16(ent + 48, w1b);
          }
          tc_wait_st();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(sffull0 + 8 * sfb);
          if (++sfb == kSfBufs) { sfb = 0; sfphase ^= 1; }
        } else {
          ok = false;
        }
      }
    }
    cp_async_wait<0>();
  } else if (kHw && warp >= 2 + 4 * kEpi) {
    // ---------------- scale-factor warps: warp w fills TMEM lanes [32*(w%4), +32) ----------------
    const int lane = (int)lane_id();
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    TileSched sched(args.groups, args.M, n_blocks, mm_tab, rs_tab, base_tab, cm.mb_rot, kTileM, prank);
    int sfb = 0; uint32_t sfphase = 0; int grp, mb, nb;
    bool ok = true, first = true;
    for (int tile = tile0; ok && sched.get(tile, grp, mb, nb); tile += tile_stride) {
      if (first && kFold) {
        // B's scale factors: the constant 1 (UE8M0 byte 127), written once
        const uint32_t ones[4] = {0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu, 0x7f7f7f7fu};
        tmem_st_32x32b_x4(tmem_base + lane_addr + kSfbCol, ones);
      }
      first = false;
      // rows lane + 32 g of the tile; rows past the group's end read the tile's first row (their results are never stored)
      const int rows_here = sched.rows(grp) - mb * kBlockM;
      // (a pair's second CTA may stand past the group's last row: it reads the group's first row instead)
      const float* sa = args.sa + (long long)grp * args.sa_group_stride + sched.row0(grp) + (rows_here > 0 ? mb * kBlockM : 0) + (long long)kb_begin * args.sa_ld;
      // weight blocks under the tile: one when folded, up to three under a wide tile
      constexpr int kNB = kFold ? 1 : 3;
      const int nblk = (args.N + 127) / 128, b0 = nb * BLOCK_N / 128;
      const float* sb[kNB];
#pragma unroll
      for (int i = 0; i < kNB; i++)
        sb[i] = args.sb + (long long)grp * args.sb_group_stride + (long long)min(b0 + i, nblk - 1) * total_kb + kb_begin;
      int roff[4], bsel[8];
#pragma unroll
      for (int g = 0; g < 4; g++) roff[g] = lane + 32 * g < rows_here ? lane + 32 * g : 0;
#pragma unroll
      for (int g = 0; g < 8; g++) bsel[g] = kFold ? 0 : min((nb * BLOCK_N + lane + 32 * g) / 128 - b0, kNB - 1);
      // The scale arrays are read kSfGroup chunks at a time, and the loads of the next batch are in flight while this one is
      // converted and stored: a single chunk per round trip to L2 (about a microsecond) would feed the tensor pipe at half
      // the rate it consumes them.
      const int n_chunks = (num_kb + 3) >> 2;
      uint32_t ra[kSfGroup][4][4], rb[kSfGroup][4][kNB];    // raw bits: [chunk][K block][row group], [chunk][K block][weight block]
      auto fetch = [&](int c0) {
#pragma unroll
        for (int u = 0; u < kSfGroup; u++) {
#pragma unroll
          for (int j = 0; j < 4; j++) {
            const int kb = (c0 + u) * 4 + j;
            const bool in = kb < num_kb;
#pragma unroll
            for (int i = 0; i < kNB; i++) rb[u][j][i] = in ? __float_as_uint(__ldg(sb[i] + kb)) : 0u;
#pragma unroll
            for (int g = 0; g < 4; g++) ra[u][j][g] = in ? __float_as_uint(__ldg(sa + (long long)kb * args.sa_ld + roff[g])) : 0u;
          }
        }
      };
      fetch(0);
      for (int c0 = 0; c0 < n_chunks && ok; c0 += kSfGroup) {
        uint32_t w[kSfGroup][4], wb[kSfGroup][8];
#pragma unroll
        for (int u = 0; u < kSfGroup; u++) {
#pragma unroll
          for (int g = 0; g < 4; g++) {
            uint32_t word = 0u;
#pragma unroll
            for (int j = 0; j < 4; j++) {
              const int e = (int)((ra[u][j][g] >> 23) & 0xffu) + (kFold ? (int)((rb[u][j][0] >> 23) & 0xffu) - 127 : 0);
              word |= (uint32_t)min(max(e, 0), 254) << (8 * j);
            }
            w[u][g] = word;
          }
          if (!kFold) {
#pragma unroll
            for (int g = 0; g < 8; g++) {
              uint32_t word = 0u;
#pragma unroll
              for (int j = 0; j < 4; j++) {
                const uint32_t bits = bsel[g] == 0 ? rb[u][j][0] : (bsel[g] == 1 ? rb[u][j][kNB > 1 ? 1 : 0] : rb[u][j][kNB - 1]);
                word |= min((bits >> 23) & 0xffu, 254u) << (8 * j);
              }
              wb[u][g] = word;
            }
          }
        }
        if (c0 + kSfGroup < n_chunks) fetch(c0 + kSfGroup);
#pragma unroll
        for (int u = 0; u < kSfGroup; u++) {
          if (c0 + u < n_chunks && ok) {
            if (mbar_wait(sfempty0 + 8 * sfb, sfphase ^ 1, abort_flag, kKernelGemm, 510 + sfb)) {
              tc_fence_after();
              tmem_st_32x32b_x4(tmem_base + lane_addr + kSfaCol + kSfEntry * sfb, w[u]);
              if (!kFold) tmem_st_32x32b_x8(tmem_base + lane_addr + kSfaCol + kSfEntry * sfb + 4, wb[u]);
              tc_wait_st();
              tc_fence_before();
              __syncwarp();
              if (lane == 0) arrive_lead(sffull0 + 8 * sfb);
              if (++sfb == kSfBufs) { sfb = 0; sfphase ^= 1; }
            } else {
              ok = false;
            }
          }
        }
      }
    }
  } else {
    // ---------------- epilogue: 4 warps per group, warp w may touch TMEM lanes [32*(w%4), +32) ----------------
    const int wq = warp & 3;
    const int cbase = ((warp - 2) >> 2) * kCols;   // column offset of this warp's group inside the tile
    const int row_in_tile = wq * 32 + (int)lane_id();
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    TileSched sched(args.groups, args.M, n_blocks, mm_tab, rs_tab, base_tab, cm.mb_rot, kTileM, prank);
    int buf = 0; uint32_t bphase = 0; int grp, mb, nb;
    bool ok = true;
    bool pre_tf = false;                               // result of an early test of the next accumulator's "full" barrier
    for (int tile = tile0; ok && sched.get(tile, grp, mb, nb); tile += tile_stride) {
      const bool row_ok = mb * kBlockM + row_in_tile < sched.rows(grp);
      const int row = sched.row0(grp) + mb * kBlockM + row_in_tile;      // row inside the group's (or the flat) matrix
      const int n0 = nb * BLOCK_N;
      if (kBlockScaled) {
        float acc[kCols];
#pragma unroll
        for (int j = 0; j < kCols; j++) acc[j] = 0.f;
        const float* sa = args.sa + (long long)grp * args.sa_group_stride + (row_ok ? row : 0) + (long long)kb_begin * args.sa_ld;
        const float* sb = args.sb + (long long)grp * args.sb_group_stride + (long long)(n0 / 128) * total_kb + kb_begin;
        // scale factors are fetched four K blocks ahead so their L2 latency hides behind the promotion work
        constexpr int kPf = 4;
        float nxt[kPf];
#pragma unroll
        for (int j = 0; j < kPf; j++) nxt[j] = j < num_kb ? __ldg(sa + (long long)j * args.sa_ld) * __ldg(sb + j) : 0.f;
        for (int kb0 = 0; kb0 < num_kb && ok; kb0 += kPf) {
          float cur[kPf];
#pragma unroll
          for (int j = 0; j < kPf; j++) {
            cur[j] = nxt[j];
            const int kn = kb0 + kPf + j;
            nxt[j] = kn < num_kb ? __ldg(sa + (long long)kn * args.sa_ld) * __ldg(sb + kn) : 0.f;
          }
#pragma unroll
        for (int jj = 0; jj < kPf; jj++) {
          if (kb0 + jj >= num_kb || !ok) break;
          const float s = cur[jj];
          if (!pre_tf && !mbar_wait(tfull0 + 8 * buf, bphase, abort_flag, kKernelGemm, 400 + buf)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int c = 0; c < kCols / 32; c += 2) {
            // two TMEM loads in flight per wait
            uint32_t r0[32], r1[32];
            tmem_ld_32x32b_x32(tmem_base + lane_addr + buf * BLOCK_N + cbase + c * 32, r0);
            if (c + 1 < kCols / 32) tmem_ld_32x32b_x32(tmem_base + lane_addr + buf * BLOCK_N + cbase + (c + 1) * 32, r1);
            // the next accumulator's barrier is tested while the loads and the promotion of this one are in flight
            if (c == 0) pre_tf = mbar_test(tfull0 + 8 * (buf + 1 == kAcc ? 0 : buf + 1), buf + 1 == kAcc ? bphase ^ 1 : bphase);
            tc_wait_ld();
#pragma unroll
            for (int j = 0; j < 32; j++) acc[c * 32 + j] = fmaf(s, __uint_as_float(r0[j]), acc[c * 32 + j]);
            if (c + 1 < kCols / 32) {
#pragma unroll
              for (int j = 0; j < 32; j++) acc[(c + 1) * 32 + j] = fmaf(s, __uint_as_float(r1[j]), acc[(c + 1) * 32 + j]);
            }
          }
          tc_fence_before();
          __syncwarp();
          if (lane_id() == 0) mbar_arrive(tempty0 + 8 * buf);
          if (++buf == kAcc) { buf = 0; bphase ^= 1; }
        }
        }
        if (!ok) break;
        if (kSplit) {
          // park the partial tile: [128 rows][BLOCK_N / 4 chunks of 16 bytes], chunk index xor-ed with the row so the
          // 32 rows a warp writes at once land in different banks
          float4* P = reinterpret_cast<float4*>(smem);
#pragma unroll
          for (int c4 = 0; c4 < kCols / 4; c4++) {
            const int chunk = cbase / 4 + c4;
            P[row_in_tile * (BLOCK_N / 4) + (chunk ^ (row_in_tile & 7))] = make_float4(acc[c4 * 4], acc[c4 * 4 + 1], acc[c4 * 4 + 2], acc[c4 * 4 + 3]);
          }
        } else {
          const long long off = (long long)grp * args.d_group_stride + (long long)row * args.ldd + n0 + cbase;
          if (args.out_fp32) {
            if (row_ok) {
#pragma unroll
              for (int c = 0; c < kCols / 8; c++) {
                if (n0 + cbase + c * 8 < args.N) {
                  float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(args.D) + off + c * 8);
                  p[0] = make_float4(acc[c * 8], acc[c * 8 + 1], acc[c * 8 + 2], acc[c * 8 + 3]);
                  p[1] = make_float4(acc[c * 8 + 4], acc[c * 8 + 5], acc[c * 8 + 6], acc[c * 8 + 7]);
                }
              }
            }
          } else {
            __nv_bfloat16* dbf = scatter_row(args, grp, row, row_ok, sc_parity, reinterpret_cast<__nv_bfloat16*>(args.D) + off - n0 - cbase) + n0 + cbase;
            uint8_t* stg = staging + (warp - 2) * kStgWarpBytes;
            const EpiRows erows = epi_rows(row_ok, dbf);
#pragma unroll
            for (int cc = 0; cc < kCols / 32; cc++) {
              float v[32];
#pragma unroll
              for (int j = 0; j < 32; j++) v[j] = acc[cc * 32 + j];
              epi_store32_bf16(stg, v, erows, cc * 32, args.N - (n0 + cbase + cc * 32));
            }
          }
        }
      } else {
        if (!mbar_wait(tfull0 + 8 * buf, bphase, abort_flag, kKernelGemm, 410 + buf)) { ok = false; break; }
        tc_fence_after();
        long long off = (long long)grp * args.d_group_stride + (long long)row * args.ldd + n0;
        __nv_bfloat16* dbf = scatter_row(args, grp, row, row_ok, sc_parity, reinterpret_cast<__nv_bfloat16*>(args.D) + off - n0) + n0;
        EpiRows erows;
        if (!kSplit && args.out_fp32 == 0) erows = epi_rows(row_ok, dbf);
        const float al = args.alpha ? __ldg(args.alpha + grp) : 1.f;
#pragma unroll
        for (int c = 0; c < BLOCK_N / 32; c++) {
          uint32_t r[32];
          tmem_ld_32x32b_x32(tmem_base + lane_addr + buf * BLOCK_N + c * 32, r);
          tc_wait_ld();
          if (kFp4) {
#pragma unroll
            for (int j = 0; j < 32; j++) r[j] = __float_as_uint(__uint_as_float(r[j]) * al);
          }
          if (kSplit) {
            float4* P = reinterpret_cast<float4*>(smem);
#pragma unroll
            for (int q = 0; q < 8; q++)
              P[row_in_tile * (BLOCK_N / 4) + ((c * 8 + q) ^ (row_in_tile & 7))] =
                  make_float4(__uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]), __uint_as_float(r[q * 4 + 3]));
          } else if (args.out_fp32 == 2) {
            // 32 columns = 32 bytes of this thread's row: one full sector, written straight from registers
            if (row_ok && n0 + c * 32 < args.N) {
              uint4* p = reinterpret_cast<uint4*>(reinterpret_cast<uint8_t*>(args.D) + off + c * 32);
              uint32_t w[8];
#pragma unroll
              for (int q = 0; q < 8; q++)
                w[q] = pack_e4m3x4(__uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]), __uint_as_float(r[q * 4 + 3]));
              p[0] = make_uint4(w[0], w[1], w[2], w[3]);
              p[1] = make_uint4(w[4], w[5], w[6], w[7]);
            }
          } else if (args.out_fp32) {
            if (row_ok) {
#pragma unroll
              for (int q = 0; q < 4; q++) {
                if (n0 + c * 32 + q * 8 < args.N) {
                  float4* p = reinterpret_cast<float4*>(reinterpret_cast<float*>(args.D) + off + c * 32 + q * 8);
                  p[0] = make_float4(__uint_as_float(r[q * 8]), __uint_as_float(r[q * 8 + 1]), __uint_as_float(r[q * 8 + 2]), __uint_as_float(r[q * 8 + 3]));
                  p[1] = make_float4(__uint_as_float(r[q * 8 + 4]), __uint_as_float(r[q * 8 + 5]), __uint_as_float(r[q * 8 + 6]), __uint_as_float(r[q * 8 + 7]));
                }
              }
            }
          } else {
            float v[32];
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]);
            epi_store32_bf16(staging + (warp - 2) * kStgWarpBytes, v, erows, c * 32, args.N - (n0 + c * 32));
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane_id() == 0) arrive_lead(tempty0 + 8 * buf);
        if (++buf == kAcc) { buf = 0; bphase ^= 1; }
      }
    }
  }

  if (kSplit) {
    // ---------------- cross-CTA reduction of the partial tiles ----------------
    cluster_sync_all();
    if (warp >= 2 && warp < 2 + 4 * kEpi) {
      const int mb = tile0 / n_blocks, nb = tile0 % n_blocks;      // split-K runs single-row-block GEMMs: no rotation to apply
      const int R = (kBlockM + split - 1) / split;
      constexpr int kChunks = BLOCK_N / 4;
      const int nthr = 128 * kEpi, te = (int)threadIdx.x - 64;
      for (int item = te; item < R * kChunks; item += nthr) {
        const int r = srank * R + item / kChunks, chunk = item % kChunks;
        const int grow = mb * kBlockM + r, n = nb * BLOCK_N + chunk * 4;
        if (r >= kBlockM || grow >= args.M || n >= args.N) continue;
        const uint32_t local = smem_base + (uint32_t)(r * kChunks + (chunk ^ (r & 7))) * 16u;
        float4 s4 = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int pr = 0; pr < split; pr++) {
          const float4 v = ld_dsmem_f4(mapa_shared(local, (uint32_t)pr));
          s4.x += v.x; s4.y += v.y; s4.z += v.z; s4.w += v.w;
        }
        const long long off = (long long)grow * args.ldd + n;
        if (args.out_fp32) *reinterpret_cast<float4*>(reinterpret_cast<float*>(args.D) + off) = s4;
        else *reinterpret_cast<uint2*>(scatter_row(args, 0, grow, true, sc_parity, reinterpret_cast<__nv_bfloat16*>(args.D) + (long long)grow * args.ldd) + n) =
            make_uint2(pack_bf16x2(s4.x, s4.y), pack_bf16x2(s4.z, s4.w));
      }
    }
    cluster_sync_all();           // nobody leaves while a peer may still read its partial tile
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (*abort_flag && threadIdx.x == 0) {
    // give copies still in flight time to land before the shared memory is handed back
    for (int i = 0; i < 2000; i++) __nanosleep(1000);
  }
  __syncthreads();
  if (kPair) cluster_sync_all();          // neither CTA frees its TMEM or leaves while the other may still signal it or read its tiles
  if (warp == 1) {
    tc_fence_after();
    if (kPair) tmem_dealloc_pair(tmem_base, kTmemCols); else tmem_dealloc(tmem_base, kTmemCols);
  }
  if (cm.tail_counter) {
    // every thread orders its own (possibly peer-memory) stores before the count; the CTA that counts last speaks for the grid
    __threadfence_system();
    __syncthreads();
    __shared__ int s_last;
    if (threadIdx.x == 0) s_last = (atomicAdd(cm.tail_counter, 1) == (int)gridDim.x - 1) ? 1 : 0;
    __syncthreads();
    if (s_last) {
      const int ep = *cm.tail_epoch + 1;
      for (int i = threadIdx.x; i < cm.tail_clear_n; i += blockDim.x) cm.tail_clear[i] = 0;
      __threadfence_system();
      __syncthreads();
      if ((int)threadIdx.x < cm.tail_world) st_release_sys(reinterpret_cast<int*>(cm.tail_flag[threadIdx.x]), ep);
      if (threadIdx.x == 0) { *cm.tail_counter = 0; if (cm.tail_advance) *cm.tail_advance += 1; }
    }
  }
}

// ---- host side ---------------------------------------------------------------------------------
struct TmapKey {
  const void* p; uint64_t d0, d1, d2, s1, s2; uint32_t b0, b1; int dt;
  bool operator==(const TmapKey& o) const {
    return p == o.p && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && s1 == o.s1 && s2 == o.s2 && b0 == o.b0 && b1 == o.b1 && dt == o.dt;
  }
};
struct TmapKeyHash {
  size_t operator()(const TmapKey& k) const {
    size_t h = (size_t)k.p;
    for (uint64_t v : {k.d0, k.d1, k.d2, k.s1, k.s2, (uint64_t)k.b0, (uint64_t)k.b1, (uint64_t)k.dt}) h = h * 1000003u ^ (size_t)v;
    return h;
  }
};

// [groups][rows][K] K-major tensor -> 4-D map {128 bytes of K, rows, groups, K chunk} with box {128 B, box_rows, 1, kG}
// (kG = K blocks per pipeline stage of the kernel that will use the map) and 128B swizzle; K in bytes must be a multiple of 128.  The chunk dimension's stride (128 B) is smaller than the row
// stride, which the encoder accepts.
static int get_tmap_kmajor(CUtensorMap* out, const void* base, bool fp8, uint64_t K, uint64_t rows, uint64_t groups,
                           uint64_t row_stride_elems, uint64_t group_stride_elems, uint32_t box_rows, int kg) {
  const bool flat = (K * (fp8 ? 1 : 2)) % kKBytes != 0;       // see GemmArgs::k_flat
  if (flat) kg = 1;
  static std::mutex mu;
  static std::unordered_map<TmapKey, CUtensorMap, TmapKeyHash> cache;
  const uint64_t es = fp8 ? 1 : 2;
  TmapKey key{base, K, rows, groups, row_stride_elems * es, group_stride_elems * es, (uint32_t)(kKBytes / es), box_rows | ((uint32_t)kg << 16) | (flat ? 1u << 24 : 0u), fp8 ? TMA_U8 : TMA_BF16};
  std::lock_guard<std::mutex> lk(mu);
  auto it = cache.find(key);
  if (it != cache.end()) { *out = it->second; return 0; }
  uint64_t dims[4] = {flat ? K : kKBytes / es, rows, groups, flat ? 1 : K * es / kKBytes};
  uint64_t strides[3] = {row_stride_elems * es, group_stride_elems * es, (uint64_t)kKBytes};
  uint32_t box[4] = {(uint32_t)(kKBytes / es), box_rows, 1, (uint32_t)kg};
  if (groups > 1 && group_stride_elems < row_stride_elems) {
    // heads interleaved inside a row ([rows, groups, K] memory order): groups become the faster dimension, the kernel swaps coordinates
    dims[1] = groups; dims[2] = rows; strides[0] = group_stride_elems * es; strides[1] = row_stride_elems * es;
    box[1] = 1; box[2] = box_rows;
  }
  if (groups == 1) strides[1] = rows * row_stride_elems * es;      // unused, but must be a legal stride
  int rc = make_tmap(out, base, fp8 ? TMA_U8 : TMA_BF16, 4, dims, strides, box, TMA_SW_128);
  if (rc == 0) { if (cache.size() > 8192) cache.clear(); cache.emplace(key, *out); }
  return rc;
}

static bool g_split_k_enabled = true;
static bool g_pair_enabled = true;

static int num_sms() {
  static int n = 0;
  if (!n) { int dev; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev); }
  return n;
}

template <int BLOCK_N, bool kFP8, bool kBS, int kMode = 0>
static int launch(const CUtensorMap* tas, const CUtensorMap& tb, const GemmArgs& a, int grid, cudaStream_t st) {
  auto kern = gemm_kernel<BLOCK_N, kFP8, kBS, false, kMode>;
  using S = Smem<BLOCK_N, kMode == 2>;
  constexpr bool kHw = kMode != 0;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return (int)launch_pdl(kern, dim3((unsigned)grid), dim3(EpiCfg<BLOCK_N, kBS, kHw>::kThreads), S::kBytes, st, tas[0], tas[1], tas[2], tb, a);
}

// CTA-pair form of the tensor-core-scaled fp8 GEMM: clusters of two CTAs, one 256-row tile per pair
template <int BLOCK_N>
static int launch_pair(const CUtensorMap* tas, const CUtensorMap& tb, const GemmArgs& a, int pairs, cudaStream_t st) {
  auto kern = gemm_kernel<BLOCK_N, true, false, false, 1, true>;
  using S = Smem<BLOCK_N, false, true>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(pairs * 2), 1, 1);
  cfg.blockDim = dim3(EpiCfg<BLOCK_N, false, true>::kThreads, 1, 1);
  cfg.dynamicSmemBytes = S::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  // one pair per two SMs that can host a cluster: asked of the driver once (74 on a B200; 72 if it does not say)
  static int resident = 0;
  if (!resident) {
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    resident = (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) == cudaSuccess && n > 0) ? n : (num_sms() / 16) * 8;
  }
  if (pairs > resident) pairs = resident;
  cfg.gridDim = dim3((unsigned)(pairs * 2), 1, 1);
  pdl_attr(cfg, attr, 1);
  return (int)cudaLaunchKernelEx(&cfg, kern, tas[0], tas[1], tas[2], tb, a);
}

// split-K form: `tiles` clusters of `split` CTAs
template <int BLOCK_N, bool kFP8, bool kBS>
static int launch_split(const CUtensorMap* tas, const CUtensorMap& tb, const GemmArgs& a, int tiles, int split, cudaStream_t st) {
  constexpr bool kHw = false;
  auto kern = gemm_kernel<BLOCK_N, kFP8, kBS, true, 0>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<BLOCK_N>::kBytes);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(tiles * split), 1, 1);
  cfg.blockDim = dim3(EpiCfg<BLOCK_N, kBS, kHw>::kThreads, 1, 1);
  cfg.dynamicSmemBytes = Smem<BLOCK_N>::kBytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)split; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  pdl_attr(cfg, attr, 1);
  return (int)cudaLaunchKernelEx(&cfg, kern, tas[0], tas[1], tas[2], tb, a);
}

// Split-K plan for a dense GEMM with at most 128 rows.  The cost of a candidate is the bytes one CTA pulls through its
// L2 port (activation + weight slices of every tile it runs) plus a fixed charge per wave and for the reduction; the
// 128-wide tile halves the activation re-reads of the 64-wide one, and the split brings the idle SMs back.
static void plan_small_m(int N, int num_kb, bool fp8, int* bn_out, int* split_out) {
  double best = 1e30;
  *bn_out = 128; *split_out = 1;
  for (int bn : {256, 128, 64, 32}) {
    for (int sp = 1; sp <= 8; sp++) {
      if (bn == 256 && (fp8 || sp > 1 || N % 256 != 0)) continue;       // the widest tile exists for plain bf16 only
      if (num_kb % sp || (sp > 1 && num_kb / sp < 4)) continue;
      const long long tiles = (N + bn - 1) / bn;
      const long long ctas = tiles * sp;
      const int cap = sp > 1 ? (num_sms() / 8 / sp) * sp * 8 : num_sms();      // clusters do not straddle the 8 GPCs
      if (cap <= 0) continue;
      const long long waves = (ctas + cap - 1) / cap;
      const double unit_kb = (double)(kBlockM + bn) * kKBytes * (num_kb / sp) / 1024.0;
      const double cost = (double)waves * (unit_kb / 64.0 + 1.0) + (sp > 1 ? 2.0 : 0.0);    // ~64 KB/us per SM
      if (cost < best - 1e-9) { best = cost; *bn_out = bn; *split_out = sp; }
    }
  }
}

}  // namespace ne

using namespace ne;

// dtype: 0 = bf16 operands, 1 = fp8 e4m3 operands with block scales (sa/sb required), 2 = the same with the promise that every
// scale is a power of two: the tensor cores apply them (see kHw).
// A [groups, M, K] (row stride lda, group stride a_gs), B [groups, N, K] (contiguous), D [groups, M, N] (row stride ldd).
// masked_m: device int32 [groups] or null.  row_start: device int32 [groups] for the contiguous grouped layout (A and D
// are then flat [M, *] matrices and masked_m holds the per-group row counts) or null.
// Returns 0 or a CUDA / argument error code.
static int gemm_impl(const void* A, long long lda, long long a_gs, const void* B, void* D, long long ldd, long long d_gs,
                     int M, int N, int K, int groups, const int* masked_m, const int* row_start, int dtype, const float* sa, int sa_ld,
                     long long sa_gs, const float* sb, int out_fp32, int block_n_hint, const long long* row_dst, const GemmComm* comm,
                     int a_rows_total, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  if (comm) {
    if (comm->wait_flags && (groups > kSchedCache || comm->wait_world > 16 || !masked_m)) return 1007;
    if (comm->gate_flags && (groups != 1 || row_start || masked_m || comm->gate_world > 16 || comm->gate_rpr < 1)) return 1008;
    if (comm->scatter_mode && (out_fp32 || row_dst)) return 1005;
    if (comm->scatter_mode == 3 && (groups != 1 || comm->scatter_rpr < 1)) return 1009;
    if (comm->tail_counter && comm->tail_world > 16) return 1010;
  }
  // Tensor-core scaling pays where tiles follow one another on an SM (prefill): it frees the CUDA cores but drains a whole
  // accumulator at the end of every tile, and its scale fetch delays a CTA's first tile.  A GEMM of at most 128 rows per
  // group is one wave of tiles bound by the weight stream, where the promotion path (which takes any scales) is faster.
  // (Not with a gated A operand: the scale warps would read the scales of rows whose source rank has not delivered them yet.)
  const bool fp8 = dtype >= 1, hw = dtype == 2 && (row_start ? M / groups : M) > 128 && !(comm && comm->gate_flags);
  if (N % 8 != 0 || (K * (fp8 ? 1 : 2)) % 16 != 0 || (lda * (fp8 ? 1 : 2)) % 16 != 0) return 1001;
  if (fp8 && (K % 128 != 0 || !sa || !sb)) return 1002;
  if ((ldd * (out_fp32 == 1 ? 4 : (out_fp32 == 2 ? 1 : 2))) % 16 != 0) return 1003;
  if (out_fp32 == 2 && (fp8 || N % 32 != 0)) return 1006;      // e4m3 output: plain bf16 GEMMs, whole 32-column chunks
  const int m_blocks = (M + kBlockM - 1) / kBlockM;
  // pick the widest N tile that still yields about one tile per SM; fp8 promotion keeps BLOCK_N accumulators in registers
  int bn = block_n_hint;
  int split = 1;
  const int num_kb_host = (K * (fp8 ? 1 : 2) + kKBytes - 1) / kKBytes;
  const bool can_split = groups == 1 && !row_start && !masked_m && !row_dst && m_blocks == 1 && N % 4 == 0 &&
                         (K * (fp8 ? 1 : 2)) % kKBytes == 0 && g_split_k_enabled && out_fp32 != 2 &&
                         (!comm || (comm->scatter_mode != 2 && !comm->wait_flags));
  if (bn == 0 && can_split) {
    plan_small_m(N, num_kb_host, fp8, &bn, &split);
  } else if (bn == 0) {
    if (fp8 && !hw && !row_start && !masked_m) {
      // dense block-scaled GEMM: the serial K loop of a tile dominates at small M, so take the fewest waves of
      // tiles and, among equals, the narrowest tile (more SMs pulling weights at the same time)
      long long best_waves = 1ll << 60;
      bn = 128;
      for (int c : {128, 64, 32}) {
        long long tiles = (long long)groups * m_blocks * ((N + c - 1) / c);
        long long waves = (tiles + num_sms() - 1) / num_sms();
        if (waves <= best_waves) { best_waves = waves; bn = c; }
      }
    } else {
      const int cands[4] = {256, 128, 64, 32};
      bn = 32;
      for (int c : cands) {
        if (fp8 && c > 128) continue;
        long long tiles = (long long)groups * m_blocks * ((N + c - 1) / c);
        if (tiles >= num_sms() || c == 32) { bn = c; break; }
      }
      if (!fp8 && bn == 256 && N % 256 != 0 && N < 2048) bn = 128;
    }
  }
  if (hw && bn == 0) bn = 128;
  if (hw && !block_n_hint) {
    // Wide tile where it lowers the operand bytes an SM pulls through its fill path over the whole GEMM: waves of tiles times
    // the bytes of one K block of a tile.
    const long long gm = row_start ? m_blocks : (long long)groups * m_blocks;
    auto cost = [&](int w) { const long long t = gm * ((N + w - 1) / w); return ((t + num_sms() - 1) / num_sms()) * (long long)(kBlockM + w); };
    if (N >= 224 && cost(224) < cost(bn)) bn = 224;
  }
  if (fp8 && bn > 128 && !(hw && bn == 224)) bn = 128;
  // CTA pairs (256-row tiles) where every group has rows for several of them; not with a fused collective
  // and a long K loop to spread the two-CTA hand-overs of a tile over (measured: +2 % at K = 7168 / 16384 with N >= 4096, -13 % at
  // K = 2048)
  const bool pair = hw && bn == 224 && g_pair_enabled && !comm && !row_dst && (row_start ? M / groups : M) >= 512 && K >= 4096 && N >= 4096;
  const int kg = pair ? 2 : (bn >= 192 ? 1 : 2);      // KGroup<bn>::value
  CUtensorMap ta[3], tb;       // activation maps with 128-, 64- and 32-row boxes
  if (row_start || groups == 1) a_gs = (long long)(a_rows_total > 0 ? a_rows_total : M) * lda;
  int rc = 0;
  for (int i = 0; i < 3 && !rc; i++)
    rc = get_tmap_kmajor(&ta[i], A, fp8, (uint64_t)K, (uint64_t)(a_rows_total > 0 ? a_rows_total : M), (uint64_t)(row_start ? 1 : groups), (uint64_t)lda,
                         (uint64_t)a_gs, kBlockM >> i, kg);
  if (rc) return 2000 + rc;
  rc = get_tmap_kmajor(&tb, B, fp8, (uint64_t)K, (uint64_t)N, (uint64_t)groups, (uint64_t)K, (uint64_t)N * K, (uint32_t)(pair ? bn / 2 : bn), kg);
  if (rc) return 3000 + rc;
  GemmArgs a;
  a.a_group_inner = (!row_start && groups > 1 && a_gs < lda) ? 1 : 0;
  a.k_flat = (K * (fp8 ? 1 : 2)) % kKBytes != 0 ? 1 : 0;
  a.M = M; a.N = N; a.K = K; a.groups = groups; a.masked_m = masked_m; a.row_start = row_start; a.D = D; a.ldd = ldd; a.d_group_stride = d_gs;
  if (row_start) { a.d_group_stride = 0; sa_gs = 0; if (!masked_m) return 1004; }
  a.sa = sa; a.sa_ld = sa_ld; a.sa_group_stride = sa_gs; a.sb = sb;
  a.sb_group_stride = (long long)((N + 127) / 128) * (K / 128); a.out_fp32 = out_fp32; a.alpha = nullptr;
  a.row_dst = row_dst; a.rd_group_stride = row_start ? 0 : M;
  if (row_dst && out_fp32) return 1005;
  if (comm) { a.comm = *comm; if (m_blocks <= 1 || groups != 1) a.comm.mb_rot = 0; else a.comm.mb_rot %= m_blocks; }
  else memset(&a.comm, 0, sizeof(a.comm));
  long long tiles = (long long)groups * m_blocks * ((N + bn - 1) / bn);
  int grid = (int)(tiles < num_sms() ? tiles : num_sms());
  if (pair) {
    const long long ptiles = (row_start ? (long long)(M + 255) / 256 + groups : (long long)groups * ((M + 255) / 256)) * ((N + bn - 1) / bn);
    return launch_pair<224>(ta, tb, a, (int)(ptiles < 4096 ? ptiles : 4096), stream);      // capped at the resident pairs by the launcher
  }
  if (hw) {
    switch (bn) {
      case 224: return launch<224, true, false, 1>(ta, tb, a, grid, stream);
      case 128: return launch<128, true, false, 1>(ta, tb, a, grid, stream);
      case 64: return launch<64, true, false, 1>(ta, tb, a, grid, stream);
      default: return launch<32, true, false, 1>(ta, tb, a, grid, stream);
    }
  }
  if (split > 1) {
    if (fp8) {
      switch (bn) {
        case 128: return launch_split<128, true, true>(ta, tb, a, (int)tiles, split, stream);
        case 64: return launch_split<64, true, true>(ta, tb, a, (int)tiles, split, stream);
        default: return launch_split<32, true, true>(ta, tb, a, (int)tiles, split, stream);
      }
    }
    switch (bn) {
      case 128: return launch_split<128, false, false>(ta, tb, a, (int)tiles, split, stream);
      case 64: return launch_split<64, false, false>(ta, tb, a, (int)tiles, split, stream);
      default: return launch_split<32, false, false>(ta, tb, a, (int)tiles, split, stream);
    }
  }
  if (fp8) {
    switch (bn) {
      case 128: return launch<128, true, true>(ta, tb, a, grid, stream);
      case 64: return launch<64, true, true>(ta, tb, a, grid, stream);
      default: return launch<32, true, true>(ta, tb, a, grid, stream);
    }
  }
  switch (bn) {
    case 256: return launch<256, false, false>(ta, tb, a, grid, stream);
    case 128: return launch<128, false, false>(ta, tb, a, grid, stream);
    case 64: return launch<64, false, false>(ta, tb, a, grid, stream);
    default: return launch<32, false, false>(ta, tb, a, grid, stream);
  }
}

extern "C" int ne_gemm(const void* A, long long lda, long long a_gs, const void* B, void* D, long long ldd, long long d_gs,
                       int M, int N, int K, int groups, const int* masked_m, const int* row_start, int dtype, const float* sa, int sa_ld,
                       long long sa_gs, const float* sb, int out_fp32, int block_n_hint, const long long* row_dst, cudaStream_t stream) {
  return gemm_impl(A, lda, a_gs, B, D, ldd, d_gs, M, N, K, groups, masked_m, row_start, dtype, sa, sa_ld, sa_gs, sb, out_fp32, block_n_hint, row_dst,
                   nullptr, 0, stream);
}

// The same GEMM with a collective fused in (see GemmComm).  `a_rows_total` > 0 gives the number of rows the A tensor map must
// cover when that is more than M (the double-buffered gather area of the gated form).
extern "C" int ne_gemm_comm(const void* A, long long lda, long long a_gs, const void* B, void* D, long long ldd, long long d_gs,
                            int M, int N, int K, int groups, const int* masked_m, const int* row_start, int dtype, const float* sa, int sa_ld,
                            long long sa_gs, const float* sb, int out_fp32, int block_n_hint, const GemmComm* comm, int a_rows_total,
                            cudaStream_t stream) {
  return gemm_impl(A, lda, a_gs, B, D, ldd, d_gs, M, N, K, groups, masked_m, row_start, dtype, sa, sa_ld, sa_gs, sb, out_fp32, block_n_hint, nullptr,
                   comm, a_rows_total, stream);
}
extern "C" int ne_gemm_comm_size() { return (int)sizeof(GemmComm); }

// NVFP4 GEMM (see kMode 2): A [rows, K] and B [groups, N, K] packed e2m1 (K / 2 bytes per row), SFA [rows, K / 16] and
// SFB [groups, N, K / 16] e4m3 bytes, alpha [groups] fp32 (or null), D bf16 (out_fp32 = 1: fp32).  Layouts as ne_gemm: one dense
// group, masked groups [groups, M, *] (masked_m) or the contiguous grouped form (row_start + masked_m over flat [M, *] matrices).
extern "C" int ne_gemm_nvfp4(const void* A, const void* B, void* D, long long ldd, int M, int N, int K, int groups, const int* masked_m,
                             const int* row_start, const void* sfa, const void* sfb, const float* alpha, int out_fp32, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || groups <= 0) return 0;
  if (K % 256 != 0 || N % 8 != 0 || !sfa || !sfb || (row_start && !masked_m)) return 1001;
  if ((ldd * (out_fp32 ? 4 : 2)) % 16 != 0) return 1003;
  const int Kb = K / 2;                 // bytes per operand row: the kernel's unit of K
  constexpr int bn = 128;
  const int m_blocks = (M + kBlockM - 1) / kBlockM;
  CUtensorMap ta[3], tb;
  const long long a_gs = (row_start || groups == 1) ? (long long)M * Kb : (long long)M * Kb;
  int rc = 0;
  for (int i = 0; i < 3 && !rc; i++)
    rc = get_tmap_kmajor(&ta[i], A, true, (uint64_t)Kb, (uint64_t)M, (uint64_t)(row_start ? 1 : groups), (uint64_t)Kb, (uint64_t)a_gs, kBlockM >> i, 1);
  if (rc) return 2000 + rc;
  rc = get_tmap_kmajor(&tb, B, true, (uint64_t)Kb, (uint64_t)N, (uint64_t)groups, (uint64_t)Kb, (uint64_t)N * Kb, (uint32_t)bn, 1);
  if (rc) return 3000 + rc;
  GemmArgs a;
  memset(&a, 0, sizeof(a));
  a.M = M; a.N = N; a.K = Kb; a.groups = groups; a.masked_m = masked_m; a.row_start = row_start; a.D = D; a.ldd = ldd;
  a.d_group_stride = row_start ? 0 : (long long)M * ldd;
  a.sa = reinterpret_cast<const float*>(sfa); a.sa_group_stride = row_start ? 0 : M;      // NVFP4: byte arrays; the stride counts rows
  a.sb = reinterpret_cast<const float*>(sfb);
  a.alpha = alpha; a.out_fp32 = out_fp32 ? 1 : 0;
  a.rd_group_stride = row_start ? 0 : M;
  const long long tiles = (row_start ? (long long)m_blocks + groups : (long long)groups * m_blocks) * ((N + bn - 1) / bn);
  const int grid = (int)(tiles < num_sms() ? tiles : num_sms());
  return launch<128, true, false, 2>(ta, tb, a, grid, stream);
}

// 1: every fp8 activation quantiser of this library rounds its group scales up to powers of two (the form dtype 2 of
// ne_gemm needs); 0: plain amax / 448.  Returns the previous setting.  Kernels captured in a CUDA graph keep the setting
// they were captured with.
extern "C" int ne_set_scale_pow2(int on) { int was = g_scale_pow2; g_scale_pow2 = on ? 1 : 0; return was; }

// Turn the cluster split-K plan of small-M dense GEMMs on or off (on by default); returns the previous setting.
extern "C" int ne_gemm_set_split_k(int on) { int was = g_split_k_enabled ? 1 : 0; g_split_k_enabled = on != 0; return was; }

// Turn the CTA-pair form of the tensor-core-scaled fp8 GEMM on or off (on by default); returns the previous setting.
extern "C" int ne_gemm_set_pair(int on) { int was = g_pair_enabled ? 1 : 0; g_pair_enabled = on != 0; return was; }

// Debug build only: register the bounds the checked kernels compare their table entries with (0 = leave unchecked).  Returns 1 when
// this library was built with the checks, 0 otherwise (the call is then a no-op).
extern "C" int ne_debug_set_bounds(long long cache_rows, long long cache_pages, long long state_slots, long long experts) {
#ifdef NE_DEBUG_BOUNDS
  long long b[BK_COUNT] = {cache_rows, cache_pages, state_slots, experts};
  cudaMemcpyToSymbol(g_bounds, b, sizeof(b));
  return 1;
#else
  (void)cache_rows; (void)cache_pages; (void)state_slots; (void)experts;
  return 0;
#endif
}

extern "C" int ne_get_status(int* out8) {
  return (int)cudaMemcpyFromSymbol(out8, g_status, sizeof(int) * 8);
}
extern "C" int ne_clear_status() {
  int z[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  return (int)cudaMemcpyToSymbol(g_status, z, sizeof(z));
}
