// Hot / cold tiering of the sparse-attention latent cache (HiSparse).
//
// The full latent cache of every sequence lives in pinned host memory ("cold", addressed by the scheduler's logical pages);
// the device keeps, per sequence slot and layer, a small buffer of `hot_rows` latent rows ("hot") that the sparse attention
// kernel reads.  Each decode step the indexer lists the top-k key positions of every sequence; `hisparse_stage_kernel` turns
// that list into hot row ids: positions already resident are stamped as used in this step, the others take over rows that
// were not used in this step (in ring order from a per-slot cursor, so rows idle the longest go first) and are copied in
// from the cold tier through the unified address space.  The position of the token being decoded gets a row as well; the
// key kernel writes its latent row there and `hisparse_writeback_kernel` copies it to the cold tier.  Everything is
// device-side and shape-stable, so the step replays from a CUDA graph.
//
// Replaces in the reference: runtime/context/cache/hisparse.py:154-221,294-316,352-391 and
// kernel/jit/sgl/include/sgl_kernel/hisparse/hisparse.cuh:11 (ring slot mapping), :56 (load of the selected rows), :273
// (write-back).
#include "ptx.cuh"

namespace ne {

constexpr int kHsMaxTopk = 4096;
constexpr int kKernelHs = 11;

struct HsArgs {
  int* pos_to_hot;            // [slots, max_ctx]   hot row of a key position or -1
  int* hot_to_pos;            // [slots, hot_rows]  key position held by a hot row or -1
  int* stamp;                 // [slots, hot_rows]  step in which the row was last used
  int* cursor;                // [slots]
  int* step;                  // [2] step counter, finished-CTA counter
  const uint8_t* cold;        // this layer's cold pages [pages, page_rows, row_bytes] (pinned host memory)
  uint8_t* hot;               // this layer's hot rows [slots * hot_rows, row_bytes]
  const int* sel; int topk;   // [B, topk] key positions, -1 padded
  const int* slots;           // [B]
  const int* context_lens;    // [B] (the token being decoded sits at context_len - 1)
  const int* block_tables; int bt_stride;
  int* out;                   // [B, topk] hot row ids (slot * hot_rows + row) or -1
  long long* new_slot;        // [B] hot row id of the token being decoded
  int max_ctx, hot_rows, row_bytes, page_rows, B;
};

__global__ void __launch_bounds__(256) hisparse_stage_kernel(const HsArgs a) {
  __shared__ int s_miss[kHsMaxTopk];
  __shared__ int s_vict[kHsMaxTopk + 1];
  __shared__ int s_nmiss, s_inew, s_need_new, s_hnew, s_wcnt[8], s_base, s_scanned;
  const int b = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int slot = a.slots[b];
  const int step = a.step[0] + 1;
  const int new_pos = a.context_lens[b] - 1;
  int* p2h = a.pos_to_hot + (long long)slot * a.max_ctx;
  int* h2p = a.hot_to_pos + (long long)slot * a.hot_rows;
  int* stp = a.stamp + (long long)slot * a.hot_rows;
  const int* sel = a.sel + (long long)b * a.topk;
  int* out = a.out + (long long)b * a.topk;
  const long long row0 = (long long)slot * a.hot_rows;
  if (tid == 0) { s_nmiss = 0; s_inew = -1; s_need_new = 0; s_hnew = -1; s_base = 0; s_scanned = 0; }
  __syncthreads();
  // A: hits are stamped, misses are listed in list order (ordered compaction: the same victims go to the same positions on
  // every run, and the tables equal those of the plain PyTorch statement)
  for (int i0 = 0; i0 < a.topk; i0 += 256) {
    const int i = i0 + tid;
    bool miss = false;
    if (i < a.topk) {
      const int p = sel[i];
      if (p < 0 || p >= a.max_ctx) out[i] = -1;
      else if (p == new_pos) s_inew = i;
      else {
        const int h = p2h[p];
        if (h >= 0) { stp[h] = step; out[i] = (int)(row0 + h); }
        else miss = true;
      }
    }
    const unsigned bal = __ballot_sync(0xffffffffu, miss);
    if (lane == 0) s_wcnt[warp] = __popc(bal);
    __syncthreads();
    int off = s_nmiss;
    for (int w = 0; w < warp; w++) off += s_wcnt[w];
    if (miss) s_miss[off + __popc(bal & ((1u << lane) - 1u))] = i;
    __syncthreads();
    if (tid == 0) { int t = 0; for (int w = 0; w < 8; w++) t += s_wcnt[w]; s_nmiss += t; }
    __syncthreads();
  }
  if (tid == 0 && new_pos >= 0 && new_pos < a.max_ctx) {
    const int h = p2h[new_pos];
    if (h >= 0) { stp[h] = step; s_hnew = h; } else s_need_new = 1;
  }
  __syncthreads();
  const int need_new = s_need_new, n_miss = s_nmiss, need = n_miss + need_new;
  // B: the first `need` rows, in ring order from the cursor, that were not used in this step
  const int cur = a.cursor[slot];
  for (int j0 = 0; j0 < a.hot_rows && s_base < need; j0 += 256) {
    const int j = j0 + tid;
    int h = cur + j;
    if (h >= a.hot_rows) h -= a.hot_rows;
    const bool free_row = j < a.hot_rows && stp[h] != step;
    const unsigned bal = __ballot_sync(0xffffffffu, free_row);
    if (lane == 0) s_wcnt[warp] = __popc(bal);
    __syncthreads();
    int off = s_base;
    for (int w = 0; w < warp; w++) off += s_wcnt[w];
    if (free_row) {
      const int v = off + __popc(bal & ((1u << lane) - 1u));
      if (v < need) { s_vict[v] = h; atomicMax(&s_scanned, j + 1); }
    }
    __syncthreads();
    if (tid == 0) { int t = 0; for (int w = 0; w < 8; w++) t += s_wcnt[w]; s_base += t; }
    __syncthreads();
  }
  const int got = s_base < need ? s_base : need;
  if (tid == 0 && got < need) report(ST_BAD_ARG, kKernelHs, need, got);        // hot buffer smaller than one step's demand
  // C: the token being decoded takes the first victim (nothing to copy: the key kernel writes the row)
  if (tid == 0) {
    int hn = s_hnew;
    if (need_new && got > 0) {
      hn = s_vict[0];
      const int old = h2p[hn];
      if (old >= 0) p2h[old] = -1;
      h2p[hn] = new_pos; p2h[new_pos] = hn; stp[hn] = step;
    }
    a.new_slot[b] = hn >= 0 ? row0 + hn : row0;        // row 0 of the slot if nothing could be had (reported above)
    if (s_inew >= 0) out[s_inew] = hn >= 0 ? (int)(row0 + hn) : -1;
    a.cursor[slot] = (cur + s_scanned) % a.hot_rows;
  }
  // every other miss: one warp evicts, maps and copies a row
  const int chunks = a.row_bytes / 16;
  for (int m = warp; m < n_miss; m += 8) {
    const int i = s_miss[m];
    const int v = m + need_new;
    if (v >= got) { if (lane == 0) out[i] = -1; continue; }
    const int p = sel[i], h = s_vict[v];
    if (lane == 0) {
      const int old = h2p[h];
      if (old >= 0) p2h[old] = -1;
      h2p[h] = p; p2h[p] = h; stp[h] = step;
      out[i] = (int)(row0 + h);
    }
    const long long page = a.block_tables[(long long)b * a.bt_stride + p / a.page_rows];
    const uint4* src = reinterpret_cast<const uint4*>(a.cold + (page * a.page_rows + p % a.page_rows) * a.row_bytes);
    uint4* dst = reinterpret_cast<uint4*>(a.hot + (row0 + h) * a.row_bytes);
    for (int c = lane; c < chunks; c += 32) dst[c] = src[c];
  }
  // the last CTA to finish publishes the step number
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    if (atomicAdd(&a.step[1], 1) == a.B - 1) { a.step[1] = 0; a.step[0] = step; }
  }
}

// hot row new_slot[b] -> cold row slot_mapping[b] (the logical cache row of the token just written)
__global__ void __launch_bounds__(64) hisparse_writeback_kernel(const uint8_t* __restrict__ hot, uint8_t* __restrict__ cold,
                                                               const long long* __restrict__ new_slot, const long long* __restrict__ slot_mapping,
                                                               int row_bytes) {
  const long long h = new_slot[blockIdx.x], c = slot_mapping[blockIdx.x];
  if (h < 0 || c < 0) return;
  const uint4* src = reinterpret_cast<const uint4*>(hot + h * row_bytes);
  uint4* dst = reinterpret_cast<uint4*>(cold + c * row_bytes);
  for (int i = threadIdx.x; i < row_bytes / 16; i += 64) dst[i] = src[i];
}

}  // namespace ne

using namespace ne;

extern "C" int ne_hisparse_stage(int* pos_to_hot, int* hot_to_pos, int* stamp, int* cursor, int* step, const void* cold, void* hot, const int* sel,
                                 int topk, const int* slots, const int* context_lens, const int* block_tables, int bt_stride, int* out,
                                 long long* new_slot, int max_ctx, int hot_rows, int row_bytes, int page_rows, int B, cudaStream_t st) {
  if (B <= 0) return 0;
  if (topk < 1 || topk > kHsMaxTopk || row_bytes % 16 || hot_rows < 1 || page_rows < 1) return 1001;
  HsArgs a;
  a.pos_to_hot = pos_to_hot; a.hot_to_pos = hot_to_pos; a.stamp = stamp; a.cursor = cursor; a.step = step; a.cold = (const uint8_t*)cold;
  a.hot = (uint8_t*)hot; a.sel = sel; a.topk = topk; a.slots = slots; a.context_lens = context_lens; a.block_tables = block_tables;
  a.bt_stride = bt_stride; a.out = out; a.new_slot = new_slot; a.max_ctx = max_ctx; a.hot_rows = hot_rows; a.row_bytes = row_bytes;
  a.page_rows = page_rows; a.B = B;
  hisparse_stage_kernel<<<B, 256, 0, st>>>(a);
  return (int)cudaGetLastError();
}

extern "C" int ne_hisparse_writeback(const void* hot, void* cold, const long long* new_slot, const long long* slot_mapping, int row_bytes, int B,
                                     cudaStream_t st) {
  if (B <= 0) return 0;
  if (row_bytes % 16) return 1001;
  hisparse_writeback_kernel<<<B, 64, 0, st>>>((const uint8_t*)hot, (uint8_t*)cold, new_slot, slot_mapping, row_bytes);
  return (int)cudaGetLastError();
}
