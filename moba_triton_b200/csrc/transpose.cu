// Transpose: regroups per-query selections (CSR, block_idx) by key/value block
// (CSC) with a *stable* counting sort, so a column lists its queries ordered by
// (query head, row) on every run.
//
//   1. count    one CTA per (row chunk, sequence, query head): shared-memory
//               histogram over blocks -> tile_counts[seq,kvh][block][g*C + chunk]
//   2. colscan  one warp per (sequence, kv head, block): exclusive scan of that
//               block's tile counts in (g, chunk) order; total -> col_nnz
//   3. offsets  per (sequence, kv head): exclusive scan over blocks ->
//               col_offsets, and the longest-first dispatch order (stable
//               descending sort of col_nnz, by rank counting)
//   4. items    per (sequence, kv head): walks the columns in dispatch order and cuts
//               each into work items of at most chunk_tiles tiles; a split column's
//               items get consecutive dK/dV partial slots
//   5. scatter  one CTA per (row chunk, sequence, query head): its warps split the
//               chunk's rows into consecutive runs; a per-warp histogram and a scan
//               over the warps give each warp its own cursors, and every warp then
//               walks its run in order, ranks equal blocks inside the warp with
//               match.any and writes (row, head, slot) at cursor[block]++.
//
// Stands in for count_columns_kernel / offsets_and_order_kernel /
// scatter_pairs_kernel of the reference (src/moba/kernels/routing.py:138-301),
// which claim positions with an atomic cursor and therefore leave the order
// inside a column to the scheduler.
#include "common.cuh"
#include "sm100.cuh"

#include <mutex>

namespace moba {

struct TransposeGeom {
  int chunk_rows;   // R, a power of two
  int chunks;       // C = cdiv(max_seqlen, R)
};
static inline TransposeGeom transpose_geom(const moba_b200_problem& p) {
  int r = 256;
  while ((p.max_seqlen + r - 1) / r > 256) r <<= 1;
  return TransposeGeom{r, (p.max_seqlen + r - 1) / r};
}
static inline size_t tile_count_bytes(const moba_b200_problem& p) {
  const TransposeGeom g = transpose_geom(p);
  const size_t group = p.q_heads / p.kv_heads;
  return (size_t)p.n_seq * p.kv_heads * p.num_blocks * group * g.chunks * sizeof(int32_t);
}
// the per-chunk histograms, then one 16-byte cell holding the counter of dK/dV partial slots
size_t transpose_scratch_bytes(const moba_b200_problem& p) { return ((tile_count_bytes(p) + 15) & ~size_t(15)) + 16; }

__device__ __forceinline__ size_t block_idx_row(const moba_b200_problem& p, int seq, int hq,
                                                int bos, int row) {
  const size_t b = p.packed ? 0 : (size_t)seq;
  return ((b * p.q_heads + hq) * p.tokens + bos + row) * (size_t)p.slots;
}

__global__ void __launch_bounds__(256)
count_kernel(const int32_t* __restrict__ block_idx, const int32_t* __restrict__ cu,
             int32_t* __restrict__ tile_counts, int32_t* __restrict__ slot_counter, moba_b200_problem p, int R, int C) {
  extern __shared__ int hist[];
  if (blockIdx.x == 0 && threadIdx.x == 0) *slot_counter = 0;     // claimed from by work_items_kernel, two launches on
  const int chunk = blockIdx.x % C, y = blockIdx.x / C;
  const int seq = y / p.q_heads, hq = y % p.q_heads;
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  const int row0 = chunk * R;
  if (row0 >= sp.len) return;
  const int rows = min(R, sp.len - row0);
  const int nb_lim = (row0 + rows - 1) / p.block_size + 1;
  for (int i = threadIdx.x; i < nb_lim; i += 256) hist[i] = 0;
  __syncthreads();
  const int32_t* src = block_idx + block_idx_row(p, seq, hq, sp.bos, row0);
  // only the rows inside the query window are listed (all of them without a window)
  const int w_lo = max(0, p.win_begin - row0), w_hi = min(rows, (p.win_rows > 0 ? p.win_begin + p.win_rows : sp.len) - row0);
  const int n = max(w_lo, w_hi) * p.slots;
  for (int e = w_lo * p.slots + threadIdx.x; e < n; e += 256) {
    const int blk = src[e];
    if (blk >= 0 && blk < nb_lim) atomicAdd(&hist[blk], 1);
  }
  __syncthreads();
  const int group = p.q_heads / p.kv_heads;
  const int kvh = hq / group, g = hq % group;
  int32_t* dst = tile_counts + ((size_t)(seq * p.kv_heads + kvh) * p.num_blocks) * (group * C) + g * C + chunk;
  for (int i = threadIdx.x; i < nb_lim; i += 256) dst[(size_t)i * (group * C)] = hist[i];
}

// One warp per column. Replaces the column's tile counts by their exclusive
// prefix (in (g, chunk) order) and writes the column total.
__global__ void __launch_bounds__(128)
colscan_kernel(const int32_t* __restrict__ cu, int32_t* __restrict__ tile_counts,
               int32_t* __restrict__ col_nnz, moba_b200_problem p, int R, int C, int ctas_per_row) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = (int)(blockIdx.x % ctas_per_row) * 4 + warp;
  const int kv_row = (int)(blockIdx.x / ctas_per_row);       // (sequence, kv head)
  if (col >= p.num_blocks) return;
  const int seq = kv_row / p.kv_heads;
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  int32_t* out_nnz = col_nnz + (size_t)kv_row * p.num_blocks + col;
  if ((size_t)col * p.block_size >= (size_t)sp.len) {
    if (lane == 0) *out_nnz = 0;
    return;
  }
  const int group = p.q_heads / p.kv_heads;
  const int c_lo = (int)(((size_t)col * p.block_size) / R);
  const int c_hi = (sp.len + R - 1) / R;                    // exclusive
  const int span = c_hi - c_lo;
  int32_t* base = tile_counts + ((size_t)kv_row * p.num_blocks + col) * (group * C);
  int running = 0;
  const int total = group * span;
  for (int i0 = 0; i0 < total; i0 += 32) {
    const int i = i0 + lane;
    int v = 0;
    int32_t* ptr = nullptr;
    if (i < total) {
      ptr = base + (i / span) * C + c_lo + (i % span);
      v = *ptr;
    }
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (ptr) *ptr = running + incl - v;
    running += __shfl_sync(0xffffffffu, incl, 31);
  }
  if (lane == 0) *out_nnz = running;
}

// (sequence, kv head) x (128 columns): col_offsets (first CTA of the row) and the dispatch order.
__global__ void __launch_bounds__(1024)
offsets_order_kernel(const int32_t* __restrict__ col_nnz, int32_t* __restrict__ col_offsets,
                     int32_t* __restrict__ order, int nb) {
  extern __shared__ int cnt[];              // [nb]
  __shared__ int warp_sums[32];
  __shared__ int carry_s;
  const int32_t* nnz = col_nnz + (size_t)blockIdx.x * nb;
  int32_t* off = col_offsets + (size_t)blockIdx.x * (nb + 1);
  int32_t* ord = order + (size_t)blockIdx.x * nb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int i0 = 0; i0 < nb; i0 += 1024) {
    const int i = i0 + threadIdx.x;
    const int v = (i < nb) ? nnz[i] : 0;
    if (i < nb) cnt[i] = v;
    int incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
      int w = warp_sums[lane];
      int wi = w;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, wi, o);
        if (lane >= o) wi += t;
      }
      warp_sums[lane] = wi - w;             // exclusive over warps
    }
    __syncthreads();
    const int carry = carry_s;
    if (i < nb && blockIdx.y == 0) off[i] = carry + warp_sums[warp] + incl - v;
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + warp_sums[warp] + incl;
    __syncthreads();
  }
  if (threadIdx.x == 0 && blockIdx.y == 0) off[nb] = carry_s;
  // stable descending rank: position of column i = #{j : n_j > n_i or (n_j == n_i and j < i)}.
  // nb^2 comparisons in all: CTA y of the row ranks columns [128 y, 128 y + 128), eight
  // threads per column over interleaved j.
  const int i = (int)blockIdx.y * 128 + (int)(threadIdx.x >> 3), part = threadIdx.x & 7;
  int rank = 0;
  if (i < nb) {
    const int ni = cnt[i];
    for (int j = part; j < nb; j += 8) {
      const int nj = cnt[j];
      rank += (nj > ni || (nj == ni && j < i)) ? 1 : 0;
    }
  }
  rank += __shfl_xor_sync(0xffffffffu, rank, 1);
  rank += __shfl_xor_sync(0xffffffffu, rank, 2);
  rank += __shfl_xor_sync(0xffffffffu, rank, 4);
  if (i < nb && part == 0) ord[rank] = i;
}

// One CTA per (sequence, kv head) row: the row's work items, largest first. A column of more
// than `tc` tiles becomes ceil(tiles / tc) items, each with a dK/dV partial slot of its own:
// pieces of `tc` tiles and a last, shorter one. The kernels deal the list out to their CTAs in
// alternating direction, which balances a list that is sorted by size; so the full pieces come
// first and the last pieces of the cut columns are merged, by size, into the (already sorted)
// uncut columns: without that a CTA's share was off by up to 18 % when a CTA gets only some
// eight items. The slots of a row are consecutive and claimed from a counter, so rows may
// claim in any order: slot numbers name scratch memory, results do not depend on them, nor on
// the order of the list. A row with more than kMaxCut cut columns keeps its columns' pieces
// side by side, in column order (it has items enough for the order not to matter).
constexpr int kMaxCut = 2048;
__global__ void __launch_bounds__(1024)
work_items_kernel(const int32_t* __restrict__ col_nnz, const int32_t* __restrict__ order, int4* __restrict__ items,
                  int32_t* __restrict__ slot_counter, int nb, int items_per_row, int tc, int slot_cap,
                  unsigned* error_word) {
  __shared__ long long warp_sums[32];
  __shared__ long long carry_s;
  __shared__ int base_s;
  __shared__ int rem_s[kMaxCut], rank_s[kMaxCut], sorted_s[kMaxCut], slot_s[kMaxCut];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int32_t* nnz = col_nnz + (size_t)blockIdx.x * nb;
  const int32_t* ord = order + (size_t)blockIdx.x * nb;
  int4* out = items + (size_t)blockIdx.x * items_per_row;
  auto tiles_of = [&](int r) { return (nnz[ord[r]] + 127) / 128; };
  auto chunks_of = [&](int r, int& blk, int& tiles) {
    blk = ord[r];
    tiles = (nnz[blk] + 127) / 128;
    return tiles <= tc ? 1 : (tiles + tc - 1) / tc;
  };
  // exclusive prefix of a 64-bit value over the CTA, and the CTA's total
  auto block_scan = [&](long long v, long long& total) {
    long long incl = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const long long t = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += t;
    }
    __syncthreads();
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    long long before = 0, all = 0;
    for (int w = 0; w < 32; ++w) {
      const long long s = warp_sums[w];
      before += (w < warp) ? s : 0;
      all += s;
    }
    total = all;
    return before + incl - v;
  };
  // pass 1: cut columns (a prefix of the dispatch order) and the partial slots the row needs
  long long mine = 0;
  for (int r = threadIdx.x; r < nb; r += 1024) {
    int blk, tiles;
    const int c = chunks_of(r, blk, tiles);
    if (c > 1) mine += 1LL | ((long long)c << 32);
  }
  long long row_total;
  block_scan(mine, row_total);
  const int n_cut = (int)(row_total & 0xffffffffLL);
  const int row_slots = (int)(row_total >> 32);
  if (threadIdx.x == 0) {
    base_s = row_slots > 0 ? atomicAdd(slot_counter, row_slots) : 0;
    carry_s = 0;
    if (row_slots > 0 && (long long)base_s + row_slots > slot_cap) atomicOr(error_word, 2u);   // sizes were promised by the host
  }
  __syncthreads();
  const int base = base_s;
  // beyond the promised capacity (flagged above) an item falls back to "whole column": wrong
  // sums, reported through the error word, but no access outside the scratch
  auto slot_or_none = [&](int s) { return s < slot_cap ? s : -1; };
  auto put = [&](int at, int4 it) {
    if (at >= 0 && at < items_per_row) out[at] = it;
    else atomicOr(error_word, 2u);
  };

  if (n_cut <= kMaxCut) {
    const int n_full = row_slots - n_cut;                   // pieces of exactly tc tiles: they lead the list
    // the cut columns: full pieces in column order, the last piece's size and slot for later
    for (int r0 = 0; r0 < n_cut; r0 += 1024) {
      const int r = r0 + threadIdx.x;
      int blk = 0, tiles = 0, c = 0;
      if (r < n_cut) c = chunks_of(r, blk, tiles);
      long long total;
      const long long carry = carry_s;
      const int slot0 = (int)(carry + block_scan((long long)c, total));   // pieces of the cut columns before this one
      if (r < n_cut) {
        const int full0 = slot0 - r;                        // each earlier cut column has one piece that is not full
        for (int i = 0; i + 1 < c; ++i) put(full0 + i, make_int4(blk, i * tc, tc, slot_or_none(base + slot0 + i)));
        rem_s[r] = tiles - (c - 1) * tc;
        slot_s[r] = slot0;
      }
      __syncthreads();
      if (threadIdx.x == 0) carry_s = carry + total;
      __syncthreads();
    }
    // rank of each last piece among the last pieces: larger first, ties in column order
    for (int r = threadIdx.x; r < n_cut; r += 1024) {
      const int mine_rem = rem_s[r];
      int rank = 0;
      for (int q = 0; q < n_cut; ++q) {
        const int o = rem_s[q];
        rank += (o > mine_rem || (o == mine_rem && q < r)) ? 1 : 0;
      }
      rank_s[r] = rank;
      sorted_s[rank] = mine_rem;
    }
    __syncthreads();
    // last pieces of the cut columns: behind the uncut columns that are larger
    for (int r = threadIdx.x; r < n_cut; r += 1024) {
      const int mine_rem = rem_s[r];
      int lo = n_cut, hi = nb;                              // first uncut column with tiles <= mine_rem
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (tiles_of(mid) > mine_rem) lo = mid + 1; else hi = mid;
      }
      int blk, tiles;
      const int c = chunks_of(r, blk, tiles);
      put(n_full + rank_s[r] + (lo - n_cut), make_int4(blk, (c - 1) * tc, mine_rem, slot_or_none(base + slot_s[r] + c - 1)));
    }
    // uncut columns: behind the last pieces that are at least as large
    for (int r = n_cut + threadIdx.x; r < nb; r += 1024) {
      int blk, tiles;
      chunks_of(r, blk, tiles);
      int lo = 0, hi = n_cut;                               // first last piece smaller than this column
      while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (sorted_s[mid] >= tiles) lo = mid + 1; else hi = mid;
      }
      put(n_full + (r - n_cut) + lo, make_int4(blk, 0, tiles, -1));
    }
    for (int j = n_full + nb + threadIdx.x; j < items_per_row; j += 1024) out[j] = make_int4(0, 0, 0, -2);   // padding
    return;
  }

  // more cut columns than the tables hold: each column's pieces side by side, in column order
  for (int r0 = 0; r0 < nb; r0 += 1024) {
    const int r = r0 + threadIdx.x;
    int blk = 0, tiles = 0, c = 0;
    if (r < nb) c = chunks_of(r, blk, tiles);
    const long long v = (long long)c | ((long long)(c > 1 ? c : 0) << 32);
    long long total;
    const long long carry = carry_s;
    const long long at = carry + block_scan(v, total);
    const int item0 = (int)(at & 0xffffffffLL), slot0 = (int)(at >> 32);
    for (int i = 0; i < c; ++i)
      put(item0 + i, make_int4(blk, i * tc, tiles == 0 ? 0 : min(tc, tiles - i * tc), c > 1 ? slot_or_none(base + slot0 + i) : -1));
    __syncthreads();
    if (threadIdx.x == 0) carry_s = carry + total;
    __syncthreads();
  }
  const int used = (int)(carry_s & 0xffffffffLL);
  for (int j = used + threadIdx.x; j < items_per_row; j += 1024) out[j] = make_int4(0, 0, 0, -2);   // padding
}

// One CTA of W warps per (row chunk, sequence, query head). The walk of a run is one
// dependent chain per warp (match, cursor, store), so the chunk is cut into W runs that are
// walked side by side: a histogram per run and a scan over the runs (both in shared memory)
// turn the chunk's cursors into cursors per run. The order inside a column stays
// (query head, row): runs are consecutive rows and keep the chunk's order.
template <int W>
__global__ void __launch_bounds__(32 * W)
scatter_kernel(const int32_t* __restrict__ block_idx, const int32_t* __restrict__ cu,
               const int32_t* __restrict__ tile_prefix, const int32_t* __restrict__ col_offsets,
               int32_t* __restrict__ rows_out, int32_t* __restrict__ heads_out,
               int32_t* __restrict__ slots_out, moba_b200_problem p, int R, int C,
               long long capacity) {
  extern __shared__ int cursor_all[];                        // [W][nb_lim]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = blockIdx.x % C, y = blockIdx.x / C;
  const int seq = y / p.q_heads, hq = y % p.q_heads;
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  const int row0 = chunk * R;
  if (row0 >= sp.len) return;                                // the whole CTA
  const int rows = min(R, sp.len - row0);
  const int nb_lim = (row0 + rows - 1) / p.block_size + 1;
  const int group = p.q_heads / p.kv_heads;
  const int kvh = hq / group, g = hq % group;
  const size_t kv_row = (size_t)seq * p.kv_heads + kvh;
  const int32_t* pre = tile_prefix + (kv_row * p.num_blocks) * (group * C) + g * C + chunk;
  const int32_t* off = col_offsets + kv_row * (p.num_blocks + 1);
  // this warp's run of rows
  // the chunk's rows inside the query window (all of them without a window), cut into W runs
  const int w_lo = max(0, p.win_begin - row0);
  const int w_hi = max(w_lo, min(rows, (p.win_rows > 0 ? p.win_begin + p.win_rows : sp.len) - row0));
  const int run = (w_hi - w_lo + W - 1) / W;
  const int r_lo = min(w_hi, w_lo + warp * run), r_hi = min(w_hi, r_lo + run);
  const int32_t* src = block_idx + block_idx_row(p, seq, hq, sp.bos, row0 + r_lo);
  const int n = (r_hi - r_lo) * p.slots;
  int* cursor = cursor_all + warp * nb_lim;

  for (int i = threadIdx.x; i < W * nb_lim; i += 32 * W) cursor_all[i] = 0;
  __syncthreads();
  for (int e = lane; e < n; e += 32) {
    const int blk = src[e];
    if (blk >= 0 && blk < nb_lim) atomicAdd(&cursor[blk], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < nb_lim; i += 32 * W) {
    int at = off[i] + pre[(size_t)i * (group * C)];
#pragma unroll
    for (int w = 0; w < W; ++w) {
      const int t = cursor_all[w * nb_lim + i];
      cursor_all[w * nb_lim + i] = at;
      at += t;
    }
  }
  __syncthreads();

  int32_t* ro = rows_out + kv_row * capacity;
  int32_t* ho = heads_out + kv_row * capacity;
  int32_t* so = slots_out + kv_row * capacity;
  const unsigned lt = (1u << lane) - 1u;
  const int first_row = sp.bos + row0 + r_lo;
  // The entries are fetched a batch of kBatch steps ahead: one memory latency per batch
  // instead of one per step.
  constexpr int kBatch = 4;
  int nxt[kBatch];
#pragma unroll
  for (int j = 0; j < kBatch; ++j) {
    const int e = j * 32 + lane;
    nxt[j] = (e < n) ? src[e] : -1;
  }
  for (int e0 = 0; e0 < n; e0 += 32 * kBatch) {
    int cur[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      cur[j] = nxt[j];
      const int e = e0 + 32 * kBatch + j * 32 + lane;
      nxt[j] = (e < n) ? src[e] : -1;
    }
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
      const int e = e0 + j * 32 + lane;
      if (e0 + j * 32 >= n) break;                         // warp-uniform
      const int blk = cur[j];
      const bool valid = blk >= 0 && blk < nb_lim;
      const int key = valid ? blk : (0x40000000 + lane);
      const unsigned same = __match_any_sync(0xffffffffu, key);
      int base = 0;
      if (valid) base = cursor[blk];
      __syncwarp();
      if (valid && (same & lt) == 0) cursor[blk] = base + __popc(same);
      __syncwarp();
      if (valid) {
        const long long dst = base + __popc(same & lt);
        if (dst < capacity) {
          ro[dst] = first_row + e / p.slots;
          ho[dst] = hq;
          so[dst] = e % p.slots;
        }
      }
    }
  }
}

// warps per scatter CTA: as many runs side by side as their cursor arrays leave room for
static inline int scatter_warps_for(const moba_b200_problem& p) {
  const size_t hist_bytes = (size_t)p.num_blocks * sizeof(int);
  if (8 * hist_bytes <= 64 * 1024) return 8;
  if (4 * hist_bytes <= 200 * 1024) return 4;
  return 1;
}
void transpose_plan(const moba_b200_problem& p, int* chunk_rows, int* chunks, int* scatter_warps) {
  const TransposeGeom g = transpose_geom(p);
  *chunk_rows = g.chunk_rows; *chunks = g.chunks; *scatter_warps = scatter_warps_for(p);
}

template <int W>
static int launch_scatter(const moba_b200_problem& p, const int32_t* block_idx, const int32_t* cu,
                          const int32_t* tiles, const int32_t* col_offsets, int32_t* rows, int32_t* heads,
                          int32_t* slots, const TransposeGeom& g, long long capacity, cudaStream_t st) {
  const size_t smem = (size_t)W * p.num_blocks * sizeof(int);
  if (smem > 48 * 1024)
    MOBA_CUDA_OK(cudaFuncSetAttribute(scatter_kernel<W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const long long ctas = (long long)g.chunks * p.n_seq * p.q_heads;
  scatter_kernel<W><<<(unsigned)ctas, 32 * W, smem, st>>>(block_idx, cu, tiles, col_offsets, rows, heads, slots, p,
                                                           g.chunk_rows, g.chunks, capacity);
  MOBA_LAUNCH_OK("scatter_kernel");
  return MOBA_B200_OK;
}

int launch_transpose(const moba_b200_problem& p, const int32_t* block_idx, const int32_t* cu,
                     int32_t* col_nnz, int32_t* col_offsets, int32_t* order, int32_t* rows,
                     int32_t* heads, int32_t* slots, int32_t* work_items, void* scratch, size_t scratch_bytes,
                     cudaStream_t st) {
  const TransposeGeom g = transpose_geom(p);
  if (scratch_bytes < transpose_scratch_bytes(p)) {
    set_error("transpose: scratch has %zu bytes, needs %zu", scratch_bytes,
              transpose_scratch_bytes(p));
    return MOBA_B200_ESCRATCH;
  }
  const size_t hist_bytes = (size_t)p.num_blocks * sizeof(int);
  if (hist_bytes > 200 * 1024) {
    set_error("transpose: %d blocks per sequence exceed the shared-memory histogram", p.num_blocks);
    return MOBA_B200_EUNSUPPORTED;
  }
  const long long row_ctas = (long long)g.chunks * p.n_seq * p.q_heads;
  if (row_ctas > 0x7fffffffLL) {
    set_error("transpose: %lld (row chunk, sequence, head) units exceed the grid limit", row_ctas);
    return MOBA_B200_EUNSUPPORTED;
  }
  int32_t* tiles = static_cast<int32_t*>(scratch);
  int32_t* slot_counter = reinterpret_cast<int32_t*>(static_cast<unsigned char*>(scratch) + ((tile_count_bytes(p) + 15) & ~size_t(15)));
  if (sched_items_per_row(p) > 0x7fffffffLL || sched_part_slots(p) > 0x7fffffffLL) {
    set_error("transpose: chunk_tiles %d cuts the problem into too many work items", sched_chunk_tiles(p));
    return MOBA_B200_EUNSUPPORTED;
  }
  const int group = p.q_heads / p.kv_heads;
  const long long capacity = (long long)group * (p.win_rows > 0 ? p.win_rows : p.max_seqlen) * p.slots;
  if (hist_bytes > 48 * 1024) {
    MOBA_CUDA_OK(cudaFuncSetAttribute(count_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hist_bytes));
    MOBA_CUDA_OK(cudaFuncSetAttribute(offsets_order_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)hist_bytes));
  }
  { KernelTimer t__("count_kernel", st);
  count_kernel<<<(unsigned)row_ctas, 256, hist_bytes, st>>>(block_idx, cu, tiles, slot_counter, p, g.chunk_rows, g.chunks);
  MOBA_LAUNCH_OK("count_kernel"); }
  { KernelTimer t__("colscan_kernel", st);
  const unsigned per_row = (unsigned)((p.num_blocks + 3) / 4);
  colscan_kernel<<<per_row * (unsigned)(p.n_seq * p.kv_heads), 128, 0, st>>>(cu, tiles, col_nnz, p, g.chunk_rows, g.chunks, (int)per_row);
  MOBA_LAUNCH_OK("colscan_kernel"); }
  { KernelTimer t__("offsets_order_kernel", st);
  offsets_order_kernel<<<dim3(p.n_seq * p.kv_heads, (p.num_blocks + 127) / 128), 1024, hist_bytes, st>>>(
      col_nnz, col_offsets, order, p.num_blocks);
  MOBA_LAUNCH_OK("offsets_order_kernel"); }
  if (work_items != nullptr) {
    KernelTimer t__("work_items_kernel", st);
    unsigned* err = device_error_word();
    if (err == nullptr) { set_error("transpose: no device error word"); return MOBA_B200_ECUDA; }
    work_items_kernel<<<p.n_seq * p.kv_heads, 1024, 0, st>>>(col_nnz, order, reinterpret_cast<int4*>(work_items), slot_counter,
                                                            p.num_blocks, (int)sched_items_per_row(p), sched_chunk_tiles(p),
                                                            (int)sched_part_slots(p), err);
    MOBA_LAUNCH_OK("work_items_kernel");
  }
  { KernelTimer t__("scatter_kernel", st);
  const int w = scatter_warps_for(p);
  if (w == 8) return launch_scatter<8>(p, block_idx, cu, tiles, col_offsets, rows, heads, slots, g, capacity, st);
  if (w == 4) return launch_scatter<4>(p, block_idx, cu, tiles, col_offsets, rows, heads, slots, g, capacity, st);
  return launch_scatter<1>(p, block_idx, cu, tiles, col_offsets, rows, heads, slots, g, capacity, st); }
}

// ---------------------------------------------------------------------------
// Transpose for callers that cannot hand over scratch memory.
//
// Some hosts of this library may not allocate device memory at all: a serving
// process that lays out every byte of the GPU at start-up and forbids cudaMalloc
// afterwards (it synchronises the device and can fail once memory is
// fragmented), or a plugin that is handed nothing but its input and output
// buffers and has no allocator to ask. For them the per-chunk histogram of the
// transpose lives in this fixed array inside the library image. Every GPU that
// loads the library keeps these 8 MiB until the process exits.
//
// `g_transpose_scratch` names the array in device code. In host code the same
// name is only a handle for cudaGetSymbolAddress: passing it to a kernel as a
// pointer would hand the kernel a host address.
// ---------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_transpose_scratch[kStaticScratchBytes];

// Device address of the array on the current device; looked up once per device,
// with that device current, and cached.
static int static_scratch_address(void** out) {
  static void* table[64] = {nullptr};
  static std::mutex mu;
  int dev = -1;
  MOBA_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { set_error("device ordinal %d out of range", dev); return MOBA_B200_EUNSUPPORTED; }
  std::lock_guard<std::mutex> lock(mu);
  if (table[dev] == nullptr) {
    void* ptr = nullptr;
    MOBA_CUDA_OK(cudaGetSymbolAddress(&ptr, g_transpose_scratch));
    table[dev] = ptr;
  }
  *out = table[dev];
  return MOBA_B200_OK;
}

int launch_transpose_noalloc(const moba_b200_problem& p, const int32_t* block_idx, const int32_t* cu,
                             int32_t* col_nnz, int32_t* col_offsets, int32_t* order, int32_t* rows,
                             int32_t* heads, int32_t* slots, int32_t* work_items, cudaStream_t st) {
  const size_t need = transpose_scratch_bytes(p);
  if (need > kStaticScratchBytes) {
    set_error("transpose without caller scratch: this problem needs %zu bytes of scratch, the built-in "
              "array holds %zu; use moba_b200_transpose with a caller buffer", need, kStaticScratchBytes);
    return MOBA_B200_EUNSUPPORTED;
  }
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != MOBA_B200_OK) return rc;
  // Nothing in the array has to be cleared by the caller: the count pass writes every entry
  // the scan pass reads and resets the slot counter, so the previous call's contents are
  // simply overwritten.
  return launch_transpose(p, block_idx, cu, col_nnz, col_offsets, order, rows, heads, slots, work_items, scratch,
                          kStaticScratchBytes, st);
}

}  // namespace moba
