// Forward attention on tcgen05 tensor cores (bf16/f16, block_size 128,
// head_dim 64 or 128).
//
// Persistent CTAs (one per SM) walk the (sequence, kv head, block) columns in
// longest-first order, round-robin. Work is cut into tiles of 128 gathered
// queries; NB tiles (4 at head_dim 64, 2 at 128) are in flight per SM, each on
// its own TMEM buffer, output staging tile and softmax warpgroup, because one tile
// is a long chain of short dependent steps (gather -> MMA -> softmax -> MMA ->
// epilogue) and only several chains side by side keep the SM busy.
//   loader   (1 warp)    walks the work list, publishes each item's descriptor in shared
//                        memory one item ahead of its loads, TMA-loads its K block and V
//                        block (two buffers each at head_dim 64); zeroes the rows of a
//                        block that its sequence cuts short
//   mma      (2 threads) one issues S = Q K^T (M128 N128 K=D) tile after tile, the other
//                        O = P V (M128 N=D K128) with P as operand A **from TMEM**; each
//                        blocks on what its next tile needs, so a tile that becomes ready
//                        is issued without a polling round
//   movers   (head_dim 128 only: NB x 4 warps) copy the query rows of their warpgroup's next
//                        tile in and the staged output rows of its previous tile out; at
//                        head_dim 64 the softmax warps do both themselves (below)
//   softmax  (NB x 4 warps; warpgroup w owns tiles t = w mod NB)
//            - gathers the 128 query rows of its *next* tile with 16-byte asynchronous
//              copies, issued between the two passes over the current tile's scores: a
//              warp sustains only about 3 bytes per clock of such copies, so the copying
//              is spread over all 4 NB warps instead of a few dedicated ones;
//            - tcgen05.ld S, mask, exp2, row sum, P (16-bit pairs) -> tcgen05.st over the
//              scores already read (P never touches shared memory); then tcgen05.ld O,
//              normalise, stage in smem and store the partial output rows (eight or
//              sixteen lanes per row) and their log2-sum-exp at the (query, slot) addresses
// TMEM columns of a buffer: S [0,128), P over [0,64), O in [64,128) at head_dim 64 and in
// a second 128 columns at head_dim 128.
// A (query, block) pair is complete inside one tile, so nothing is rescaled
// here; the merge kernel combines a query's slots.
//
// Stands in for moba_fwd_kernel of the reference (src/moba/kernels/moba_fwd.py:229-425).
#include "common.cuh"
#include "sm100.cuh"

#include <type_traits>

namespace moba {
using namespace sm100;

namespace {

constexpr int kTile = 128;                 // queries per tile == keys per block
constexpr int kSub = kTile * 128;          // bytes of one [128 rows][64 elems] swizzled sub-tile

template <int D> struct FwdCfg {
  static constexpr int kSubs = D / 64;                 // sub-tiles per operand along the head dim
  static constexpr int kOperand = kSubs * kSub;        // bytes of K, V or one Q stage
  // Tiles in flight (TMEM buffers, output staging tiles, softmax warpgroups).
  static constexpr int kBufs = tensor_core_plan(D).fwd_tiles_in_flight;
  // Q stages form a ring over the CTA's tile sequence (tile t lives in stage t mod kQStages);
  // shared memory has no room for one stage per buffer at head_dim 64.
  static constexpr int kQStages = tensor_core_plan(D).fwd_q_stages;
  // P never goes through shared memory: it is written back to TMEM over the scores it was
  // computed from and read from there as operand A of P V. What each tile in flight keeps in
  // shared memory is a staging tile for its 16-bit output rows.
  static constexpr int kStageBytes = kOperand;         // [128][D] 16-bit
  // K and V buffers: with two, the next item's blocks load while this item's last tiles run.
  static constexpr int kKvBufs = (D == 64) ? 2 : 1;
  static constexpr int kSmemData = 2 * kKvBufs * kOperand + kQStages * kOperand + kBufs * kStageBytes;
  static constexpr int kSmem = kSmemData + 1024 /*align*/ + 10240 /*barriers, row tables*/;
  static constexpr int kMmaWarp = 4 * kBufs, kPvWarp = kMmaWarp + 1, kLoadWarp = kMmaWarp + 2;
  // With two tiles in flight the softmax warps are only eight, and copying the next tile's
  // query rows in and this tile's output rows out took half of a tile's time on them. There a
  // second set of warps ("movers", four per tile in flight) does both, beside the softmax warps.
  static constexpr bool kMovers = (kBufs == 2);
  static constexpr int kMoverWarp0 = kLoadWarp + 1;
  static constexpr int kMoverWarps = 4;                // per tile in flight (six were slower: 0.55 vs 0.49 ms on one KV head of cfg3)
  static constexpr int kThreads = (4 * kBufs + 3 + (kMovers ? kMoverWarps * kBufs : 0)) * 32;
};

struct Column {                            // one unit of work
  int kv_row, blk, n, lo, key0, keys, bos;
  size_t b;
};

struct Bars {
  uint64_t k_full[2], v_full[2], k_free[2], v_free[2], k_fix, v_fix;
  uint64_t q_full[4];                      // per buffer: the warpgroup's gathered Q tile has landed
  uint64_t q_empty[4];                     // per stage: the S MMA that read it has retired
  uint64_t s_full[4], p_full[4], o_full[4], so_free[4];
  uint64_t o_staged[2], stage_free[2];     // movers: a tile's output rows are staged / have left the staging tile
  uint64_t sp_free[2];                     // head_dim 128: the S / P columns of a buffer are free (its P V has retired)
  uint64_t col_full[8];                    // column descriptors published by the loader
  uint64_t drain[2];                       // all MMAs of an issuing thread have completed
  uint32_t tmem_base;
  int abort;
  Column cols[8];                          // ring: cols[i & 7] describes the CTA's i-th column; n < 0 ends the stream
  unsigned char* out_ptr[4][kTile];        // destination rows of the tile each warpgroup is storing
  int q_row[4][2][kTile];                  // per warpgroup, two gathers deep: row of the [B*T*Hq][D] view of q, -1 = none
};

// AND of a predicate over the 128 threads of a warpgroup (named barrier `id`). Every decision
// that steers a warpgroup past one of its own barriers is taken through this, so that a wait
// that gave up in some threads only can never leave the others alone at a barrier.
__device__ __forceinline__ bool group_all(bool pred, int id, int threads = 128) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.u32 q, %1, 0;\n\t"
      "bar.red.and.pred p, %2, %3, q;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(r) : "r"((uint32_t)pred), "r"(id), "r"(threads) : "memory");
  return r != 0;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// Work item `item` of the launch: the items of the (sequence, kv head) rows interleaved, each
// row's in its dispatch order (heaviest first). To this kernel an item is a column of its
// own: a block and a range of the block's pair list.
__device__ __forceinline__ bool load_column(Column& c, int item, const moba_b200_index& ix,
                                            const moba_b200_problem& p, const int32_t* cu, int n_kv_rows) {
  c.kv_row = item % n_kv_rows;
  WorkItem w;
  if (!load_work_item(w, ix, ix.col_nnz + (size_t)c.kv_row * p.num_blocks, c.kv_row, item / n_kv_rows)) {
    c.n = 0; c.keys = 0;
    return false;
  }
  c.blk = w.blk;
  c.n = w.n;
  c.lo = ix.col_offsets[(size_t)c.kv_row * (p.num_blocks + 1) + c.blk] + w.first;
  const int seq = c.kv_row / p.kv_heads;
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  c.b = p.packed ? 0 : (size_t)seq;
  c.bos = sp.bos;
  c.key0 = sp.bos + c.blk * kTile;
  c.keys = min(kTile, sp.bos + sp.len - c.key0);
  return c.n > 0 && c.keys > 0;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, typename T, typename TP>
__global__ void __launch_bounds__(FwdCfg<D>::kThreads, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                 const T* __restrict__ q, moba_b200_index ix, const int32_t* __restrict__ cu,
                 TP* __restrict__ part_o, float* __restrict__ part_lse, moba_b200_problem p, int n_items,
                 unsigned* error_word) {
  using Cfg = FwdCfg<D>;
  constexpr int NQ = Cfg::kQStages, NB = Cfg::kBufs, NKV = Cfg::kKvBufs;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = smem;                                     // NKV buffers
  unsigned char* sV = sK + NKV * Cfg::kOperand;
  unsigned char* sQ = sV + NKV * Cfg::kOperand;                 // NQ stages
  unsigned char* sO = sQ + NQ * Cfg::kOperand;                  // NB output staging tiles
  Bars* bars = reinterpret_cast<Bars*>(sO + NB * Cfg::kStageBytes);
  static_assert(sizeof(Bars) <= 10240, "barrier block outgrew its reservation");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_kv_rows = p.n_seq * p.kv_heads;
#ifdef MOBA_WAIT_STATS
  __shared__ unsigned long long wait_stats[32];
  if (threadIdx.x < 32) wait_stats[threadIdx.x] = 0;
  const long long kernel_t0 = clock64();
  const WaitCtx wc{&bars->abort, error_word, wait_stats};
#else
  const WaitCtx wc{&bars->abort, error_word};
#endif

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->k_full[i], 1); mbar_init(&bars->v_full[i], 1);
      mbar_init(&bars->k_free[i], 1); mbar_init(&bars->v_free[i], 1);
    }
    mbar_init(&bars->k_fix, 1); mbar_init(&bars->v_fix, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars->q_full[i], Cfg::kMovers ? Cfg::kMoverWarps : 4); mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->p_full[i], 4);
      mbar_init(&bars->o_full[i], 1); mbar_init(&bars->so_free[i], 4);
    }
    for (int i = 0; i < 8; ++i) mbar_init(&bars->col_full[i], 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->o_staged[i], 4); mbar_init(&bars->stage_free[i], Cfg::kMoverWarps); mbar_init(&bars->sp_free[i], 1);
    }
    mbar_init(&bars->drain[0], 1); mbar_init(&bars->drain[1], 1);
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == Cfg::kMmaWarp) tmem_alloc(&bars->tmem_base, 512);
  if (warp == Cfg::kLoadWarp && lane == 0) { tma_prefetch_desc(&k_map); tma_prefetch_desc(&v_map); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  const float cs = rsqrtf((float)D) * kLog2e;
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

  const bool is_mover = Cfg::kMovers && warp >= Cfg::kMoverWarp0;
  if (warp < 4 * NB || is_mover) {
    // ================ gather + softmax + epilogue warpgroups (and their movers) ================
    // warp group: four softmax warps, or kMoverWarps movers, of tile buffer wg
    const int gwarps = is_mover ? Cfg::kMoverWarps : 4;
    const int gw = is_mover ? warp - Cfg::kMoverWarp0 : warp;
    const int wg = gw / gwarps;                       // owns tiles with t % NB == wg and buffer wg
    const int gtid = (gw % gwarps) * 32 + lane;       // thread of the group
    const int gthreads = gwarps * 32;
    const int r = gtid;                               // row of the tile == TMEM lane (softmax warps; movers beyond 127 own no row)
    const int bar_id = 2 + wg + (is_mover ? NB : 0);  // named barrier of this group
    const uint32_t tbuf = tmem + ((uint32_t)((gtid >> 5 & 3) * 32) << 16) + wg * ((D == 64) ? 128 : 256);
    unsigned char* myO = sO + wg * Cfg::kStageBytes;            // staging of this warpgroup's output rows
    // TMEM columns of a buffer: scores [0, 128); P, 16-bit pairs, over [0, 64); O in [128 - D, 128)
    // at head_dim 64 and in a second 128 columns at head_dim 128.
    constexpr uint32_t kOCol = (D == 64) ? 64 : 128;
    constexpr uint32_t kBufCols = (D == 64) ? 128 : 256;
    constexpr int CPR = D / 8;                        // 16-byte chunks per gathered row
    constexpr int RPP = 128 / CPR;                    // rows per pass of the warpgroup

    // Position in the CTA's tile sequence: tile `t` is tile t - t0 of the CTA's `it`-th column.
    struct Cur { uint32_t it, t0, t; int nt; bool have; Column c; };
    // Moves `k` to the column that holds tile k.t. Returns 1 when found, 0 at the end of the
    // stream (or after a wait gave up), -1 when `blocking` is false and the descriptor has
    // not been published yet. The answer is the same in all 128 threads.
    auto locate = [&](Cur& k, bool blocking) -> int {
      for (;;) {
        if (!k.have) {
          bool ok = blocking ? mbar_wait(&bars->col_full[k.it & 7], (k.it >> 3) & 1, wc, 1)
                             : mbar_try_wait(&bars->col_full[k.it & 7], (k.it >> 3) & 1);
          ok = group_all(ok, bar_id, gthreads);
          if (!ok) return blocking ? 0 : -1;
          k.c = bars->cols[k.it & 7];
          if (k.c.n < 0) return 0;
          k.nt = (k.c.n + kTile - 1) / kTile;
          k.have = true;
        }
        if (k.t < k.t0 + (uint32_t)k.nt) return 1;
        k.t0 += (uint32_t)k.nt; ++k.it; k.have = false;
      }
    };
    // This thread's index entry (row r of tile k.t): query position, head, slot.
    auto load_entry = [&](const Cur& k, int& row, int& head, int& slot) {
      const int e = (int)(k.t - k.t0) * kTile + r;
      row = head = slot = 0;
      if (r < kTile && e < k.c.n) {
        const size_t o = (size_t)k.c.kv_row * ix.capacity + k.c.lo + e;
        row = ld_nc_pinned(ix.row_indices + o); head = ld_nc_pinned(ix.head_indices + o);
        slot = ld_nc_pinned(ix.slot_of_pair + o);
      }
    };
    // Copies the 128 query rows of tile k.t into its stage. `n_gather` alternates the row
    // table, so one barrier per gather is enough (the table of gather g is rewritten by
    // gather g + 2, behind the barrier of gather g + 1).
    uint32_t n_gather = 0;
    const uint64_t keep = l2_policy_evict_last();
    auto gather = [&](const Cur& k, int row, int head) {
      const bool live = r < kTile && (int)(k.t - k.t0) * kTile + r < k.c.n;
      int* tab = bars->q_row[wg][n_gather & 1];
      ++n_gather;
      if (r < kTile) tab[r] = live ? (int)((k.c.b * p.tokens + row) * p.q_heads + head) : -1;
      asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(gthreads) : "memory");
      const uint32_t qs = k.t % NQ, uq = k.t / NQ;
      if (uq >= 1) mbar_wait(&bars->q_empty[qs], (uq - 1) & 1, wc, 9);
      const uint32_t stage = smem_u32(sQ) + qs * Cfg::kOperand;
      if constexpr (Cfg::kMovers && Cfg::kMoverWarps != 4) {   // any number of threads: a row's pieces on neighbouring threads
        for (int j = gtid; j < kTile * CPR; j += gthreads) {
          const int rr = j / CPR, cc = j % CPR;
          const int ri = tab[rr];
          cp_async16_hint(stage + (cc >> 3) * kSub + swz128(rr, cc & 7), q + (size_t)(ri < 0 ? 0 : ri) * D + cc * 8,
                          ri < 0 ? 0u : 16u, keep);
        }
      } else {
        const int cc = r % CPR;
#pragma unroll
        for (int pass = 0; pass < CPR; ++pass) {
          const int rr = pass * RPP + r / CPR;
          const int ri = tab[rr];
          cp_async16_hint(stage + (cc >> 3) * kSub + swz128(rr, cc & 7), q + (size_t)(ri < 0 ? 0 : ri) * D + cc * 8,
                          ri < 0 ? 0u : 16u, keep);
        }
      }
      cp_async_commit();
    };

    // The staged 16-bit output rows of a tile -> global memory, eight or sixteen lanes per row.
    auto store_rows = [&](bool ok) {
      constexpr int CPRO = D / 8;                    // 16-byte chunks per output row
      if constexpr (Cfg::kMovers && Cfg::kMoverWarps != 4) {
        for (int j = gtid; j < kTile * CPRO; j += gthreads) {
          const int rr = j / CPRO, cc = j % CPRO;
          unsigned char* op = bars->out_ptr[wg][rr];
          const uint4 w = *reinterpret_cast<const uint4*>(myO + (cc >> 3) * kSub + swz128(rr, cc & 7));
          if (op != nullptr && ok) st_global_stream16(op + cc * 16, w);
        }
      } else {
        constexpr int RPPO = 128 / CPRO;             // rows per pass of the warpgroup
        const int cc = r % CPRO;
#pragma unroll
        for (int pass = 0; pass < CPRO; ++pass) {
          const int rr = pass * RPPO + r / CPRO;
          unsigned char* op = bars->out_ptr[wg][rr];
          const uint4 w = *reinterpret_cast<const uint4*>(myO + (cc >> 3) * kSub + swz128(rr, cc & 7));
          if (op != nullptr && ok) st_global_stream16(op + cc * 16, w);
        }
      }
    };

    Cur pf{0u, 0u, (uint32_t)wg, 0, false, Column{}};
    int n_row = 0, n_head = 0, n_slot = 0;
    bool more = locate(pf, true) == 1;
    if (more) load_entry(pf, n_row, n_head, n_slot);
    if (is_mover) {
      // ---- movers: copy the rows of this warpgroup's tiles in, a tile ahead of the softmax
      // warps, and the staged output rows of the tile before out ----
      for (uint32_t j = 0;; ++j) {
        const bool have_tile = more;
        if (have_tile) {
          gather(pf, n_row, n_head);
          cp_async_wait<0>();
          fence_proxy_async();
          mbar_arrive_warp(&bars->q_full[wg]);
        }
        if (j >= 1 && sizeof(TP) == 2) {
          const bool ok = mbar_wait(&bars->o_staged[wg], (j - 1) & 1, wc, 10);
          store_rows(ok);
          mbar_arrive_warp(&bars->stage_free[wg]);
        }
        if (!have_tile) break;
        pf.t += NB;
        more = locate(pf, true) == 1;
        if (more) load_entry(pf, n_row, n_head, n_slot);
      }
    } else {
    bool gathered = false;
    PHASE_CLOCK(ph);
    while (more) {
      const Cur cur = pf;
      const Column& c = cur.c;
      const int row = n_row, head = n_head, slot = n_slot;
      const uint32_t u = cur.t / NB;                   // how often this buffer has been used before
      const bool live = (int)(cur.t - cur.t0) * kTile + r < c.n;
      if (!Cfg::kMovers && !gathered) {                // first tile, or its descriptor came late
        gather(cur, row, head);
        cp_async_wait<0>();
        fence_proxy_async();
        mbar_arrive_warp(&bars->q_full[wg]);
      }
      PHASE_ADD(wc, 10, ph);                           // late gather
      TRACE(error_word, cur.t, 0);
      int jmax = c.keys - 1;
      if (p.causal && live && (row - c.bos) / kTile == c.blk) jmax = min(jmax, row - c.key0);
      // Away from the diagonal block and the ragged ends every row keeps all 128 keys; such
      // a warp runs without the per-element comparison.
      const bool all_open = __all_sync(0xffffffffu, jmax >= kTile - 1);

      const bool s_ok = mbar_wait(&bars->s_full[wg], u & 1, wc, 2);
      tc_fence_after();
      // The next tile of this warpgroup: its index entries are requested now and used after
      // the first pass over the scores; its rows are copied while the second pass runs.
      pf.t += NB;
      const int nxt = locate(pf, false);
      if (nxt == 1) load_entry(pf, n_row, n_head, n_slot);
      PHASE_ADD(wc, 11, ph);                           // s_full wait, next tile located
      TRACE(error_word, cur.t, 1);

      uint32_t v[32];
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        tmem_ld32(tbuf + ch * 32, v);
        tmem_ld_wait();
        if (all_open) {
#pragma unroll
          for (int k = 0; k < 32; k += 2)
            mx4[(k >> 1) & 3] = max3(mx4[(k >> 1) & 3], __uint_as_float(v[k]), __uint_as_float(v[k + 1]));
        } else {
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const float s = (ch * 32 + k <= jmax) ? __uint_as_float(v[k]) : -INFINITY;
            mx4[k & 3] = fmaxf(mx4[k & 3], s);
          }
        }
      }
      const float m2 = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * cs;

      PHASE_ADD(wc, 12, ph);                           // first pass (row maximum)
      TRACE(error_word, cur.t, 2);
      if (!Cfg::kMovers && nxt == 1) gather(pf, n_row, n_head);
      PHASE_ADD(wc, 13, ph);                           // copies of the next tile issued
      TRACE(error_word, cur.t, 3);

      float l4[4] = {0.f, 0.f, 0.f, 0.f};
      auto exp_pass = [&](auto masked) {
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(tbuf + ch * 32, v);
          tmem_ld_wait();
          // P of these 32 keys goes back over scores that have been read: chunk ch's 16-bit
          // pairs land in columns [16 ch, 16 ch + 16), all of them below column 32 (ch + 1).
          uint32_t pk[16];
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float pe[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float x = ex2(fmaf(__uint_as_float(v[g * 8 + k]), cs, -m2));
              if constexpr (decltype(masked)::value) pe[k] = (ch * 32 + g * 8 + k <= jmax) ? x : 0.f;
              else pe[k] = x;
              l4[k & 3] += pe[k];
            }
            pk[g * 4 + 0] = pack2<T>(pe[0], pe[1]); pk[g * 4 + 1] = pack2<T>(pe[2], pe[3]);
            pk[g * 4 + 2] = pack2<T>(pe[4], pe[5]); pk[g * 4 + 3] = pack2<T>(pe[6], pe[7]);
          }
          tmem_st16(tbuf + ch * 16, pk);
        }
        tmem_st_wait();
      };
      if (all_open) exp_pass(std::false_type{}); else exp_pass(std::true_type{});
      const float l = (l4[0] + l4[1]) + (l4[2] + l4[3]);
      PHASE_ADD(wc, 14, ph);                           // second pass (exp, P)
      TRACE(error_word, cur.t, 4);
      if (!Cfg::kMovers && nxt == 1) { cp_async_wait<0>(); fence_proxy_async(); }   // the next tile's rows have landed and are visible to the MMA
      tc_fence_before();
      mbar_arrive_warp(&bars->p_full[wg]);
      if (!Cfg::kMovers && nxt == 1) mbar_arrive_warp(&bars->q_full[wg]);
      PHASE_ADD(wc, 15, ph);                           // copies landed, fences, arrivals
      TRACE(error_word, cur.t, 5);

      // ---- epilogue of the same tile: O sits in the first D columns of this buffer ----
      const float inv = 1.f / l;
      const size_t dst_row = part_row(p, c.b, head, row) * (size_t)p.slots + slot;
      TP* dst = part_o + dst_row * D;
      // A wait that gave up leaves TMEM unspecified: the tile then stores nothing.
      const bool o_ok = mbar_wait(&bars->o_full[wg], u & 1, wc, 3) && s_ok;
      tc_fence_after();
      PHASE_ADD(wc, 16, ph);                           // o_full wait
      TRACE(error_word, cur.t, 6);
      // the movers have taken the previous tile's rows out of the staging tile
      if (Cfg::kMovers && sizeof(TP) == 2 && u >= 1) mbar_wait(&bars->stage_free[wg], (u - 1) & 1, wc, 11);
#pragma unroll 1
      for (int ch = 0; ch < D / 32; ++ch) {
        tmem_ld32(tbuf + kOCol + ch * 32, v);
        tmem_ld_wait();
        if (sizeof(TP) == 2) {
          // Stage the 16-bit tile in shared memory: one row per thread straight to global
          // memory would touch 32 lines per instruction.
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
            w.y = pack2<T>(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
            w.z = pack2<T>(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
            w.w = pack2<T>(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(myO + (ch >> 1) * kSub + swz128(r, (ch & 1) * 4 + g)) = w;
          }
        } else if (live && o_ok) {
          float4* d4 = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(dst) + ch * 128);
#pragma unroll
          for (int g = 0; g < 8; ++g)
            d4[g] = make_float4(__uint_as_float(v[g * 4 + 0]) * inv, __uint_as_float(v[g * 4 + 1]) * inv,
                                __uint_as_float(v[g * 4 + 2]) * inv, __uint_as_float(v[g * 4 + 3]) * inv);
        }
      }
      tc_fence_before();
      mbar_arrive_warp(&bars->so_free[wg]);               // the TMEM buffer may be overwritten
      PHASE_ADD(wc, 17, ph);                           // O read and staged
      TRACE(error_word, cur.t, 7);
      if (live && o_ok) st_global_stream_f32(part_lse + dst_row, m2 + log2f(l));
      if (sizeof(TP) == 2) {
        bars->out_ptr[wg][r] = (live && o_ok) ? reinterpret_cast<unsigned char*>(dst) : nullptr;
        if constexpr (Cfg::kMovers) {
          mbar_arrive_warp(&bars->o_staged[wg]);       // (releasing: the movers see the rows and the table)
        } else {
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
          store_rows(true);
          asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");   // the staging tile may be written again
        }
      }
      PHASE_ADD(wc, 18, ph);                           // partial rows stored
      TRACE(error_word, cur.t, 8);

      if (nxt == 1) { gathered = true; continue; }
      if (nxt == 0) break;
      more = locate(pf, true) == 1;                    // the descriptor was not there in time
      if (more) load_entry(pf, n_row, n_head, n_slot);
      gathered = false;
    }
    }
  }
  else if (warp == Cfg::kMmaWarp || warp == Cfg::kPvWarp) {
    // ============================== MMA issuers ==============================
    // Two threads feed the tensor core, each walking the CTA's tiles in order and blocking
    // on exactly what its next MMA needs: a tile is issued as soon as its inputs are there.
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(0, 128, 128, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(0, 128, D, 0, 1);
      const uint32_t fbits = (fmt << 7) | (fmt << 10);
      const uint32_t aQ = smem_u32(sQ);
      constexpr uint32_t kOCol = (D == 64) ? 64 : 128, kBufCols = (D == 64) ? 128 : 256;
      const bool is_s = warp == Cfg::kMmaWarp;
      uint32_t t = 0, pt = 0;                                   // tiles issued, cut-short columns seen
      for (uint32_t it = 0;; ++it) {
        if (!mbar_wait(&bars->col_full[it & 7], (it >> 3) & 1, wc, 20)) break;
        const int n = bars->cols[it & 7].n;
        if (n < 0) break;
        const int nt = (n + kTile - 1) / kTile;
        const bool partial = bars->cols[it & 7].keys < kTile;
        const uint32_t kb = it % NKV, ku = it / NKV;             // K/V buffer of the item, its earlier uses
        const uint32_t aK = smem_u32(sK) + kb * Cfg::kOperand, aV = smem_u32(sV) + kb * Cfg::kOperand;
        for (int i = 0; i < nt; ++i, ++t) {
          const uint32_t b = t % NB, u = t / NB;
          if (is_s) {
            // ---- S = Q K^T of tile t ----
            const uint32_t qs = t % NQ;
            mbar_wait(&bars->q_full[b], u & 1, wc, 21);
            // The buffer's columns: where O has columns of its own (head_dim 128) the scores of
            // the next tile only wait for P V of the previous one, not for its O to be read out.
            if (u >= 1) mbar_wait(D == 128 ? &bars->sp_free[b] : &bars->so_free[b], (u - 1) & 1, wc, 22);
            if (i == 0) {
              mbar_wait(&bars->k_full[kb], ku & 1, wc, 23);
              if (partial) mbar_wait(&bars->k_fix, pt & 1, wc, 23);
            }
            tc_fence_after();
            TRACE(error_word, t, 0);
            const uint32_t qb = aQ + qs * Cfg::kOperand;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const uint32_t o = (ks >> 2) * kSub + (ks & 3) * 32;
              umma_f16(tmem + b * kBufCols, make_sdesc(qb + o, 16, 1024), make_sdesc(aK + o, 16, 1024),
                       idesc_s | fbits, ks > 0);
            }
            TRACE(error_word, t, 1);
            umma_commit(&bars->s_full[b]);
            umma_commit(&bars->q_empty[qs]);
            if (i == nt - 1) umma_commit(&bars->k_free[kb]);
          } else {
            // ---- O = P V of tile t ----
            mbar_wait(&bars->p_full[b], u & 1, wc, 24);
            if (D == 128 && u >= 1) mbar_wait(&bars->so_free[b], (u - 1) & 1, wc, 24);   // the O columns have been read out
            if (i == 0) {
              mbar_wait(&bars->v_full[kb], ku & 1, wc, 25);
              if (partial) mbar_wait(&bars->v_fix, pt & 1, wc, 25);
            }
            tc_fence_after();
            TRACE(error_word, t, 0);
            // operand A: P from TMEM, 16 keys (eight columns of 16-bit pairs) per step
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
              umma_f16_ts(tmem + b * kBufCols + kOCol, tmem + b * kBufCols + ks * 8,
                          make_sdesc(aV + ks * 2048, kSub, 1024), idesc_o | fbits, ks > 0);
            }
            TRACE(error_word, t, 1);
            umma_commit(&bars->o_full[b]);
            if (D == 128) umma_commit(&bars->sp_free[b]);
            if (i == nt - 1) umma_commit(&bars->v_free[kb]);
          }
        }
        if (partial) ++pt;
      }
      // Every MMA of this thread has completed before the CTA lets go of its TMEM, also on
      // the way out of a run that gave up on a wait.
      umma_commit(&bars->drain[is_s ? 0 : 1]);
      mbar_wait_quiet(&bars->drain[is_s ? 0 : 1], 0);
    }
    __syncwarp();
  } else {
    // ================== work-list walker and K/V TMA loader ==================
    // The only warp that resolves columns (three dependent global loads each); it runs
    // ahead of everybody and publishes the descriptors through a ring in shared memory.
    // All 32 lanes run the loop; lane 0 publishes and issues the loads, and the whole warp
    // zeroes the rows of a block that the end of its sequence cuts short (they belong to
    // the next sequence, or to the next batch row).
    uint32_t it_cnt = 0;
    const uint64_t keep = l2_policy_evict_last();
    // The list is sorted longest first; CTAs take it in alternating direction
    // (0..G-1, G-1..0, ...) so that no CTA collects the largest of every round.
    const int G = (int)gridDim.x;
    const size_t index_elems = (size_t)n_kv_rows * ix.capacity;
    auto item_of = [&](int round) { return round * G + ((round & 1) ? (G - 1 - (int)blockIdx.x) : (int)blockIdx.x); };
    // The index entries of a column are read by the softmax warps a tile at a time, straight
    // from global memory; asking the L2 for them a column ahead turns a DRAM round trip per
    // tile into an L2 hit.
    auto prefetch_entries = [&](int round) {
      const int item = item_of(round);
      Column c;
      if (round * G >= n_items || item >= n_items || !load_column(c, item, ix, p, cu, n_kv_rows)) return;
      if (lane < 3) {
        const int32_t* arr = lane == 0 ? ix.row_indices : (lane == 1 ? ix.head_indices : ix.slot_of_pair);
        l2_prefetch_i32(arr, (size_t)c.kv_row * ix.capacity + c.lo, c.n, index_elems);
      }
    };
    // The next item with pairs at or after `round` (its round is returned, -1 at the end).
    auto find = [&](Column& c, int round) {
      for (; round * G < n_items; ++round) {
        const int item = item_of(round);
        if (item < n_items && load_column(c, item, ix, p, cu, n_kv_rows)) return round;
      }
      return -1;
    };
    // Descriptor number `n` of the stream. The ring holds eight and the descriptors run one
    // item ahead of the K/V loads: a descriptor is overwritten when the MMAs of the item five
    // places behind it have long retired.
    auto publish = [&](const Column& c, uint32_t n) {
      __syncwarp();
      if (lane == 0) {
        bars->cols[n & 7] = c;
        mbar_arrive(&bars->col_full[n & 7]);
      }
    };
    Column c, c_next;
    int round = find(c, 0);
    if (round >= 0) { prefetch_entries(round); publish(c, 0); }
    while (round >= 0) {
      // The softmax warps look for their next tile while they work on the current one; at the
      // last tiles of an item that is a tile of the next item, so its descriptor (and, in the
      // L2, its index entries) must be there before this item's K and V are even loaded.
      const int round_next = find(c_next, round + 1);
      if (round_next >= 0) { prefetch_entries(round_next); publish(c_next, it_cnt + 1); }
      if (*wc.abort) break;                                 // no new loads once a wait gave up
      const int kvh = c.kv_row % p.kv_heads;
      const int tok0 = (int)(c.b * p.tokens) + c.key0;
      const uint32_t kb = it_cnt % NKV, ku = it_cnt / NKV;     // buffer of this item, its earlier uses
      unsigned char* bK = sK + kb * Cfg::kOperand;
      unsigned char* bV = sV + kb * Cfg::kOperand;
      if (ku >= 1) mbar_wait(&bars->k_free[kb], (ku - 1) & 1, wc, 4);
      if (lane == 0) {
        mbar_expect_tx(&bars->k_full[kb], Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d_hint(bK + s * kSub, &k_map, &bars->k_full[kb], s * 64, kvh, tok0, keep);
      }
      if (ku >= 1) mbar_wait(&bars->v_free[kb], (ku - 1) & 1, wc, 5);
      if (lane == 0) {
        mbar_expect_tx(&bars->v_full[kb], Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d_hint(bV + s * kSub, &v_map, &bars->v_full[kb], s * 64, kvh, tok0, keep);
      }
      if (c.keys < kTile) {
        const int dead = kTile - c.keys;
        mbar_wait(&bars->k_full[kb], ku & 1, wc, 7);
        for (int i = lane; i < dead * 8 * Cfg::kSubs; i += 32) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(bK + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive_warp(&bars->k_fix);
        mbar_wait(&bars->v_full[kb], ku & 1, wc, 8);
        for (int i = lane; i < dead * 8 * Cfg::kSubs; i += 32) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(bV + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive_warp(&bars->v_fix);
      }
      ++it_cnt;
      c = c_next;
      round = round_next;
    }
    __syncwarp();
    if (lane == 0) {
      bars->cols[it_cnt & 7].n = -1;                          // end of the stream
      mbar_arrive(&bars->col_full[it_cnt & 7]);
      // No load may be in flight into this CTA's shared memory when it exits.
      for (uint32_t back = 1; back <= (uint32_t)NKV && back <= it_cnt; ++back) {
        const uint32_t n = it_cnt - back;
        mbar_wait_quiet(&bars->k_full[n % NKV], (n / NKV) & 1);
        mbar_wait_quiet(&bars->v_full[n % NKV], (n / NKV) & 1);
      }
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == Cfg::kMmaWarp) tmem_dealloc(tmem, 512);
#ifdef MOBA_WAIT_STATS
  if (threadIdx.x < 32) {
    unsigned long long* out = reinterpret_cast<unsigned long long*>(error_word + 64) + (size_t)blockIdx.x * 32;
    out[threadIdx.x] = threadIdx.x == 31 ? (unsigned long long)(clock64() - kernel_t0) : wait_stats[threadIdx.x];
  }
#endif
}

template <int D, typename T, typename TP>
int launch_one(const moba_b200_problem& p, const CUtensorMap& km, const CUtensorMap& vm, const void* q,
               const moba_b200_index& ix, const int32_t* cu, void* part_o, float* part_lse, int n_items,
               unsigned* err, cudaStream_t st) {
  auto kern = fwd_sm100_kernel<D, T, TP>;
  MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<D>::kSmem));
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = n_items < sms ? n_items : sms;
  kern<<<grid, FwdCfg<D>::kThreads, FwdCfg<D>::kSmem, st>>>(km, vm, (const T*)q, ix, cu, (TP*)part_o, part_lse, p,
                                                             n_items, err);
  MOBA_LAUNCH_OK("fwd_sm100_kernel");
  return MOBA_B200_OK;
}

}  // namespace

bool fwd_sm100_supported(const moba_b200_problem& p) {
  return (p.dtype == MOBA_B200_BF16 || p.dtype == MOBA_B200_F16) && p.block_size == 128 &&
         (p.head_dim == 64 || p.head_dim == 128) &&
         (long long)p.batch * p.tokens * p.q_heads < 0x7fffffffLL;
}

int launch_fwd_sm100(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                     const moba_b200_index& ix, const int32_t* cu, void* part_o, float* part_lse,
                     cudaStream_t st) {
  KernelTimer timer__("fwd_sm100_kernel", st);
  unsigned* err = device_error_word();
  if (err == nullptr) { set_error("forward: no device error word"); return MOBA_B200_ECUDA; }
  CUtensorMap km, vm;
  const uint64_t rows = (uint64_t)p.batch * p.tokens;
  int rc = encode_rows_map(&km, k, rows, p.kv_heads, p.head_dim, 128);
  if (rc) return rc;
  rc = encode_rows_map(&vm, v, rows, p.kv_heads, p.head_dim, 128);
  if (rc) return rc;
  if (ix.work_items == nullptr || ix.items_per_row <= 0) {
    set_error("forward: the index carries no work items (build it with moba_b200_transpose)");
    return MOBA_B200_EINVAL;
  }
  const long long n_items_ll = (long long)ix.items_per_row * p.n_seq * p.kv_heads;
  if (n_items_ll > 0x7fffffffLL) { set_error("forward: too many work items"); return MOBA_B200_EUNSUPPORTED; }
  const int n_items = (int)n_items_ll;
  const bool bf = p.dtype == MOBA_B200_BF16;
#define GO(D, T, TP) return launch_one<D, T, TP>(p, km, vm, q, ix, cu, part_o, part_lse, n_items, err, st)
  if (p.head_dim == 64) {
    if (bf) { if (p.part_f32) GO(64, __nv_bfloat16, float); else GO(64, __nv_bfloat16, __nv_bfloat16); }
    else { if (p.part_f32) GO(64, __half, float); else GO(64, __half, __half); }
  } else {
    if (bf) { if (p.part_f32) GO(128, __nv_bfloat16, float); else GO(128, __nv_bfloat16, __nv_bfloat16); }
    else { if (p.part_f32) GO(128, __half, float); else GO(128, __half, __half); }
  }
#undef GO
  return MOBA_B200_OK;
}

}  // namespace moba
