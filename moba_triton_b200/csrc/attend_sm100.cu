// Forward attention on tcgen05 tensor cores (bf16/f16, block_size 128,
// head_dim 64 or 128).
//
// Persistent CTAs (one per SM) walk the (sequence, kv head, block) columns in
// longest-first order, round-robin. Work is cut into tiles of 128 gathered
// queries; NB tiles (4 at head_dim 64, 2 at 128) are in flight per SM, each on
// its own TMEM buffer, P buffer and softmax warpgroup, because one tile is a
// long chain of short dependent steps (MMA -> softmax -> MMA -> epilogue) and
// only several chains side by side keep the SM busy.
//   loader   (1 thread)  walks the work list, publishes each column's descriptor in
//                        shared memory, TMA-loads its K block and V block
//   gather   (2 warps)   128 selected query rows per tile -> swizzled smem, by TMA
//                        tile::gather4 (warp 0, which resolves the rows) and by 16-byte
//                        asynchronous copies (warp 1) side by side
//   mma      (1 thread)  S = Q K^T (M128 N128 K=D), then O = P V (M128 N=D K128) written
//                        over the first D columns of the same TMEM buffer
//   softmax  (NB x 4 warps; warpgroup w owns tiles t = w mod NB) tcgen05.ld S,
//            mask, exp2, row sum, P (16-bit) -> smem; then tcgen05.ld O, normalise,
//            stage in smem and store the partial output rows (eight or sixteen lanes
//            per row) and their log2-sum-exp at the (query, slot) addresses
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
  // Tiles in flight (TMEM / P buffers, softmax warpgroups). At head_dim 64 twenty warps of 96
  // registers fit: 4 warpgroups + 2 gather warps measured 0.45 ms at [1,131072,4,64] (the gather
  // warps are the busy ones), 3 + 6 measured 0.49 ms (then the softmax warps are).
  static constexpr int kBufs = (D == 64) ? 4 : 2;
  static constexpr int kQStages = (D == 64) ? (kBufs >= 4 ? 3 : 4) : 2;
  // Gather warps: warp 0 resolves rows and requests the first kTmaRows of a tile by TMA,
  // the others share the 16-byte copies of the rest (a warp sustains ~3 B/clk of those).
  static constexpr int kGatherWarps = 2;
  static constexpr int kGatherThreads = 32 * kGatherWarps;
  static constexpr int kTmaRows = 72;                  // 64 ... 104 measured; 72 (and 64) best
  static constexpr int kPBytes = 2 * kSub;             // [128][128] 16-bit
  static constexpr int kSmemData = 2 * kOperand + kQStages * kOperand + kBufs * kPBytes;
  static constexpr int kSmem = kSmemData + 1024 /*align*/ + 10240 /*barriers, pointers*/;
  static constexpr int kMmaWarp = 4 * kBufs, kLoadWarp = kMmaWarp + 1, kGatherWarp0 = kMmaWarp + 2;
  static constexpr int kThreads = (4 * kBufs + 2 + kGatherWarps) * 32;
};

struct Column {                            // one unit of work
  int kv_row, blk, n, lo, key0, keys, bos;
  size_t b;
};

struct Bars {
  uint64_t k_full, v_full, k_fix, v_fix, k_free, v_free;
  uint64_t q_full[4], q_empty[4];
  uint64_t s_full[4], p_full[4], o_full[4], so_free[4];
  uint64_t col_full[4];                    // column descriptors published by the loader thread
  uint64_t drain;                          // all MMAs of the CTA have completed
  uint32_t tmem_base;
  int abort;
  Column cols[4];                          // ring: cols[i & 3] describes the CTA's i-th column; n < 0 ends the stream
  unsigned char* out_ptr[4][kTile];        // destination rows of the tile each warpgroup is storing
  alignas(16) int row_idx[2][kTile];       // rows of the [batch * tokens * heads] view of q, two consecutive tiles
};

__device__ __forceinline__ bool load_column(Column& c, int item, const moba_b200_index& ix,
                                            const moba_b200_problem& p, const int32_t* cu, int n_kv_rows) {
  const int r = item / n_kv_rows;
  c.kv_row = item % n_kv_rows;
  c.blk = ix.order[(size_t)c.kv_row * p.num_blocks + r];
  c.n = ix.col_nnz[(size_t)c.kv_row * p.num_blocks + c.blk];
  c.lo = ix.col_offsets[(size_t)c.kv_row * (p.num_blocks + 1) + c.blk];
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
                 const __grid_constant__ CUtensorMap q_map, const T* __restrict__ q, moba_b200_index ix, const int32_t* __restrict__ cu,
                 TP* __restrict__ part_o, float* __restrict__ part_lse, moba_b200_problem p, int n_items,
                 unsigned* error_word) {
  using Cfg = FwdCfg<D>;
  constexpr int NQ = Cfg::kQStages, NB = Cfg::kBufs;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = smem;
  unsigned char* sV = sK + Cfg::kOperand;
  unsigned char* sQ = sV + Cfg::kOperand;                       // NQ stages
  unsigned char* sP = sQ + NQ * Cfg::kOperand;                  // NB buffers
  Bars* bars = reinterpret_cast<Bars*>(sP + NB * Cfg::kPBytes);

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
    mbar_init(&bars->k_full, 1); mbar_init(&bars->v_full, 1);
    mbar_init(&bars->k_fix, Cfg::kGatherThreads); mbar_init(&bars->v_fix, Cfg::kGatherThreads);
    mbar_init(&bars->k_free, 1); mbar_init(&bars->v_free, 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bars->q_full[i], Cfg::kGatherWarps); mbar_init(&bars->q_empty[i], 1);
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->p_full[i], 128);
      mbar_init(&bars->o_full[i], 1); mbar_init(&bars->so_free[i], 128);
      mbar_init(&bars->col_full[i], 1);
    }
    mbar_init(&bars->drain, 1);
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == Cfg::kMmaWarp) tmem_alloc(&bars->tmem_base, 512);
  if (warp == Cfg::kLoadWarp && lane == 0) { tma_prefetch_desc(&k_map); tma_prefetch_desc(&v_map); tma_prefetch_desc(&q_map); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  const float cs = rsqrtf((float)D) * kLog2e;
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

  if (warp < 4 * NB) {
    // ===================== softmax + epilogue warpgroups =====================
    const int wg = warp >> 2;                         // owns tiles with t % NB == wg and buffer wg
    const int r = (warp & 3) * 32 + lane;             // row of the tile == TMEM lane
    const uint32_t tbuf = tmem + ((uint32_t)((warp & 3) * 32) << 16) + wg * 128;
    unsigned char* myP = sP + wg * Cfg::kPBytes;
    uint32_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
      mbar_wait(&bars->col_full[it & 3], (it >> 2) & 1, wc, 1);
      const Column c = bars->cols[it & 3];
      if (c.n < 0) break;
      const int nt = (c.n + kTile - 1) / kTile;
      const int32_t* rows_i = ix.row_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      const int32_t* heads_i = ix.head_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      const int32_t* slots_i = ix.slot_of_pair + (size_t)c.kv_row * ix.capacity + c.lo;
      // Index entries of this warpgroup's next tile are fetched one tile ahead.
      const int i_first = (int)((wg + NB - (t0 % NB)) % NB);
      int n_row = 0, n_head = 0, n_slot = 0;
      if (i_first < nt && i_first * kTile + r < c.n) {
        const int e0 = i_first * kTile + r;
        n_row = rows_i[e0]; n_head = heads_i[e0]; n_slot = slots_i[e0];
      }
      for (int i = i_first; i < nt; i += NB) {
        const uint32_t u = (t0 + i) / NB;             // how often this buffer has been used before
        const int e = i * kTile + r;
        const bool live = e < c.n;
        const int row = n_row, head = n_head, slot = n_slot;
        {
          const int e2 = e + NB * kTile;
          n_row = n_head = n_slot = 0;
          if (i + NB < nt && e2 < c.n) {
            n_row = ld_nc_pinned(rows_i + e2); n_head = ld_nc_pinned(heads_i + e2); n_slot = ld_nc_pinned(slots_i + e2);
          }
        }
        int jmax = c.keys - 1;
        if (p.causal && live && (row - c.bos) / kTile == c.blk) jmax = min(jmax, row - c.key0);

        mbar_wait(&bars->s_full[wg], u & 1, wc, 2);
        tc_fence_after();
        uint32_t v[32];
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(tbuf + ch * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const float s = (ch * 32 + k <= jmax) ? __uint_as_float(v[k]) : -INFINITY;
            mx4[k & 3] = fmaxf(mx4[k & 3], s);
          }
        }
        const float m2 = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * cs;
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          tmem_ld32(tbuf + ch * 32, v);
          tmem_ld_wait();
          unsigned char* dst_sub = myP + (ch >> 1) * kSub;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float pe[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float x = ex2(fmaf(__uint_as_float(v[g * 8 + k]), cs, -m2));
              pe[k] = (ch * 32 + g * 8 + k <= jmax) ? x : 0.f;
              l4[k & 3] += pe[k];
            }
            uint4 w;
            w.x = pack2<T>(pe[0], pe[1]); w.y = pack2<T>(pe[2], pe[3]);
            w.z = pack2<T>(pe[4], pe[5]); w.w = pack2<T>(pe[6], pe[7]);
            *reinterpret_cast<uint4*>(dst_sub + swz128(r, (ch & 1) * 4 + g)) = w;
          }
        }
        const float l = (l4[0] + l4[1]) + (l4[2] + l4[3]);
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(&bars->p_full[wg]);

        // ---- epilogue of the same tile: O sits in the first D columns of this buffer ----
        const float inv = 1.f / l;
        const size_t dst_row = ((c.b * p.q_heads + head) * p.tokens + row) * (size_t)p.slots + slot;
        TP* dst = part_o + dst_row * D;
        mbar_wait(&bars->o_full[wg], u & 1, wc, 3);
        tc_fence_after();
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          tmem_ld32(tbuf + ch * 32, v);
          tmem_ld_wait();
          if (sizeof(TP) == 2) {
            // Stage the 16-bit tile in this buffer's P region (its MMA has retired): one row
            // per thread straight to global memory would touch 32 lines per instruction.
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint4 w;
              w.x = pack2<T>(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
              w.y = pack2<T>(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
              w.z = pack2<T>(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
              w.w = pack2<T>(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
              *reinterpret_cast<uint4*>(myP + (ch >> 1) * kSub + swz128(r, (ch & 1) * 4 + g)) = w;
            }
          } else if (live) {
            float4* d4 = reinterpret_cast<float4*>(reinterpret_cast<unsigned char*>(dst) + ch * 128);
#pragma unroll
            for (int g = 0; g < 8; ++g)
              d4[g] = make_float4(__uint_as_float(v[g * 4 + 0]) * inv, __uint_as_float(v[g * 4 + 1]) * inv,
                                  __uint_as_float(v[g * 4 + 2]) * inv, __uint_as_float(v[g * 4 + 3]) * inv);
          }
        }
        tc_fence_before();
        mbar_arrive(&bars->so_free[wg]);               // the TMEM buffer may be overwritten
        if (live) part_lse[dst_row] = m2 + log2f(l);
        if (sizeof(TP) == 2) {
          bars->out_ptr[wg][r] = live ? reinterpret_cast<unsigned char*>(dst) : nullptr;
          asm volatile("bar.sync %0, 128;" ::"r"(2 + wg) : "memory");
          constexpr int CPRO = D / 8;                  // 16-byte chunks per output row
          constexpr int RPPO = 128 / CPRO;             // rows per pass of the warpgroup
          const int cc = r % CPRO;
#pragma unroll
          for (int pass = 0; pass < CPRO; ++pass) {
            const int rr = pass * RPPO + r / CPRO;
            unsigned char* op = bars->out_ptr[wg][rr];
            const uint4 w = *reinterpret_cast<const uint4*>(myP + (cc >> 3) * kSub + swz128(rr, cc & 7));
            if (op != nullptr) *reinterpret_cast<uint4*>(op + cc * 16) = w;
          }
          asm volatile("bar.sync %0, 128;" ::"r"(2 + wg) : "memory");   // the staging area is P again
        }
      }
      t0 += nt;
    }
  }
  else if (warp == Cfg::kMmaWarp) {
    // ============================== MMA issuer ==============================
    // One thread feeds the tensor core. It polls instead of blocking so that whichever of
    // "next S tile" and "next P.V tile" becomes possible first is issued first.
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(0, 128, 128, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(0, 128, D, 0, 1);
      const uint32_t fbits = (fmt << 7) | (fmt << 10);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aP = smem_u32(sP);
      struct Cursor { uint32_t it, pt; int i, nt, partial; bool have, end; };
      Cursor cs_{0, 0, 0, 0, 0, false, false}, cp_{0, 0, 0, 0, 0, false, false};
      auto refill = [&](Cursor& k) {
        if (k.have || k.end) return;
        if (!mbar_try_wait(&bars->col_full[k.it & 3], (k.it >> 2) & 1)) return;
        const int n = bars->cols[k.it & 3].n;
        if (n < 0) { k.end = true; return; }
        k.nt = (n + kTile - 1) / kTile;
        k.partial = bars->cols[k.it & 3].keys < kTile;
        k.i = 0;
        k.have = true;
      };
      auto step = [&](Cursor& k) {
        if (++k.i == k.nt) { k.have = false; ++k.it; if (k.partial) ++k.pt; }
      };
      uint32_t ns = 0, np = 0, idle = 0;
      while (true) {
        bool progressed = false;
        // ---- S = Q K^T of tile ns ----
        refill(cs_);
        if (cs_.have) {
          const uint32_t b = ns % NB, u = ns / NB, qs = ns % NQ, uq = ns / NQ;
          bool ok = mbar_try_wait(&bars->q_full[qs], uq & 1);
          if (ok && u >= 1) ok = mbar_try_wait(&bars->so_free[b], (u - 1) & 1);
          if (ok && cs_.i == 0) {
            ok = mbar_try_wait(&bars->k_full, cs_.it & 1);
            if (ok && cs_.partial) ok = mbar_try_wait(&bars->k_fix, cs_.pt & 1);
          }
          if (ok) {
            tc_fence_after();
            const uint32_t qb = aQ + qs * Cfg::kOperand;
#pragma unroll
            for (int ks = 0; ks < D / 16; ++ks) {
              const uint32_t o = (ks >> 2) * kSub + (ks & 3) * 32;
              umma_f16(tmem + b * 128, make_sdesc(qb + o, 16, 1024), make_sdesc(aK + o, 16, 1024),
                       idesc_s | fbits, ks > 0);
            }
            umma_commit(&bars->s_full[b]);
            umma_commit(&bars->q_empty[qs]);
            if (cs_.i == cs_.nt - 1) umma_commit(&bars->k_free);
            step(cs_);
            ++ns;
            progressed = true;
          }
        }
        // ---- O = P V of tile np ----
        if (np < ns) {
          refill(cp_);
          if (cp_.have) {
            const uint32_t b = np % NB, u = np / NB;
            bool ok = mbar_try_wait(&bars->p_full[b], u & 1);
            if (ok && cp_.i == 0) {
              ok = mbar_try_wait(&bars->v_full, cp_.it & 1);
              if (ok && cp_.partial) ok = mbar_try_wait(&bars->v_fix, cp_.pt & 1);
            }
            if (ok) {
              tc_fence_after();
              const uint32_t pb = aP + b * Cfg::kPBytes;
#pragma unroll
              for (int ks = 0; ks < 8; ++ks) {
                umma_f16(tmem + b * 128, make_sdesc(pb + (ks >> 2) * kSub + (ks & 3) * 32, 16, 1024),
                         make_sdesc(aV + ks * 2048, kSub, 1024), idesc_o | fbits, ks > 0);
              }
              umma_commit(&bars->o_full[b]);
              if (cp_.i == cp_.nt - 1) umma_commit(&bars->v_free);
              step(cp_);
              ++np;
              progressed = true;
            }
          }
        }
        if (cs_.end && np == ns) break;
        if (progressed) { idle = 0; continue; }
        if ((++idle & 1023u) == 0u) {
          if (*wc.abort) break;
          if (idle >= (1u << 24)) {                     // bounded: give up, flag the error
            *wc.abort = 1;
            atomicOr(error_word, kErrWaitTimeout);
            break;
          }
        }
      }
      // Every MMA has completed before the CTA lets go of its TMEM, also on the way out of
      // a run that gave up on a wait.
      umma_commit(&bars->drain);
      mbar_wait_quiet(&bars->drain, 0);
    }
    __syncwarp();
  } else if (warp == Cfg::kLoadWarp) {
    // ================== work-list walker and K/V TMA loader ==================
    // The only thread that resolves columns (three dependent global loads each); it runs
    // ahead of everybody and publishes the descriptors through a ring in shared memory.
    if (lane == 0) {
      uint32_t it_cnt = 0;
      // The list is sorted longest first; CTAs take it in alternating direction
      // (0..G-1, G-1..0, ...) so that no CTA collects the largest of every round.
      const int G = (int)gridDim.x;
      for (int round = 0; round * G < n_items; ++round) {
        const int item = round * G + ((round & 1) ? (G - 1 - (int)blockIdx.x) : (int)blockIdx.x);
        if (item >= n_items) continue;
        Column c;
        if (!load_column(c, item, ix, p, cu, n_kv_rows)) continue;
        if (*wc.abort) break;                                 // no new loads once a wait gave up
        bars->cols[it_cnt & 3] = c;
        mbar_arrive(&bars->col_full[it_cnt & 3]);
        const int kvh = c.kv_row % p.kv_heads;
        const int tok0 = (int)(c.b * p.tokens) + c.key0;
        if (it_cnt >= 1) mbar_wait(&bars->k_free, (it_cnt - 1) & 1, wc, 4);
        mbar_expect_tx(&bars->k_full, Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d(sK + s * kSub, &k_map, &bars->k_full, s * 64, kvh, tok0);
        if (it_cnt >= 1) mbar_wait(&bars->v_free, (it_cnt - 1) & 1, wc, 5);
        mbar_expect_tx(&bars->v_full, Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d(sV + s * kSub, &v_map, &bars->v_full, s * 64, kvh, tok0);
        ++it_cnt;
      }
      bars->cols[it_cnt & 3].n = -1;                          // end of the stream
      mbar_arrive(&bars->col_full[it_cnt & 3]);
      // No load may be in flight into this CTA's shared memory when it exits.
      if (it_cnt >= 1) {
        mbar_wait_quiet(&bars->k_full, (it_cnt - 1) & 1);
        mbar_wait_quiet(&bars->v_full, (it_cnt - 1) & 1);
      }
    }
    __syncwarp();
  }
  else {
    // ============================ query gatherers ============================
    // A tile's Q rows arrive by two routes at once, because neither is fast enough alone
    // (about 6 bytes per clock each): rows [0, kTmaRows) by TMA (tile::gather4, four rows
    // per request, bytes counted on q_full), the rest by 16-byte asynchronous copies.
    // Warp 0 resolves the rows (four per lane, fetched a tile ahead) and issues the TMA
    // requests; the other warps only copy, so that their waits for copies sit out no other
    // load.
    // Rows past the end of a column are asked for outside the tensor (TMA) or zero-filled.
    const int gw = warp - Cfg::kGatherWarp0;
    const int pt = threadIdx.x - Cfg::kGatherWarp0 * 32;
    constexpr int kTmaRows = Cfg::kTmaRows, kCopyWarps = Cfg::kGatherWarps - 1;
    static_assert(kTmaRows % 4 == 0 && kTmaRows <= kTile, "TMA rows come four at a time");
    const int oob_row = p.batch * p.tokens * p.q_heads;
    constexpr int CPR = D / 8;                            // 16-byte chunks per row
    constexpr int RPI = 32 / CPR;                         // rows per copy instruction of the warp
    constexpr int kCopyPasses = (kTile - kTmaRows) / RPI;
    uint32_t t = 0;
    static_assert((kTile - kTmaRows) % RPI == 0, "whole copy instructions");
    uint32_t issued = 0, arrived = 0;                     // copying warps: tiles copied / published so far
    auto publish_all = [&]() {                            // copying warps: never block with copies unpublished
      if (gw >= 1 && issued > arrived) {
        cp_async_wait<0>();
        fence_proxy_async();
        __syncwarp();
        for (; arrived < issued; ++arrived)
          if (lane == 0) mbar_arrive(&bars->q_full[arrived % NQ]);
      }
    };
    for (uint32_t it = 0;; ++it) {
      // The next descriptor appears only after MMAs that consume the copies have run.
      if (gw >= 1 && __shfl_sync(0xffffffffu, mbar_try_wait(&bars->col_full[it & 3], (it >> 2) & 1) ? 0 : 1, 0)) publish_all();
      mbar_wait(&bars->col_full[it & 3], (it >> 2) & 1, wc, 6);
      const Column c = bars->cols[it & 3];
      if (c.n < 0) break;
      const int nt = (c.n + kTile - 1) / kTile;
      if (c.keys < kTile) {
        // The block is cut short by the end of its sequence: zero the rows of K and V past
        // it (they belong to the next sequence). Outstanding copies go first; the K load
        // awaited here is issued only after their MMAs have run.
        publish_all();
        const int dead = kTile - c.keys;
        mbar_wait(&bars->k_full, it & 1, wc, 7);
        for (int i = pt; i < dead * 8 * Cfg::kSubs; i += Cfg::kGatherThreads) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(sK + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive(&bars->k_fix);
        mbar_wait(&bars->v_full, it & 1, wc, 8);
        for (int i = pt; i < dead * 8 * Cfg::kSubs; i += Cfg::kGatherThreads) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(sV + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive(&bars->v_fix);
      }
      const int32_t* rows_i = ix.row_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      const int32_t* heads_i = ix.head_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      int n_row[4] = {0, 0, 0, 0}, n_head[4] = {0, 0, 0, 0};   // warp 0: entries of rows 4 lane .. + 3 of the next tile
      if (gw == 0) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const int e = lane * 4 + k;
          if (e < c.n) { n_row[k] = ld_nc_pinned(rows_i + e); n_head[k] = ld_nc_pinned(heads_i + e); }
        }
      }
      for (int i = 0; i < nt; ++i, ++t) {
        if (*wc.abort) break;                              // no new requests once a wait gave up
        const uint32_t qs = t % NQ, uq = t / NQ;
        int* ridx = bars->row_idx[t & 1];                  // double-buffered: one barrier per tile
        int r4[4] = {0, 0, 0, 0};
        if (gw == 0) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int e = i * kTile + lane * 4 + k;
            r4[k] = e < c.n ? (int)((c.b * p.tokens + n_row[k]) * p.q_heads + n_head[k]) : oob_row;
            if (e + kTile < c.n) { n_row[k] = ld_nc_pinned(rows_i + e + kTile); n_head[k] = ld_nc_pinned(heads_i + e + kTile); }
          }
          *reinterpret_cast<int4*>(ridx + lane * 4) = make_int4(r4[0], r4[1], r4[2], r4[3]);
        }
        if (uq >= 1) mbar_wait(&bars->q_empty[qs], (uq - 1) & 1, wc, 9);
        if (pt == 0) mbar_expect_tx(&bars->q_full[qs], kTmaRows * D * 2);
        asm volatile("bar.sync 1, %0;" ::"n"(Cfg::kGatherThreads) : "memory");   // the row list of this tile is in shared memory
        if (gw == 0) {
          if (lane < kTmaRows / 4) {
#pragma unroll
            for (int sub = 0; sub < Cfg::kSubs; ++sub)
              tma_gather4(sQ + qs * Cfg::kOperand + sub * kSub + lane * 512, &q_map, &bars->q_full[qs], sub * 64, r4[0],
                          r4[1], r4[2], r4[3]);
          }
        } else {
          const uint32_t stage = smem_u32(sQ) + qs * Cfg::kOperand;
          const int cc = lane % CPR;
#pragma unroll
          for (int pass = gw - 1; pass < kCopyPasses; pass += kCopyWarps) {
            const int rr = kTmaRows + pass * RPI + lane / CPR;
            const int ri = ridx[rr];
            const bool live = ri != oob_row;
            cp_async16(stage + (cc >> 3) * kSub + swz128(rr, cc & 7), q + (size_t)(live ? ri : 0) * D + cc * 8, live ? 16u : 0u);
          }
          cp_async_commit();
          ++issued;
          if (issued - arrived > 1) {                      // publish the older tile in flight
            cp_async_wait<1>();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars->q_full[arrived % NQ]);
            ++arrived;
          }
        }
      }
      if (*wc.abort) break;
    }
    publish_all();
    // No request may be in flight into this CTA's shared memory when it exits.
    for (uint32_t k = 0; k < (uint32_t)NQ && k < t; ++k) {
      const uint32_t u = t - 1 - k;
      mbar_wait_quiet(&bars->q_full[u % NQ], (u / NQ) & 1);
    }
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
int launch_one(const moba_b200_problem& p, const CUtensorMap& km, const CUtensorMap& vm, const CUtensorMap& qm, const void* q,
               const moba_b200_index& ix, const int32_t* cu, void* part_o, float* part_lse, int n_items,
               unsigned* err, cudaStream_t st) {
  auto kern = fwd_sm100_kernel<D, T, TP>;
  MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, FwdCfg<D>::kSmem));
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = n_items < sms ? n_items : sms;
  kern<<<grid, FwdCfg<D>::kThreads, FwdCfg<D>::kSmem, st>>>(km, vm, qm, (const T*)q, ix, cu, (TP*)part_o, part_lse, p,
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
  CUtensorMap km, vm, qm;
  const uint64_t rows = (uint64_t)p.batch * p.tokens;
  int rc = encode_rows_map(&km, k, rows, p.kv_heads, p.head_dim, 128);
  if (rc) return rc;
  rc = encode_rows_map(&vm, v, rows, p.kv_heads, p.head_dim, 128);
  if (rc) return rc;
  rc = encode_2d_map(&qm, q, rows * p.q_heads, p.head_dim, 1);         // rows gathered four at a time
  if (rc) return rc;
  const int n_items = p.num_blocks * p.n_seq * p.kv_heads;
  const bool bf = p.dtype == MOBA_B200_BF16;
#define GO(D, T, TP) return launch_one<D, T, TP>(p, km, vm, qm, q, ix, cu, part_o, part_lse, n_items, err, st)
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
