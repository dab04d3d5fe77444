// Gate scorer on tcgen05 tensor cores (bf16/f16, block_size 128, head_dim
// 64/128, at most 8 ranked blocks per query).
//
// Persistent CTAs (two per SM) walk the (128-query tile, sequence, query head)
// units, heaviest first, in alternating direction per round. With 128-token
// blocks a tile is exactly one block, so every row of a tile has the same
// candidates: the blocks before the tile's own. Roles:
//   loader (1 thread)  TMA: the unit's Q tile, then block-mean chunks of 128 blocks
//   mma    (1 thread)  S = Q Kbar^T (M128 N128 K=D) into one of two TMEM buffers: the first
//                      two chunks of the unit (bounding pass), then every chunk (ranking pass)
//   select (2 x 4 warps; warpgroup w takes columns [64 w, 64 w + 64) of every chunk)
//          tcgen05.ld, one row per thread. The first two chunks of a unit are scored twice.
//          The first pass only keeps, per row, the maxima of eight interleaved subsets
//          of the scores (one max per score): the L-th largest of them is a score that
//          at least L candidates reach, so nothing below it can be selected. The second
//          pass tests every score against that bound with one compare and appends the
//          few that pass, by predicated stores, to a small per-thread buffer in shared
//          memory; the buffer is emptied into the row's sorted register list of L keys
//          whenever some lane of the warp is about to run out of room, which also
//          raises the bound to the score of the list's last entry (candidates arrive
//          in ascending block order, so an equal score never wins). A key is the score
//          rounded to the input dtype and made monotone in the high half and
//          0xFFFF - block id in the low half, so "score descending, ties to the lower
//          id" is plain integer order. Scoring two chunks twice costs tensor-core time the
//          gate has to spare; ranking every score would cost issue slots it has not.
// At the end of a unit the two warpgroups' lists are merged and each thread emits
// its ids plus the own block, ascending, -1 padded.
//
// Scores are float32 tensor-core sums rounded to the input dtype; the portable
// gate rounds the exact sum. The two differ only when a float32 partial sum
// straddles a rounding boundary of the input dtype.
//
// Stands in for gate_kernel of the reference (src/moba/kernels/gating.py:92-335).
#include "common.cuh"
#include "sm100.cuh"

#include <type_traits>

namespace moba {
using namespace sm100;

namespace {

constexpr int kTile = 128;
constexpr int kSub = kTile * 128;
constexpr int kMmaWarp = 8, kLoadWarp = 9;
constexpr int kThreads = 10 * 32;
constexpr int kMaxTake = 8;
constexpr int kEmpty = 0x7fffffff;

template <int D> struct GateCfg {
  static constexpr int kSubs = D / 64;
  static constexpr int kOperand = kSubs * kSub;
  // Per-thread buffer of scores that passed the entry test, in slots of 8 bytes, and how
  // many columns are tested between two checks for room. Two CTAs share an SM, which at
  // head_dim 128 leaves room for 7 slots only.
  static constexpr int kCap = tensor_core_plan(D).gate_slots;
  static constexpr int kStep = tensor_core_plan(D).gate_step;
  static constexpr int kBufBytes = kCap * kTile * 8;                       // per warpgroup
  static constexpr int kSmem = 3 * kOperand + 2 * kBufBytes + 1024 + 512;  // Q + two Kbar stages + buffers
};

struct Bars {
  uint64_t q_full, q_free, kb_full[2], kb_empty[2], s_full[2], s_free[2], drain;
  uint32_t tmem_base;
  int abort;
};

// Sorted (descending) register list of the L best keys seen so far.
template <int L>
__device__ __forceinline__ void list_offer(uint32_t (&t)[L], uint32_t x) {
#pragma unroll
  for (int i = 0; i < L; ++i) {
    const uint32_t hi = max(t[i], x);
    x = min(t[i], x);
    t[i] = hi;
  }
}

template <typename T> __device__ __forceinline__ uint32_t round16(float a);
template <> __device__ __forceinline__ uint32_t round16<__nv_bfloat16>(float a) {
  return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(a));
}
template <> __device__ __forceinline__ uint32_t round16<__half>(float a) {
  return (uint32_t)__half_as_ushort(__float2half_rn(a));
}
template <typename T> __device__ __forceinline__ float widen16(uint32_t bits);
template <> __device__ __forceinline__ float widen16<__nv_bfloat16>(uint32_t bits) { return __uint_as_float(bits << 16); }
template <> __device__ __forceinline__ float widen16<__half>(uint32_t bits) {
  return __half2float(__ushort_as_half((unsigned short)bits));
}

// Score (rounded to T) and block id -> sortable key; never 0 for a real candidate
// (the low half of a key is 0xFFFF - id with id <= 0xFFFE).
template <typename T>
__device__ __forceinline__ uint32_t make_key(float score, uint32_t block) {
  const uint32_t b = round16<T>(score);
  const uint32_t mono = (b & 0x8000u) ? (~b & 0xFFFFu) : (b | 0x8000u);
  return (mono << 16) | (0xFFFFu - block);
}
// The score a candidate has to exceed to get past `key` (the list's last entry):
// -inf while the list has room.
template <typename T>
__device__ __forceinline__ float entry_bar(uint32_t key) {
  if (key == 0u) return -INFINITY;
  const uint32_t mono = key >> 16;
  const uint32_t b = (mono & 0x8000u) ? (mono & 0x7FFFu) : (~mono & 0xFFFFu);
  return widen16<T>(b);
}

// The largest score that is certainly below every score whose rounding to T is at least
// round_T(m): one step of T under round_T(m), widened back to float.
template <typename T>
__device__ __forceinline__ float one_step_below(float m) {
  if (!(m > -INFINITY)) return -INFINITY;
  const uint32_t key = make_key<T>(m, 0u);
  const uint32_t mono = key >> 16;
  if (mono == 0u) return -INFINITY;
  return entry_bar<T>(((mono - 1u) << 16) | 1u);
}

// Which unit a CTA takes in its `round`-th turn: heaviest units first, alternating
// direction, so that no CTA collects the heaviest unit of every round.
__device__ __forceinline__ int unit_of(int round) {
  const int g = (int)gridDim.x, c = (int)blockIdx.x;
  return round * g + ((round & 1) ? (g - 1 - c) : c);
}

struct Unit {
  int tile, seq, hq, row0, n_chunks, bos, len;
  int n_lo, c_hi0;          // chunks [0, n_lo) and [c_hi0, ...) of the Kbar row are visited
  int n_first;              // chunks the bounding pass scores before the ranking pass scores all
  // chunk of the Kbar row that step `s` of a pass scores
  __device__ __forceinline__ int chunk_of(int s) const { return s < n_lo ? s : c_hi0 + (s - n_lo); }
  // a unit takes n_first + n_chunks steps: the bounding pass, then the ranking pass
  __device__ __forceinline__ int steps() const { return n_first + n_chunks; }
  __device__ __forceinline__ int chunk_of_step(int step) const { return chunk_of(step < n_first ? step : step - n_first); }
};
// The bounding pass looks at the first two chunks only: 256 candidates give a bar that about
// one score in ten of a later chunk passes until the first flush raises it, and scoring a long
// row of block means twice would cost more tensor-core time than the tighter bar saves.
constexpr int kBoundChunks = 2;
__device__ __forceinline__ bool load_unit(Unit& u, int idx, const moba_b200_problem& p, const int32_t* cu,
                                          int n_tiles) {
  const int ny = p.n_seq * p.q_heads;
  u.tile = n_tiles - 1 - idx / ny;                              // long tiles first
  const int y = idx % ny;
  u.seq = y / p.q_heads; u.hq = y % p.q_heads;
  const SeqSpan sp = seq_span(cu, p.packed, u.seq, p.tokens);
  u.bos = sp.bos; u.len = sp.len;
  u.row0 = u.tile * kTile;
  // Candidates are blocks [0, tile); with a candidate window only [0, sinks) and
  // [tile - window, tile), so only the chunks that hold some of those are scored.
  const int total = (p.take > 0) ? (u.tile + kTile - 1) / kTile : 0;
  if (p.gate_window <= 0) {
    u.n_lo = total; u.c_hi0 = total;
  } else {
    const int recent0 = max(0, u.tile - p.gate_window);         // first block of the recent window
    u.n_lo = min(total, (min(p.gate_sinks, recent0) + kTile - 1) / kTile);
    u.c_hi0 = max(u.n_lo, recent0 / kTile);
  }
  u.n_chunks = u.n_lo + (total - u.c_hi0);
  u.n_first = min(u.n_chunks, kBoundChunks);
  return u.row0 < sp.len;
}

template <int D, typename T, int L>
__global__ void __launch_bounds__(kThreads, 2)
gate_sm100_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kb_map,
                  const int32_t* __restrict__ cu, int32_t* __restrict__ block_idx, moba_b200_problem p,
                  int n_tiles, int n_units, unsigned* error_word) {
  using Cfg = GateCfg<D>;
  constexpr int CAP = Cfg::kCap, STEP = Cfg::kStep;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem;
  unsigned char* sKb = sQ + Cfg::kOperand;                    // two stages
  unsigned char* sBuf = sKb + 2 * Cfg::kOperand;              // two warpgroups' buffers
  Bars* bars = reinterpret_cast<Bars*>(sBuf + 2 * Cfg::kBufBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = p.q_heads / p.kv_heads;
  const int take = p.take;
#ifdef MOBA_WAIT_STATS
  __shared__ unsigned long long wait_stats[32];
  if (threadIdx.x < 32) wait_stats[threadIdx.x] = 0;
  const long long kernel_t0 = clock64();
  const WaitCtx wc{&bars->abort, error_word, wait_stats};
#else
  const WaitCtx wc{&bars->abort, error_word};
#endif

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1); mbar_init(&bars->q_free, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->kb_full[i], 1); mbar_init(&bars->kb_empty[i], 1);
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->s_free[i], 8);
    }
    mbar_init(&bars->drain, 1);
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) tmem_alloc(&bars->tmem_base, 256);
  if (warp == kLoadWarp && lane == 0) { tma_prefetch_desc(&q_map); tma_prefetch_desc(&kb_map); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  // Every role walks the same units and counts the same steps: a unit of n chunks takes 2 n
  // steps (chunk `step mod n`), `gc` is the number of steps of all earlier units of this CTA,
  // and a step uses Kbar stage and TMEM buffer (gc + step) & 1.
  if (warp < 8) {
    // ================================ select ================================
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    // This thread's buffer: slot s is the 8 bytes at buf0 + s * kSlot (shared-memory address).
    constexpr uint32_t kSlot = kTile * 8;
    const uint32_t buf0 = smem_u32(sBuf + wg * Cfg::kBufBytes) + (uint32_t)r * 8u;
    // List exchange at the end of a unit: thread r of warpgroup 1 leaves its list in the
    // (empty) buffer slots of thread r of warpgroup 0, two keys per slot, so a thread of
    // warpgroup 0 only ever reads and overwrites words of its own.
    const uint32_t xk0 = smem_u32(sBuf) + (uint32_t)r * 8u;
    static_assert((L + 1) / 2 <= CAP, "a list fits the slots of one thread");
    uint32_t gc = 0;
    PHASE_CLOCK(ph);
    for (int round = 0; round * (int)gridDim.x < n_units; ++round) {
      const int ui = unit_of(round);
      if (ui >= n_units) continue;
      Unit u;
      if (!load_unit(u, ui, p, cu, n_tiles)) continue;
      uint32_t best[L];
#pragma unroll
      for (int e = 0; e < L; ++e) best[e] = 0u;                 // 0 sorts below every real key
      float mx[8];                                              // first pass: maxima of 8 column subsets
#pragma unroll
      for (int e = 0; e < 8; ++e) mx[e] = -INFINITY;
      float bar = -INFINITY;                                    // a score must exceed this to be appended
      uint32_t wa = buf0;                                       // address of the next free slot
      auto flush = [&]() {                                      // whole warp: empty the buffers into the lists
        PHASE_CLOCK(fl);
        while (__any_sync(0xffffffffu, wa != buf0)) {
          uint32_t key = 0u;
          if (wa != buf0) {
            wa -= kSlot;
            uint32_t sx, sy;
            asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(sx), "=r"(sy) : "r"(wa));
            key = make_key<T>(__uint_as_float(sx), sy);
          }
          list_offer<L>(best, key);
        }
        bar = fmaxf(bar, entry_bar<T>(best[L - 1]));
        PHASE_ADD(wc, 4, fl);                                   // flushes (also counted in their phase)
      };
      PHASE_ADD(wc, 1, ph);                                     // unit set-up
      for (int step = 0; step < u.steps(); ++step) {
        const uint32_t gidx = gc + (uint32_t)step, st = gidx & 1u;
        const bool second = step >= u.n_first;
        const int c = u.chunk_of_step(step);
        if (step == u.n_first) {
          // The L-th largest of the eight subset maxima: at least L candidates reach it.
          float lo1 = INFINITY, lo2 = INFINITY;                 // smallest and second smallest
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            lo2 = fminf(lo2, fmaxf(lo1, mx[e]));
            lo1 = fminf(lo1, mx[e]);
          }
          bar = one_step_below<T>(L >= 8 ? lo1 : lo2);
        }
        const bool s_ok = mbar_wait(&bars->s_full[st], (gidx >> 1) & 1u, wc, 9);
        tc_fence_after();
        PHASE_ADD(wc, 2, ph);                                   // s_full wait
        const int c0 = c * kTile + wg * 64;                     // first column (block) of this warpgroup's half
        const bool run = __all_sync(0xffffffffu, s_ok);         // a wait gave up: rank nothing unseen
        uint32_t v[32];
#pragma unroll 1
        for (int h = 0; h < 2; ++h) {
          tmem_ld32(tmem + lane_off + st * 128 + wg * 64 + h * 32, v);
          tmem_ld_wait();
          if (h == 1) { tc_fence_before(); mbar_arrive_warp(&bars->s_free[st]); }   // the scores are in registers
          // which of these 32 blocks are candidates of the tile: all, none, or some
          const int g0 = c0 + h * 32;
          const bool none = g0 >= u.tile || (p.gate_window > 0 && g0 >= p.gate_sinks && g0 + 32 <= u.tile - p.gate_window);
          if (!run || none) continue;
          const bool all = g0 + 32 <= u.tile &&
                           (p.gate_window <= 0 || g0 + 32 <= p.gate_sinks || g0 >= u.tile - p.gate_window);
          if (!all) {
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (!gate_candidate(p, g0 + k, u.tile)) v[k] = 0xff800000u;   // -inf: never passes
          }
          if (!second) {
#pragma unroll
            for (int k = 0; k < 32; ++k) mx[k & 7] = fmaxf(mx[k & 7], __uint_as_float(v[k]));
            continue;
          }
          const uint32_t col0 = (uint32_t)(c0 + h * 32);
#pragma unroll
          for (int k0 = 0; k0 < 32; k0 += STEP) {
            if (__any_sync(0xffffffffu, wa > buf0 + (CAP - STEP) * kSlot)) flush();   // room for STEP more
#pragma unroll
            for (int k = k0; k < k0 + STEP; ++k) {
              // if (score > bar) { slot <- (score, block id); next slot }, predicated: a branch
              // here would be taken by some lane of the warp at almost every score
              asm volatile(
                  "{\n\t.reg .pred p;\n\t"
                  "setp.gt.f32 p, %1, %2;\n\t"
                  "@p st.shared.v2.b32 [%0], {%3, %4};\n\t"
                  "@p add.u32 %0, %0, %5;\n\t}"
                  : "+r"(wa)
                  : "f"(__uint_as_float(v[k])), "f"(bar), "r"(v[k]), "r"(col0 + (uint32_t)k), "n"(kTile * 8)
                  : "memory");
            }
          }
        }
        PHASE_ADD(wc, 3, ph);                                   // loads, maxima / tests and appends, flushes
      }
      flush();
      gc += (uint32_t)u.steps();
      // ---- merge the two warpgroups' lists (warpgroup 1 -> warpgroup 0's empty buffer) ----
      asm volatile("bar.sync 2, 256;" ::: "memory");            // warpgroup 0 has emptied its buffer
      if (wg == 1) {
#pragma unroll
        for (int e = 0; e < L; ++e)
          asm volatile("st.shared.b32 [%0], %1;" ::"r"(xk0 + (uint32_t)(e >> 1) * kSlot + (uint32_t)(e & 1) * 4u), "r"(best[e]) : "memory");
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");
      if (wg == 0 && u.row0 + r < u.len) {
#pragma unroll
        for (int e = 0; e < L; ++e) {
          uint32_t other;
          asm volatile("ld.shared.b32 %0, [%1];" : "=r"(other) : "r"(xk0 + (uint32_t)(e >> 1) * kSlot + (uint32_t)(e & 1) * 4u));
          list_offer<L>(best, other);
        }
        // ---- emit: the best `take` ids plus the own block, ascending, -1 padded ----
        int ids[L];
        int kept = 0;
#pragma unroll
        for (int e = 0; e < L; ++e) {
          const bool ok = e < take && best[e] != 0u;
          ids[e] = ok ? (int)(0xFFFFu - (best[e] & 0xFFFFu)) : kEmpty;
          kept += ok ? 1 : 0;
        }
        const size_t b = p.packed ? 0 : (size_t)u.seq;
        int32_t* dst = block_idx + ((b * p.q_heads + u.hq) * p.tokens + u.bos + u.row0 + r) * (size_t)p.slots;
#pragma unroll
        for (int e = 0; e < L; ++e) {                           // rank by id: position in the output
          if (ids[e] == kEmpty) continue;
          int rank = 0;
#pragma unroll
          for (int f = 0; f < L; ++f) rank += (ids[f] < ids[e]) ? 1 : 0;
          dst[rank] = ids[e];
        }
        if (p.always_current) dst[kept++] = u.tile;             // the own block is past every candidate
        for (int e = kept; e < p.slots; ++e) dst[e] = -1;
      }
      // Warpgroup 0 reads the exchange area (its own buffer) before it appends to it again;
      // warpgroup 1 writes there only behind the first barrier of the next unit.
      PHASE_ADD(wc, 5, ph);                                     // last flush, merge, emit
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0) {
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc = make_idesc(0, 128, 128, 0, 0) | (fmt << 7) | (fmt << 10);
      const uint32_t aQ = smem_u32(sQ);
      uint32_t gc = 0, nq = 0;                                  // steps / Q tiles consumed so far
      for (int round = 0; round * (int)gridDim.x < n_units; ++round) {
        const int ui = unit_of(round);
        if (ui >= n_units) continue;
        Unit u;
        if (!load_unit(u, ui, p, cu, n_tiles) || u.n_chunks == 0) continue;
        mbar_wait(&bars->q_full, nq & 1, wc);
        for (int step = 0; step < u.steps(); ++step, ++gc) {
          const uint32_t st = gc & 1, use = gc >> 1;
          const uint32_t aK = smem_u32(sKb) + st * Cfg::kOperand;
          mbar_wait(&bars->kb_full[st], use & 1, wc);
          if (use >= 1) mbar_wait(&bars->s_free[st], (use - 1) & 1, wc);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t o = (ks >> 2) * kSub + (ks & 3) * 32;
            umma_f16(tmem + st * 128, make_sdesc(aQ + o, 16, 1024), make_sdesc(aK + o, 16, 1024), idesc, ks > 0);
          }
          umma_commit(&bars->s_full[st]);
          umma_commit(&bars->kb_empty[st]);
        }
        umma_commit(&bars->q_free);                             // the Q tile may be replaced
        ++nq;
      }
      // Every MMA has completed before the CTA lets go of its TMEM, also on the way out of
      // a run that gave up on a wait.
      umma_commit(&bars->drain);
      mbar_wait_quiet(&bars->drain, 0);
    }
    __syncwarp();
  } else {
    if (lane == 0) {
      uint32_t gc = 0, nq = 0;
      for (int round = 0; round * (int)gridDim.x < n_units; ++round) {
        const int ui = unit_of(round);
        if (ui >= n_units) continue;
        Unit u;
        if (!load_unit(u, ui, p, cu, n_tiles) || u.n_chunks == 0) continue;
        if (*wc.abort) break;                                   // no new loads once a wait gave up
        const size_t b = p.packed ? 0 : (size_t)u.seq;
        const int kv_row = u.seq * p.kv_heads + u.hq / group;
        const int tok0 = (int)(b * p.tokens) + u.bos + u.row0;
        if (nq >= 1) mbar_wait(&bars->q_free, (nq - 1) & 1, wc);
        mbar_expect_tx(&bars->q_full, Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d(sQ + s * kSub, &q_map, &bars->q_full, s * 64, u.hq, tok0);
        ++nq;
        for (int step = 0; step < u.steps(); ++step, ++gc) {
          const uint32_t st = gc & 1, use = gc >> 1;
          const int c = u.chunk_of_step(step);
          if (use >= 1) mbar_wait(&bars->kb_empty[st], (use - 1) & 1, wc);
          if (*wc.abort) break;
          mbar_expect_tx(&bars->kb_full[st], Cfg::kOperand);
          for (int s = 0; s < Cfg::kSubs; ++s)
            tma_load_3d(sKb + st * Cfg::kOperand + s * kSub, &kb_map, &bars->kb_full[st], s * 64, c * kTile, kv_row);
        }
        if (*wc.abort) break;
      }
      // No load may be in flight into this CTA's shared memory when it exits.
      if (nq >= 1) mbar_wait_quiet(&bars->q_full, (nq - 1) & 1);
      for (uint32_t k = 1; k <= 2 && k <= gc; ++k) {
        const uint32_t c = gc - k;
        mbar_wait_quiet(&bars->kb_full[c & 1], (c >> 1) & 1);
      }
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, 256);
#ifdef MOBA_WAIT_STATS
  if (threadIdx.x < 32 && blockIdx.x < 148) {
    unsigned long long* out = reinterpret_cast<unsigned long long*>(error_word + 64) + (size_t)blockIdx.x * 32;
    out[threadIdx.x] = threadIdx.x == 31 ? (unsigned long long)(clock64() - kernel_t0) : wait_stats[threadIdx.x];
  }
#endif
}


template <int D, typename T, int L>
int launch_one(const moba_b200_problem& p, const CUtensorMap& qm, const CUtensorMap& km, const int32_t* cu,
               int32_t* block_idx, unsigned* err, cudaStream_t st) {
  auto kern = gate_sm100_kernel<D, T, L>;
  MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GateCfg<D>::kSmem));
  const int n_tiles = (p.max_seqlen + kTile - 1) / kTile;
  const long long n_units = (long long)n_tiles * p.n_seq * p.q_heads;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = (int)(n_units < 2LL * sms ? n_units : 2LL * sms);
  kern<<<grid, kThreads, GateCfg<D>::kSmem, st>>>(qm, km, cu, block_idx, p, n_tiles, (int)n_units, err);
  MOBA_LAUNCH_OK("gate_sm100_kernel");
  return MOBA_B200_OK;
}

}  // namespace

bool gate_sm100_supported(const moba_b200_problem& p) {
  return (p.dtype == MOBA_B200_BF16 || p.dtype == MOBA_B200_F16) && p.block_size == 128 &&
         (p.head_dim == 64 || p.head_dim == 128) && p.take <= kMaxTake && p.slots <= kMaxTake + 1 &&
         p.num_blocks <= 0xFFFF &&
         (long long)p.batch * p.tokens < 0x7fffffffLL &&
         (long long)((p.max_seqlen + 127) / 128) * p.n_seq * p.q_heads < 0x7fffffffLL;
}

int encode_kbar_map_impl(CUtensorMap* out, const void* base, uint64_t kv_rows, uint64_t nb, uint64_t dim);

int launch_gate_sm100(const moba_b200_problem& p, const void* q, const void* kbar, const int32_t* cu,
                      int32_t* block_idx, cudaStream_t st) {
  KernelTimer timer__("gate_sm100_kernel", st);
  unsigned* err = device_error_word();
  if (err == nullptr) { set_error("gate: no device error word"); return MOBA_B200_ECUDA; }
  CUtensorMap qm, km;
  int rc = encode_rows_map(&qm, q, (uint64_t)p.batch * p.tokens, p.q_heads, p.head_dim, 128);
  if (rc) return rc;
  rc = encode_kbar_map_impl(&km, kbar, (uint64_t)p.n_seq * p.kv_heads, p.num_blocks, p.head_dim);
  if (rc) return rc;
  const bool bf = p.dtype == MOBA_B200_BF16;
#define GO(D, T) return (p.take <= 7) ? launch_one<D, T, 7>(p, qm, km, cu, block_idx, err, st) \
                                      : launch_one<D, T, 8>(p, qm, km, cu, block_idx, err, st)
  if (p.head_dim == 64) { if (bf) GO(64, __nv_bfloat16); else GO(64, __half); }
  if (bf) GO(128, __nv_bfloat16); else GO(128, __half);
#undef GO
}

}  // namespace moba
