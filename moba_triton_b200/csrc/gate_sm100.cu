// Gate scorer on tcgen05 tensor cores (bf16/f16, block_size 128, head_dim
// 64/128, at most 8 ranked blocks per query).
//
// One CTA per (128-query tile, sequence, query head); with 128-token blocks a
// tile is exactly one block, so every row of the tile has the same candidates:
// the blocks before the tile's own. Roles:
//   loader (1 thread)  TMA: the Q tile once, then block-mean chunks of 128 blocks
//   mma    (1 thread)  S = Q Kbar^T (M128 N128 K=D) into one of two TMEM buffers
//   select (2 x 4 warps, alternating chunks) tcgen05.ld one row per thread,
//          round to the input dtype, compare with the row's entry bar; the rare
//          winner enters a per-thread list (ties: admission needs strictly
//          greater, eviction drops the highest id among the weakest)
// At the end each thread emits its list plus the own block, ascending, -1 padded.
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
  static constexpr int kSmem = 3 * kOperand + 1024 + 512;     // Q + two Kbar stages
};

struct Bars {
  uint64_t q_full, kb_full[2], kb_empty[2], s_full[2], s_free[2];
  uint32_t tmem_base;
  int abort;
};

// Offers (s, blk) to the list; returns the new entry bar (the weakest kept score,
// -inf while a slot is empty). Kept out of line: it runs a few dozen times per row.
__device__ __noinline__ float list_insert(float* vals, int* ids, int take, float s, int blk) {
  int w = 0;
  for (int e = 1; e < take; ++e)
    if (vals[e] < vals[w] || (vals[e] == vals[w] && ids[e] > ids[w])) w = e;
  vals[w] = s;
  ids[w] = blk;
  float m = vals[0];
  for (int e = 1; e < take; ++e) m = fminf(m, vals[e]);
  return m;
}

template <int D, typename T>
__global__ void __launch_bounds__(kThreads, 2)
gate_sm100_kernel(const __grid_constant__ CUtensorMap q_map, const __grid_constant__ CUtensorMap kb_map,
                  const int32_t* __restrict__ cu, int32_t* __restrict__ block_idx, moba_b200_problem p,
                  int n_tiles, unsigned* error_word) {
  using Cfg = GateCfg<D>;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sQ = smem;
  unsigned char* sKb = sQ + Cfg::kOperand;                    // two stages
  Bars* bars = reinterpret_cast<Bars*>(sKb + 2 * Cfg::kOperand);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = n_tiles - 1 - (int)blockIdx.x;             // long tiles first
  const int seq = blockIdx.y / p.q_heads, hq = blockIdx.y % p.q_heads;
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  const int row0 = tile * kTile;
  if (row0 >= sp.len) return;                                 // whole CTA leaves before any barrier
  const int group = p.q_heads / p.kv_heads;
  const int kv_row = seq * p.kv_heads + hq / group;
  const size_t b = p.packed ? 0 : (size_t)seq;
  const int take = p.take;
  const int n_chunks = (take > 0) ? (tile + kTile - 1) / kTile : 0;   // candidates: blocks [0, tile)
  const WaitCtx wc{&bars->abort, error_word};

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->kb_full[i], 1); mbar_init(&bars->kb_empty[i], 1);
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->s_free[i], 128);
    }
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) tmem_alloc(&bars->tmem_base, 256);
  if (warp == kLoadWarp && lane == 0) { tma_prefetch_desc(&q_map); tma_prefetch_desc(&kb_map); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp < 8) {
    // ================================ select ================================
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    float vals[kMaxTake];
    int ids[kMaxTake];
#pragma unroll
    for (int e = 0; e < kMaxTake; ++e) { vals[e] = -INFINITY; ids[e] = kEmpty; }
    float thr = -INFINITY;
    // The two warpgroups take alternate chunks of the same 128 rows, so each keeps
    // its own list per row; the lists are merged at the end through shared memory.
    for (int c = wg; c < n_chunks; c += 2) {
      const uint32_t u = (uint32_t)c >> 1;
      mbar_wait(&bars->s_full[wg], u & 1, wc);
      tc_fence_after();
      const int c0 = c * kTile;
      const int cmax = tile - c0;                               // columns [0, cmax) are candidates
      uint32_t v[32];
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        tmem_ld32(tmem + lane_off + wg * 128 + ch * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const int col = ch * 32 + k;
          const float s = Elem<T>::round_f(__uint_as_float(v[k]));
          if (col < cmax && s > thr) thr = list_insert(vals, ids, take, s, c0 + col);
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->s_free[wg]);
    }
    // ---- merge the two warpgroups' lists (warpgroup 1 -> shared -> warpgroup 0) ----
    float* xv = reinterpret_cast<float*>(sKb);                  // Kbar stages are idle now
    int* xi = reinterpret_cast<int*>(sKb + kTile * kMaxTake * 4);
    asm volatile("bar.sync 2, 256;" ::: "memory");              // every S MMA has been consumed
    if (wg == 1) {
      for (int e = 0; e < take; ++e) { xv[r * kMaxTake + e] = vals[e]; xi[r * kMaxTake + e] = ids[e]; }
    }
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (wg == 0 && row0 + r < sp.len) {
      // The final selection is the best `take` of the union of both lists. Rebuild
      // it by offering the union in ascending block order, so the admission rule
      // (strictly greater: the earlier block wins a tie) applies unchanged.
      float av[2 * kMaxTake];
      int ai[2 * kMaxTake];
      int n = 0;
      for (int e = 0; e < take; ++e) if (ids[e] != kEmpty) { av[n] = vals[e]; ai[n] = ids[e]; ++n; }
      for (int e = 0; e < take; ++e) {
        const int id = xi[r * kMaxTake + e];
        if (id != kEmpty) { av[n] = xv[r * kMaxTake + e]; ai[n] = id; ++n; }
      }
      for (int i = 1; i < n; ++i) {                             // insertion sort by id
        const float tv = av[i]; const int ti = ai[i];
        int j = i - 1;
        while (j >= 0 && ai[j] > ti) { av[j + 1] = av[j]; ai[j + 1] = ai[j]; --j; }
        av[j + 1] = tv; ai[j + 1] = ti;
      }
      for (int e = 0; e < take; ++e) { vals[e] = -INFINITY; ids[e] = kEmpty; }
      thr = -INFINITY;
      for (int i = 0; i < n; ++i)
        if (av[i] > thr) thr = list_insert(vals, ids, take, av[i], ai[i]);
      // ---- emit: kept ids plus the own block, ascending, -1 padded ----
      int out[kMaxTake + 1];
      int m = 0;
      for (int e = 0; e < take; ++e) if (ids[e] != kEmpty) out[m++] = ids[e];
      for (int i = 1; i < m; ++i) {
        const int ti = out[i];
        int j = i - 1;
        while (j >= 0 && out[j] > ti) { out[j + 1] = out[j]; --j; }
        out[j + 1] = ti;
      }
      if (p.always_current) out[m++] = tile;                    // larger than every candidate
      int32_t* dst = block_idx + ((b * p.q_heads + hq) * p.tokens + sp.bos + row0 + r) * (size_t)p.slots;
      for (int e = 0; e < p.slots; ++e) dst[e] = (e < m) ? out[e] : -1;
    }
  } else if (warp == kMmaWarp) {
    if (lane == 0 && n_chunks > 0) {
      const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;
      const uint32_t idesc = make_idesc(0, 128, 128, 0, 0) | (fmt << 7) | (fmt << 10);
      const uint32_t aQ = smem_u32(sQ);
      mbar_wait(&bars->q_full, 0, wc);
      for (int c = 0; c < n_chunks; ++c) {
        const uint32_t st = c & 1, u = (uint32_t)c >> 1;
        const uint32_t aK = smem_u32(sKb) + st * Cfg::kOperand;
        mbar_wait(&bars->kb_full[st], u & 1, wc);
        if (u >= 1) mbar_wait(&bars->s_free[st], (u - 1) & 1, wc);
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t o = (ks >> 2) * kSub + (ks & 3) * 32;
          umma_f16(tmem + st * 128, make_sdesc(aQ + o, 16, 1024), make_sdesc(aK + o, 16, 1024), idesc, ks > 0);
        }
        umma_commit(&bars->s_full[st]);
        umma_commit(&bars->kb_empty[st]);
      }
    }
    __syncwarp();
  } else {
    if (lane == 0 && n_chunks > 0) {
      const int tok0 = (int)(b * p.tokens) + sp.bos + row0;
      mbar_expect_tx(&bars->q_full, Cfg::kOperand);
      for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d(sQ + s * kSub, &q_map, &bars->q_full, s * 64, hq, tok0);
      for (int c = 0; c < n_chunks; ++c) {
        const uint32_t st = c & 1, u = (uint32_t)c >> 1;
        if (u >= 1) mbar_wait(&bars->kb_empty[st], (u - 1) & 1, wc);
        mbar_expect_tx(&bars->kb_full[st], Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s)
          tma_load_3d(sKb + st * Cfg::kOperand + s * kSub, &kb_map, &bars->kb_full[st], s * 64, c * kTile, kv_row);
      }
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, 256);
}


template <int D, typename T>
int launch_one(const moba_b200_problem& p, const CUtensorMap& qm, const CUtensorMap& km, const int32_t* cu,
               int32_t* block_idx, unsigned* err, cudaStream_t st) {
  auto kern = gate_sm100_kernel<D, T>;
  MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GateCfg<D>::kSmem));
  const int n_tiles = (p.max_seqlen + kTile - 1) / kTile;
  dim3 grid(n_tiles, p.n_seq * p.q_heads);
  kern<<<grid, kThreads, GateCfg<D>::kSmem, st>>>(qm, km, cu, block_idx, p, n_tiles, err);
  MOBA_LAUNCH_OK("gate_sm100_kernel");
  return MOBA_B200_OK;
}

}  // namespace

bool gate_sm100_supported(const moba_b200_problem& p) {
  return (p.dtype == MOBA_B200_BF16 || p.dtype == MOBA_B200_F16) && p.block_size == 128 &&
         (p.head_dim == 64 || p.head_dim == 128) && p.take <= kMaxTake && p.slots <= kMaxTake + 1 &&
         (long long)p.batch * p.tokens < 0x7fffffffLL;
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
  if (p.head_dim == 64) {
    if (bf) return launch_one<64, __nv_bfloat16>(p, qm, km, cu, block_idx, err, st);
    return launch_one<64, __half>(p, qm, km, cu, block_idx, err, st);
  }
  if (bf) return launch_one<128, __nv_bfloat16>(p, qm, km, cu, block_idx, err, st);
  return launch_one<128, __half>(p, qm, km, cu, block_idx, err, st);
}

}  // namespace moba
