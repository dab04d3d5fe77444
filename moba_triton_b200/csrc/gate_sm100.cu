// Gate scorer on tcgen05 tensor cores (bf16/f16, block_size 128, head_dim
// 64/128, at most 8 ranked blocks per query).
//
// One CTA per (128-query tile, sequence, query head); with 128-token blocks a
// tile is exactly one block, so every row of the tile has the same candidates:
// the blocks before the tile's own. Roles:
//   loader (1 thread)  TMA: the Q tile once, then block-mean chunks of 128 blocks
//   mma    (1 thread)  S = Q Kbar^T (M128 N128 K=D) into one of two TMEM buffers
//   select (2 x 4 warps, alternating chunks) tcgen05.ld one row per thread,
//          round each score to the input dtype and pack it with its block id
//          into one sortable 32-bit key (score bits made monotone in the high
//          half, 0xFFFF - id in the low half), so "score descending, ties to
//          the lower id" is plain integer order. Each thread keeps its best
//          keys in a sorted register list; groups of four keys are skipped
//          with one compare when none can enter.
// At the end the two warpgroups' lists are merged and each thread emits its
// ids plus the own block, ascending, -1 padded.
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
  uint64_t q_full, kb_full[2], kb_empty[2], s_full[2], s_free[2], drain;
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

// Two 16-bit floats (packed) -> two 16-bit keys whose unsigned order is the
// numeric order: negative values have all bits flipped, the others only the sign.
__device__ __forceinline__ uint32_t monotone16x2(uint32_t w) {
  const uint32_t neg = ((w >> 15) & 0x00010001u) * 0x7FFFu;
  return w ^ (neg | 0x80008000u);
}

template <typename T> __device__ __forceinline__ uint32_t round_pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t round_pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t round_pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, typename T, int L>
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
#ifdef MOBA_WAIT_STATS
  const WaitCtx wc{&bars->abort, error_word, nullptr};
#else
  const WaitCtx wc{&bars->abort, error_word};
#endif

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->kb_full[i], 1); mbar_init(&bars->kb_empty[i], 1);
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->s_free[i], 128);
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

  if (warp < 8) {
    // ================================ select ================================
    const int wg = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t best[L];
#pragma unroll
    for (int e = 0; e < L; ++e) best[e] = 0u;                   // 0 sorts below every real key
    // The two warpgroups take alternate chunks of the same 128 rows, so each keeps
    // its own list per row; the lists are merged at the end through shared memory.
    for (int c = wg; c < n_chunks; c += 2) {
      const uint32_t u = (uint32_t)c >> 1;
      mbar_wait(&bars->s_full[wg], u & 1, wc);
      tc_fence_after();
      const int c0 = c * kTile;
      const int cmax = tile - c0;                               // columns [0, cmax) are candidates
      const bool full = cmax >= kTile;
      uint32_t v[32];
#pragma unroll 1
      for (int ch = 0; ch < 4; ++ch) {
        tmem_ld32(tmem + lane_off + wg * 128 + ch * 32, v);
        tmem_ld_wait();
        const uint32_t inv0 = 0xFFFFu - (uint32_t)(c0 + ch * 32);   // low half of column 0's key
#pragma unroll
        for (int g = 0; g < 8; ++g) {
          const uint32_t w0 = monotone16x2(round_pack2<T>(__uint_as_float(v[g * 4 + 0]), __uint_as_float(v[g * 4 + 1])));
          const uint32_t w1 = monotone16x2(round_pack2<T>(__uint_as_float(v[g * 4 + 2]), __uint_as_float(v[g * 4 + 3])));
          uint32_t k0 = (w0 << 16) | (inv0 - (g * 4 + 0));
          uint32_t k1 = (w0 & 0xFFFF0000u) | (inv0 - (g * 4 + 1));
          uint32_t k2 = (w1 << 16) | (inv0 - (g * 4 + 2));
          uint32_t k3 = (w1 & 0xFFFF0000u) | (inv0 - (g * 4 + 3));
          if (!full) {
            const int col = ch * 32 + g * 4;
            k0 = (col + 0 < cmax) ? k0 : 0u;
            k1 = (col + 1 < cmax) ? k1 : 0u;
            k2 = (col + 2 < cmax) ? k2 : 0u;
            k3 = (col + 3 < cmax) ? k3 : 0u;
          }
          // Mostly at most one key of a group enters the list: offer the largest, and the
          // other three only if one of them still beats the list's last entry. Keys are
          // distinct (the column is in the low half), so exactly one equals the maximum.
          const uint32_t m = max(max(k0, k1), max(k2, k3));
          if (m > best[L - 1]) {
            list_offer<L>(best, m);
            k0 = (k0 == m) ? 0u : k0;
            k1 = (k1 == m) ? 0u : k1;
            k2 = (k2 == m) ? 0u : k2;
            k3 = (k3 == m) ? 0u : k3;
            if (max(max(k0, k1), max(k2, k3)) > best[L - 1]) {
              list_offer<L>(best, k0);
              list_offer<L>(best, k1);
              list_offer<L>(best, k2);
              list_offer<L>(best, k3);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->s_free[wg]);
    }
    // ---- merge the two warpgroups' lists (warpgroup 1 -> shared -> warpgroup 0) ----
    uint32_t* xk = reinterpret_cast<uint32_t*>(sKb);            // the Kbar stages are idle by now
    asm volatile("bar.sync 2, 256;" ::: "memory");              // every S MMA has been consumed
    if (wg == 1) {
#pragma unroll
      for (int e = 0; e < L; ++e) xk[e * kTile + r] = best[e];
    }
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (wg == 0 && row0 + r < sp.len) {
#pragma unroll
      for (int e = 0; e < L; ++e) list_offer<L>(best, xk[e * kTile + r]);
      // ---- emit: the best `take` ids plus the own block, ascending, -1 padded ----
      int ids[L];
      int kept = 0;
#pragma unroll
      for (int e = 0; e < L; ++e) {
        const bool ok = e < take && best[e] != 0u;
        ids[e] = ok ? (int)(0xFFFFu - (best[e] & 0xFFFFu)) : kEmpty;
        kept += ok ? 1 : 0;
      }
      int32_t* dst = block_idx + ((b * p.q_heads + hq) * p.tokens + sp.bos + row0 + r) * (size_t)p.slots;
#pragma unroll
      for (int e = 0; e < L; ++e) {                             // rank by id: position in the output
        if (ids[e] == kEmpty) continue;
        int rank = 0;
#pragma unroll
        for (int f = 0; f < L; ++f) rank += (ids[f] < ids[e]) ? 1 : 0;
        dst[rank] = ids[e];
      }
      if (p.always_current) dst[kept++] = tile;                 // the own block is past every candidate
      for (int e = kept; e < p.slots; ++e) dst[e] = -1;
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
      // Every MMA has completed before the CTA lets go of its TMEM, also on the way out of
      // a run that gave up on a wait.
      umma_commit(&bars->drain);
      mbar_wait_quiet(&bars->drain, 0);
    }
    __syncwarp();
  } else {
    if (lane == 0 && n_chunks > 0) {
      const int tok0 = (int)(b * p.tokens) + sp.bos + row0;
      mbar_expect_tx(&bars->q_full, Cfg::kOperand);
      for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d(sQ + s * kSub, &q_map, &bars->q_full, s * 64, hq, tok0);
      int issued = 0;
      for (int c = 0; c < n_chunks; ++c) {
        const uint32_t st = c & 1, u = (uint32_t)c >> 1;
        if (u >= 1) mbar_wait(&bars->kb_empty[st], (u - 1) & 1, wc);
        if (*wc.abort) break;                            // no new loads once a wait gave up
        mbar_expect_tx(&bars->kb_full[st], Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s)
          tma_load_3d(sKb + st * Cfg::kOperand + s * kSub, &kb_map, &bars->kb_full[st], s * 64, c * kTile, kv_row);
        issued = c + 1;
      }
      // No load may be in flight into this CTA's shared memory when it exits.
      mbar_wait_quiet(&bars->q_full, 0);
      for (int k = 1; k <= 2 && k <= issued; ++k) {
        const int c = issued - k;
        mbar_wait_quiet(&bars->kb_full[c & 1], ((uint32_t)c >> 1) & 1);
      }
    }
    __syncwarp();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, 256);
}


template <int D, typename T, int L>
int launch_one(const moba_b200_problem& p, const CUtensorMap& qm, const CUtensorMap& km, const int32_t* cu,
               int32_t* block_idx, unsigned* err, cudaStream_t st) {
  auto kern = gate_sm100_kernel<D, T, L>;
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
         p.num_blocks <= 0xFFFF &&
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
#define GO(D, T) return (p.take <= 7) ? launch_one<D, T, 7>(p, qm, km, cu, block_idx, err, st) \
                                      : launch_one<D, T, 8>(p, qm, km, cu, block_idx, err, st)
  if (p.head_dim == 64) { if (bf) GO(64, __nv_bfloat16); else GO(64, __half); }
  if (bf) GO(128, __nv_bfloat16); else GO(128, __half);
#undef GO
}

}  // namespace moba
