// Backward on tcgen05 tensor cores (bf16/f16, block_size 128, head_dim 64/128).
//
// Persistent CTAs walk the (sequence, kv head, block) columns longest-first,
// round-robin; the CTA that takes a column owns its dK and dV, which stay in
// TMEM for the whole column and are stored once.
// Per tile of 128 gathered queries (five MMAs, all M = 128):
//   S  = Q K^T            A Q  (K-major)   B K  (K-major)   N 128  -> TMEM [0,128)
//   dP = dO V^T           A dO (K-major)   B V  (K-major)   N 128  -> TMEM [128,256)
//   P  = exp2(S c - lse), dS = P (dP - delta)   (256 threads, 64 columns each) -> smem, 16-bit
//   dV += P^T dO          A P  (M-major)   B dO (N-major)   N D    -> TMEM [256,256+D)
//   dK += dS^T Q          A dS (M-major)   B Q  (N-major)   N D    -> TMEM [256+D,256+2D)
//   dQ  = dS K            A dS (K-major)   B K  (N-major)   N D    -> TMEM [0,D)  (over S)
// dQ rows go to the (query, slot) partial buffer; a later pass sums the slots.
//
// Stands in for moba_bwd_kernel of the reference (src/moba/kernels/moba_bwd.py:215-394),
// which splits a block into 64-key sub-tiles for lack of shared memory.
#include "common.cuh"
#include "sm100.cuh"

#include <type_traits>

namespace moba {
using namespace sm100;

namespace {

constexpr int kTile = 128;
constexpr int kSub = kTile * 128;
constexpr int kMmaWarp = 8, kLoadWarp = 9, kGatherWarp0 = 10;
constexpr int kThreads = 14 * 32;

template <int D> struct BwdCfg {
  static constexpr int kSubs = D / 64;
  static constexpr int kOperand = kSubs * kSub;          // K, V, one Q stage, one dO stage
  static constexpr int kStages = (D == 64) ? 2 : 1;      // Q / dO gather stages
  static constexpr int kKvBufs = (D == 64) ? 2 : 1;
  static constexpr int kPBytes = 2 * kSub;
  // At head_dim 64 there is room for a staging tile of dQ of its own, so dQ can be the first
  // of a tile's last three MMAs and be written out while dV and dK run; at 128 it is staged
  // in the P buffer, after dV has read that.
  static constexpr bool kOwnStage = (D == 64);
  static constexpr int kStageBytes = kOwnStage ? kSub * (D / 64) : 0;
  static constexpr int kSmemData = 2 * kKvBufs * kOperand + 2 * kStages * kOperand + 2 * kPBytes + kStageBytes;
  static constexpr int kSmem = kSmemData + 1024 + 8192;
};

struct Bars {
  uint64_t k_full[2], v_full[2], kv_free[2], k_fix, v_fix;
  uint64_t qd_full[2], qd_empty[2];
  uint64_t sp_full, pds_full, dq_full, dq_read, acc_full, acc_read, drain;
  uint32_t tmem_base;
  int abort;
  // Per gathered row of each stage, written by the gather warps before they publish the
  // stage: {token row or -1, head << 8 | slot, lse, delta}. The elementwise warps never
  // touch global memory for these.
  int4 meta[2][kTile];
  unsigned char* out_ptr[kTile];            // destination dQ rows of the tile being stored
  long long row_off[kTile];                 // element offset of the gathered row in q / dout, -1 = dead
};

struct Column {
  int kv_row, blk, n, lo, key0, keys, bos;
  size_t b;
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

// The work list is sorted longest first; CTAs take it in alternating direction
// (0..G-1, G-1..0, ...) so that no CTA collects the largest column of every round.
__device__ __forceinline__ int snake_item(int round) {
  const int g = (int)gridDim.x, c = (int)blockIdx.x;
  return round * g + ((round & 1) ? (g - 1 - c) : c);
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

// 32 float32 columns of a TMEM row -> 32 T values * scale -> 64 contiguous bytes
template <typename T>
__device__ __forceinline__ void store_row32(unsigned char* dst, const uint32_t (&v)[32], float scale) {
  uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 w;
    w.x = pack2<T>(__uint_as_float(v[g * 8 + 0]) * scale, __uint_as_float(v[g * 8 + 1]) * scale);
    w.y = pack2<T>(__uint_as_float(v[g * 8 + 2]) * scale, __uint_as_float(v[g * 8 + 3]) * scale);
    w.z = pack2<T>(__uint_as_float(v[g * 8 + 4]) * scale, __uint_as_float(v[g * 8 + 5]) * scale);
    w.w = pack2<T>(__uint_as_float(v[g * 8 + 6]) * scale, __uint_as_float(v[g * 8 + 7]) * scale);
    d4[g] = w;
  }
}

template <int D, typename T>
__global__ void __launch_bounds__(kThreads, 1)
bwd_sm100_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                 const T* __restrict__ q, const T* __restrict__ dout, const float* __restrict__ lse,
                 const float* __restrict__ delta, moba_b200_index ix, const int32_t* __restrict__ cu,
                 T* __restrict__ dq_part, T* __restrict__ dk, T* __restrict__ dv, moba_b200_problem p,
                 int n_items, unsigned* error_word) {
  using Cfg = BwdCfg<D>;
  constexpr int NST = Cfg::kStages, NKV = Cfg::kKvBufs;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = smem;                                  // NKV buffers
  unsigned char* sV = sK + NKV * Cfg::kOperand;
  unsigned char* sQ = sV + NKV * Cfg::kOperand;              // NST stages
  unsigned char* sG = sQ + NST * Cfg::kOperand;              // dO, NST stages
  unsigned char* sP = sG + NST * Cfg::kOperand;
  unsigned char* sS = sP + Cfg::kPBytes;                     // dS
  unsigned char* sO = Cfg::kOwnStage ? sS + Cfg::kPBytes : sP;   // staging of the 16-bit dQ tile
  Bars* bars = reinterpret_cast<Bars*>(sS + Cfg::kPBytes + Cfg::kStageBytes);

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
      mbar_init(&bars->k_full[i], 1); mbar_init(&bars->v_full[i], 1); mbar_init(&bars->kv_free[i], 1);
      mbar_init(&bars->qd_full[i], 128); mbar_init(&bars->qd_empty[i], 1);
    }
    mbar_init(&bars->k_fix, 128); mbar_init(&bars->v_fix, 128);
    mbar_init(&bars->sp_full, 1); mbar_init(&bars->pds_full, 256);
    mbar_init(&bars->dq_full, 1); mbar_init(&bars->dq_read, 256);
    mbar_init(&bars->acc_full, 1); mbar_init(&bars->acc_read, 256); mbar_init(&bars->drain, 1);
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) tmem_alloc(&bars->tmem_base, 512);
  if (warp == kLoadWarp && lane == 0) { tma_prefetch_desc(&k_map); tma_prefetch_desc(&v_map); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  // At head_dim 64 TMEM has room for dQ columns of their own; at 128 dQ lands on S.
  constexpr uint32_t cS = 0, cDP = 128, cDV = 256, cDK = 256 + D, cDQ = Cfg::kOwnStage ? 256 + 2 * D : 0;

  const float softmax_scale = rsqrtf((float)D);
  const float cs = softmax_scale * kLog2e;
  const uint32_t fmt = std::is_same<T, __nv_bfloat16>::value ? 1u : 0u;

  if (warp < 8) {
    // =========================== elementwise warps ===========================
    const int wg = warp >> 2;                          // column half of the tile
    const int r = (warp & 3) * 32 + lane;              // tile row == TMEM lane
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t t = 0, it_cnt = 0;
    for (int round = 0; round * (int)gridDim.x < n_items; ++round) {
      const int item = snake_item(round);
      if (item >= n_items) continue;
      Column c;
      const bool work = load_column(c, item, ix, p, cu, n_kv_rows);
      const int kvh = c.kv_row % p.kv_heads;
      if (!work) {
        if (c.keys > 0 && r < c.keys) {                // nobody selected this block: exact zeros
          T* base = (wg == 0 ? dv : dk) + ((c.b * p.tokens + c.key0 + r) * p.kv_heads + kvh) * (size_t)D;
          for (int i = 0; i < D / 8; ++i) reinterpret_cast<uint4*>(base)[i] = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      const int nt = (c.n + kTile - 1) / kTile;
      for (int i = 0; i < nt; ++i, ++t) {
        // The stage's metadata was written before the gather warps published the stage, the
        // MMA warp waited for that before issuing S / dP, and sp_full follows those MMAs.
        // A wait that gave up leaves the stage's metadata stale or never written: the row then
        // counts as dead, so that no address is ever built from it.
        const bool sp_ok = mbar_wait(&bars->sp_full, t & 1, wc, 1);
        const int4 mt = sp_ok ? bars->meta[t % NST][r] : make_int4(-1, 0, 0, 0);
        const int row = mt.x < 0 ? 0 : mt.x, head = mt.y >> 8, slot = mt.y & 0xff;
        const bool live = mt.x >= 0;
        const float lse_r = __int_as_float(mt.z), delta_r = __int_as_float(mt.w);
        const size_t qrow = (c.b * p.q_heads + head) * p.tokens + row;
        int jmax = live ? c.keys - 1 : -1;             // dead rows contribute nothing
        if (p.causal && live && (row - c.bos) / kTile == c.blk) jmax = min(jmax, row - c.key0);

        tc_fence_after();
        uint32_t sv[32], pv[32];
        // Away from the diagonal block and the ragged ends every lane keeps all 128 keys;
        // such a tile runs without the per-element comparison.
        const bool all_open = __all_sync(0xffffffffu, jmax >= kTile - 1);
        auto p_ds_half = [&](int hc, auto masked) {
          const int col0 = wg * 64 + hc * 32;
          tmem_ld32(tmem + lane_off + cS + col0, sv);
          tmem_ld32(tmem + lane_off + cDP + col0, pv);
          tmem_ld_wait();
          unsigned char* p_sub = sP + wg * kSub;       // keys [64 wg, 64 wg + 64) live in sub-tile wg
          unsigned char* s_sub = sS + wg * kSub;
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            float pe[8], ds[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float x = ex2(fmaf(__uint_as_float(sv[g * 8 + k]), cs, -lse_r));
              if constexpr (decltype(masked)::value) pe[k] = (col0 + g * 8 + k <= jmax) ? x : 0.f;
              else pe[k] = x;
              ds[k] = pe[k] * (__uint_as_float(pv[g * 8 + k]) - delta_r);
            }
            uint4 wp, wd;
            wp.x = pack2<T>(pe[0], pe[1]); wp.y = pack2<T>(pe[2], pe[3]);
            wp.z = pack2<T>(pe[4], pe[5]); wp.w = pack2<T>(pe[6], pe[7]);
            wd.x = pack2<T>(ds[0], ds[1]); wd.y = pack2<T>(ds[2], ds[3]);
            wd.z = pack2<T>(ds[4], ds[5]); wd.w = pack2<T>(ds[6], ds[7]);
            const uint32_t off = swz128(r, hc * 4 + g);
            *reinterpret_cast<uint4*>(p_sub + off) = wp;
            *reinterpret_cast<uint4*>(s_sub + off) = wd;
          }
        };
        if (all_open) {
#pragma unroll 1
          for (int hc = 0; hc < 2; ++hc) p_ds_half(hc, std::false_type{});
        } else {
#pragma unroll 1
          for (int hc = 0; hc < 2; ++hc) p_ds_half(hc, std::true_type{});
        }
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(&bars->pds_full);

        // ---- dQ rows of this tile: this warpgroup stores columns [wg D/2, (wg+1) D/2) ----
        const bool dq_ok = mbar_wait(&bars->dq_full, t & 1, wc, 2);
        tc_fence_after();
        // Stage the 16-bit dQ tile in shared memory (a tile of its own, or the P buffer once
        // dV has read it) so that eight or sixteen adjacent lanes write each row; one row per
        // thread straight to global memory would touch 32 lines per instruction.
#pragma unroll 1
        for (int ch = 0; ch < D / 64; ++ch) {
          tmem_ld32(tmem + lane_off + cDQ + wg * (D / 2) + ch * 32, sv);
          tmem_ld_wait();
          const int c16 = wg * (D / 16) + ch * 4;          // first 16-byte chunk of these 32 columns
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(sv[g * 8 + 0]) * softmax_scale, __uint_as_float(sv[g * 8 + 1]) * softmax_scale);
            w.y = pack2<T>(__uint_as_float(sv[g * 8 + 2]) * softmax_scale, __uint_as_float(sv[g * 8 + 3]) * softmax_scale);
            w.z = pack2<T>(__uint_as_float(sv[g * 8 + 4]) * softmax_scale, __uint_as_float(sv[g * 8 + 5]) * softmax_scale);
            w.w = pack2<T>(__uint_as_float(sv[g * 8 + 6]) * softmax_scale, __uint_as_float(sv[g * 8 + 7]) * softmax_scale);
            *reinterpret_cast<uint4*>(sO + ((c16 + g) >> 3) * kSub + swz128(r, (c16 + g) & 7)) = w;
          }
        }
        tc_fence_before();
        mbar_arrive(&bars->dq_read);                     // S / dQ columns may be overwritten
        if (wg == 0) bars->out_ptr[r] = (live && dq_ok) ? reinterpret_cast<unsigned char*>(
                                                   dq_part + ((qrow * p.slots) + slot) * (size_t)D) : nullptr;
        asm volatile("bar.sync 2, 256;" ::: "memory");
        {
          constexpr int CPRO = D / 8;                    // 16-byte chunks per row
          constexpr int RPPO = 256 / CPRO;               // rows per pass of the 256 threads
          const int tid = wg * 128 + r;
          const int cc = tid % CPRO;
#pragma unroll
          for (int pass = 0; pass < kTile / RPPO; ++pass) {
            const int rr = pass * RPPO + tid / CPRO;
            unsigned char* op = bars->out_ptr[rr];
            const uint4 w = *reinterpret_cast<const uint4*>(sO + (cc >> 3) * kSub + swz128(rr, cc & 7));
            if (op != nullptr) *reinterpret_cast<uint4*>(op + cc * 16) = w;
          }
        }
        asm volatile("bar.sync 2, 256;" ::: "memory");   // the staging tile may be written again
      }
      // ---- the column's dV (warpgroup 0) and dK (warpgroup 1), one key row per thread ----
      const bool acc_ok = mbar_wait(&bars->acc_full, it_cnt & 1, wc, 3);
      tc_fence_after();
      {
        unsigned char* dst = reinterpret_cast<unsigned char*>(
            (wg == 0 ? dv : dk) + ((c.b * p.tokens + c.key0 + r) * p.kv_heads + kvh) * (size_t)D);
        const uint32_t col = (wg == 0) ? cDV : cDK;
        const float sc = (wg == 0) ? 1.f : softmax_scale;
        uint32_t av[32];
#pragma unroll 1
        for (int ch = 0; ch < D / 32; ++ch) {
          tmem_ld32(tmem + lane_off + col + ch * 32, av);
          tmem_ld_wait();
          if (acc_ok && r < c.keys) store_row32<T>(dst + ch * 64, av, sc);
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->acc_read);
      ++it_cnt;
    }
  } else if (warp == kMmaWarp) {
    // ============================== MMA issuer ==============================
    {
      const bool leader = elect_one();                 // all 32 lanes run the loop, one issues
      const uint32_t fbits = (fmt << 7) | (fmt << 10);
      const uint32_t id_s = make_idesc(0, 128, 128, 0, 0) | fbits;     // S, dP
      const uint32_t id_acc = make_idesc(0, 128, D, 1, 1) | fbits;     // dV, dK
      const uint32_t id_dq = make_idesc(0, 128, D, 0, 1) | fbits;      // dQ
      const uint32_t aP = smem_u32(sP), aS = smem_u32(sS);
      uint32_t t = 0, it_cnt = 0, pt_cnt = 0;
      for (int round = 0; round * (int)gridDim.x < n_items; ++round) {
      const int item = snake_item(round);
      if (item >= n_items) continue;
        Column c;
        if (!load_column(c, item, ix, p, cu, n_kv_rows)) continue;
        const int nt = (c.n + kTile - 1) / kTile;
        const bool partial = c.keys < kTile;
        const uint32_t kb = it_cnt % NKV, ku = it_cnt / NKV;
        const uint32_t aK = smem_u32(sK) + kb * Cfg::kOperand, aV = smem_u32(sV) + kb * Cfg::kOperand;
        mbar_wait(&bars->k_full[kb], ku & 1, wc, 4);
        mbar_wait(&bars->v_full[kb], ku & 1, wc, 5);
        if (partial) { mbar_wait(&bars->k_fix, pt_cnt & 1, wc, 6); mbar_wait(&bars->v_fix, pt_cnt & 1, wc, 6); }
        for (int i = 0; i < nt; ++i, ++t) {
          const uint32_t st = t % NST, us = t / NST;
          const uint32_t aQ = smem_u32(sQ) + st * Cfg::kOperand, aG = smem_u32(sG) + st * Cfg::kOperand;
          mbar_wait(&bars->qd_full[st], us & 1, wc, 8);
          // Where dQ shares the S columns and its staging the P tile, S of this tile waits for
          // the previous dQ to be read out. With columns and a staging tile of its own, S and
          // dP run while the elementwise warps write dQ out: they finished reading S and dP
          // before pds_full, and sp_full also covers the dV / dK that read P and dS.
          if (!Cfg::kOwnStage && t >= 1) mbar_wait(&bars->dq_read, (t - 1) & 1, wc, 9);
          tc_fence_after();
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t o = (ks >> 2) * kSub + (ks & 3) * 32;
            if (leader) umma_f16(tmem + cS, make_sdesc(aQ + o, 16, 1024), make_sdesc(aK + o, 16, 1024), id_s, ks > 0);
          }
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t o = (ks >> 2) * kSub + (ks & 3) * 32;
            if (leader) umma_f16(tmem + cDP, make_sdesc(aG + o, 16, 1024), make_sdesc(aV + o, 16, 1024), id_s, ks > 0);
          }
          if (leader) umma_commit(&bars->sp_full);

          mbar_wait(&bars->pds_full, t & 1, wc, 10);
          // the previous column's dK / dV have been read out (S and dP of this tile did not need that)
          if (i == 0 && it_cnt >= 1) mbar_wait(&bars->acc_read, (it_cnt - 1) & 1, wc, 7);
          tc_fence_after();
          auto issue_dv = [&]() {
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {          // 16 queries per step
              if (leader) umma_f16(tmem + cDV, make_sdesc(aP + ks * 2048, kSub, 1024), make_sdesc(aG + ks * 2048, kSub, 1024),
                       id_acc, (i > 0 || ks > 0));
            }
          };
          // dQ is what the elementwise warps wait for: first if it has a staging tile of its
          // own, else right after dV, whose operand P the staging overwrites. dK (and dV) run
          // while they write dQ out.
          if (!Cfg::kOwnStage) issue_dv();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {            // 16 keys per step
            if (leader) umma_f16(tmem + cDQ, make_sdesc(aS + (ks >> 2) * kSub + (ks & 3) * 32, 16, 1024),
                     make_sdesc(aK + ks * 2048, kSub, 1024), id_dq, ks > 0);
          }
          if (leader) umma_commit(&bars->dq_full);
          if (Cfg::kOwnStage) issue_dv();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            if (leader) umma_f16(tmem + cDK, make_sdesc(aS + ks * 2048, kSub, 1024), make_sdesc(aQ + ks * 2048, kSub, 1024),
                     id_acc, (i > 0 || ks > 0));
          }
          if (leader) umma_commit(&bars->qd_empty[st]);
          if (i == nt - 1) { if (leader) umma_commit(&bars->acc_full); if (leader) umma_commit(&bars->kv_free[kb]); }
        }
        ++it_cnt;
        if (partial) ++pt_cnt;
      }
      // Every MMA has completed before the CTA lets go of its TMEM, also on the way out of
      // a run that gave up on a wait.
      if (leader) umma_commit(&bars->drain);
      mbar_wait_quiet(&bars->drain, 0);
    }
    __syncwarp();
  } else if (warp == kLoadWarp) {
    // ============================ K/V TMA loader ============================
    if (lane == 0) {
      uint32_t it_cnt = 0;
      for (int round = 0; round * (int)gridDim.x < n_items; ++round) {
      const int item = snake_item(round);
      if (item >= n_items) continue;
        Column c;
        if (!load_column(c, item, ix, p, cu, n_kv_rows)) continue;
        if (*wc.abort) break;                            // no new loads once a wait gave up
        const int kvh = c.kv_row % p.kv_heads;
        const int tok0 = (int)(c.b * p.tokens) + c.key0;
        const uint32_t kb = it_cnt % NKV, ku = it_cnt / NKV;
        if (ku >= 1) mbar_wait(&bars->kv_free[kb], (ku - 1) & 1, wc, 11);
        mbar_expect_tx(&bars->k_full[kb], Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s)
          tma_load_3d(sK + kb * Cfg::kOperand + s * kSub, &k_map, &bars->k_full[kb], s * 64, kvh, tok0);
        mbar_expect_tx(&bars->v_full[kb], Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s)
          tma_load_3d(sV + kb * Cfg::kOperand + s * kSub, &v_map, &bars->v_full[kb], s * 64, kvh, tok0);
        ++it_cnt;
      }
      // No load may be in flight into this CTA's shared memory when it exits.
      for (uint32_t k = 1; k <= (uint32_t)NKV && k <= it_cnt; ++k) {
        const uint32_t c = it_cnt - k;
        mbar_wait_quiet(&bars->k_full[c % NKV], (c / NKV) & 1);
        mbar_wait_quiet(&bars->v_full[c % NKV], (c / NKV) & 1);
      }
    }
    __syncwarp();
  } else {
    // ========================= query / dO row gatherers =========================
    const int pt = threadIdx.x - kGatherWarp0 * 32;
    constexpr int CPR = D / 8, RPP = 128 / CPR;
    uint32_t t = 0, it_cnt = 0;
    for (int round = 0; round * (int)gridDim.x < n_items; ++round) {
      const int item = snake_item(round);
      if (item >= n_items) continue;
      Column c;
      if (!load_column(c, item, ix, p, cu, n_kv_rows)) continue;
      const int nt = (c.n + kTile - 1) / kTile;
      const uint32_t kb = it_cnt % NKV, ku = it_cnt / NKV;
      if (c.keys < kTile) {
        const int dead = kTile - c.keys;
        mbar_wait(&bars->k_full[kb], ku & 1, wc, 12);
        for (int i = pt; i < dead * 8 * Cfg::kSubs; i += 128) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(sK + kb * Cfg::kOperand + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive(&bars->k_fix);
        mbar_wait(&bars->v_full[kb], ku & 1, wc, 12);
        for (int i = pt; i < dead * 8 * Cfg::kSubs; i += 128) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(sV + kb * Cfg::kOperand + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive(&bars->v_fix);
      }
      const int32_t* rows_i = ix.row_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      const int32_t* heads_i = ix.head_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      const int32_t* slots_i = ix.slot_of_pair + (size_t)c.kv_row * ix.capacity + c.lo;
      int n_row = 0, n_head = 0, n_slot = 0;               // index entry of the next tile, fetched ahead
      if (pt < c.n) { n_row = rows_i[pt]; n_head = heads_i[pt]; n_slot = slots_i[pt]; }
      for (int i = 0; i < nt; ++i, ++t) {
        const uint32_t st = t % NST, us = t / NST;
        const int e = i * kTile + pt;
        long long off = -1;
        int4 mt = make_int4(-1, 0, 0, 0);
        if (e < c.n) {
          off = (long long)(((c.b * p.tokens + n_row) * p.q_heads + n_head) * (size_t)D);
          const size_t qr = (c.b * p.q_heads + n_head) * p.tokens + n_row;
          mt = make_int4(n_row, (n_head << 8) | n_slot, __float_as_int(lse[qr]), __float_as_int(delta[qr]));
        }
        if (e + kTile < c.n) { n_row = rows_i[e + kTile]; n_head = heads_i[e + kTile]; n_slot = slots_i[e + kTile]; }
        if (us >= 1) mbar_wait(&bars->qd_empty[st], (us - 1) & 1, wc, 13);
        bars->meta[st][pt] = mt;
        bars->row_off[pt] = off;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const uint32_t stage_q = smem_u32(sQ) + st * Cfg::kOperand;
        const uint32_t stage_g = smem_u32(sG) + st * Cfg::kOperand;
        const int cc = pt % CPR;
#pragma unroll
        for (int pass = 0; pass < CPR; ++pass) {
          const int rr = pass * RPP + pt / CPR;
          const long long ro = bars->row_off[rr];
          const uint32_t o = (cc >> 3) * kSub + swz128(rr, cc & 7);
          const long long eo = (ro < 0 ? 0 : ro) + cc * 8;
          cp_async16(stage_q + o, q + eo, ro < 0 ? 0u : 16u);
          cp_async16(stage_g + o, dout + eo, ro < 0 ? 0u : 16u);
        }
        cp_async_commit();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // Published as soon as it has landed: these warps have nothing else to do until the
        // next stage frees, and a tile held back until then costs the MMA warp a wait.
        cp_async_wait<0>();
        fence_proxy_async();
        mbar_arrive(&bars->qd_full[st]);
      }
      ++it_cnt;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, 512);
#ifdef MOBA_WAIT_STATS
  if (threadIdx.x < 32) {
    unsigned long long* out = reinterpret_cast<unsigned long long*>(error_word + 64) + (size_t)blockIdx.x * 32;
    out[threadIdx.x] = threadIdx.x == 31 ? (unsigned long long)(clock64() - kernel_t0) : wait_stats[threadIdx.x];
  }
#endif
}

template <int D, typename T>
int launch_one(const moba_b200_problem& p, const CUtensorMap& km, const CUtensorMap& vm, const void* q,
               const void* dout, const float* lse, const float* delta, const moba_b200_index& ix,
               const int32_t* cu, void* dq_part, void* dk, void* dv, int n_items, unsigned* err,
               cudaStream_t st) {
  auto kern = bwd_sm100_kernel<D, T>;
  MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<D>::kSmem));
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = n_items < sms ? n_items : sms;
  kern<<<grid, kThreads, BwdCfg<D>::kSmem, st>>>(km, vm, (const T*)q, (const T*)dout, lse, delta, ix, cu,
                                                  (T*)dq_part, (T*)dk, (T*)dv, p, n_items, err);
  MOBA_LAUNCH_OK("bwd_sm100_kernel");
  return MOBA_B200_OK;
}

}  // namespace

bool bwd_sm100_supported(const moba_b200_problem& p) {
  return (p.dtype == MOBA_B200_BF16 || p.dtype == MOBA_B200_F16) && p.block_size == 128 &&
         (p.head_dim == 64 || p.head_dim == 128) && (long long)p.batch * p.tokens < 0x7fffffffLL;
}

int launch_bwd_sm100(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                     const void* dout, const float* lse, const float* delta, const moba_b200_index& ix,
                     const int32_t* cu, void* dq_part, void* dk, void* dv, cudaStream_t st) {
  KernelTimer timer__("bwd_sm100_kernel", st);
  unsigned* err = device_error_word();
  if (err == nullptr) { set_error("backward: no device error word"); return MOBA_B200_ECUDA; }
  CUtensorMap km, vm;
  const uint64_t rows = (uint64_t)p.batch * p.tokens;
  int rc = encode_rows_map(&km, k, rows, p.kv_heads, p.head_dim, 128);
  if (rc) return rc;
  rc = encode_rows_map(&vm, v, rows, p.kv_heads, p.head_dim, 128);
  if (rc) return rc;
  const int n_items = p.num_blocks * p.n_seq * p.kv_heads;
  const bool bf = p.dtype == MOBA_B200_BF16;
  if (p.head_dim == 64) {
    if (bf) return launch_one<64, __nv_bfloat16>(p, km, vm, q, dout, lse, delta, ix, cu, dq_part, dk, dv, n_items, err, st);
    return launch_one<64, __half>(p, km, vm, q, dout, lse, delta, ix, cu, dq_part, dk, dv, n_items, err, st);
  }
  if (bf) return launch_one<128, __nv_bfloat16>(p, km, vm, q, dout, lse, delta, ix, cu, dq_part, dk, dv, n_items, err, st);
  return launch_one<128, __half>(p, km, vm, q, dout, lse, delta, ix, cu, dq_part, dk, dv, n_items, err, st);
}

}  // namespace moba
