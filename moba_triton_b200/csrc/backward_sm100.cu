// Backward on tcgen05 tensor cores (bf16/f16, block_size 128, head_dim 64/128).
//
// Persistent CTAs walk the (sequence, kv head, block) columns longest-first,
// round-robin; the CTA that takes a column owns its dK and dV, which stay in
// TMEM for the whole column and are stored once.
// Per tile of 128 gathered queries (five MMAs, all M = 128):
//   S  = Q K^T            A Q  (K-major)   B K  (K-major)   N 128  -> TMEM [0,128)
//   dP = dO V^T           A dO (K-major)   B V  (K-major)   N 128  -> TMEM [128,256)
//   P  = exp2(S c - lse), dS = P (dP - delta)   (512 threads, 32 columns each) -> smem, 16-bit
//   dV += P^T dO          A P  (M-major)   B dO (N-major)   N D    -> TMEM [256,256+D)
//   dK += dS^T Q          A dS (M-major)   B Q  (N-major)   N D    -> TMEM [256+D,256+2D)
//   dQ  = dS K            A dS (from TMEM, written back over dP)   B K  (N-major)   N D    -> TMEM [0,D)  (over S)
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
constexpr int kElemWarps = 16;                           // four key quarters x four row groups
constexpr int kElemThreads = 32 * kElemWarps;
constexpr int kMmaWarp = kElemWarps, kLoadWarp = kMmaWarp + 1, kGatherWarp0 = kMmaWarp + 2;
constexpr int kThreads = (kElemWarps + 6) * 32;

template <int D> struct BwdCfg {
  static constexpr int kSubs = D / 64;
  static constexpr int kOperand = kSubs * kSub;          // K, V, one Q stage, one dO stage
  static constexpr int kStages = tensor_core_plan(D).bwd_gather_stages;   // Q / dO gather stages
  static constexpr int kKvBufs = tensor_core_plan(D).bwd_kv_buffers;
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
  int slot;      // dK/dV partial slot of this work item, -1: the item is the whole column
  size_t b;
};

// Work item `item` of the launch: the items of the (sequence, kv head) rows interleaved, each
// row's in its dispatch order (heaviest first). An item is a block and a range of the block's
// pair list; the items of a split column each own a dK/dV partial slot.
__device__ __forceinline__ bool load_column(Column& c, int item, const moba_b200_index& ix,
                                            const moba_b200_problem& p, const int32_t* cu, int n_kv_rows) {
  c.kv_row = item % n_kv_rows;
  WorkItem w;
  if (!load_work_item(w, ix, ix.col_nnz + (size_t)c.kv_row * p.num_blocks, c.kv_row, item / n_kv_rows)) {
    c.n = 0; c.keys = 0; c.slot = -1;                  // padding: nothing to do, nothing to zero
    return false;
  }
  c.blk = w.blk;
  c.n = w.n;
  c.slot = w.slot;
  c.lo = ix.col_offsets[(size_t)c.kv_row * (p.num_blocks + 1) + c.blk] + w.first;
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
                 T* __restrict__ dq_part, float* __restrict__ dkv_scratch, T* __restrict__ dk, T* __restrict__ dv,
                 moba_b200_problem p, int n_items, unsigned* error_word) {
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
      mbar_init(&bars->qd_full[i], 4); mbar_init(&bars->qd_empty[i], 1);
    }
    mbar_init(&bars->k_fix, 4); mbar_init(&bars->v_fix, 4);
    mbar_init(&bars->sp_full, 1); mbar_init(&bars->pds_full, kElemWarps);
    mbar_init(&bars->dq_full, 1); mbar_init(&bars->dq_read, kElemWarps);
    mbar_init(&bars->acc_full, 1); mbar_init(&bars->acc_read, kElemWarps); mbar_init(&bars->drain, 1);
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

  if (warp < kElemWarps) {
    // =========================== elementwise warps ===========================
    // Sixteen warps: warp w works on TMEM lanes (tile rows) [32 (w mod 4), +32) and on key
    // quarter w / 4 of the tile, i.e. 32 of a row's 128 scores. The tile's P / dS work is a
    // fixed number of instructions; spread over sixteen warps, the loads from TMEM of one
    // warp run under the arithmetic of the others.
    const int wq = warp >> 2;                          // key quarter of the tile
    const int r = (warp & 3) * 32 + lane;              // tile row == TMEM lane
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    uint32_t t = 0, it_cnt = 0;
    PHASE_CLOCK(ph);
    for (int round = 0; round * (int)gridDim.x < n_items; ++round) {
      const int item = snake_item(round);
      if (item >= n_items) continue;
      Column c;
      const bool work = load_column(c, item, ix, p, cu, n_kv_rows);
      const int kvh = c.kv_row % p.kv_heads;
      if (!work) {
        if (c.keys > 0 && r < c.keys && wq < 2) {      // nobody selected this block: exact zeros
          T* base = (wq == 0 ? dv : dk) + ((c.b * p.tokens + c.key0 + r) * p.kv_heads + kvh) * (size_t)D;
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
        PHASE_ADD(wc, 16, ph);                           // between tiles
        const bool sp_ok = mbar_wait(&bars->sp_full, t & 1, wc, 1);
        PHASE_ADD(wc, 17, ph);                           // sp_full wait
        TRACE(error_word, t, 0);
        const int4 mt = sp_ok ? bars->meta[t % NST][r] : make_int4(-1, 0, 0, 0);
        const int row = mt.x < 0 ? 0 : mt.x, head = mt.y >> 8, slot = mt.y & 0xff;
        const bool live = mt.x >= 0;
        const float lse_r = __int_as_float(mt.z), delta_r = __int_as_float(mt.w);
        int jmax = live ? c.keys - 1 : -1;             // dead rows contribute nothing
        if (p.causal && live && (row - c.bos) / kTile == c.blk) jmax = min(jmax, row - c.key0);

        tc_fence_after();
        // Away from the diagonal block and the ragged ends every lane keeps all 128 keys;
        // such a tile runs without the per-element comparison.
        const bool all_open = __all_sync(0xffffffffu, jmax >= kTile - 1);
        PHASE_ADD(wc, 18, ph);                           // row metadata
        {
          unsigned char* p_sub = sP + (wq >> 1) * kSub;   // keys [64 h, 64 h + 64) live in sub-tile h
          unsigned char* s_sub = sS + (wq >> 1) * kSub;
          auto p_ds = [&](auto masked) {
#pragma unroll
            for (int hc = 0; hc < 2; ++hc) {              // sixteen columns at a time: few live registers
              uint32_t sv[16], pv[16], dsk[8];
              const int col0 = wq * 32 + hc * 16;
              tmem_ld16(tmem + lane_off + cS + col0, sv);
              tmem_ld16(tmem + lane_off + cDP + col0, pv);
              tmem_ld_wait();
#pragma unroll
              for (int g = 0; g < 2; ++g) {
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
                const uint32_t off = swz128(r, (wq & 1) * 4 + hc * 2 + g);
                *reinterpret_cast<uint4*>(p_sub + off) = wp;
                *reinterpret_cast<uint4*>(s_sub + off) = wd;
                dsk[g * 4 + 0] = wd.x; dsk[g * 4 + 1] = wd.y; dsk[g * 4 + 2] = wd.z; dsk[g * 4 + 3] = wd.w;
              }
              // dS also goes back to TMEM, over the dP columns this thread has just read: dQ = dS K
              // takes it from there as operand A (keys [16 ks, +16) in the eight columns from 16 ks).
              tmem_st8(tmem + lane_off + cDP + col0, dsk);
            }
            tmem_st_wait();
          };
          if (all_open) p_ds(std::false_type{}); else p_ds(std::true_type{});
        }
        PHASE_ADD(wc, 19, ph);                           // P, dS: loads, arithmetic, stores
        TRACE(error_word, t, 1);
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive_warp(&bars->pds_full);
        PHASE_ADD(wc, 20, ph);                           // fences, arrival
        TRACE(error_word, t, 2);

        // ---- dQ rows of this tile: this quarter stores columns [wq D/4, (wq+1) D/4) ----
        const bool dq_ok = mbar_wait(&bars->dq_full, t & 1, wc, 2);
        tc_fence_after();
        PHASE_ADD(wc, 21, ph);                           // dq_full wait
        TRACE(error_word, t, 3);
        // Stage the 16-bit dQ tile in shared memory (a tile of its own, or the P buffer once
        // dV has read it) so that eight or sixteen adjacent lanes write each row; one row per
        // thread straight to global memory would touch 32 lines per instruction.
        {
          constexpr int QC = D / 4;                      // dQ columns of a quarter: 16 or 32
          uint32_t qv[QC];
          if constexpr (QC == 16) tmem_ld16(tmem + lane_off + cDQ + wq * QC, qv);
          else tmem_ld32(tmem + lane_off + cDQ + wq * QC, qv);
          tmem_ld_wait();
          const int c16 = wq * (QC / 8);                 // first 16-byte chunk of these columns
#pragma unroll
          for (int g = 0; g < QC / 8; ++g) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(qv[g * 8 + 0]) * softmax_scale, __uint_as_float(qv[g * 8 + 1]) * softmax_scale);
            w.y = pack2<T>(__uint_as_float(qv[g * 8 + 2]) * softmax_scale, __uint_as_float(qv[g * 8 + 3]) * softmax_scale);
            w.z = pack2<T>(__uint_as_float(qv[g * 8 + 4]) * softmax_scale, __uint_as_float(qv[g * 8 + 5]) * softmax_scale);
            w.w = pack2<T>(__uint_as_float(qv[g * 8 + 6]) * softmax_scale, __uint_as_float(qv[g * 8 + 7]) * softmax_scale);
            *reinterpret_cast<uint4*>(sO + ((c16 + g) >> 3) * kSub + swz128(r, (c16 + g) & 7)) = w;
          }
        }
        tc_fence_before();
        mbar_arrive_warp(&bars->dq_read);                     // S / dQ columns may be overwritten
        if (wq == 0) bars->out_ptr[r] = (live && dq_ok) ? reinterpret_cast<unsigned char*>(
                                                   dq_part + (part_row(p, c.b, head, row) * p.slots + slot) * (size_t)D) : nullptr;
        PHASE_ADD(wc, 22, ph);                           // dQ read and staged
        TRACE(error_word, t, 4);
        asm volatile("bar.sync 2, %0;" ::"n"(kElemThreads) : "memory");
        TRACE(error_word, t, 5);
        {
          constexpr int CPRO = D / 8;                    // 16-byte chunks per row
          constexpr int RPPO = kElemThreads / CPRO;      // rows per pass of the elementwise threads
          const int tid = wq * 128 + r;
          const int cc = tid % CPRO;
#pragma unroll
          for (int pass = 0; pass < kTile / RPPO; ++pass) {
            const int rr = pass * RPPO + tid / CPRO;
            unsigned char* op = bars->out_ptr[rr];
            const uint4 w = *reinterpret_cast<const uint4*>(sO + (cc >> 3) * kSub + swz128(rr, cc & 7));
            if (op != nullptr) st_global_stream16(op + cc * 16, w);
          }
        }
        asm volatile("bar.sync 2, %0;" ::"n"(kElemThreads) : "memory");   // the staging tile may be written again
        PHASE_ADD(wc, 23, ph);                           // barriers and dQ stores
        TRACE(error_word, t, 6);
      }
      // ---- the column's dV (quarters 0, 1) and dK (quarters 2, 3): half of a key row per thread ----
      const bool acc_ok = mbar_wait(&bars->acc_full, it_cnt & 1, wc, 3);
      tc_fence_after();
      {
        constexpr int HC = D / 2;                        // columns of a half
        const uint32_t col = ((wq < 2) ? cDV : cDK) + (wq & 1) * HC;
        const float sc = (wq < 2) ? 1.f : softmax_scale;
        uint32_t av[32];
        if (c.slot < 0) {                                // the item is the whole column: final values
          unsigned char* dst = reinterpret_cast<unsigned char*>(
              (wq < 2 ? dv : dk) + ((c.b * p.tokens + c.key0 + r) * p.kv_heads + kvh) * (size_t)D + (wq & 1) * HC);
#pragma unroll 1
          for (int ch = 0; ch < HC / 32; ++ch) {
            tmem_ld32(tmem + lane_off + col + ch * 32, av);
            tmem_ld_wait();
            if (acc_ok && r < c.keys) store_row32<T>(dst + ch * 64, av, sc);
          }
        } else {                                         // one of several items of the column: float32 partial
          float* dst = dkv_scratch + (((size_t)c.slot * 2 + (wq < 2 ? 0 : 1)) * kTile + r) * D + (wq & 1) * HC;
#pragma unroll 1
          for (int ch = 0; ch < HC / 32; ++ch) {
            tmem_ld32(tmem + lane_off + col + ch * 32, av);
            tmem_ld_wait();
            if (acc_ok && r < c.keys) {
#pragma unroll
              for (int g = 0; g < 8; ++g)
                reinterpret_cast<float4*>(dst + ch * 32)[g] =
                    make_float4(__uint_as_float(av[g * 4 + 0]) * sc, __uint_as_float(av[g * 4 + 1]) * sc,
                                __uint_as_float(av[g * 4 + 2]) * sc, __uint_as_float(av[g * 4 + 3]) * sc);
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive_warp(&bars->acc_read);
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
          TRACE(error_word, t, 0);
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
          TRACE(error_word, t, 1);

          mbar_wait(&bars->pds_full, t & 1, wc, 10);
          TRACE(error_word, t, 2);
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
          for (int ks = 0; ks < 8; ++ks) {            // 16 keys per step, dS from TMEM
            if (leader) umma_f16_ts(tmem + cDQ, tmem + cDP + 16 * ks,
                     make_sdesc(aK + ks * 2048, kSub, 1024), id_dq, ks > 0);
          }
          if (leader) umma_commit(&bars->dq_full);
          TRACE(error_word, t, 3);
          if (Cfg::kOwnStage) issue_dv();
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            if (leader) umma_f16(tmem + cDK, make_sdesc(aS + ks * 2048, kSub, 1024), make_sdesc(aQ + ks * 2048, kSub, 1024),
                     id_acc, (i > 0 || ks > 0));
          }
          if (leader) umma_commit(&bars->qd_empty[st]);
          TRACE(error_word, t, 4);
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
      const uint64_t keep = l2_policy_evict_last();
      const size_t index_elems = (size_t)n_kv_rows * ix.capacity;
      // The gather warps read a column's index entries a tile at a time from global memory;
      // asking the L2 for them a column ahead saves them a DRAM round trip per tile.
      auto prefetch_entries = [&](int round) {
        const int item = snake_item(round);
        Column c;
        if (round * (int)gridDim.x >= n_items || item >= n_items || !load_column(c, item, ix, p, cu, n_kv_rows)) return;
        const size_t lo = (size_t)c.kv_row * ix.capacity + c.lo;
        l2_prefetch_i32(ix.row_indices, lo, c.n, index_elems);
        l2_prefetch_i32(ix.head_indices, lo, c.n, index_elems);
        l2_prefetch_i32(ix.slot_of_pair, lo, c.n, index_elems);
      };
      prefetch_entries(0);
      for (int round = 0; round * (int)gridDim.x < n_items; ++round) {
      prefetch_entries(round + 1);
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
          tma_load_3d_hint(sK + kb * Cfg::kOperand + s * kSub, &k_map, &bars->k_full[kb], s * 64, kvh, tok0, keep);
        mbar_expect_tx(&bars->v_full[kb], Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s)
          tma_load_3d_hint(sV + kb * Cfg::kOperand + s * kSub, &v_map, &bars->v_full[kb], s * 64, kvh, tok0, keep);
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
    const uint64_t keep = l2_policy_evict_last();
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
        mbar_arrive_warp(&bars->k_fix);
        mbar_wait(&bars->v_full[kb], ku & 1, wc, 12);
        for (int i = pt; i < dead * 8 * Cfg::kSubs; i += 128) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(sV + kb * Cfg::kOperand + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive_warp(&bars->v_fix);
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
        TRACE(error_word, t, 0);
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
          cp_async16_hint(stage_q + o, q + eo, ro < 0 ? 0u : 16u, keep);
          cp_async16_hint(stage_g + o, dout + eo, ro < 0 ? 0u : 16u, keep);
        }
        cp_async_commit();
        TRACE(error_word, t, 1);
        if (NST == 1 && e + kTile < c.n) {
          // With one stage the copies of the next tile's rows cannot start before this tile's
          // last MMA has retired, and the MMA warp then waits for them. The rows are asked into
          // the L2 now (the index entry has arrived while this tile's copies were issued), so
          // that those copies find them there instead of in DRAM. With two stages the copies
          // run a tile ahead anyway and the extra requests only cost (0.72 -> 0.73 ms at D=64).
          const size_t nxt = ((c.b * p.tokens + n_row) * p.q_heads + n_head) * (size_t)D;
#pragma unroll
          for (int line = 0; line < D * 2 / 128; ++line) {
            l2_prefetch_line(q + nxt + line * 64);
            l2_prefetch_line(dout + nxt + line * 64);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // Published as soon as it has landed: these warps have nothing else to do until the
        // next stage frees, and a tile held back until then costs the MMA warp a wait.
        cp_async_wait<0>();
        fence_proxy_async();
        mbar_arrive_warp(&bars->qd_full[st]);
        TRACE(error_word, t, 2);
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

// dK / dV of the columns that were cut into several work items. CTA (x, y) looks at 256
// consecutive work items of one (sequence, kv head) row, one per thread, and of the first
// items of split columns it finds there takes every gridDim.y-th, starting at y, and of
// each such column the z-th part of its sums: it adds the column's float32 partials in item
// order and stores the result. Split columns are the heaviest ones and therefore neighbours in
// the dispatch order, hence the slicing; most CTAs find nothing and leave.
constexpr int kReduceSlices = 16;                       // at most; fewer when the rows give CTAs enough
template <int D, typename T>
__global__ void __launch_bounds__(256)
dkv_reduce_kernel(const float* __restrict__ dkv_scratch, moba_b200_index ix, const int32_t* __restrict__ cu,
                  T* __restrict__ dk, T* __restrict__ dv, moba_b200_problem p, int ctas_per_row) {
  __shared__ int4 found[256];
  __shared__ int n_found;
  const int kv_row = blockIdx.x / ctas_per_row;
  const int j = (blockIdx.x % ctas_per_row) * 256 + threadIdx.x;
  if (threadIdx.x == 0) n_found = 0;
  __syncthreads();
  int4 it = make_int4(0, 0, 0, -2);
  if (j < ix.items_per_row)
    it = __ldg(reinterpret_cast<const int4*>(ix.work_items) + (size_t)kv_row * ix.items_per_row + j);
  const bool first = it.w >= 0 && it.y == 0;               // the first item of a split column
  // position among the CTA's finds, in item order (so that the slices are the same on every run)
  const unsigned ballot = __ballot_sync(0xffffffffu, first);
  __shared__ int warp_finds[8];
  if ((threadIdx.x & 31) == 0) warp_finds[threadIdx.x >> 5] = __popc(ballot);
  __syncthreads();
  int before = __popc(ballot & ((1u << (threadIdx.x & 31)) - 1u));
  for (int w = 0; w < (int)(threadIdx.x >> 5); ++w) before += warp_finds[w];
  if (first) found[before] = it;
  if (threadIdx.x == 255) n_found = before + (first ? 1 : 0);
  __syncthreads();
  const int seq = kv_row / p.kv_heads, kvh = kv_row % p.kv_heads;
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  const size_t b = p.packed ? 0 : (size_t)seq;
  for (int f = blockIdx.y; f < n_found; f += (int)gridDim.y) {
    const int4 col = found[f];
    const int nnz = ix.col_nnz[(size_t)kv_row * p.num_blocks + col.x];
    const int tiles = (nnz + kTile - 1) / kTile;
    const int n_chunks = (tiles + ix.chunk_tiles - 1) / ix.chunk_tiles;
    const int key0 = sp.bos + col.x * kTile;
    const int keys = min(kTile, sp.bos + sp.len - key0);
    constexpr int V4 = D / 4;                              // float4 per row
    constexpr int kAhead = 4;                              // elements per thread in flight
    for (int i0 = (int)blockIdx.z * 256 * kAhead + threadIdx.x; i0 < 2 * kTile * V4; i0 += 256 * kAhead * (int)gridDim.z) {
      float4 acc[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) acc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int c = 0; c < n_chunks; ++c) {
#pragma unroll
        for (int u = 0; u < kAhead; ++u) {
          const int i = i0 + u * 256;
          const int which = i / (kTile * V4), row = (i / V4) % kTile, c4 = i % V4;
          if (row >= keys) continue;
          const float4 x = __ldcs(reinterpret_cast<const float4*>(
              dkv_scratch + (((size_t)(col.w + c) * 2 + which) * kTile + row) * D) + c4);
          acc[u].x += x.x; acc[u].y += x.y; acc[u].z += x.z; acc[u].w += x.w;
        }
      }
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int i = i0 + u * 256;
        const int which = i / (kTile * V4), row = (i / V4) % kTile, c4 = i % V4;
        if (row >= keys) continue;
        T* dst = (which == 0 ? dv : dk) + ((b * p.tokens + key0 + row) * p.kv_heads + kvh) * (size_t)D + c4 * 4;
        uint2 w;
        w.x = pack2<T>(acc[u].x, acc[u].y);
        w.y = pack2<T>(acc[u].z, acc[u].w);
        *reinterpret_cast<uint2*>(dst) = w;
      }
    }
  }
}

template <int D, typename T>
int launch_one(const moba_b200_problem& p, const CUtensorMap& km, const CUtensorMap& vm, const void* q,
               const void* dout, const float* lse, const float* delta, const moba_b200_index& ix,
               const int32_t* cu, void* dq_part, float* dkv_scratch, void* dk, void* dv, int n_items, unsigned* err,
               cudaStream_t st) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = n_items < sms ? n_items : sms;
  {
    KernelTimer timer__("bwd_sm100_kernel", st);
    auto kern = bwd_sm100_kernel<D, T>;
    MOBA_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdCfg<D>::kSmem));
    kern<<<grid, kThreads, BwdCfg<D>::kSmem, st>>>(km, vm, (const T*)q, (const T*)dout, lse, delta, ix, cu,
                                                    (T*)dq_part, dkv_scratch, (T*)dk, (T*)dv, p, n_items, err);
    MOBA_LAUNCH_OK("bwd_sm100_kernel");
  }
  KernelTimer timer__("dkv_reduce_kernel", st);
  const int ctas_per_row = (ix.items_per_row + 255) / 256;
  // z: the 2 x 128 x D sums of a column in parts of at least 1024 float4; fewer parts when the
  // rows alone give CTAs enough (every CTA first looks through its 256 items)
  const int x_ctas = ctas_per_row * p.n_seq * p.kv_heads;
  int slices = 4096 / x_ctas;
  slices = slices < 1 ? 1 : (slices > kReduceSlices ? kReduceSlices : slices);
  int parts = 4096 / (x_ctas * slices);
  parts = parts < 1 ? 1 : (parts > D / 16 ? D / 16 : parts);
  dkv_reduce_kernel<D, T><<<dim3(x_ctas, slices, parts), 256, 0, st>>>(
      dkv_scratch, ix, cu, (T*)dk, (T*)dv, p, ctas_per_row);
  MOBA_LAUNCH_OK("dkv_reduce_kernel");
  return MOBA_B200_OK;
}

}  // namespace

bool bwd_sm100_supported(const moba_b200_problem& p) {
  return (p.dtype == MOBA_B200_BF16 || p.dtype == MOBA_B200_F16) && p.block_size == 128 &&
         (p.head_dim == 64 || p.head_dim == 128) && (long long)p.batch * p.tokens < 0x7fffffffLL;
}

int launch_bwd_sm100(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                     const void* dout, const float* lse, const float* delta, const moba_b200_index& ix,
                     const int32_t* cu, void* dq_part, float* dkv_scratch, void* dk, void* dv, cudaStream_t st) {
  unsigned* err = device_error_word();
  if (err == nullptr) { set_error("backward: no device error word"); return MOBA_B200_ECUDA; }
  CUtensorMap km, vm;
  const uint64_t rows = (uint64_t)p.batch * p.tokens;
  int rc = encode_rows_map(&km, k, rows, p.kv_heads, p.head_dim, 128);
  if (rc) return rc;
  rc = encode_rows_map(&vm, v, rows, p.kv_heads, p.head_dim, 128);
  if (rc) return rc;
  if (ix.work_items == nullptr || ix.items_per_row <= 0 || ix.chunk_tiles <= 0) {
    set_error("backward: the index carries no work items (build it with moba_b200_transpose)");
    return MOBA_B200_EINVAL;
  }
  if (dkv_scratch == nullptr) { set_error("backward: dkv_scratch is NULL"); return MOBA_B200_EINVAL; }
  const long long n_items_ll = (long long)ix.items_per_row * p.n_seq * p.kv_heads;
  if (n_items_ll > 0x7fffffffLL) { set_error("backward: too many work items"); return MOBA_B200_EUNSUPPORTED; }
  const int n_items = (int)n_items_ll;
  const bool bf = p.dtype == MOBA_B200_BF16;
  if (p.head_dim == 64) {
    if (bf) return launch_one<64, __nv_bfloat16>(p, km, vm, q, dout, lse, delta, ix, cu, dq_part, dkv_scratch, dk, dv, n_items, err, st);
    return launch_one<64, __half>(p, km, vm, q, dout, lse, delta, ix, cu, dq_part, dkv_scratch, dk, dv, n_items, err, st);
  }
  if (bf) return launch_one<128, __nv_bfloat16>(p, km, vm, q, dout, lse, delta, ix, cu, dq_part, dkv_scratch, dk, dv, n_items, err, st);
  return launch_one<128, __half>(p, km, vm, q, dout, lse, delta, ix, cu, dq_part, dkv_scratch, dk, dv, n_items, err, st);
}

}  // namespace moba
