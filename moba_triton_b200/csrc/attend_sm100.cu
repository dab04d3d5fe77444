// Forward attention on tcgen05 tensor cores (bf16/f16, block_size 128,
// head_dim 64 or 128).
//
// Persistent CTAs (one per SM) walk the (sequence, kv head, block) columns in
// longest-first order, round-robin. Per column:
//   loader   (1 thread)  TMA: the K block and the V block -> swizzled smem, once
//   gather   (2 warps)   cp.async: 128 selected query rows per tile -> swizzled smem
//   mma      (1 thread)  S = Q K^T (M128 N128 K=D) and O = P V (M128 N=D K128) into TMEM
//   softmax  (2 x 4 warps, alternating tiles) tcgen05.ld S, mask, exp2, row sum,
//            P (16-bit) -> smem; then tcgen05.ld O, normalise, store the partial
//            output row and its log2-sum-exp at the (query, slot) address
// TMEM: S[2] at columns 0/128, O[2] at 256 / 256+D (float32).
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
constexpr int kMmaWarp = 8, kLoadWarp = 9, kGatherWarp0 = 10;
constexpr int kGatherThreads = 64;           // two gather warps, two rows of a tile per thread
constexpr int kThreads = 12 * 32;            // 384 threads: up to 168 registers each

template <int D> struct FwdCfg {
  static constexpr int kSubs = D / 64;                 // sub-tiles per operand along the head dim
  static constexpr int kOperand = kSubs * kSub;        // bytes of K, V or one Q stage
  static constexpr int kQStages = (D == 64) ? 3 : 2;
  static constexpr int kPBytes = 2 * kSub;             // [128][128] 16-bit
  static constexpr int kSmemData = 2 * kOperand + kQStages * kOperand + 2 * kPBytes;
  static constexpr int kSmem = kSmemData + 1024 /*align*/ + 6144 /*barriers, pointers*/;
};

struct Bars {
  uint64_t k_full, v_full, k_fix, v_fix, k_free, v_free;
  uint64_t q_full[3], q_empty[3];
  uint64_t s_full[2], p_full[2], o_full[2], so_free[2];
  uint32_t tmem_base;
  int abort;
#ifdef MOBA_WAIT_STATS
  unsigned long long stats[16];            // debug builds: cycles per wait site / section
#endif
  unsigned char* out_ptr[2][kTile];        // destination rows of the tile each warpgroup is storing
  const void* row_ptr[2][kTile];           // gather sources of two consecutive tiles (nullptr = dead row)
};

struct Column {                            // one unit of work
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
__global__ void __launch_bounds__(kThreads, 1)
fwd_sm100_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map,
                 const T* __restrict__ q, moba_b200_index ix, const int32_t* __restrict__ cu,
                 TP* __restrict__ part_o, float* __restrict__ part_lse, moba_b200_problem p, int n_items,
                 unsigned* error_word) {
  using Cfg = FwdCfg<D>;
  constexpr int NQ = Cfg::kQStages;
  extern __shared__ unsigned char smem_dyn[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  unsigned char* sK = smem;
  unsigned char* sV = sK + Cfg::kOperand;
  unsigned char* sQ = sV + Cfg::kOperand;                       // NQ stages
  unsigned char* sP = sQ + NQ * Cfg::kOperand;                  // 2 buffers
  Bars* bars = reinterpret_cast<Bars*>(sP + 2 * Cfg::kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_kv_rows = p.n_seq * p.kv_heads;
#ifdef MOBA_WAIT_STATS
  const WaitCtx wc{&bars->abort, error_word, bars->stats};
  if (threadIdx.x < 16) bars->stats[threadIdx.x] = 0;
  const long long kernel_t0 = clock64();
#define STAT_T0() long long st0__ = clock64()
#define STAT_ADD(site) do { long long n__ = clock64(); atomicAdd(&bars->stats[site], (unsigned long long)(n__ - st0__)); st0__ = clock64(); } while (0)
#else
  const WaitCtx wc{&bars->abort, error_word};
#define STAT_T0() do {} while (0)
#define STAT_ADD(site) do {} while (0)
#endif

  if (threadIdx.x == 0) {
    mbar_init(&bars->k_full, 1); mbar_init(&bars->v_full, 1);
    mbar_init(&bars->k_fix, kGatherThreads); mbar_init(&bars->v_fix, kGatherThreads);
    mbar_init(&bars->k_free, 1); mbar_init(&bars->v_free, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&bars->q_full[i], kGatherThreads); mbar_init(&bars->q_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars->s_full[i], 1); mbar_init(&bars->p_full[i], 128);
      mbar_init(&bars->o_full[i], 1); mbar_init(&bars->so_free[i], 128);
    }
    bars->abort = 0;
    fence_barrier_init();
  }
  if (warp == kMmaWarp) tmem_alloc(&bars->tmem_base, 512);
  if (warp == kLoadWarp && lane == 0) { tma_prefetch_desc(&k_map); tma_prefetch_desc(&v_map); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;

  const float cs = rsqrtf((float)D) * kLog2e;
  const uint32_t fmt = (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) ? 1u : 0u;

  if (warp < 8) {
    // ===================== softmax + epilogue warpgroups =====================
    const int wg = warp >> 2;                         // handles tiles with (t & 1) == wg
    const int r = (warp & 3) * 32 + lane;             // row of the tile == TMEM lane
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;
    unsigned char* myP = sP + wg * Cfg::kPBytes;
    int t0 = 0;
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      Column c;
      if (!load_column(c, item, ix, p, cu, n_kv_rows)) continue;
      const int nt = (c.n + kTile - 1) / kTile;
      const int32_t* rows_i = ix.row_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      const int32_t* heads_i = ix.head_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      const int32_t* slots_i = ix.slot_of_pair + (size_t)c.kv_row * ix.capacity + c.lo;
      // Index entries of this warpgroup's next tile are fetched one tile ahead, so their
      // latency hides behind the current tile.
      const int i_first = ((t0 & 1) == wg) ? 0 : 1;
      int n_row = 0, n_head = 0, n_slot = 0;
      if (i_first < nt && i_first * kTile + r < c.n) {
        const int e0 = i_first * kTile + r;
        n_row = rows_i[e0]; n_head = heads_i[e0]; n_slot = slots_i[e0];
      }
      for (int i = i_first; i < nt; i += 2) {
        const int t = t0 + i;
        const uint32_t u = (uint32_t)t >> 1;
        const int e = i * kTile + r;
        const bool live = e < c.n;
        const int row = n_row, head = n_head, slot = n_slot;
        {
          const int e2 = e + 2 * kTile;
          const bool live2 = (i + 2 < nt) && e2 < c.n;
          n_row = n_head = n_slot = 0;
          if (live2) { n_row = ld_nc_pinned(rows_i + e2); n_head = ld_nc_pinned(heads_i + e2); n_slot = ld_nc_pinned(slots_i + e2); }
        }
        STAT_T0();
        int jmax = c.keys - 1;
        if (p.causal && live && (row - c.bos) / kTile == c.blk) jmax = min(jmax, row - c.key0);

        STAT_ADD(0); mbar_wait(&bars->s_full[wg], u & 1, wc); STAT_ADD(1);
        tc_fence_after();
        const uint32_t ts = tmem + lane_off + wg * 128;
        // The whole 128-column row of S sits in registers: four loads in flight, one wait.
        uint32_t v[128];
        tmem_ld32(ts, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
        tmem_ld32(ts + 32, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
        tmem_ld32(ts + 64, *reinterpret_cast<uint32_t(*)[32]>(&v[64]));
        tmem_ld32(ts + 96, *reinterpret_cast<uint32_t(*)[32]>(&v[96]));
        tmem_ld_wait();
        if (jmax < kTile - 1) {                       // tail block or the query's own block: mask
#pragma unroll
          for (int j = 0; j < kTile; ++j) v[j] = (j <= jmax) ? v[j] : 0xff800000u;   // -inf
        }
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int j = 0; j < kTile; j += 4) {
#pragma unroll
          for (int a = 0; a < 4; ++a) mx4[a] = fmaxf(mx4[a], __uint_as_float(v[j + a]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
        const float m2 = mx * cs;
        STAT_ADD(2);
        float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int c16 = 0; c16 < 16; ++c16) {          // 16-byte chunks of the P row
          float pe[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            pe[k] = ex2(fmaf(__uint_as_float(v[c16 * 8 + k]), cs, -m2));   // ex2(-inf) = 0 for masked keys
            l4[k & 3] += pe[k];
          }
          uint4 w;
          w.x = pack2<T>(pe[0], pe[1]); w.y = pack2<T>(pe[2], pe[3]);
          w.z = pack2<T>(pe[4], pe[5]); w.w = pack2<T>(pe[6], pe[7]);
          *reinterpret_cast<uint4*>(myP + (c16 >> 3) * kSub + swz128(r, c16 & 7)) = w;
        }
        const float l = (l4[0] + l4[1]) + (l4[2] + l4[3]);
        STAT_ADD(3);
        fence_proxy_async();
        tc_fence_before();
        mbar_arrive(&bars->p_full[wg]);

        // ---- epilogue of the same tile ----
        STAT_ADD(4); mbar_wait(&bars->o_full[wg], u & 1, wc); STAT_ADD(5);
        tc_fence_after();
        const uint32_t to = tmem + lane_off + 256 + wg * D;
        const float inv = 1.f / l;
        const size_t dst_row = ((c.b * p.q_heads + head) * p.tokens + row) * (size_t)p.slots + slot;
        TP* dst = part_o + dst_row * D;
#pragma unroll
        for (int ch = 0; ch < D / 32; ++ch) tmem_ld32(to + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(&v[ch * 32]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&bars->so_free[wg]);               // S and O columns of this buffer are free again
        STAT_ADD(6);
        if (live) part_lse[dst_row] = m2 + log2f(l);
        if (sizeof(TP) == 2) {
          // Stores of one row per thread would touch 32 different lines per instruction.
          // Stage the 16-bit tile in this warpgroup's P buffer (its MMA has retired) and
          // let eight (D=64) or sixteen (D=128) adjacent lanes write each row.
          unsigned char* stage = myP;                  // [128 rows][D/64 x 128 bytes], swizzled per 128 B
#pragma unroll
          for (int g = 0; g < D / 8; ++g) {
            uint4 w;
            w.x = pack2<T>(__uint_as_float(v[g * 8 + 0]) * inv, __uint_as_float(v[g * 8 + 1]) * inv);
            w.y = pack2<T>(__uint_as_float(v[g * 8 + 2]) * inv, __uint_as_float(v[g * 8 + 3]) * inv);
            w.z = pack2<T>(__uint_as_float(v[g * 8 + 4]) * inv, __uint_as_float(v[g * 8 + 5]) * inv);
            w.w = pack2<T>(__uint_as_float(v[g * 8 + 6]) * inv, __uint_as_float(v[g * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(stage + (g >> 3) * kSub + swz128(r, g & 7)) = w;
          }
          bars->out_ptr[wg][r] = live ? reinterpret_cast<unsigned char*>(dst) : nullptr;
          STAT_ADD(7);
          asm volatile("bar.sync %0, 128;" ::"r"(2 + wg) : "memory");
          STAT_ADD(8);
          constexpr int CPRO = D / 8;                  // 16-byte chunks per output row
          constexpr int RPPO = 128 / CPRO;             // rows per pass of the warpgroup
          const int tid = (warp & 3) * 32 + lane;
          const int cc = tid % CPRO;
#pragma unroll
          for (int pass = 0; pass < CPRO; ++pass) {
            const int rr = pass * RPPO + tid / CPRO;
            unsigned char* op = bars->out_ptr[wg][rr];
            const uint4 w = *reinterpret_cast<const uint4*>(stage + (cc >> 3) * kSub + swz128(rr, cc & 7));
            if (op != nullptr) *reinterpret_cast<uint4*>(op + cc * 16) = w;
          }
          STAT_ADD(9);
          asm volatile("bar.sync %0, 128;" ::"r"(2 + wg) : "memory");   // staging is P again from here on
          STAT_ADD(10);
        } else if (live) {
          float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
          for (int g = 0; g < D / 4; ++g)
            d4[g] = make_float4(__uint_as_float(v[g * 4 + 0]) * inv, __uint_as_float(v[g * 4 + 1]) * inv,
                                __uint_as_float(v[g * 4 + 2]) * inv, __uint_as_float(v[g * 4 + 3]) * inv);
        }
      }
      t0 += nt;
    }
  } else if (warp == kMmaWarp) {
    // ============================== MMA issuer ==============================
    if (lane == 0) {
      constexpr uint32_t idesc_s = make_idesc(0, 128, 128, 0, 0);
      constexpr uint32_t idesc_o = make_idesc(0, 128, D, 0, 1);
      const uint32_t fbits = (fmt << 7) | (fmt << 10);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aP = smem_u32(sP);
      uint32_t t = 0, it_cnt = 0, pt_cnt = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        Column c;
        if (!load_column(c, item, ix, p, cu, n_kv_rows)) continue;
        const int nt = (c.n + kTile - 1) / kTile;
        const bool partial = c.keys < kTile;
        mbar_wait(&bars->k_full, it_cnt & 1, wc);
        if (partial) mbar_wait(&bars->k_fix, pt_cnt & 1, wc);
        bool v_ready = false;
        auto issue_pv = [&](uint32_t tt) {
          const uint32_t b = tt & 1, u = tt >> 1;
          if (!v_ready) {
            mbar_wait(&bars->v_full, it_cnt & 1, wc);
            if (partial) mbar_wait(&bars->v_fix, pt_cnt & 1, wc);
            v_ready = true;
          }
          mbar_wait(&bars->p_full[b], u & 1, wc);
          tc_fence_after();
          const uint32_t pb = aP + b * Cfg::kPBytes;
#pragma unroll
          for (int ks = 0; ks < 8; ++ks) {
            const uint64_t da = make_sdesc(pb + (ks >> 2) * kSub + (ks & 3) * 32, 16, 1024);
            const uint64_t db = make_sdesc(aV + ks * 2048, kSub, 1024);
            umma_f16(tmem + 256 + b * D, da, db, idesc_o | fbits, ks > 0);
          }
          umma_commit(&bars->o_full[b]);
        };
        for (int i = 0; i < nt; ++i, ++t) {
          const uint32_t b = t & 1, u = t >> 1, qs = t % NQ, uq = t / NQ;
          mbar_wait(&bars->q_full[qs], uq & 1, wc);
          if (u >= 1) mbar_wait(&bars->so_free[b], (u - 1) & 1, wc);
          tc_fence_after();
          const uint32_t qb = aQ + qs * Cfg::kOperand;
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint64_t da = make_sdesc(qb + (ks >> 2) * kSub + (ks & 3) * 32, 16, 1024);
            const uint64_t db = make_sdesc(aK + (ks >> 2) * kSub + (ks & 3) * 32, 16, 1024);
            umma_f16(tmem + b * 128, da, db, idesc_s | fbits, ks > 0);
          }
          umma_commit(&bars->s_full[b]);
          umma_commit(&bars->q_empty[qs]);
          if (i == nt - 1) umma_commit(&bars->k_free);
          if (i >= 1) issue_pv(t - 1);
        }
        issue_pv(t - 1);
        umma_commit(&bars->v_free);
        ++it_cnt;
        if (partial) ++pt_cnt;
      }
    }
    __syncwarp();
  } else if (warp == kLoadWarp) {
    // ============================ K/V TMA loader ============================
    if (lane == 0) {
      uint32_t it_cnt = 0;
      for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
        Column c;
        if (!load_column(c, item, ix, p, cu, n_kv_rows)) continue;
        const int kvh = c.kv_row % p.kv_heads;
        const int tok0 = (int)(c.b * p.tokens) + c.key0;
        if (it_cnt >= 1) mbar_wait(&bars->k_free, (it_cnt - 1) & 1, wc);
        mbar_expect_tx(&bars->k_full, Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d(sK + s * kSub, &k_map, &bars->k_full, s * 64, kvh, tok0);
        if (it_cnt >= 1) mbar_wait(&bars->v_free, (it_cnt - 1) & 1, wc);
        mbar_expect_tx(&bars->v_full, Cfg::kOperand);
        for (int s = 0; s < Cfg::kSubs; ++s) tma_load_3d(sV + s * kSub, &v_map, &bars->v_full, s * 64, kvh, tok0);
        ++it_cnt;
      }
    }
    __syncwarp();
  } else {
    // ============================ query gatherers ============================
    const int pt = threadIdx.x - kGatherWarp0 * 32;      // 0..63
    constexpr int CPR = D / 8;                            // 16-byte chunks per row
    constexpr int RPP = kGatherThreads / CPR;             // rows per pass
    constexpr int PASSES = kTile / RPP;
    constexpr int LAG = NQ - 1;                           // tiles whose copies stay in flight
    uint32_t t = 0, it_cnt = 0;
    uint32_t issued = 0, arrived = 0;                     // tiles copied / published so far
    auto publish_all = [&]() {
      if (issued > arrived) {
        cp_async_wait<0>();
        fence_proxy_async();
        for (; arrived < issued; ++arrived) mbar_arrive(&bars->q_full[arrived % NQ]);
      }
    };
    for (int item = blockIdx.x; item < n_items; item += gridDim.x) {
      Column c;
      if (!load_column(c, item, ix, p, cu, n_kv_rows)) continue;
      const int nt = (c.n + kTile - 1) / kTile;
      if (c.keys < kTile) {
        // Publish the previous column's tiles first: the K load awaited below is issued
        // only after their MMAs have run.
        publish_all();
        // zero the rows of K and V past the end of the sequence (they belong to the next one)
        const int dead = kTile - c.keys;
        mbar_wait(&bars->k_full, it_cnt & 1, wc);
        for (int i = pt; i < dead * 8 * Cfg::kSubs; i += kGatherThreads) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(sK + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive(&bars->k_fix);
        mbar_wait(&bars->v_full, it_cnt & 1, wc);
        for (int i = pt; i < dead * 8 * Cfg::kSubs; i += kGatherThreads) {
          const int s = i / (dead * 8), rr = c.keys + (i % (dead * 8)) / 8, ch = i % 8;
          *reinterpret_cast<uint4*>(sV + s * kSub + rr * 128 + ch * 16) = make_uint4(0, 0, 0, 0);
        }
        fence_proxy_async();
        mbar_arrive(&bars->v_fix);
      }
      const int32_t* rows_i = ix.row_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      const int32_t* heads_i = ix.head_indices + (size_t)c.kv_row * ix.capacity + c.lo;
      for (int i = 0; i < nt; ++i, ++t) {
        const uint32_t qs = t % NQ, uq = t / NQ;
        const void* src[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int e = i * kTile + pt + h * kGatherThreads;
          src[h] = nullptr;
          if (e < c.n) src[h] = q + ((c.b * p.tokens + rows_i[e]) * p.q_heads + heads_i[e]) * (size_t)D;
        }
        if (uq >= 1) mbar_wait(&bars->q_empty[qs], (uq - 1) & 1, wc);
        const void** ptrs = bars->row_ptr[t & 1];          // double-buffered: one barrier per tile
        ptrs[pt] = src[0];
        ptrs[pt + kGatherThreads] = src[1];
        asm volatile("bar.sync 1, 64;" ::: "memory");
        const uint32_t stage = smem_u32(sQ) + qs * Cfg::kOperand;
        const int cc = pt % CPR;
#pragma unroll
        for (int pass = 0; pass < PASSES; ++pass) {
          const int rr = pass * RPP + pt / CPR;
          const unsigned char* sp = static_cast<const unsigned char*>(ptrs[rr]);
          const uint32_t dst = stage + (cc >> 3) * kSub + swz128(rr, cc & 7);
          cp_async16(dst, sp ? sp + cc * 16 : static_cast<const void*>(q), sp ? 16u : 0u);
        }
        cp_async_commit();
        ++issued;
        if (issued - arrived > LAG) {                      // publish the oldest tile in flight
          cp_async_wait<LAG>();
          fence_proxy_async();
          mbar_arrive(&bars->q_full[arrived % NQ]);
          ++arrived;
        }
      }
      ++it_cnt;
    }
    publish_all();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) tmem_dealloc(tmem, 512);
#ifdef MOBA_WAIT_STATS
  if (threadIdx.x < 16) {
    unsigned long long* out = reinterpret_cast<unsigned long long*>(error_word + 64) + blockIdx.x * 16;
    out[threadIdx.x] = (threadIdx.x == 15) ? (unsigned long long)(clock64() - kernel_t0) : bars->stats[threadIdx.x];
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
  kern<<<grid, kThreads, FwdCfg<D>::kSmem, st>>>(km, vm, (const T*)q, ix, cu, (TP*)part_o, part_lse, p,
                                                  n_items, err);
  MOBA_LAUNCH_OK("fwd_sm100_kernel");
  return MOBA_B200_OK;
}

}  // namespace

bool fwd_sm100_supported(const moba_b200_problem& p) {
  return (p.dtype == MOBA_B200_BF16 || p.dtype == MOBA_B200_F16) && p.block_size == 128 &&
         (p.head_dim == 64 || p.head_dim == 128) &&
         (long long)p.batch * p.tokens < 0x7fffffffLL;
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
  const int n_items = p.num_blocks * p.n_seq * p.kv_heads;
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
