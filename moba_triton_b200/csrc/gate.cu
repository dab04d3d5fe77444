// Gate, portable kernels: block mean-pooling and the exact (float64) scorer with
// warp-level top-k selection. These run for every dtype / block size / head
// dim; the tcgen05 scorer in gate_sm100.cu replaces the second one for
// 16-bit inputs.
//
// Numerics contract (what makes selections comparable bit for bit):
//   block sum  = round_T(float(exact sum))      exact sum accumulated in float64
//   block mean = round_T(float(sum) / float(occupancy))
//   score      = round_T(float(exact dot))      unscaled
//   rank by (score desc, block id asc) over blocks strictly before the query's
//   own block; the own block is appended, never ranked.
// Reference behaviour being reproduced: src/moba/kernels/pooling.py:77-95 and
// src/moba/kernels/gating.py:183-335 (float32 accumulation there).
#include "common.cuh"

#include <float.h>

namespace moba {

// ---------------------------------------------------------------------------
// pool: grid (num_blocks, n_seq * Hkv), 128 threads
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
pool_kernel(const T* __restrict__ k, const int32_t* __restrict__ cu, T* __restrict__ kbar,
            int packed, int tokens, int hkv, int d, int bs, int nb) {
  constexpr int EPV = 16 / sizeof(T);            // elements per 16-byte vector
  const int blk = (int)(blockIdx.x % nb), kv_row = (int)(blockIdx.x / nb);
  const int seq = kv_row / hkv, h = kv_row % hkv;
  const SeqSpan sp = seq_span(cu, packed, seq, tokens);
  const int vpr = d / EPV;                       // vectors per row
  const int groups = 128 / vpr;
  const int c = threadIdx.x % vpr, rg = threadIdx.x / vpr;

  T* dst = kbar + ((size_t)kv_row * nb + blk) * d;
  const int lo = blk * bs;
  if (lo >= sp.len) {                            // padded slot of a short packed sequence
    if (threadIdx.x < d) dst[threadIdx.x] = Elem<T>::from_f(0.f);
    for (int i = threadIdx.x + 128; i < d; i += 128) dst[i] = Elem<T>::from_f(0.f);
    return;
  }
  const int hi = min(lo + bs, sp.len);
  const size_t batch_base = packed ? 0 : (size_t)seq * tokens;
  const T* src = k + ((batch_base + sp.bos + lo) * hkv + h) * (size_t)d + c * EPV;
  const size_t row_stride = (size_t)hkv * d;

  double acc[EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) acc[e] = 0.0;
  if (rg < groups) {
    // four rows in flight per thread: the loads do not depend on one another
    constexpr int kAhead = 4;
    for (int r0 = rg; r0 < hi - lo; r0 += groups * kAhead) {
      uint4 raw[kAhead];
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        const int r = r0 + u * groups;
        raw[u] = (r < hi - lo) ? *reinterpret_cast<const uint4*>(src + r * row_stride) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < kAhead; ++u) {
        if (r0 + u * groups < hi - lo) {
          const T* vals = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
          for (int e = 0; e < EPV; ++e) acc[e] += (double)Elem<T>::to_f(vals[e]);
        }
      }
    }
  }
  // Sums over the row groups, one output element per thread (float64 sums of these values are
  // exact, so the order of the additions does not matter).
  __shared__ double red[128 * EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) red[threadIdx.x * EPV + e] = acc[e];
  __syncthreads();
  const float occ = (float)(hi - lo);
  for (int i = threadIdx.x; i < d; i += 128) {
    double s = 0.0;
    for (int g = 0; g < groups; ++g) s += red[g * d + i];       // thread g * vpr + i / EPV, element i % EPV
    const float total = Elem<T>::round_f((float)s);
    dst[i] = Elem<T>::from_f(__fdiv_rn(total, occ));
  }
}

int launch_pool(const moba_b200_problem& p, const void* k, const int32_t* cu, void* kbar,
                cudaStream_t st) {
  KernelTimer timer__("pool_kernel", st);
  const int epv = 16 / (int)dtype_size(p.dtype);
  if (p.head_dim % epv || p.head_dim / epv > 128) {
    set_error("pool: head_dim %d unsupported", p.head_dim);
    return MOBA_B200_EUNSUPPORTED;
  }
  const long long ctas = (long long)p.num_blocks * p.n_seq * p.kv_heads;
  if (ctas > 0x7fffffffLL) { set_error("pool: %lld blocks exceed the grid limit", ctas); return MOBA_B200_EUNSUPPORTED; }
  const unsigned grid = (unsigned)ctas;
#define MOBA_POOL(T)                                                                   \
  pool_kernel<T><<<grid, 128, 0, st>>>((const T*)k, cu, (T*)kbar, p.packed, p.tokens,  \
                                       p.kv_heads, p.head_dim, p.block_size, p.num_blocks)
  if (p.dtype == MOBA_B200_F32) MOBA_POOL(float);
  else if (p.dtype == MOBA_B200_BF16) MOBA_POOL(__nv_bfloat16);
  else MOBA_POOL(__half);
#undef MOBA_POOL
  MOBA_LAUNCH_OK("pool_kernel");
  return MOBA_B200_OK;
}

// ---------------------------------------------------------------------------
// portable gate: grid (cdiv(max_seqlen, 32), n_seq * Hq), 128 threads.
// Each warp owns 8 query rows; a lane scores one candidate block of the
// current 32-block chunk for all 8 rows in float64, then the warp merges the
// chunk into each row's running list (shared memory, `take` entries).
// ---------------------------------------------------------------------------
constexpr int kGateRows = 32;
constexpr int kGateChunk = 32;
constexpr int kRowsPerWarp = 8;
constexpr int kEmptyIdx = 0x7fffffff;

struct Cand {
  float v;
  int i;
};
// best = larger score, ties to the smaller id
__device__ __forceinline__ Cand warp_best(Cand c) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, c.v, o);
    int oi = __shfl_xor_sync(0xffffffffu, c.i, o);
    if (ov > c.v || (ov == c.v && oi < c.i)) { c.v = ov; c.i = oi; }
  }
  return c;
}
// weakest = smaller score, ties to the larger id (so the lower id survives)
__device__ __forceinline__ Cand warp_weakest(Cand c, int& slot) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, c.v, o);
    int oi = __shfl_xor_sync(0xffffffffu, c.i, o);
    int os = __shfl_xor_sync(0xffffffffu, slot, o);
    if (ov < c.v || (ov == c.v && (oi > c.i || (oi == c.i && os < slot)))) {
      c.v = ov; c.i = oi; slot = os;
    }
  }
  return c;
}

template <typename T>
__global__ void __launch_bounds__(128)
gate_portable_kernel(const T* __restrict__ q, const T* __restrict__ kbar,
                     const int32_t* __restrict__ cu, int32_t* __restrict__ block_idx,
                     moba_b200_problem p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int d = p.head_dim, take = p.take, slots = p.slots;
  double* qs = reinterpret_cast<double*>(smem_raw);                       // [32][d]
  double* ks = qs + kGateRows * d;                                        // [32][d+1]
  float* lval = reinterpret_cast<float*>(ks + kGateChunk * (d + 1));      // [32][take]
  int* lidx = reinterpret_cast<int*>(lval + kGateRows * max(take, 1));    // [32][take]

  const int group = p.q_heads / p.kv_heads;
  const int seq = blockIdx.y / p.q_heads, hq = blockIdx.y % p.q_heads;
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  const int row0 = blockIdx.x * kGateRows;
  if (row0 >= sp.len) return;
  const int n_cand = (sp.len + p.block_size - 1) / p.block_size;
  const size_t batch_base = p.packed ? 0 : (size_t)seq * p.tokens;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // stage the 32 query rows as float64; dead rows are zero
  for (int i = threadIdx.x; i < kGateRows * d; i += 128) {
    const int r = i / d, c = i % d;
    double v = 0.0;
    if (row0 + r < sp.len)
      v = (double)Elem<T>::to_f(q[((batch_base + sp.bos + row0 + r) * p.q_heads + hq) * (size_t)d + c]);
    qs[i] = v;
  }
  for (int i = threadIdx.x; i < kGateRows * take; i += 128) {
    lval[i] = -INFINITY;
    lidx[i] = kEmptyIdx;
  }
  __syncthreads();

  const int last_row = min(row0 + kGateRows, sp.len) - 1;
  const int horizon = min(last_row / p.block_size, n_cand);      // blocks < horizon can be candidates
  const T* kb = kbar + ((size_t)seq * p.kv_heads + hq / group) * p.num_blocks * (size_t)d;
  float thr[kRowsPerWarp];                                       // current entry bar per row
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) thr[r] = -INFINITY;

  for (int c0 = 0; take > 0 && c0 < horizon; c0 += kGateChunk) {
    __syncthreads();
    for (int i = threadIdx.x; i < kGateChunk * d; i += 128) {
      const int j = i / d, c = i % d;
      ks[j * (d + 1) + c] = (c0 + j < n_cand) ? (double)Elem<T>::to_f(kb[(size_t)(c0 + j) * d + c]) : 0.0;
    }
    __syncthreads();

    double acc[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) acc[r] = 0.0;
    const double* krow = ks + lane * (d + 1);
    const double* qrow = qs + warp * kRowsPerWarp * d;
    for (int c = 0; c < d; ++c) {
      const double kv = krow[c];
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) acc[r] = fma(qrow[r * d + c], kv, acc[r]);
    }
    const int blk = c0 + lane;
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int lrow = warp * kRowsPerWarp + r;
      const int row = row0 + lrow;
      const int own = row / p.block_size;
      float s = Elem<T>::round_f((float)acc[r]);
      if (!(gate_candidate(p, blk, own) && blk < n_cand && row < sp.len)) s = -INFINITY;
      float* lv = lval + lrow * take;
      int* li = lidx + lrow * take;
      // offer the chunk's candidates in (score desc, id asc) order while they clear the bar
      while (__any_sync(0xffffffffu, s > thr[r])) {
        Cand best = warp_best(Cand{s, blk});
        // weakest list entry (ties: highest id; empty entries carry the largest id)
        Cand weak{INFINITY, -1};
        int wslot = 0x7fffffff;
        for (int e = lane; e < take; e += 32) {
          const float ev = lv[e];
          const int ei = li[e];
          if (ev < weak.v || (ev == weak.v && (ei > weak.i || (ei == weak.i && e < wslot)))) {
            weak.v = ev; weak.i = ei; wslot = e;
          }
        }
        weak = warp_weakest(weak, wslot);
        if (!(best.v > weak.v)) break;           // cannot happen while thr is current; safety
        if (lane == 0) { lv[wslot] = best.v; li[wslot] = best.i; }
        if (blk == best.i) s = -INFINITY;
        __syncwarp();
        // new bar = weakest entry after the insert
        float m = INFINITY;
        for (int e = lane; e < take; e += 32) m = fminf(m, lv[e]);
#pragma unroll
        for (int o = 16; o; o >>= 1) m = fminf(m, __shfl_xor_sync(0xffffffffu, m, o));
        thr[r] = m;
      }
    }
  }
  __syncwarp();

  // emit ascending ids: rank every kept entry (and the own block) by id
#pragma unroll 1
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int lrow = warp * kRowsPerWarp + r;
    const int row = row0 + lrow;
    if (row >= sp.len) continue;
    const int own = row / p.block_size;
    const int* li = lidx + lrow * take;
    const size_t b = p.packed ? 0 : (size_t)seq;
    int32_t* out = block_idx + ((b * p.q_heads + hq) * p.tokens + sp.bos + row) * (size_t)slots;
    const int n_items = take + (p.always_current ? 1 : 0);
    int kept = 0;
    for (int e = lane; e < n_items; e += 32) {
      const int id = (e < take) ? li[e] : own;
      if (id == kEmptyIdx) continue;
      int rank = 0;
      for (int f = 0; f < n_items; ++f) {
        const int other = (f < take) ? li[f] : own;
        rank += (other < id) ? 1 : 0;
      }
      out[rank] = id;
      ++kept;
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) kept += __shfl_xor_sync(0xffffffffu, kept, o);
    for (int e = kept + lane; e < slots; e += 32) out[e] = -1;
  }
}

int launch_gate_portable(const moba_b200_problem& p, const void* q, const void* kbar,
                         const int32_t* cu, int32_t* block_idx, cudaStream_t st) {
  KernelTimer timer__("gate_portable_kernel", st);
  const int d = p.head_dim;
  const size_t smem = sizeof(double) * (kGateRows * d + kGateChunk * (d + 1)) +
                      (size_t)kGateRows * (p.take > 0 ? p.take : 1) * 8;
  if (smem > 200 * 1024) {
    set_error("gate: head_dim %d / top_k %d need %zu bytes of shared memory", d, p.top_k, smem);
    return MOBA_B200_EUNSUPPORTED;
  }
  if ((long long)p.n_seq * p.q_heads > 65535) {
    set_error("portable gate: %d sequences x %d heads exceed 65535 grid rows", p.n_seq, p.q_heads);
    return MOBA_B200_EUNSUPPORTED;
  }
  dim3 grid((p.max_seqlen + kGateRows - 1) / kGateRows, p.n_seq * p.q_heads);
#define MOBA_GATE(T)                                                                          \
  do {                                                                                        \
    MOBA_CUDA_OK(cudaFuncSetAttribute(gate_portable_kernel<T>,                                \
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    gate_portable_kernel<T><<<grid, 128, smem, st>>>((const T*)q, (const T*)kbar, cu, block_idx, p); \
  } while (0)
  if (p.dtype == MOBA_B200_F32) MOBA_GATE(float);
  else if (p.dtype == MOBA_B200_BF16) MOBA_GATE(__nv_bfloat16);
  else MOBA_GATE(__half);
#undef MOBA_GATE
  MOBA_LAUNCH_OK("gate_portable_kernel");
  return MOBA_B200_OK;
}

}  // namespace moba
