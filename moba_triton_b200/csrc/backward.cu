// Backward, portable kernels: delta = rowsum(out * dout), the KV-block-owner
// gradient kernel on CUDA cores, and the dQ slot reduction. delta and the dQ
// reduction are shared with the tcgen05 backward.
//
// Numerics contract (same as the tcgen05 kernel; reference:
// src/moba/kernels/moba_bwd.py:215-394):
//   p  = exp2(q.k * D^-1/2 * log2e - lse)  (0 for masked keys and dead rows)
//   dV += round_T(p)^T dO,  dP = dO V^T,  dS = p * (dP - delta)   (float32)
//   dK += round_T(dS)^T Q,  dQ_part = round_T(dS) K * D^-1/2 -> dtype of q
//   dK is scaled by D^-1/2 once, when stored. A block nobody selected stores
//   zeros; dQ = sum of the written slots in slot order.
#include "common.cuh"

namespace moba {

// ---------------------------------------------------------------------------
// delta: one thread per 16-byte vector, shuffle-reduced across the row
// ---------------------------------------------------------------------------
// grid (row groups of one batch entry, batch). A row is (token s, head h) of batch entry b; the
// division by the head count that separates the two is a multiplication by a reciprocal the
// host prepared (exact for the 31-bit row numbers the launcher admits): generic 64-bit
// divisions had made this streaming kernel instruction-bound.
template <typename T>
__global__ void __launch_bounds__(256)
delta_kernel(const T* __restrict__ out, const T* __restrict__ dout, float* __restrict__ delta,
             unsigned rows_per_batch, int tokens, int q_heads, int d, unsigned long long heads_recip, int heads_shift) {
  constexpr int EPV = 16 / sizeof(T);
  const int tpr = d / EPV;                        // threads per row: power of two, <= 32
  const unsigned gid = blockIdx.x * 256u + threadIdx.x;
  const unsigned r = gid / (unsigned)tpr;         // row (s, h) of this batch entry; tpr is a power of two
  const int c = (int)(gid % (unsigned)tpr);
  const size_t b = blockIdx.y;
  float acc = 0.f;
  if (r < rows_per_batch) {
    const size_t at = (b * rows_per_batch + r) * (size_t)d + c * EPV;
    const uint4 a = *reinterpret_cast<const uint4*>(out + at);
    const uint4 g = *reinterpret_cast<const uint4*>(dout + at);
    const T* av = reinterpret_cast<const T*>(&a);
    const T* gv = reinterpret_cast<const T*>(&g);
#pragma unroll
    for (int e = 0; e < EPV; ++e) acc = fmaf(Elem<T>::to_f(av[e]), Elem<T>::to_f(gv[e]), acc);
  }
  for (int o = tpr >> 1; o; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (r < rows_per_batch && c == 0) {
    const unsigned s = (unsigned)(((unsigned long long)r * heads_recip) >> heads_shift);   // r / q_heads
    const unsigned h = r - s * (unsigned)q_heads;
    delta[(b * q_heads + h) * tokens + s] = acc;
  }
}

int launch_delta(const moba_b200_problem& p, const void* out, const void* dout, float* delta,
                 cudaStream_t st) {
  KernelTimer timer__("delta_kernel", st);
  const int epv = 16 / (int)dtype_size(p.dtype);
  const int tpr = p.head_dim / epv;
  if (tpr > 32 || tpr < 1 || (tpr & (tpr - 1))) {
    set_error("backward: head_dim %d unsupported for this dtype", p.head_dim);
    return MOBA_B200_EUNSUPPORTED;
  }
  const unsigned long long rows_per_batch = (unsigned long long)p.tokens * p.q_heads;
  if (rows_per_batch * tpr >= (1ull << 31) || p.batch > 65535) {
    set_error("backward: %llu rows per batch entry (or batch %d) exceed the delta kernel's grid", rows_per_batch, p.batch);
    return MOBA_B200_EUNSUPPORTED;
  }
  if (!rows_per_batch || !p.batch) return MOBA_B200_OK;
  // r / q_heads == (r * recip) >> shift for every r < 2^31, with recip = ceil(2^shift / q_heads)
  int log2h = 0;
  while ((1u << log2h) < (unsigned)p.q_heads) ++log2h;
  const int shift = 31 + log2h;
  const unsigned long long recip = ((1ull << shift) + p.q_heads - 1) / p.q_heads;
  const dim3 grid((unsigned)((rows_per_batch * tpr + 255) / 256), (unsigned)p.batch);
#define MOBA_DELTA(T) \
  delta_kernel<T><<<grid, 256, 0, st>>>((const T*)out, (const T*)dout, delta, (unsigned)rows_per_batch, p.tokens, \
                                        p.q_heads, p.head_dim, recip, shift)
  if (p.dtype == MOBA_B200_F32) MOBA_DELTA(float);
  else if (p.dtype == MOBA_B200_BF16) MOBA_DELTA(__nv_bfloat16);
  else MOBA_DELTA(__half);
#undef MOBA_DELTA
  MOBA_LAUNCH_OK("delta_kernel");
  return MOBA_B200_OK;
}

// ---------------------------------------------------------------------------
// portable backward: grid (num_blocks, n_seq * Hkv), 256 threads, tiles of 8
// gathered rows (one per warp).
//   phase 1  warp per row: scores and dP over keys (lanes), p and dS -> smem
//   phase 2  thread owns head-dim column d = tid % D and keys j = tid / D + i * 256 / D:
//            dV[j][d] += p[r][j] dO[r][d],  dK[j][d] += dS[r][j] q[r][d]
//   phase 3  warp per row: dQ[r][:] = dS[r][:] K, stored to the (query, slot) partial
// ---------------------------------------------------------------------------
constexpr int kBwdRows = 8;

template <typename T> struct Pad { static constexpr int value = 2; };   // 16-bit: odd word stride
template <> struct Pad<float> { static constexpr int value = 1; };

template <typename T>
__global__ void __launch_bounds__(256)
bwd_portable_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                    const T* __restrict__ dout, const float* __restrict__ lse,
                    const float* __restrict__ delta, moba_b200_index ix,
                    const int32_t* __restrict__ cu, T* __restrict__ dq_part, T* __restrict__ dk,
                    T* __restrict__ dv, moba_b200_problem p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int d = p.head_dim, bs = p.block_size, nb = p.num_blocks;
  const int kstride = d + Pad<T>::value;
  float* dKs = reinterpret_cast<float*>(smem_raw);          // [bs][d]
  float* dVs = dKs + bs * d;                                // [bs][d]
  float* Qs = dVs + bs * d;                                 // [8][d]
  float* Gs = Qs + kBwdRows * d;                            // [8][d]   dO rows
  float* Ps = Gs + kBwdRows * d;                            // [8][bs]
  float* Ss = Ps + kBwdRows * bs;                           // [8][bs]  dS rows
  T* Ks = reinterpret_cast<T*>(Ss + kBwdRows * bs);         // [bs][d+pad]
  T* Vs = Ks + bs * kstride;                                // [bs][d+pad]

  const int kv_row = blockIdx.y;
  const int seq = kv_row / p.kv_heads, kvh = kv_row % p.kv_heads;
  const int blk = ix.order[(size_t)kv_row * nb + blockIdx.x];
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  const size_t b = p.packed ? 0 : (size_t)seq;
  const int key0 = sp.bos + blk * bs;
  const int keys = min(bs, sp.bos + sp.len - key0);
  if (keys <= 0) return;                                    // padded column of a short sequence
  const int n = ix.col_nnz[(size_t)kv_row * nb + blk];
  const int lo = ix.col_offsets[(size_t)kv_row * (nb + 1) + blk];

  for (int i = threadIdx.x; i < bs * d; i += 256) {
    const int j = i / d, c = i % d;
    T kv = Elem<T>::from_f(0.f), vv = Elem<T>::from_f(0.f);
    if (j < keys) {
      const size_t src = ((b * p.tokens + key0 + j) * p.kv_heads + kvh) * (size_t)d + c;
      kv = k[src];
      vv = v[src];
    }
    Ks[j * kstride + c] = kv;
    Vs[j * kstride + c] = vv;
    dKs[i] = 0.f;
    dVs[i] = 0.f;
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float softmax_scale = rsqrtf((float)d);
  const float scale2 = softmax_scale * kLog2e;
  const int32_t* rows_i = ix.row_indices + (size_t)kv_row * ix.capacity + lo;
  const int32_t* heads_i = ix.head_indices + (size_t)kv_row * ix.capacity + lo;
  const int32_t* slots_i = ix.slot_of_pair + (size_t)kv_row * ix.capacity + lo;
  const int key_iters = (bs + 31) / 32;
  // phase-2 ownership: column dcol, keys jbase + i * jstep
  const int dcol = threadIdx.x % d;
  const int jbase = threadIdx.x / d, jstep = 256 / d;       // the launcher guarantees d divides 256

  for (int e0 = 0; e0 < n; e0 += kBwdRows) {
    // ---- phase 1 ----
    const int e = e0 + warp;
    const bool live = e < n;
    const int row = live ? rows_i[e] : -1;
    const int head = live ? heads_i[e] : 0;
    const int slot = live ? slots_i[e] : 0;
    float lse_r = 0.f, delta_r = 0.f;
    if (live) {
      const size_t qrow = (b * p.q_heads + head) * p.tokens + row;
      lse_r = lse[qrow];
      delta_r = delta[qrow];
    }
    for (int c = lane; c < d; c += 32) {
      float qv = 0.f, gv = 0.f;
      if (live) {
        const size_t src = ((b * p.tokens + row) * p.q_heads + head) * (size_t)d + c;
        qv = Elem<T>::to_f(q[src]);
        gv = Elem<T>::to_f(dout[src]);
      }
      Qs[warp * d + c] = qv;
      Gs[warp * d + c] = gv;
    }
    __syncwarp();
    for (int it = 0; it < key_iters; ++it) {
      const int j = it * 32 + lane;
      if (j >= bs) break;
      float s = 0.f, dp = 0.f;
      const T* kr = Ks + j * kstride;
      const T* vr = Vs + j * kstride;
      for (int c = 0; c < d; ++c) {
        s = fmaf(Qs[warp * d + c], Elem<T>::to_f(kr[c]), s);
        dp = fmaf(Gs[warp * d + c], Elem<T>::to_f(vr[c]), dp);
      }
      const bool ok = live && j < keys && (!p.causal || key0 + j <= row);
      const float pe = ok ? exp2f(s * scale2 - lse_r) : 0.f;
      const float ds = pe * (dp - delta_r);
      Ps[warp * bs + j] = Elem<T>::round_f(pe);
      Ss[warp * bs + j] = Elem<T>::round_f(ds);
    }
    __syncthreads();
    // ---- phase 2 ----
    {
      float qreg[kBwdRows], greg[kBwdRows];
#pragma unroll
      for (int r = 0; r < kBwdRows; ++r) {
        qreg[r] = Qs[r * d + dcol];
        greg[r] = Gs[r * d + dcol];
      }
      for (int j = jbase; j < keys; j += jstep) {
        float ak = dKs[j * d + dcol], av = dVs[j * d + dcol];
#pragma unroll
        for (int r = 0; r < kBwdRows; ++r) {
          av = fmaf(Ps[r * bs + j], greg[r], av);
          ak = fmaf(Ss[r * bs + j], qreg[r], ak);
        }
        dKs[j * d + dcol] = ak;
        dVs[j * d + dcol] = av;
      }
    }
    // ---- phase 3 ----
    if (live) {
      T* dst = dq_part + (part_row(p, b, head, row) * (size_t)p.slots + slot) * d;
      for (int c = lane; c < d; c += 32) {
        float acc = 0.f;
        for (int j = 0; j < keys; ++j) acc = fmaf(Ss[warp * bs + j], Elem<T>::to_f(Ks[j * kstride + c]), acc);
        dst[c] = Elem<T>::from_f(acc * softmax_scale);
      }
    }
    __syncthreads();
  }

  for (int i = threadIdx.x; i < keys * d; i += 256) {
    const int j = i / d, c = i % d;
    const size_t dst = ((b * p.tokens + key0 + j) * p.kv_heads + kvh) * (size_t)d + c;
    dk[dst] = Elem<T>::from_f(dKs[i] * softmax_scale);
    dv[dst] = Elem<T>::from_f(dVs[i]);
  }
}

int launch_bwd_portable(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                        const void* dout, const float* lse, const float* delta,
                        const moba_b200_index& ix, const int32_t* cu, void* dq_part, void* dk,
                        void* dv, cudaStream_t st) {
  KernelTimer timer__("bwd_portable_kernel", st);
  const size_t d = p.head_dim, bs = p.block_size;
  const size_t pad = p.dtype == MOBA_B200_F32 ? 1 : 2;
  const size_t smem = sizeof(float) * (2 * bs * d + 2 * kBwdRows * d + 2 * kBwdRows * bs) +
                      dtype_size(p.dtype) * 2 * bs * (d + pad);
  if (smem > 220 * 1024 || d > 256 || (256 % d) != 0) {
    set_error("backward: block_size %d with head_dim %d (%zu-byte elements) needs %zu bytes of "
              "shared memory; unsupported", p.block_size, p.head_dim, dtype_size(p.dtype), smem);
    return MOBA_B200_EUNSUPPORTED;
  }
  if ((long long)p.n_seq * p.kv_heads > 65535) {
    set_error("portable backward: %d sequences x %d heads exceed 65535 grid rows", p.n_seq, p.kv_heads);
    return MOBA_B200_EUNSUPPORTED;
  }
  dim3 grid(p.num_blocks, p.n_seq * p.kv_heads);
#define MOBA_BWD(T)                                                                            \
  do {                                                                                         \
    MOBA_CUDA_OK(cudaFuncSetAttribute(bwd_portable_kernel<T>,                                  \
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    bwd_portable_kernel<T><<<grid, 256, smem, st>>>((const T*)q, (const T*)k, (const T*)v,     \
        (const T*)dout, lse, delta, ix, cu, (T*)dq_part, (T*)dk, (T*)dv, p);                   \
  } while (0)
  if (p.dtype == MOBA_B200_F32) MOBA_BWD(float);
  else if (p.dtype == MOBA_B200_BF16) MOBA_BWD(__nv_bfloat16);
  else MOBA_BWD(__half);
#undef MOBA_BWD
  MOBA_LAUNCH_OK("bwd_portable_kernel");
  return MOBA_B200_OK;
}

// ---------------------------------------------------------------------------
// dQ reduction: sum of the written slots, in slot order, one thread per
// 16-byte vector. Reference: src/moba/kernels/moba_bwd.py:397-446.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
dq_reduce_kernel(const T* __restrict__ dq_part, const float* __restrict__ part_lse,
                 T* __restrict__ dq, int tokens, int q_heads, int d, int slots,
                 int win_begin, int win_rows) {
  // grid (row groups of one (batch entry, head), heads, batch): no division anywhere
  constexpr int EPV = 16 / sizeof(T);
  const unsigned tpr = (unsigned)(d / EPV);       // threads per row, a power of two
  const unsigned gid = blockIdx.x * 256u + threadIdx.x;
  const unsigned row = gid / tpr;                 // row of the window
  const int c = (int)(gid % tpr);
  if (row >= (unsigned)win_rows) return;
  const size_t h = blockIdx.y, b = blockIdx.z;
  const size_t r = (b * q_heads + h) * win_rows + row;   // head-major row (b, h, s) of the partials
  float acc[EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) acc[e] = 0.f;
  const float* ls = part_lse + r * slots;
  const T* src = dq_part + r * slots * (size_t)d + c * EPV;
  // eight slots at a time: all loads first (more requests in flight), then the sums in slot order
  constexpr int kAhead = 8;
  for (int i0 = 0; i0 < slots; i0 += kAhead) {
    bool live[kAhead];
    uint4 raw[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) live[u] = (i0 + u < slots) && (ls[i0 + u] > -INFINITY);
#pragma unroll
    for (int u = 0; u < kAhead; ++u)
      raw[u] = live[u] ? __ldcs(reinterpret_cast<const uint4*>(src + (size_t)(i0 + u) * d)) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (!live[u]) continue;
      const T* vals = reinterpret_cast<const T*>(&raw[u]);
#pragma unroll
      for (int e = 0; e < EPV; ++e) acc[e] += Elem<T>::to_f(vals[e]);
    }
  }
  const size_t s = (size_t)win_begin + row;
  __align__(16) T packed_out[EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) packed_out[e] = Elem<T>::from_f(acc[e]);
  *reinterpret_cast<uint4*>(dq + ((b * tokens + s) * q_heads + h) * (size_t)d + c * EPV) =
      *reinterpret_cast<const uint4*>(packed_out);
}

int launch_dq_reduce(const moba_b200_problem& p, const void* dq_part, const float* part_lse,
                     void* dq, cudaStream_t st) {
  KernelTimer timer__("dq_reduce_kernel", st);
  const int epv = 16 / (int)dtype_size(p.dtype);
  const int tpr = p.head_dim / epv;
  const long long threads = (long long)window_rows(p) * tpr;
  if (tpr < 1 || (tpr & (tpr - 1)) || threads >= (1ll << 31) || p.q_heads > 65535 || p.batch > 65535) {
    set_error("backward: head_dim %d, %d heads or batch %d outside the dQ reduction's grid", p.head_dim, p.q_heads, p.batch);
    return MOBA_B200_EUNSUPPORTED;
  }
  if (threads == 0 || p.batch == 0) return MOBA_B200_OK;
  const dim3 blocks((unsigned)((threads + 255) / 256), (unsigned)p.q_heads, (unsigned)p.batch);
#define MOBA_DQR(T) \
  dq_reduce_kernel<T><<<blocks, 256, 0, st>>>((const T*)dq_part, part_lse, (T*)dq, p.tokens, p.q_heads, p.head_dim, p.slots, \
                                              p.win_begin, window_rows(p))
  if (p.dtype == MOBA_B200_F32) MOBA_DQR(float);
  else if (p.dtype == MOBA_B200_BF16) MOBA_DQR(__nv_bfloat16);
  else MOBA_DQR(__half);
#undef MOBA_DQR
  MOBA_LAUNCH_OK("dq_reduce_kernel");
  return MOBA_B200_OK;
}

}  // namespace moba
