// Forward, portable kernels: marker fill, KV-block-major attention on CUDA
// cores (any dtype / block size / head dim that fits shared memory) and the
// log2-sum-exp merge. The merge is shared with the tcgen05 forward.
//
// Numerics contract of the attention (same as the tcgen05 kernel):
//   s = (q . k) * D^-1/2 * log2(e)  in float32, masked (tail keys, and keys
//   after the query inside the own block when causal); m = max s;
//   p = exp2(s - m); l = sum p (unrounded); p is rounded to the dtype of v
//   before p.v; the partial stores O_i = (p.v)/l and lse_i = m + log2 l.
// Reference: src/moba/kernels/moba_fwd.py:229-425 (it stores m, l and the
// unnormalised accumulator instead; the merged result is the same quantity).
#include "common.cuh"

namespace moba {

__global__ void fill_kernel(float* __restrict__ dst, size_t n, float value) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = value;
}

int launch_fill_lse(const moba_b200_problem& p, float* part_lse, cudaStream_t st) {
  KernelTimer timer__("fill_kernel", st);
  const size_t n = (size_t)p.batch * p.q_heads * window_rows(p) * p.slots;
  const int blocks = (int)((n + 1023) / 1024 < 148 * 8 ? (n + 1023) / 1024 : 148 * 8);
  fill_kernel<<<blocks > 0 ? blocks : 1, 256, 0, st>>>(part_lse, n, -INFINITY);
  MOBA_LAUNCH_OK("fill_kernel");
  return MOBA_B200_OK;
}

// ---------------------------------------------------------------------------
// portable attention: grid (num_blocks, n_seq * Hkv), 256 threads. A warp
// handles four gathered query rows at a time; lanes run over keys for the
// scores and over the head dim for p.v.
// ---------------------------------------------------------------------------
constexpr int kFwdWarps = 8;
constexpr int kFwdRows = 4;       // rows per warp iteration

template <typename T, typename TP>
__global__ void __launch_bounds__(256)
fwd_portable_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                    moba_b200_index ix, const int32_t* __restrict__ cu, TP* __restrict__ part_o,
                    float* __restrict__ part_lse, moba_b200_problem p) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int d = p.head_dim, bs = p.block_size, nb = p.num_blocks;
  const int kstride = d + 1;
  float* Ks = reinterpret_cast<float*>(smem_raw);           // [bs][d+1]
  float* Vs = Ks + bs * kstride;                            // [bs][d]
  float* Qs = Vs + bs * d;                                  // [warps][rows][d]
  float* Ps = Qs + kFwdWarps * kFwdRows * d;                // [warps][rows][bs]

  const int kv_row = blockIdx.y;
  const int seq = kv_row / p.kv_heads, kvh = kv_row % p.kv_heads;
  const int blk = ix.order[(size_t)kv_row * nb + blockIdx.x];
  const int n = ix.col_nnz[(size_t)kv_row * nb + blk];
  if (n == 0) return;
  const int lo = ix.col_offsets[(size_t)kv_row * (nb + 1) + blk];
  const SeqSpan sp = seq_span(cu, p.packed, seq, p.tokens);
  const size_t b = p.packed ? 0 : (size_t)seq;
  const int key0 = sp.bos + blk * bs;                       // token index of the block's first key
  const int keys = min(bs, sp.bos + sp.len - key0);
  if (keys <= 0) return;

  for (int i = threadIdx.x; i < bs * d; i += 256) {
    const int j = i / d, c = i % d;
    float kv = 0.f, vv = 0.f;
    if (j < keys) {
      const size_t src = ((b * p.tokens + key0 + j) * p.kv_heads + kvh) * (size_t)d + c;
      kv = Elem<T>::to_f(k[src]);
      vv = Elem<T>::to_f(v[src]);
    }
    Ks[j * kstride + c] = kv;
    Vs[j * d + c] = vv;
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float scale = rsqrtf((float)d) * kLog2e;
  const int32_t* rows_i = ix.row_indices + (size_t)kv_row * ix.capacity + lo;
  const int32_t* heads_i = ix.head_indices + (size_t)kv_row * ix.capacity + lo;
  const int32_t* slots_i = ix.slot_of_pair + (size_t)kv_row * ix.capacity + lo;
  float* qw = Qs + warp * kFwdRows * d;
  float* pw = Ps + warp * kFwdRows * bs;
  const int key_iters = (bs + 31) / 32;

  for (int e0 = warp * kFwdRows; e0 < n; e0 += kFwdWarps * kFwdRows) {
    int row[kFwdRows], head[kFwdRows], slot[kFwdRows];
#pragma unroll
    for (int r = 0; r < kFwdRows; ++r) {
      const bool live = e0 + r < n;
      row[r] = live ? rows_i[e0 + r] : -1;
      head[r] = live ? heads_i[e0 + r] : 0;
      slot[r] = live ? slots_i[e0 + r] : 0;
      for (int c = lane; c < d; c += 32)
        qw[r * d + c] = live ? Elem<T>::to_f(q[((b * p.tokens + row[r]) * p.q_heads + head[r]) * (size_t)d + c]) : 0.f;
    }
    __syncwarp();
    float m[kFwdRows], l[kFwdRows];
#pragma unroll
    for (int r = 0; r < kFwdRows; ++r) m[r] = -INFINITY;
    // scores -> Ps (raw), row maxima
    for (int it = 0; it < key_iters; ++it) {
      const int j = it * 32 + lane;
      float acc[kFwdRows];
#pragma unroll
      for (int r = 0; r < kFwdRows; ++r) acc[r] = 0.f;
      if (j < bs) {
        const float* kr = Ks + j * kstride;
        for (int c = 0; c < d; ++c) {
          const float kv = kr[c];
#pragma unroll
          for (int r = 0; r < kFwdRows; ++r) acc[r] = fmaf(qw[r * d + c], kv, acc[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < kFwdRows; ++r) {
        float s = acc[r] * scale;
        const bool ok = j < keys && row[r] >= 0 && (!p.causal || key0 + j <= row[r]);
        s = ok ? s : -INFINITY;
        if (j < bs) pw[r * bs + j] = s;
        m[r] = fmaxf(m[r], s);
      }
    }
#pragma unroll
    for (int r = 0; r < kFwdRows; ++r) {
#pragma unroll
      for (int o = 16; o; o >>= 1) m[r] = fmaxf(m[r], __shfl_xor_sync(0xffffffffu, m[r], o));
      l[r] = 0.f;
    }
    __syncwarp();
    for (int it = 0; it < key_iters; ++it) {
      const int j = it * 32 + lane;
      if (j < bs) {
#pragma unroll
        for (int r = 0; r < kFwdRows; ++r) {
          const float s = pw[r * bs + j];
          const float pe = (s == -INFINITY) ? 0.f : exp2f(s - m[r]);
          l[r] += pe;
          pw[r * bs + j] = Elem<T>::round_f(pe);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kFwdRows; ++r) {
#pragma unroll
      for (int o = 16; o; o >>= 1) l[r] += __shfl_xor_sync(0xffffffffu, l[r], o);
    }
    __syncwarp();
    // p.v, lanes over the head dim
    for (int c = lane; c < d; c += 32) {
      float o[kFwdRows];
#pragma unroll
      for (int r = 0; r < kFwdRows; ++r) o[r] = 0.f;
      for (int j = 0; j < keys; ++j) {
        const float vv = Vs[j * d + c];
#pragma unroll
        for (int r = 0; r < kFwdRows; ++r) o[r] = fmaf(pw[r * bs + j], vv, o[r]);
      }
#pragma unroll
      for (int r = 0; r < kFwdRows; ++r) {
        if (row[r] < 0) continue;
        const size_t dst = part_row(p, b, head[r], row[r]) * (size_t)p.slots + slot[r];
        part_o[dst * d + c] = Elem<TP>::from_f(o[r] / l[r]);
      }
    }
    // lane r publishes row r's log2-sum-exp
#pragma unroll
    for (int r = 0; r < kFwdRows; ++r) {
      if (lane == r && row[r] >= 0) {
        const size_t dst = part_row(p, b, head[r], row[r]) * (size_t)p.slots + slot[r];
        part_lse[dst] = m[r] + log2f(l[r]);
      }
    }
    __syncwarp();
  }
}

static size_t fwd_portable_smem(const moba_b200_problem& p) {
  const size_t d = p.head_dim, bs = p.block_size;
  return sizeof(float) * (bs * (d + 1) + bs * d + kFwdWarps * kFwdRows * (d + bs));
}

int launch_fwd_portable(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                        const moba_b200_index& ix, const int32_t* cu, void* part_o,
                        float* part_lse, cudaStream_t st) {
  KernelTimer timer__("fwd_portable_kernel", st);
  const size_t smem = fwd_portable_smem(p);
  if (smem > 220 * 1024) {
    set_error("forward: block_size %d with head_dim %d needs %zu bytes of shared memory",
              p.block_size, p.head_dim, smem);
    return MOBA_B200_EUNSUPPORTED;
  }
  if ((long long)p.n_seq * p.kv_heads > 65535) {
    set_error("portable forward: %d sequences x %d heads exceed 65535 grid rows", p.n_seq, p.kv_heads);
    return MOBA_B200_EUNSUPPORTED;
  }
  dim3 grid(p.num_blocks, p.n_seq * p.kv_heads);
#define MOBA_FWD(T, TP)                                                                        \
  do {                                                                                         \
    MOBA_CUDA_OK(cudaFuncSetAttribute(fwd_portable_kernel<T, TP>,                              \
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    fwd_portable_kernel<T, TP><<<grid, 256, smem, st>>>((const T*)q, (const T*)k, (const T*)v, \
                                                        ix, cu, (TP*)part_o, part_lse, p);     \
  } while (0)
  if (p.dtype == MOBA_B200_F32) MOBA_FWD(float, float);
  else if (p.dtype == MOBA_B200_BF16) { if (p.part_f32) MOBA_FWD(__nv_bfloat16, float); else MOBA_FWD(__nv_bfloat16, __nv_bfloat16); }
  else { if (p.part_f32) MOBA_FWD(__half, float); else MOBA_FWD(__half, __half); }
#undef MOBA_FWD
  MOBA_LAUNCH_OK("fwd_portable_kernel");
  return MOBA_B200_OK;
}

// ---------------------------------------------------------------------------
// merge: one thread per 16-byte vector of a partial row. Streams part_o once.
//   LSE = m + log2 sum_i 2^(lse_i - m),  O = sum_i 2^(lse_i - LSE) O_i
// Reference: src/moba/kernels/moba_fwd.py:428-521.
// ---------------------------------------------------------------------------
template <typename TP, typename TO>
__global__ void __launch_bounds__(256)
merge_kernel(const TP* __restrict__ part_o, const float* __restrict__ part_lse,
             TO* __restrict__ out, float* __restrict__ lse_out, int tokens,
             int q_heads, int d, int slots, int win_begin, int win_rows) {
  // grid (row groups of one (batch entry, head), heads, batch): no division anywhere (generic
  // 64-bit divisions cost this streaming kernel more instructions than its sums)
  constexpr int EPV = 16 / sizeof(TP);
  const unsigned tpr = (unsigned)(d / EPV);                  // threads per row, a power of two
  const unsigned gid = blockIdx.x * 256u + threadIdx.x;
  const unsigned row = gid / tpr;                            // row of the window
  const int c = (int)(gid % tpr);
  if (row >= (unsigned)win_rows) return;
  const size_t h = blockIdx.y, b = blockIdx.z, bh = b * q_heads + h;
  const size_t r = bh * win_rows + row;                      // head-major row (b, h, s) of the partials
  const float* ls = part_lse + r * slots;
  float mg = -INFINITY;
  for (int i = 0; i < slots; ++i) {
    const float li = ls[i];
    if (li > -INFINITY) mg = fmaxf(mg, li);
  }
  float acc[EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) acc[e] = 0.f;
  float wsum = 0.f;
  const TP* po = part_o + r * slots * (size_t)d + c * EPV;
  // One 16-byte load per thread at a time leaves the memory system short of requests, so
  // the slots are taken eight at a time: all loads first, then the sums in slot order.
  constexpr int kAhead = 8;
  for (int i0 = 0; i0 < slots; i0 += kAhead) {
    float li[kAhead];
    uint4 raw[kAhead];
#pragma unroll
    for (int u = 0; u < kAhead; ++u) li[u] = (i0 + u < slots) ? ls[i0 + u] : -INFINITY;
#pragma unroll
    for (int u = 0; u < kAhead; ++u)                           // unwritten: never touch its data
      raw[u] = (li[u] > -INFINITY) ? __ldcs(reinterpret_cast<const uint4*>(po + (size_t)(i0 + u) * d)) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < kAhead; ++u) {
      if (!(li[u] > -INFINITY)) continue;
      const float w = exp2f(li[u] - mg);
      wsum += w;
      const TP* vals = reinterpret_cast<const TP*>(&raw[u]);
#pragma unroll
      for (int e = 0; e < EPV; ++e) acc[e] = fmaf(w, Elem<TP>::to_f(vals[e]), acc[e]);
    }
  }
  const float inv = 1.f / wsum;                              // wsum == 0 -> NaN, as the reference
  const size_t s = (size_t)win_begin + row;
  TO* dst = out + ((b * tokens + s) * q_heads + h) * (size_t)d + c * EPV;
  __align__(16) TO packed_out[EPV];
#pragma unroll
  for (int e = 0; e < EPV; ++e) packed_out[e] = Elem<TO>::from_f(wsum > 0.f ? acc[e] * inv : NAN);
  if (sizeof(TO) * EPV == 16) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(packed_out);
  else *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(packed_out);
  if (lse_out != nullptr && c == 0) lse_out[bh * tokens + s] = (wsum > 0.f) ? mg + log2f(wsum) : -INFINITY;
}

int launch_merge(const moba_b200_problem& p, const void* part_o, const float* part_lse,
                 void* out, float* lse, cudaStream_t st) {
  KernelTimer timer__("merge_kernel", st);
  const bool pf32 = p.part_f32 || p.dtype == MOBA_B200_F32;
  const int epv = pf32 ? 4 : 8;
  const int tpr = p.head_dim / epv;
  const long long threads = (long long)window_rows(p) * tpr;
  if (tpr < 1 || (tpr & (tpr - 1)) || threads >= (1ll << 31) || p.q_heads > 65535 || p.batch > 65535) {
    set_error("merge: head_dim %d, %d heads or batch %d outside the kernel's grid", p.head_dim, p.q_heads, p.batch);
    return MOBA_B200_EUNSUPPORTED;
  }
  if (threads == 0 || p.batch == 0) return MOBA_B200_OK;
  const dim3 blocks((unsigned)((threads + 255) / 256), (unsigned)p.q_heads, (unsigned)p.batch);
#define MOBA_MERGE(TP, TO)                                                                      \
  merge_kernel<TP, TO><<<blocks, 256, 0, st>>>((const TP*)part_o, part_lse, (TO*)out, lse,      \
                                               p.tokens, p.q_heads, p.head_dim, p.slots,        \
                                               p.win_begin, window_rows(p))
  if (p.dtype == MOBA_B200_F32) MOBA_MERGE(float, float);
  else if (p.dtype == MOBA_B200_BF16) { if (pf32) MOBA_MERGE(float, __nv_bfloat16); else MOBA_MERGE(__nv_bfloat16, __nv_bfloat16); }
  else { if (pf32) MOBA_MERGE(float, __half); else MOBA_MERGE(__half, __half); }
#undef MOBA_MERGE
  MOBA_LAUNCH_OK("merge_kernel");
  return MOBA_B200_OK;
}

}  // namespace moba
