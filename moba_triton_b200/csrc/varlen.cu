// Packed (variable-length) batch boundary: the row gathers either side of the
// attention op.
//
//   pack    [B, S, row] + mask [B, S]  ->  [T, row] of the kept rows in (b, s) order,
//           cu_seqlens [B + 1] and the (total, longest) pair the host needs to size T
//   unpack  [T, row] + cu_seqlens      ->  [B, S, row], padding positions zeroed
//
// A row is one token's H * D elements, contiguous in the token-major layout, so
// both directions move whole rows with 16-byte accesses and no transposition.
// `pack` runs in three launches: a scan of every batch row's mask (local
// positions + row length), a scan over the row lengths (cu_seqlens, total,
// longest), and the row gather itself.
//
// Stands in for pack / unpack of the reference (src/moba/varlen.py:114-205), which
// index with the result of `nonzero()`.
#include "common.cuh"

namespace moba {

namespace {

constexpr int kScanThreads = 256;

// Exclusive prefix of `v` over the CTA (kScanThreads threads); `total` receives the sum.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_sums, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  __syncthreads();                                     // warp_sums may still be read from the last round
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  int before = 0, all = 0;
#pragma unroll
  for (int w = 0; w < kScanThreads / 32; ++w) {
    const int s = warp_sums[w];
    before += (w < warp) ? s : 0;
    all += s;
  }
  total = all;
  return before + incl - v;
}

// One CTA per batch row: dest[b, s] = how many kept tokens precede s in the row (or -1
// where the mask is zero), lengths[b] = kept tokens of the row.
template <typename M>
__global__ void __launch_bounds__(kScanThreads)
mask_scan_kernel(const M* __restrict__ mask, int seq_len, int32_t* __restrict__ dest, int32_t* __restrict__ lengths) {
  __shared__ int warp_sums[kScanThreads / 32];
  const size_t row = blockIdx.x;
  const M* m = mask + row * seq_len;
  int32_t* d = dest + row * seq_len;
  int running = 0;
  for (int s0 = 0; s0 < seq_len; s0 += kScanThreads) {
    const int s = s0 + threadIdx.x;
    const int keep = (s < seq_len && m[s] != M(0)) ? 1 : 0;
    int total;
    const int pos = block_exclusive_scan(keep, warp_sums, total);
    if (s < seq_len) d[s] = keep ? running + pos : -1;
    running += total;
  }
  if (threadIdx.x == 0) lengths[row] = running;
}

// One CTA: cu[0] = 0, cu[i + 1] = lengths[0] + ... + lengths[i]; meta = {total, longest}.
__global__ void __launch_bounds__(kScanThreads)
lengths_scan_kernel(const int32_t* __restrict__ lengths, int n, int32_t* __restrict__ cu, int32_t* __restrict__ meta) {
  __shared__ int warp_sums[kScanThreads / 32];
  __shared__ int longest_s;
  if (threadIdx.x == 0) longest_s = 0;
  __syncthreads();
  int running = 0, longest = 0;
  for (int i0 = 0; i0 < n; i0 += kScanThreads) {
    const int i = i0 + threadIdx.x;
    const int v = (i < n) ? lengths[i] : 0;
    int total;
    const int pos = block_exclusive_scan(v, warp_sums, total);
    if (i < n) cu[i + 1] = running + pos + v;
    running += total;
    longest = max(longest, v);
  }
  atomicMax(&longest_s, longest);
  __syncthreads();
  if (threadIdx.x == 0) { cu[0] = 0; meta[0] = running; meta[1] = longest_s; }
}

// meta = {cu[n], longest sequence} of an existing cu_seqlens (n sequences).
__global__ void __launch_bounds__(kScanThreads)
seq_meta_kernel(const int32_t* __restrict__ cu, int n, int32_t* __restrict__ meta) {
  __shared__ int longest_s;
  if (threadIdx.x == 0) longest_s = 0;
  __syncthreads();
  int longest = 0;
  for (int i = threadIdx.x; i < n; i += kScanThreads) longest = max(longest, cu[i + 1] - cu[i]);
  atomicMax(&longest_s, longest);
  __syncthreads();
  if (threadIdx.x == 0) { meta[0] = cu[n]; meta[1] = longest_s; }
}

// Thread per 16 bytes of a source row: kept rows go to packed[cu[b] + dest[b, s]].
__global__ void __launch_bounds__(256)
pack_rows_kernel(const uint4* __restrict__ x, const int32_t* __restrict__ dest, const int32_t* __restrict__ cu,
                 uint4* __restrict__ packed, size_t n_rows, int seq_len, int vec_per_row) {
  const size_t gid = (size_t)blockIdx.x * 256 + threadIdx.x;
  const size_t row = gid / vec_per_row;
  const int c = (int)(gid % vec_per_row);
  if (row >= n_rows) return;
  const int pos = dest[row];
  if (pos < 0) return;
  const size_t b = row / seq_len;
  packed[((size_t)cu[b] + pos) * vec_per_row + c] = __ldcs(x + row * vec_per_row + c);
}

// Thread per 16 bytes of the padded rectangle: its packed row, or zeros past the sequence.
__global__ void __launch_bounds__(256)
unpack_rows_kernel(const uint4* __restrict__ packed, const int32_t* __restrict__ cu, uint4* __restrict__ out,
                   size_t n_rows, int seq_len, int vec_per_row) {
  const size_t gid = (size_t)blockIdx.x * 256 + threadIdx.x;
  const size_t row = gid / vec_per_row;
  const int c = (int)(gid % vec_per_row);
  if (row >= n_rows) return;
  const size_t b = row / seq_len;
  const int s = (int)(row % seq_len);
  const int lo = cu[b], len = cu[b + 1] - lo;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (s < len) v = __ldcs(packed + ((size_t)lo + s) * vec_per_row + c);
  out[row * vec_per_row + c] = v;
}

int check_rows(int batch, int seq_len, size_t row_bytes, const char* what) {
  if (batch <= 0 || seq_len <= 0) { set_error("%s: batch and seq_len must be positive", what); return MOBA_B200_EINVAL; }
  if (row_bytes == 0 || row_bytes % 16) {
    set_error("%s: a row of %zu bytes is not a multiple of 16", what, row_bytes);
    return MOBA_B200_EUNSUPPORTED;
  }
  if ((unsigned long long)batch * seq_len * (row_bytes / 16) / 256 + 1 > 0x7fffffffULL) {
    set_error("%s: the batch exceeds the grid limit", what);
    return MOBA_B200_EUNSUPPORTED;
  }
  return MOBA_B200_OK;
}

}  // namespace

int launch_pack_index(const void* mask, int mask_bytes, int batch, int seq_len, int32_t* dest, int32_t* lengths,
                      int32_t* cu, int32_t* meta, cudaStream_t st) {
  { KernelTimer t__("mask_scan_kernel", st);
  if (mask_bytes == 1) mask_scan_kernel<uint8_t><<<batch, kScanThreads, 0, st>>>((const uint8_t*)mask, seq_len, dest, lengths);
  else if (mask_bytes == 4) mask_scan_kernel<int32_t><<<batch, kScanThreads, 0, st>>>((const int32_t*)mask, seq_len, dest, lengths);
  else if (mask_bytes == 8) mask_scan_kernel<long long><<<batch, kScanThreads, 0, st>>>((const long long*)mask, seq_len, dest, lengths);
  else { set_error("pack: mask elements of %d bytes are not supported (1, 4 or 8)", mask_bytes); return MOBA_B200_EUNSUPPORTED; }
  MOBA_LAUNCH_OK("mask_scan_kernel"); }
  KernelTimer t__("lengths_scan_kernel", st);
  lengths_scan_kernel<<<1, kScanThreads, 0, st>>>(lengths, batch, cu, meta);
  MOBA_LAUNCH_OK("lengths_scan_kernel");
  return MOBA_B200_OK;
}

int launch_seq_meta(const int32_t* cu, int n_seq, int32_t* meta, cudaStream_t st) {
  KernelTimer t__("seq_meta_kernel", st);
  seq_meta_kernel<<<1, kScanThreads, 0, st>>>(cu, n_seq, meta);
  MOBA_LAUNCH_OK("seq_meta_kernel");
  return MOBA_B200_OK;
}

int launch_pack_rows(const void* x, const int32_t* dest, const int32_t* cu, void* packed, int batch, int seq_len,
                     size_t row_bytes, cudaStream_t st) {
  const int rc = check_rows(batch, seq_len, row_bytes, "pack");
  if (rc) return rc;
  KernelTimer t__("pack_rows_kernel", st);
  const size_t n_rows = (size_t)batch * seq_len;
  const int vpr = (int)(row_bytes / 16);
  const unsigned blocks = (unsigned)((n_rows * vpr + 255) / 256);
  pack_rows_kernel<<<blocks, 256, 0, st>>>((const uint4*)x, dest, cu, (uint4*)packed, n_rows, seq_len, vpr);
  MOBA_LAUNCH_OK("pack_rows_kernel");
  return MOBA_B200_OK;
}

int launch_unpack_rows(const void* packed, const int32_t* cu, void* out, int batch, int seq_len, size_t row_bytes,
                       cudaStream_t st) {
  const int rc = check_rows(batch, seq_len, row_bytes, "unpack");
  if (rc) return rc;
  KernelTimer t__("unpack_rows_kernel", st);
  const size_t n_rows = (size_t)batch * seq_len;
  const int vpr = (int)(row_bytes / 16);
  const unsigned blocks = (unsigned)((n_rows * vpr + 255) / 256);
  unpack_rows_kernel<<<blocks, 256, 0, st>>>((const uint4*)packed, cu, (uint4*)out, n_rows, seq_len, vpr);
  MOBA_LAUNCH_OK("unpack_rows_kernel");
  return MOBA_B200_OK;
}

}  // namespace moba
