// Shared declarations for the MoBA sm_100a engine: the problem record, dtype
// traits, error plumbing and the launch functions each translation unit exports
// to api.cu.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/moba_b200.h"

namespace moba {

constexpr float kLog2e = 1.4426950408889634f;

void set_error(const char* fmt, ...);

#define MOBA_CUDA_OK(expr)                                                        \
  do {                                                                            \
    cudaError_t e__ = (expr);                                                     \
    if (e__ != cudaSuccess) {                                                     \
      ::moba::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                        __FILE__, __LINE__);                                      \
      return MOBA_B200_ECUDA;                                                     \
    }                                                                             \
  } while (0)

// Counts every kernel launch of the library and, when profiling is switched on
// through moba_b200_profile_enable(), brackets it with CUDA events on its stream.
struct KernelTimer {
  KernelTimer(const char* name, cudaStream_t st);
  ~KernelTimer();
  const char* name_;
  cudaStream_t st_;
  cudaEvent_t start_;
  bool on_;
};

#define MOBA_LAUNCH_OK(what)                                                      \
  do {                                                                            \
    cudaError_t e__ = cudaGetLastError();                                         \
    if (e__ != cudaSuccess) {                                                     \
      ::moba::set_error("launch of %s failed: %s", what, cudaGetErrorString(e__));\
      return MOBA_B200_ECUDA;                                                     \
    }                                                                             \
  } while (0)

// ---- element types -------------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float to_f(float x) { return x; }
  static __device__ __forceinline__ float from_f(float x) { return x; }
  static __device__ __forceinline__ float round_f(float x) { return x; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }
  static __device__ __forceinline__ __nv_bfloat16 from_f(float x) { return __float2bfloat16_rn(x); }
  static __device__ __forceinline__ float round_f(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
  }
};
template <> struct Elem<__half> {
  static __device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
  static __device__ __forceinline__ __half from_f(float x) { return __float2half_rn(x); }
  static __device__ __forceinline__ float round_f(float x) {
    return __half2float(__float2half_rn(x));
  }
};

static inline size_t dtype_size(int dtype) { return dtype == MOBA_B200_F32 ? 4 : 2; }

// Sequence geometry shared by every kernel: where sequence `seq` starts on the
// token axis and how long it is. Padded batches have n_seq == batch and every
// sequence is `tokens` long; packed batches read cu_seqlens.
struct SeqSpan {
  int bos;   // first token (index on the token axis of its batch row)
  int len;   // tokens in the sequence
};
__device__ __forceinline__ SeqSpan seq_span(const int32_t* cu, int packed, int seq, int tokens) {
  SeqSpan s;
  if (packed) {
    s.bos = cu[seq];
    s.len = cu[seq + 1] - s.bos;
  } else {
    s.bos = 0;
    s.len = tokens;
  }
  return s;
}

// ---- gate candidates ----
// Block `blk` is a candidate of a query whose own block is `own`: strictly past, and, when a
// candidate window is set, among the first gate_sinks blocks or the last gate_window before
// the own block.
__host__ __device__ inline bool gate_candidate(const moba_b200_problem& p, int blk, int own) {
  return blk < own && (p.gate_window <= 0 || blk < p.gate_sinks || blk >= own - p.gate_window);
}

// ---- query window: rows of the partial buffers ----
// A call may cover only the query rows [win_begin, win_begin + win_rows) of every batch row
// (host-side chunking along the query axis: the partial buffers, slots times the size of the
// output, then exist for one window at a time). Row (b, head, row) of part_o / part_lse /
// dq_part:
__host__ __device__ inline int window_rows(const moba_b200_problem& p) { return p.win_rows > 0 ? p.win_rows : p.tokens; }
__device__ __forceinline__ size_t part_row(const moba_b200_problem& p, size_t b, int head, int row) {
  return (b * p.q_heads + head) * (size_t)window_rows(p) + (size_t)(row - p.win_begin);
}

// ---- launch table of the tensor-core kernels: one tile plan per head_dim ----
// The kernels take their compile-time constants from this table, and moba_b200_launch_plan
// reports it, so there is one place that says what runs. Shared memory decides the entries:
// at head_dim 64 four tiles, four Q stages and double-buffered K/V fit beside the output
// staging tiles; at 128 every operand is twice as large.
struct TensorCorePlan {
  int head_dim;
  int fwd_tiles_in_flight, fwd_q_stages;
  int bwd_kv_buffers, bwd_gather_stages;
  int gate_slots, gate_step;
};
constexpr TensorCorePlan kTensorCorePlans[2] = {
    {64, 4, 4, 2, 2, 16, 8},
    {128, 2, 2, 1, 1, 7, 4},
};
constexpr const TensorCorePlan& tensor_core_plan(int head_dim) { return kTensorCorePlans[head_dim == 64 ? 0 : 1]; }

void transpose_plan(const moba_b200_problem& p, int* chunk_rows, int* chunks, int* scatter_warps);

// ---- scheduling: columns are dispatched as work items of at most chunk_tiles tiles ----
// Sizes are fixed functions of the problem record, so that the caller can allocate the
// item table and the dK/dV partial slots without reading anything back from the device.
constexpr int kSchedSMs = 148;               // the part this engine is written for
constexpr int kSchedSplit = 4;               // a column above total / (kSchedSplit * SMs) tiles is cut
constexpr int kMinChunkTiles = 8;

static inline long long sched_pairs_bound(const moba_b200_problem& p) {
  return (long long)p.batch * (p.win_rows > 0 ? p.win_rows : p.tokens) * p.q_heads * p.slots;   // every (query head, slot) pair
}
static inline int sched_chunk_tiles(const moba_b200_problem& p) {
  if (p.chunk_tiles > 0) return p.chunk_tiles;
  const long long tiles = (sched_pairs_bound(p) + 127) / 128;
  const long long t = (tiles + kSchedSplit * kSchedSMs - 1) / (kSchedSplit * kSchedSMs);
  return t < kMinChunkTiles ? kMinChunkTiles : (int)(t > 0x3fffffff ? 0x3fffffff : t);
}
// Items beyond one per column: a column of n entries adds ceil(tiles / Tc) - 1 <= n / (128 Tc).
static inline long long sched_extra_items(const moba_b200_problem& p) {
  return sched_pairs_bound(p) / (128LL * sched_chunk_tiles(p)) + 1;
}
static inline long long sched_items_per_row(const moba_b200_problem& p) { return p.num_blocks + sched_extra_items(p); }
// dK/dV partial slots: a split column of c items uses c slots, and c <= 2 (c - 1).
static inline long long sched_part_slots(const moba_b200_problem& p) { return 2 * sched_extra_items(p) + 1; }
static inline size_t sched_dkv_scratch_bytes(const moba_b200_problem& p) {
  return (size_t)sched_part_slots(p) * 2 * 128 * p.head_dim * sizeof(float);
}

// One work item as the kernels see it.
struct WorkItem {
  int blk;        // block (column) of the (sequence, kv head) row
  int first;      // first entry of the column's pair list this item covers
  int n;          // entries it covers (0: an empty column)
  int slot;       // dK/dV partial slot, -1: the item is the whole column
};
// Item `j` of row `kv_row`; false for padding. `col_nnz_row` is the row's col_nnz.
__device__ __forceinline__ bool load_work_item(WorkItem& w, const moba_b200_index& ix, const int32_t* col_nnz_row,
                                               int kv_row, int j) {
  const int4 it = __ldg(reinterpret_cast<const int4*>(ix.work_items) + (size_t)kv_row * ix.items_per_row + j);
  if (it.w == -2) return false;
  w.blk = it.x;
  w.first = it.y * 128;
  const int nnz = col_nnz_row[it.x];
  w.n = max(0, min(it.z * 128, nnz - w.first));
  w.slot = it.w;
  return true;
}

// ---- stage launchers (defined one per .cu file) -----------------------------
int launch_pool(const moba_b200_problem& p, const void* k, const int32_t* cu, void* kbar,
                cudaStream_t st);
int launch_gate_portable(const moba_b200_problem& p, const void* q, const void* kbar,
                         const int32_t* cu, int32_t* block_idx, cudaStream_t st);
int launch_gate_sm100(const moba_b200_problem& p, const void* q, const void* kbar,
                      const int32_t* cu, int32_t* block_idx, cudaStream_t st);
bool gate_sm100_supported(const moba_b200_problem& p);

size_t transpose_scratch_bytes(const moba_b200_problem& p);
int launch_transpose(const moba_b200_problem& p, const int32_t* block_idx, const int32_t* cu,
                     int32_t* col_nnz, int32_t* col_offsets, int32_t* order, int32_t* rows,
                     int32_t* heads, int32_t* slots, int32_t* work_items, void* scratch, size_t scratch_bytes,
                     cudaStream_t st);

int launch_transpose_noalloc(const moba_b200_problem& p, const int32_t* block_idx, const int32_t* cu,
                             int32_t* col_nnz, int32_t* col_offsets, int32_t* order, int32_t* rows,
                             int32_t* heads, int32_t* slots, int32_t* work_items, cudaStream_t st);

int launch_fill_lse(const moba_b200_problem& p, float* part_lse, cudaStream_t st);
int launch_fwd_portable(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                        const moba_b200_index& ix, const int32_t* cu, void* part_o,
                        float* part_lse, cudaStream_t st);
int launch_fwd_sm100(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                     const moba_b200_index& ix, const int32_t* cu, void* part_o,
                     float* part_lse, cudaStream_t st);
bool fwd_sm100_supported(const moba_b200_problem& p);
int launch_merge(const moba_b200_problem& p, const void* part_o, const float* part_lse,
                 void* out, float* lse, cudaStream_t st);

int launch_delta(const moba_b200_problem& p, const void* out, const void* dout, float* delta,
                 cudaStream_t st);
int launch_bwd_portable(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                        const void* dout, const float* lse, const float* delta,
                        const moba_b200_index& ix, const int32_t* cu, void* dq_part, void* dk,
                        void* dv, cudaStream_t st);
int launch_bwd_sm100(const moba_b200_problem& p, const void* q, const void* k, const void* v,
                     const void* dout, const float* lse, const float* delta,
                     const moba_b200_index& ix, const int32_t* cu, void* dq_part, float* dkv_scratch,
                     void* dk, void* dv, cudaStream_t st);
bool bwd_sm100_supported(const moba_b200_problem& p);
int launch_dq_reduce(const moba_b200_problem& p, const void* dq_part, const float* part_lse,
                     void* dq, cudaStream_t st);

int launch_pack_index(const void* mask, int mask_bytes, int batch, int seq_len, int32_t* dest, int32_t* lengths,
                      int32_t* cu, int32_t* meta, cudaStream_t st);
int launch_seq_meta(const int32_t* cu, int n_seq, int32_t* meta, cudaStream_t st);
int launch_pack_rows(const void* x, const int32_t* dest, const int32_t* cu, void* packed, int batch, int seq_len,
                     size_t row_bytes, cudaStream_t st);
int launch_unpack_rows(const void* packed, const int32_t* cu, void* out, int batch, int seq_len, size_t row_bytes,
                       cudaStream_t st);

}  // namespace moba
