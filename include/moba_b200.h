/*
 * moba_b200.h -- C ABI of the B200 (sm_100a) MoBA attention engine.
 *
 * Every entry point takes plain device pointers, a problem description and a
 * CUDA stream (passed as void*, a cudaStream_t). The compute entry points
 * neither allocate device memory, synchronise with the host nor throw: the
 * caller owns every buffer, work is enqueued on the given stream on the calling
 * thread's current device, and the return value is 0 on success or a negative
 * MOBA_B200_E* code (text via moba_b200_last_error()). Two service calls are
 * the exception and say so: moba_b200_device_status waits for the stream, and
 * while moba_b200_profile_enable(1) is in force every launch creates a pair of
 * CUDA events (a measurement aid, off by default).
 *
 * Each declaration names the reference function it stands in for, by the path
 * inside the ZuricZ/moba-triton checkout.
 *
 * Layouts (all contiguous):
 *   q, out, dout, dq      [B, S, Hq,  D]   (packed: [1, T, Hq, D])
 *   k, v, dk, dv          [B, S, Hkv, D]
 *   kbar                  [n_seq, Hkv, num_blocks, D]          dtype of k
 *   block_idx             [B, Hq, S, slots] int32, ascending ids, -1 padded,
 *                         ids local to the sequence
 *   col_nnz, order        [n_seq, Hkv, num_blocks]   int32
 *   col_offsets           [n_seq, Hkv, num_blocks+1] int32
 *   row/head/slot arrays  [n_seq, Hkv, capacity]     int32,
 *                         capacity = (Hq/Hkv) * max_seqlen * slots (win_rows in place
 *                         of max_seqlen when the problem names a query window)
 *   work_items            [n_seq, Hkv, items_per_row, 4]  int32
 *   part_o                [B, Hq, S, slots, D]  (dtype of q, or float32); S -> win_rows
 *                         when the problem names a query window
 *   part_lse, dq marker   [B, Hq, S, slots]     float32, log2 units, -inf = unwritten
 *   lse, delta            [B, Hq, S]            float32 (lse in log2 units)
 *   dq_part               [B, Hq, S, slots, D]  dtype of q
 */
#ifndef MOBA_B200_H_
#define MOBA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOBA_B200_ABI_VERSION 2

enum { MOBA_B200_F32 = 0, MOBA_B200_BF16 = 1, MOBA_B200_F16 = 2 };

enum {
  MOBA_B200_OK = 0,
  MOBA_B200_EINVAL = -1,      /* bad argument (shape, dtype, null pointer) */
  MOBA_B200_EUNSUPPORTED = -2,/* valid request this build has no kernel for */
  MOBA_B200_ECUDA = -3,       /* a CUDA call failed; see last_error */
  MOBA_B200_ESCRATCH = -4     /* scratch buffer too small */
};

/* Kernel family selection. AUTO picks TCGEN05 whenever the shape allows. */
enum { MOBA_B200_PATH_AUTO = 0, MOBA_B200_PATH_PORTABLE = 1, MOBA_B200_PATH_TCGEN05 = 2 };

/* Stages, for moba_b200_path_for(). */
enum { MOBA_B200_STAGE_GATE = 0, MOBA_B200_STAGE_FWD = 1, MOBA_B200_STAGE_BWD = 2 };

typedef struct moba_b200_problem {
  int32_t dtype;          /* MOBA_B200_F32 / BF16 / F16: dtype of q, k, v */
  int32_t batch;          /* B of q/k/v; 1 when packed */
  int32_t tokens;         /* S (padded) or T (packed total) */
  int32_t n_seq;          /* B, or the number of packed sequences */
  int32_t max_seqlen;     /* S, or the longest packed sequence */
  int32_t q_heads;
  int32_t kv_heads;       /* divides q_heads */
  int32_t head_dim;       /* power of two, row >= 128 bytes */
  int32_t block_size;     /* >= 16 */
  int32_t top_k;
  int32_t slots;          /* selections a query can hold: take + always_current */
  int32_t take;           /* past blocks ranked in per query */
  int32_t always_current; /* 1: the query's own block is always attended */
  int32_t num_blocks;     /* cdiv(max_seqlen, block_size) */
  int32_t causal;         /* 1: mask future keys inside the own block */
  int32_t packed;         /* 1: cu_seqlens describes the token axis */
  int32_t path;           /* MOBA_B200_PATH_* */
  int32_t part_f32;       /* 1: part_o is float32 instead of the dtype of q */
  int32_t chunk_tiles;    /* scheduling: a column is dispatched in work items of at most this many
                             128-query tiles; 0 = the library's policy (moba_b200_chunk_tiles) */
  int32_t gate_window;    /* gate candidates (an extension, 0 = off = the reference's semantics): only the */
  int32_t gate_sinks;     /* gate_window blocks before the query's own block, and the first gate_sinks
                             blocks of the sequence, are scored and ranked; the gate then costs
                             O(S * (window + sinks)) instead of O(S * num_blocks) */
  int32_t win_begin;      /* query window: the transpose lists, and the partial buffers hold, only the */
  int32_t win_rows;       /* query rows [win_begin, win_begin + win_rows) of every batch row; 0 = all rows.
                             part_o, part_lse and dq_part are then [B, Hq, win_rows, slots(, D)]. Padded
                             batches only. */
} moba_b200_problem;

typedef struct moba_b200_index {
  const int32_t* col_nnz;
  const int32_t* col_offsets;
  const int32_t* order;
  const int32_t* row_indices;
  const int32_t* head_indices;
  const int32_t* slot_of_pair;
  int64_t capacity;       /* entries per (sequence, kv head) in the three pair arrays */
  const int32_t* work_items; /* [n_seq, Hkv, items_per_row, 4]: {block, first tile, tiles, dK/dV partial
                                slot or -1 (whole column) or -2 (padding)}, in dispatch order; written
                                by moba_b200_transpose. NULL: the tensor-core kernels refuse the index */
  int32_t items_per_row;  /* moba_b200_work_items_per_row() of the problem the index was built for */
  int32_t chunk_tiles;    /* the chunk size the items were cut with */
} moba_b200_index;

/* ABI version of the loaded library (compare with MOBA_B200_ABI_VERSION). */
int moba_b200_abi_version(void);

/* Text of the calling thread's most recent failure; never NULL. */
const char* moba_b200_last_error(void);

/* Kernels launched by this library since it was loaded (all threads). */
long long moba_b200_launch_count(void);

/* Measurement aid: when enabled, every kernel launch of the library is
 * bracketed by CUDA events on its stream (returns the previous setting).
 * moba_b200_profile_read waits for the recorded launches, writes one
 * "kernel_name launches total_ms" line per kernel into buf (NUL terminated,
 * at most cap bytes), clears the record and returns the text length.
 * No counterpart in the reference (it times stages from Python,
 * bench/stages.py). */
int moba_b200_profile_enable(int on);
int moba_b200_profile_read(char* buf, size_t cap);

/* Waits for `stream`, then copies the device's error word to *word and clears
 * it. 0 means no kernel reported a problem; bit 0 = a bounded wait inside a
 * tensor-core kernel gave up (its results are then invalid). Kernels never
 * trap or spin forever; this is how such a failure is reported. No
 * counterpart in the reference. */
int moba_b200_device_status(unsigned int* word, void* stream);

/* Which kernel family (MOBA_B200_PATH_PORTABLE or _TCGEN05) a stage would run
 * for this problem, or a negative error code. */
int moba_b200_path_for(const moba_b200_problem* p, int stage);

/* The launch table: everything the library decides per problem, looked up in
 * constant time from the problem record (no measurement, no device query).
 * The tensor-core kernels have one tile plan per head_dim; the transpose and
 * the scheduler size themselves by sequence length and pair count. Choices
 * never depend on whether the batch is packed, so a packed batch and its
 * sequences run alone go through the same kernels and give the same bits.
 * Stands in for the reference's table lookup (src/moba/kernels/tuning.py:335-409,
 * tuned_configs.py:87-285), whose autotuner has no counterpart here. */
typedef struct moba_b200_plan {
  int32_t gate_path, fwd_path, bwd_path;   /* MOBA_B200_PATH_* of each stage */
  int32_t fwd_tiles_in_flight;             /* forward: 128-query tiles (TMEM buffers, softmax warpgroups) per SM */
  int32_t fwd_q_stages;                    /* forward: shared-memory stages of gathered Q */
  int32_t bwd_kv_buffers;                  /* backward: K/V buffers per SM */
  int32_t bwd_gather_stages;               /* backward: stages of gathered Q and dO */
  int32_t gate_slots, gate_step;           /* gate: per-thread buffer slots; scores tested between room checks */
  int32_t transpose_chunk_rows;            /* transpose: rows per histogram chunk */
  int32_t transpose_chunks;                /*            chunks per sequence */
  int32_t scatter_warps;                   /*            runs walked side by side per chunk */
  int32_t chunk_tiles;                     /* scheduler: tiles per work item */
  int32_t work_items_per_row;              /*            table entries per (sequence, kv head) */
} moba_b200_plan;
int moba_b200_launch_plan(const moba_b200_problem* p, moba_b200_plan* plan);

/* Bytes of scratch moba_b200_transpose needs for this problem. */
size_t moba_b200_transpose_scratch_bytes(const moba_b200_problem* p);

/* Scheduling. The persistent tensor-core kernels do not dispatch whole columns: the
 * transpose cuts every (sequence, kv head, block) column, in longest-first order, into
 * work items of at most chunk_tiles tiles of 128 queries, so that a few crowded
 * columns (the early blocks of a causal sequence, or a skewed selection) cannot hold
 * the last SMs busy while the others idle. The forward treats each item as a column
 * of its own; in the backward the items of a split column write float32 dK/dV
 * partials into `dkv_scratch`, summed in item order by a reduction pass.
 *   moba_b200_chunk_tiles         the chunk size used for this problem (the policy:
 *                                 total tiles / (4 x 148 SMs), at least 8; or p->chunk_tiles)
 *   moba_b200_work_items_per_row  entries per (sequence, kv head) of index.work_items
 *   moba_b200_dkv_scratch_bytes   bytes of dkv_scratch moba_b200_bwd needs
 * The reference orders blocks longest first and leaves the rest to the hardware
 * scheduler (src/moba/kernels/routing.py:188-247); it has no counterpart of the split. */
int moba_b200_chunk_tiles(const moba_b200_problem* p);
int moba_b200_work_items_per_row(const moba_b200_problem* p);
size_t moba_b200_dkv_scratch_bytes(const moba_b200_problem* p);

/* Mean key of every block.
 * Replaces pool_blocks / pool_blocks_kernel (src/moba/kernels/pooling.py:25-163). */
int moba_b200_pool(const moba_b200_problem* p, const void* k, const int32_t* cu_seqlens,
                   void* kbar, void* stream);

/* Scores every query against the block means of its past blocks, keeps the
 * best `take` (ties to the lower id), adds the own block, emits ascending ids.
 * Replaces gate_select / gate_kernel (src/moba/kernels/gating.py:92-448). */
int moba_b200_gate(const moba_b200_problem* p, const void* q, const void* kbar,
                   const int32_t* cu_seqlens, int32_t* block_idx, void* stream);

/* CSR -> CSC regrouping of the selections by (sequence, kv head, block):
 * histogram, prefix scan (+ longest-first order), stable scatter.
 * Replaces build_csc_from_indices and its three kernels
 * (src/moba/kernels/routing.py:138-427). */
int moba_b200_transpose(const moba_b200_problem* p, const int32_t* block_idx,
                        const int32_t* cu_seqlens, int32_t* col_nnz, int32_t* col_offsets,
                        int32_t* order, int32_t* row_indices, int32_t* head_indices,
                        int32_t* slot_of_pair, int32_t* work_items, void* scratch,
                        size_t scratch_bytes, void* stream);

/* moba_b200_transpose for callers that cannot allocate device memory -- a
 * server that fixes its whole memory plan at start-up and forbids cudaMalloc
 * later, or a plugin that receives only its input and output buffers. The
 * scratch is an 8 MiB array built into the library (each GPU that loads the
 * library holds it until the process exits); problems whose
 * moba_b200_transpose_scratch_bytes() exceeds 8 MiB are refused with
 * MOBA_B200_EUNSUPPORTED. Inputs and outputs are the caller's, exactly as for
 * moba_b200_transpose, and the results are identical. The call allocates and
 * frees nothing. The first call on a device looks up the array's device
 * address (with that device current); make that first call before starting
 * any stream capture. All calls share the one array and nothing in it needs
 * clearing between calls, but two calls that overlap on the same GPU (two
 * streams, two threads) race on it: serialise them.
 * This entry point has no counterpart in the reference. */
int moba_b200_transpose_noalloc(const moba_b200_problem* p, const int32_t* block_idx,
                                const int32_t* cu_seqlens, int32_t* col_nnz, int32_t* col_offsets,
                                int32_t* order, int32_t* row_indices, int32_t* head_indices,
                                int32_t* slot_of_pair, int32_t* work_items, void* stream);

/* KV-block-major attention: one K/V block resident per CTA, the queries that
 * selected it gathered through the index; writes normalised partial outputs and
 * their log2-sum-exp per (query, slot). Resets part_lse to -inf first.
 * Replaces attend_partials / moba_fwd_kernel (src/moba/kernels/moba_fwd.py:229-425,566-665). */
int moba_b200_fwd(const moba_b200_problem* p, const void* q, const void* k, const void* v,
                  const moba_b200_index* index, const int32_t* cu_seqlens,
                  void* part_o, float* part_lse, void* stream);

/* Merges a query's partials: LSE = log2 sum 2^lse_i, O = sum 2^(lse_i-LSE) O_i.
 * lse may be NULL. Unwritten slots (part_lse == -inf) are skipped by selection,
 * never by multiplication. Replaces combine_partials / moba_combine_kernel
 * (src/moba/kernels/moba_fwd.py:428-521,668-725). */
int moba_b200_merge(const moba_b200_problem* p, const void* part_o, const float* part_lse,
                    void* out, float* lse, void* stream);

/* Backward: delta = rowsum(out*dout); per KV block dK/dV owned by one CTA and
 * stored once (zeros for unselected blocks) -- or, for a column cut into several
 * work items, accumulated per item in `dkv_scratch` (moba_b200_dkv_scratch_bytes)
 * and summed in item order; dQ written as per-(query, slot) partials and summed in
 * slot order. `part_lse` is the forward's buffer, used as the written-slot marker.
 * Replaces compute_delta, moba_backward / moba_bwd_kernel and reduce_dq
 * (src/moba/kernels/moba_bwd.py:134-160,215-579). */
int moba_b200_bwd(const moba_b200_problem* p, const void* q, const void* k, const void* v,
                  const void* out, const void* dout, const float* lse, const float* part_lse,
                  const moba_b200_index* index, const int32_t* cu_seqlens,
                  float* delta, void* dq_part, void* dkv_scratch, void* dq, void* dk, void* dv,
                  void* stream);

/* Packed (variable-length) batches, the step either side of the op. A "row" is
 * one token's H*D elements (row_bytes, a multiple of 16), contiguous in the
 * token-major layout.
 *
 * moba_b200_pack_index scans a [batch, seq_len] mask (elements of 1, 4 or 8
 * bytes, nonzero = keep): dest[b, s] = position of token s among the kept tokens
 * of row b, or -1; lengths[b]; cu_seqlens[batch + 1]; meta = {total kept tokens,
 * longest row}, which the host reads once to size the packed buffer.
 * moba_b200_pack_rows then copies the kept rows of x [batch, seq_len, row] to
 * packed [total, row] in (b, s) order.
 * Replace pack (src/moba/varlen.py:114-156). */
int moba_b200_pack_index(const void* mask, int mask_elem_bytes, int batch, int seq_len,
                         int32_t* dest, int32_t* lengths, int32_t* cu_seqlens, int32_t* meta,
                         void* stream);
int moba_b200_pack_rows(const void* x, const int32_t* dest, const int32_t* cu_seqlens,
                        void* packed, int batch, int seq_len, size_t row_bytes, void* stream);

/* Inverse: out [batch, seq_len, row] takes row cu_seqlens[b] + s of packed where
 * s is inside sequence b and zeros elsewhere.
 * Replaces unpack (src/moba/varlen.py:159-205). */
int moba_b200_unpack_rows(const void* packed, const int32_t* cu_seqlens, void* out, int batch,
                          int seq_len, size_t row_bytes, void* stream);

/* meta = {cu_seqlens[n_seq], longest sequence} of an existing cu_seqlens; what
 * from_nested (src/moba/varlen.py:208-236) reads back to report max_seqlen. */
int moba_b200_seq_meta(const int32_t* cu_seqlens, int n_seq, int32_t* meta, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MOBA_B200_H_ */
