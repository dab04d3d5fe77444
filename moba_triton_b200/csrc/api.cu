// extern "C" surface of libmoba_b200.so: argument checks, kernel-family
// selection and the per-thread error text. Declarations and the reference
// functions each entry point stands in for are in include/moba_b200.h.
#include "common.cuh"
#include "sm100.cuh"

#include <stdarg.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <string>
#include <vector>

namespace moba {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

// ---- launch counter and optional per-kernel event timing --------------------
static std::atomic<long long> g_launches{0};
static std::atomic<int> g_profile{0};
struct TimedLaunch { const char* name; cudaEvent_t a, b; };
static std::mutex g_prof_mu;
static std::vector<TimedLaunch> g_timed;

KernelTimer::KernelTimer(const char* name, cudaStream_t st) : name_(name), st_(st), start_(nullptr), on_(false) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (g_profile.load(std::memory_order_relaxed)) {
    if (cudaEventCreate(&start_) == cudaSuccess) {
      cudaEventRecord(start_, st_);
      on_ = true;
    }
  }
}
KernelTimer::~KernelTimer() {
  if (!on_) return;
  cudaEvent_t stop;
  if (cudaEventCreate(&stop) != cudaSuccess) { cudaEventDestroy(start_); return; }
  cudaEventRecord(stop, st_);
  std::lock_guard<std::mutex> lk(g_prof_mu);
  g_timed.push_back(TimedLaunch{name_, start_, stop});
}

static bool is_pow2(int x) { return x > 0 && (x & (x - 1)) == 0; }

static int check_problem(const moba_b200_problem* p) {
  if (p == nullptr) { set_error("problem is NULL"); return MOBA_B200_EINVAL; }
  if (p->dtype < MOBA_B200_F32 || p->dtype > MOBA_B200_F16) {
    set_error("unknown dtype code %d", p->dtype); return MOBA_B200_EINVAL;
  }
  if (p->batch <= 0 || p->tokens <= 0 || p->n_seq <= 0 || p->max_seqlen <= 0) {
    set_error("batch/tokens/n_seq/max_seqlen must be positive"); return MOBA_B200_EINVAL;
  }
  if (p->packed ? p->batch != 1 : (p->n_seq != p->batch || p->max_seqlen != p->tokens)) {
    set_error("inconsistent packing fields (packed=%d batch=%d n_seq=%d tokens=%d max_seqlen=%d)",
              p->packed, p->batch, p->n_seq, p->tokens, p->max_seqlen);
    return MOBA_B200_EINVAL;
  }
  if (p->q_heads <= 0 || p->kv_heads <= 0 || p->q_heads % p->kv_heads) {
    set_error("query heads %d must be divisible by key/value heads %d", p->q_heads, p->kv_heads);
    return MOBA_B200_EINVAL;
  }
  if (!is_pow2(p->head_dim) || p->head_dim * (int)dtype_size(p->dtype) < 128) {
    set_error("head_dim %d must be a power of two with rows of at least 128 bytes", p->head_dim);
    return MOBA_B200_EINVAL;
  }
  if (p->block_size < 16) { set_error("block_size %d below the minimum of 16", p->block_size); return MOBA_B200_EINVAL; }
  if (p->top_k <= 0 || p->slots <= 0 || p->take < 0 || p->take + (p->always_current ? 1 : 0) > p->slots) {
    set_error("inconsistent top_k/slots/take (%d/%d/%d)", p->top_k, p->slots, p->take);
    return MOBA_B200_EINVAL;
  }
  if (p->slots > 128) { set_error("more than 128 selections per query are not supported"); return MOBA_B200_EUNSUPPORTED; }
  if (p->num_blocks != (p->max_seqlen + p->block_size - 1) / p->block_size) {
    set_error("num_blocks %d does not match max_seqlen %d / block_size %d", p->num_blocks, p->max_seqlen, p->block_size);
    return MOBA_B200_EINVAL;
  }
  if (p->chunk_tiles < 0) { set_error("chunk_tiles must not be negative"); return MOBA_B200_EINVAL; }
  if (p->gate_window < 0 || p->gate_sinks < 0 || (p->gate_window == 0 && p->gate_sinks != 0)) {
    set_error("gate_window / gate_sinks must not be negative, and sinks need a window"); return MOBA_B200_EINVAL;
  }
  if (p->win_begin < 0 || p->win_rows < 0 || (p->win_rows == 0 && p->win_begin != 0) ||
      (long long)p->win_begin + p->win_rows > p->tokens) {
    set_error("query window [%d, %d + %d) does not lie inside the %d rows", p->win_begin, p->win_begin, p->win_rows, p->tokens);
    return MOBA_B200_EINVAL;
  }
  if (p->win_rows > 0 && p->packed) { set_error("a query window needs a padded batch, not a packed one"); return MOBA_B200_EUNSUPPORTED; }
  if ((long long)(p->q_heads / p->kv_heads) * p->max_seqlen * p->slots > 0x7fffffffLL) {
    set_error("a (sequence, kv head) column list would exceed 2^31 entries"); return MOBA_B200_EUNSUPPORTED;
  }
  return MOBA_B200_OK;
}

static int need(const void* ptr, const char* name) {
  if (ptr == nullptr) { set_error("%s is NULL", name); return MOBA_B200_EINVAL; }
  return MOBA_B200_OK;
}

static int pick(const moba_b200_problem& p, bool fast_ok, const char* stage) {
  if (p.path == MOBA_B200_PATH_PORTABLE) return MOBA_B200_PATH_PORTABLE;
  if (p.path == MOBA_B200_PATH_TCGEN05) {
    if (!fast_ok) { set_error("%s: tcgen05 kernels do not cover this shape/dtype", stage); return MOBA_B200_EUNSUPPORTED; }
    return MOBA_B200_PATH_TCGEN05;
  }
  return fast_ok ? MOBA_B200_PATH_TCGEN05 : MOBA_B200_PATH_PORTABLE;
}

}  // namespace moba

using namespace moba;

#define MOBA_TRY(expr) do { int rc__ = (expr); if (rc__ != MOBA_B200_OK) return rc__; } while (0)

extern "C" {

int moba_b200_abi_version(void) { return MOBA_B200_ABI_VERSION; }

const char* moba_b200_last_error(void) { return g_error; }

long long moba_b200_launch_count(void) { return g_launches.load(); }

int moba_b200_profile_enable(int on) {
  const int old = g_profile.exchange(on ? 1 : 0);
  return old;
}

int moba_b200_profile_read(char* buf, size_t cap) {
  // Synchronises with every recorded launch, then writes "name launches total_ms\n" lines.
  std::lock_guard<std::mutex> lk(g_prof_mu);
  struct Row { const char* name; int n; double ms; };
  std::vector<Row> rows;
  for (auto& t : g_timed) {
    float ms = 0.f;
    if (cudaEventSynchronize(t.b) == cudaSuccess) cudaEventElapsedTime(&ms, t.a, t.b);
    cudaEventDestroy(t.a);
    cudaEventDestroy(t.b);
    bool found = false;
    for (auto& r : rows) if (strcmp(r.name, t.name) == 0) { r.n++; r.ms += ms; found = true; break; }
    if (!found) rows.push_back(Row{t.name, 1, ms});
  }
  g_timed.clear();
  std::string out;
  char line[160];
  for (auto& r : rows) { snprintf(line, sizeof(line), "%s %d %.6f\n", r.name, r.n, r.ms); out += line; }
  if (buf == nullptr || cap == 0) return (int)out.size();
  const size_t n = out.size() < cap - 1 ? out.size() : cap - 1;
  memcpy(buf, out.data(), n);
  buf[n] = 0;
  return (int)n;
}

int moba_b200_device_status(unsigned int* word, void* stream) {
  // Waits for the stream, then reads and clears the current device's error word.
  if (word == nullptr) { set_error("word is NULL"); return MOBA_B200_EINVAL; }
  unsigned* dev_word = device_error_word();
  if (dev_word == nullptr) { set_error("no device error word (no CUDA device?)"); return MOBA_B200_ECUDA; }
  cudaStream_t st = (cudaStream_t)stream;
  MOBA_CUDA_OK(cudaMemcpyAsync(word, dev_word, sizeof(unsigned), cudaMemcpyDeviceToHost, st));
  MOBA_CUDA_OK(cudaMemsetAsync(dev_word, 0, sizeof(unsigned), st));
  MOBA_CUDA_OK(cudaStreamSynchronize(st));
  if (*word) set_error("device error word 0x%x (1 = a bounded wait inside a kernel gave up)", *word);
  return MOBA_B200_OK;
}

int moba_b200_path_for(const moba_b200_problem* p, int stage) {
  MOBA_TRY(check_problem(p));
  switch (stage) {
    case MOBA_B200_STAGE_GATE: return pick(*p, gate_sm100_supported(*p), "gate");
    case MOBA_B200_STAGE_FWD: return pick(*p, fwd_sm100_supported(*p), "forward");
    case MOBA_B200_STAGE_BWD: return pick(*p, bwd_sm100_supported(*p), "backward");
  }
  set_error("unknown stage %d", stage);
  return MOBA_B200_EINVAL;
}

int moba_b200_launch_plan(const moba_b200_problem* p, moba_b200_plan* plan) {
  MOBA_TRY(check_problem(p));
  if (plan == nullptr) { set_error("plan is NULL"); return MOBA_B200_EINVAL; }
  memset(plan, 0, sizeof(*plan));
  plan->gate_path = pick(*p, gate_sm100_supported(*p), "gate");
  plan->fwd_path = pick(*p, fwd_sm100_supported(*p), "forward");
  plan->bwd_path = pick(*p, bwd_sm100_supported(*p), "backward");
  if (plan->gate_path < 0 || plan->fwd_path < 0 || plan->bwd_path < 0) return MOBA_B200_EUNSUPPORTED;
  const TensorCorePlan& t = tensor_core_plan(p->head_dim);
  if (plan->fwd_path == MOBA_B200_PATH_TCGEN05) { plan->fwd_tiles_in_flight = t.fwd_tiles_in_flight; plan->fwd_q_stages = t.fwd_q_stages; }
  if (plan->bwd_path == MOBA_B200_PATH_TCGEN05) { plan->bwd_kv_buffers = t.bwd_kv_buffers; plan->bwd_gather_stages = t.bwd_gather_stages; }
  if (plan->gate_path == MOBA_B200_PATH_TCGEN05) { plan->gate_slots = t.gate_slots; plan->gate_step = t.gate_step; }
  transpose_plan(*p, &plan->transpose_chunk_rows, &plan->transpose_chunks, &plan->scatter_warps);
  plan->chunk_tiles = sched_chunk_tiles(*p);
  const long long per_row = sched_items_per_row(*p);
  plan->work_items_per_row = per_row > 0x7fffffffLL ? -1 : (int)per_row;
  return MOBA_B200_OK;
}

size_t moba_b200_transpose_scratch_bytes(const moba_b200_problem* p) {
  if (check_problem(p) != MOBA_B200_OK) return 0;
  return transpose_scratch_bytes(*p);
}

int moba_b200_chunk_tiles(const moba_b200_problem* p) {
  MOBA_TRY(check_problem(p));
  return sched_chunk_tiles(*p);
}

int moba_b200_work_items_per_row(const moba_b200_problem* p) {
  MOBA_TRY(check_problem(p));
  const long long n = sched_items_per_row(*p);
  if (n > 0x7fffffffLL) { set_error("chunk_tiles %d cuts the problem into too many work items", sched_chunk_tiles(*p)); return MOBA_B200_EUNSUPPORTED; }
  return (int)n;
}

size_t moba_b200_dkv_scratch_bytes(const moba_b200_problem* p) {
  if (check_problem(p) != MOBA_B200_OK) return 0;
  return sched_dkv_scratch_bytes(*p);
}

int moba_b200_pool(const moba_b200_problem* p, const void* k, const int32_t* cu_seqlens,
                   void* kbar, void* stream) {
  MOBA_TRY(check_problem(p));
  MOBA_TRY(need(k, "k")); MOBA_TRY(need(kbar, "kbar"));
  if (p->packed) MOBA_TRY(need(cu_seqlens, "cu_seqlens"));
  return launch_pool(*p, k, cu_seqlens, kbar, (cudaStream_t)stream);
}

int moba_b200_gate(const moba_b200_problem* p, const void* q, const void* kbar,
                   const int32_t* cu_seqlens, int32_t* block_idx, void* stream) {
  MOBA_TRY(check_problem(p));
  MOBA_TRY(need(q, "q")); MOBA_TRY(need(kbar, "kbar")); MOBA_TRY(need(block_idx, "block_idx"));
  if (p->packed) MOBA_TRY(need(cu_seqlens, "cu_seqlens"));
  const int path = pick(*p, gate_sm100_supported(*p), "gate");
  if (path < 0) return path;
  if (path == MOBA_B200_PATH_TCGEN05)
    return launch_gate_sm100(*p, q, kbar, cu_seqlens, block_idx, (cudaStream_t)stream);
  return launch_gate_portable(*p, q, kbar, cu_seqlens, block_idx, (cudaStream_t)stream);
}

int moba_b200_transpose(const moba_b200_problem* p, const int32_t* block_idx,
                        const int32_t* cu_seqlens, int32_t* col_nnz, int32_t* col_offsets,
                        int32_t* order, int32_t* row_indices, int32_t* head_indices,
                        int32_t* slot_of_pair, int32_t* work_items, void* scratch, size_t scratch_bytes,
                        void* stream) {
  MOBA_TRY(check_problem(p));
  MOBA_TRY(need(block_idx, "block_idx")); MOBA_TRY(need(col_nnz, "col_nnz"));
  MOBA_TRY(need(col_offsets, "col_offsets")); MOBA_TRY(need(order, "order"));
  MOBA_TRY(need(row_indices, "row_indices")); MOBA_TRY(need(head_indices, "head_indices"));
  MOBA_TRY(need(slot_of_pair, "slot_of_pair")); MOBA_TRY(need(work_items, "work_items"));
  MOBA_TRY(need(scratch, "scratch"));
  if (p->packed) MOBA_TRY(need(cu_seqlens, "cu_seqlens"));
  return launch_transpose(*p, block_idx, cu_seqlens, col_nnz, col_offsets, order, row_indices,
                          head_indices, slot_of_pair, work_items, scratch, scratch_bytes, (cudaStream_t)stream);
}

int moba_b200_transpose_noalloc(const moba_b200_problem* p, const int32_t* block_idx,
                                const int32_t* cu_seqlens, int32_t* col_nnz, int32_t* col_offsets,
                                int32_t* order, int32_t* row_indices, int32_t* head_indices,
                                int32_t* slot_of_pair, int32_t* work_items, void* stream) {
  MOBA_TRY(check_problem(p));
  MOBA_TRY(need(block_idx, "block_idx")); MOBA_TRY(need(col_nnz, "col_nnz"));
  MOBA_TRY(need(col_offsets, "col_offsets")); MOBA_TRY(need(order, "order"));
  MOBA_TRY(need(row_indices, "row_indices")); MOBA_TRY(need(head_indices, "head_indices"));
  MOBA_TRY(need(slot_of_pair, "slot_of_pair")); MOBA_TRY(need(work_items, "work_items"));
  if (p->packed) MOBA_TRY(need(cu_seqlens, "cu_seqlens"));
  return launch_transpose_noalloc(*p, block_idx, cu_seqlens, col_nnz, col_offsets, order, row_indices,
                                  head_indices, slot_of_pair, work_items, (cudaStream_t)stream);
}

static int check_index(const moba_b200_problem* p, const moba_b200_index* ix) {
  MOBA_TRY(need(ix, "index"));
  MOBA_TRY(need(ix->col_nnz, "index.col_nnz")); MOBA_TRY(need(ix->col_offsets, "index.col_offsets"));
  MOBA_TRY(need(ix->order, "index.order")); MOBA_TRY(need(ix->row_indices, "index.row_indices"));
  MOBA_TRY(need(ix->head_indices, "index.head_indices")); MOBA_TRY(need(ix->slot_of_pair, "index.slot_of_pair"));
  if (ix->capacity <= 0) { set_error("index.capacity must be positive"); return MOBA_B200_EINVAL; }
  if (ix->work_items != nullptr &&
      (ix->items_per_row != sched_items_per_row(*p) || ix->chunk_tiles != sched_chunk_tiles(*p))) {
    set_error("index.work_items was cut for another problem (items_per_row %d, chunk_tiles %d; this call: %lld, %d)",
              ix->items_per_row, ix->chunk_tiles, sched_items_per_row(*p), sched_chunk_tiles(*p));
    return MOBA_B200_EINVAL;
  }
  return MOBA_B200_OK;
}

int moba_b200_fwd(const moba_b200_problem* p, const void* q, const void* k, const void* v,
                  const moba_b200_index* index, const int32_t* cu_seqlens, void* part_o,
                  float* part_lse, void* stream) {
  MOBA_TRY(check_problem(p));
  MOBA_TRY(check_index(p, index));
  MOBA_TRY(need(q, "q")); MOBA_TRY(need(k, "k")); MOBA_TRY(need(v, "v"));
  MOBA_TRY(need(part_o, "part_o")); MOBA_TRY(need(part_lse, "part_lse"));
  if (p->packed) MOBA_TRY(need(cu_seqlens, "cu_seqlens"));
  const int path = pick(*p, fwd_sm100_supported(*p), "forward");
  if (path < 0) return path;
  cudaStream_t st = (cudaStream_t)stream;
  MOBA_TRY(launch_fill_lse(*p, part_lse, st));
  if (path == MOBA_B200_PATH_TCGEN05)
    return launch_fwd_sm100(*p, q, k, v, *index, cu_seqlens, part_o, part_lse, st);
  return launch_fwd_portable(*p, q, k, v, *index, cu_seqlens, part_o, part_lse, st);
}

int moba_b200_merge(const moba_b200_problem* p, const void* part_o, const float* part_lse,
                    void* out, float* lse, void* stream) {
  MOBA_TRY(check_problem(p));
  MOBA_TRY(need(part_o, "part_o")); MOBA_TRY(need(part_lse, "part_lse")); MOBA_TRY(need(out, "out"));
  return launch_merge(*p, part_o, part_lse, out, lse, (cudaStream_t)stream);
}

int moba_b200_bwd(const moba_b200_problem* p, const void* q, const void* k, const void* v,
                  const void* out, const void* dout, const float* lse, const float* part_lse,
                  const moba_b200_index* index, const int32_t* cu_seqlens, float* delta,
                  void* dq_part, void* dkv_scratch, void* dq, void* dk, void* dv, void* stream) {
  MOBA_TRY(check_problem(p));
  MOBA_TRY(check_index(p, index));
  MOBA_TRY(need(q, "q")); MOBA_TRY(need(k, "k")); MOBA_TRY(need(v, "v"));
  MOBA_TRY(need(out, "out")); MOBA_TRY(need(dout, "dout")); MOBA_TRY(need(lse, "lse"));
  MOBA_TRY(need(part_lse, "part_lse")); MOBA_TRY(need(delta, "delta"));
  MOBA_TRY(need(dq_part, "dq_part")); MOBA_TRY(need(dq, "dq")); MOBA_TRY(need(dk, "dk")); MOBA_TRY(need(dv, "dv"));
  if (p->packed) MOBA_TRY(need(cu_seqlens, "cu_seqlens"));
  const int path = pick(*p, bwd_sm100_supported(*p), "backward");
  if (path < 0) return path;
  cudaStream_t st = (cudaStream_t)stream;
  MOBA_TRY(launch_delta(*p, out, dout, delta, st));
  if (path == MOBA_B200_PATH_TCGEN05)
    MOBA_TRY(launch_bwd_sm100(*p, q, k, v, dout, lse, delta, *index, cu_seqlens, dq_part,
                              static_cast<float*>(dkv_scratch), dk, dv, st));
  else
    MOBA_TRY(launch_bwd_portable(*p, q, k, v, dout, lse, delta, *index, cu_seqlens, dq_part, dk, dv, st));
  return launch_dq_reduce(*p, dq_part, part_lse, dq, st);
}

int moba_b200_pack_index(const void* mask, int mask_elem_bytes, int batch, int seq_len, int32_t* dest,
                         int32_t* lengths, int32_t* cu_seqlens, int32_t* meta, void* stream) {
  MOBA_TRY(need(mask, "mask")); MOBA_TRY(need(dest, "dest")); MOBA_TRY(need(lengths, "lengths"));
  MOBA_TRY(need(cu_seqlens, "cu_seqlens")); MOBA_TRY(need(meta, "meta"));
  if (batch <= 0 || seq_len <= 0) { set_error("pack: batch and seq_len must be positive"); return MOBA_B200_EINVAL; }
  return launch_pack_index(mask, mask_elem_bytes, batch, seq_len, dest, lengths, cu_seqlens, meta, (cudaStream_t)stream);
}

int moba_b200_pack_rows(const void* x, const int32_t* dest, const int32_t* cu_seqlens, void* packed, int batch,
                        int seq_len, size_t row_bytes, void* stream) {
  MOBA_TRY(need(x, "x")); MOBA_TRY(need(dest, "dest")); MOBA_TRY(need(cu_seqlens, "cu_seqlens"));
  MOBA_TRY(need(packed, "packed"));
  return launch_pack_rows(x, dest, cu_seqlens, packed, batch, seq_len, row_bytes, (cudaStream_t)stream);
}

int moba_b200_unpack_rows(const void* packed, const int32_t* cu_seqlens, void* out, int batch, int seq_len,
                          size_t row_bytes, void* stream) {
  MOBA_TRY(need(packed, "packed")); MOBA_TRY(need(cu_seqlens, "cu_seqlens")); MOBA_TRY(need(out, "out"));
  return launch_unpack_rows(packed, cu_seqlens, out, batch, seq_len, row_bytes, (cudaStream_t)stream);
}

int moba_b200_seq_meta(const int32_t* cu_seqlens, int n_seq, int32_t* meta, void* stream) {
  MOBA_TRY(need(cu_seqlens, "cu_seqlens")); MOBA_TRY(need(meta, "meta"));
  if (n_seq <= 0) { set_error("seq_meta: n_seq must be positive"); return MOBA_B200_EINVAL; }
  return launch_seq_meta(cu_seqlens, n_seq, meta, (cudaStream_t)stream);
}

}  // extern "C"
