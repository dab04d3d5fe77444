// sm_100a building blocks used by the tensor-core kernels: mbarriers with
// bounded waits, TMA tile loads, tcgen05 (TMEM allocation, MMA, commit, loads),
// shared-memory matrix descriptors for the 128-byte swizzle, and host-side
// tensor-map encoding.
//
// Every wait is bounded: a wait that runs out of tries sets `abort` in shared
// memory and a device-wide error word, after which every later wait of the CTA
// returns at once, the CTA runs its (bounded) loops to the end, frees its TMEM
// and exits. Nothing in this file can spin forever.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace moba {
namespace sm100 {

// ---------------------------------------------------------------------------
// device error word (per device; read by moba_b200_device_status)
// ---------------------------------------------------------------------------
enum : unsigned { kErrWaitTimeout = 1u, kErrBadIndex = 2u };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One arrival for a whole warp: every lane has done its own writes and fences; the warp
// barrier orders them before lane 0's (releasing) arrival. 32 arrivals on one barrier word
// would be 32 serialised shared-memory atomics.
__device__ __forceinline__ void mbar_arrive_warp(uint64_t* bar) {
  __syncwarp();
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

struct WaitCtx {
  volatile int* abort;        // shared-memory flag of the CTA
  unsigned* error_word;       // global
#ifdef MOBA_WAIT_STATS
  unsigned long long* stats;  // shared-memory cycle counters, one per wait site (debug builds)
#endif
};

// Debug builds (MOBA_WAIT_STATS) also time the phases of a role: PHASE_CLOCK(t) starts a
// clock, PHASE_ADD(ctx, site, t) adds the clocks since to counter `site` (lane 0 of each warp)
// and restarts it. Both vanish from normal builds.
#ifdef MOBA_WAIT_STATS
#define PHASE_CLOCK(t) long long t = clock64()
#define PHASE_ADD(ctx, site, t)                                                              \
  do {                                                                                        \
    const long long now__ = clock64();                                                        \
    if ((ctx).stats != nullptr && (threadIdx.x & 31) == 0) atomicAdd(&(ctx).stats[site], (unsigned long long)(now__ - t)); \
    t = now__;                                                                                \
  } while (0)
#else
#define PHASE_CLOCK(t) do {} while (0)
#define PHASE_ADD(ctx, site, t) do {} while (0)
#endif

// Trace builds (MOBA_TRACE) record the clock of lane 0 of every warp of CTA 0 at numbered
// points of eight consecutive tiles, behind the wait counters of the device error buffer.
#ifdef MOBA_TRACE
constexpr int kTraceT0 = 20;
constexpr int kTraceWordOffset = 64 + 2 * 32 * 160;
#define TRACE(err, tile, ev)                                                                   \
  do {                                                                                         \
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (int)(tile) >= kTraceT0 && (int)(tile) < kTraceT0 + 8) \
      reinterpret_cast<unsigned long long*>((err) + kTraceWordOffset)[(((int)(tile) - kTraceT0) * 32 + (threadIdx.x >> 5)) * 16 + (ev)] = clock64(); \
  } while (0)
#else
#define TRACE(err, tile, ev) do {} while (0)
#endif

constexpr long long kWaitCycles = 1ll << 31;   // about a second of SM clock
constexpr uint32_t kSuspendNs = 4000;          // a try may sleep this long; completion wakes it at once

// try_wait with a suspend-time hint: a waiting warp sleeps in hardware instead of taking
// issue slots from the warps that do the work.
__device__ __forceinline__ bool mbar_try_wait_sleep(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendNs)
      : "memory");
  return ok != 0;
}

// Waits for the phase with the given parity to complete. Returns false (and
// latches the abort flag) if it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx, int site = 0) {
  if (mbar_try_wait(bar, parity)) return true;        // already complete: no flag read, no clock read, no suspend hint
  if (*ctx.abort) return false;
  const long long t0__ = clock64();
  for (;;) {
    if (mbar_try_wait_sleep(bar, parity)) {
#ifdef MOBA_WAIT_STATS
      if (ctx.stats != nullptr && (threadIdx.x & 31) == 0) atomicAdd(&ctx.stats[site], (unsigned long long)(clock64() - t0__));
#endif
      return true;
    }
    if (*ctx.abort) return false;
    if (clock64() - t0__ > kWaitCycles) break;
  }
  *ctx.abort = 1;
  atomicCAS(ctx.error_word, 0u, ((unsigned)site << 8));   // the first wait that gave up names itself
  atomicOr(ctx.error_word, kErrWaitTimeout);
  return false;
}

// Bounded wait that ignores the abort flag: used on the way out of a kernel, for
// asynchronous work that must have landed before the CTA may exit.
__device__ __forceinline__ void mbar_wait_quiet(uint64_t* bar, uint32_t parity) {
  const long long t0__ = clock64();
  while (!mbar_try_wait_sleep(bar, parity))
    if (clock64() - t0__ > kWaitCycles) return;
}

__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// generic-proxy writes (st.shared, cp.async) -> visible to the async proxy (TMA, tcgen05.mma)
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------
// cp.async (16-byte, zero-fill when src_bytes == 0)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// L2 eviction policies. Rows that are gathered again and again (Q, dO, K, V) are loaded
// "evict last"; the partial buffers, which are written once and read once by a later
// kernel, are stored "evict first", so that their stream does not push the reused rows
// out of the L2.
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void cp_async16_hint(uint32_t dst_smem, const void* src, uint32_t src_bytes, uint64_t pol) {
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;" ::"r"(dst_smem), "l"(src), "r"(src_bytes), "l"(pol)
               : "memory");
}
__device__ __forceinline__ void st_global_stream16(void* dst, const uint4& w) {
  asm volatile("st.global.cs.v4.b32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "r"(w.x), "r"(w.y), "r"(w.z), "r"(w.w) : "memory");
}
__device__ __forceinline__ void st_global_stream_f32(float* dst, float v) {
  asm volatile("st.global.cs.f32 [%0], %1;" ::"l"(dst), "f"(v) : "memory");
}

// Bulk copy shared -> global (both 16-byte aligned, size a multiple of 16) by the copy engine;
// the issuing thread groups its copies and waits until they have read their source.
__device__ __forceinline__ void bulk_store(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

// Asks the L2 to fetch [p, p + bytes) (both multiples of 16); nothing waits for it.
__device__ __forceinline__ void l2_prefetch_bulk(const void* p, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// Asks the L2 for the 128-byte line that holds `p` (an ordinary load-store-unit request: cheap
// to issue, unlike the bulk form above, which goes through the copy engine one request at a time).
__device__ __forceinline__ void l2_prefetch_line(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p) : "memory");
}
// Prefetches elements [lo, lo + n) of an int32 array of `total` elements.
__device__ __forceinline__ void l2_prefetch_i32(const int32_t* base, size_t lo, int n, size_t total) {
  const size_t b0 = (lo * 4) & ~size_t(15);
  size_t b1 = ((lo + (size_t)n) * 4 + 15) & ~size_t(15);
  const size_t end = (total * 4) & ~size_t(15);
  if (b1 > end) b1 = end;
  if (b1 > b0) l2_prefetch_bulk(reinterpret_cast<const unsigned char*>(base) + b0, (uint32_t)(b1 - b0));
}

// A global load the compiler may not move: used to fetch index entries a tile or two before
// they are needed (a plain load may be sunk to its first use, which defeats the prefetch).
__device__ __forceinline__ int ld_nc_pinned(const int32_t* p) {
  int v;
  asm volatile("ld.global.nc.b32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

__device__ __forceinline__ float ld_nc_pinned_f(const float* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

// ---------------------------------------------------------------------------
// TMA tile loads (no multicast anywhere in this engine)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_3d_hint(void* dst_smem, const CUtensorMap* m, uint64_t* bar, int c0,
                                                 int c1, int c2, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4, %5}], [%2], %6;"
      ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst_smem, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// Four rows of a 2-D tensor (map with a box of one row) -> four consecutive 128-byte rows
// of a swizzled tile. Rows outside the tensor read as zeros.
__device__ __forceinline__ void tma_gather4(void* dst_smem, const CUtensorMap* m, uint64_t* bar, int col,
                                            int r0, int r1, int r2, int r3) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(dst_smem)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(col), "r"(r0), "r"(r1),
        "r"(r2), "r"(r3)
      : "memory");
}

// ---------------------------------------------------------------------------
// tcgen05: TMEM allocation, MMA, commit, loads, fences
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {   // one full warp
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {     // same warp
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// True in exactly one lane of a converged warp. The MMA-issuing warp runs its loop with all
// 32 lanes (so addresses and descriptors stay warp-uniform) and lets this lane issue.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}

// D[tmem] (+)= A[smem] * B[smem], 16-bit inputs, float32 accumulate
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A is a 128-lane block of TMEM, row m in lane m, 16-bit
// elements 2 j and 2 j + 1 of the row in the low and high half of column j
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// the mbarrier arrives once every MMA issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 consecutive float32 columns: thread i of the warp gets lane (base_lane + i)
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
// 32 lanes x 16 consecutive float32 columns
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 32 lanes x 16 consecutive 32-bit columns, registers -> TMEM: thread i of the warp writes lane (base_lane + i)
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// the same for 8 columns
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Same wait, but also names registers of the load it guards as in/out operands, so the compiler
// cannot schedule their first use above the wait.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[7]), "+r"(r[8]), "+r"(r[15]), "+r"(r[16]), "+r"(r[23]), "+r"(r[24]), "+r"(r[31])
               :: "memory");
}

// ---------------------------------------------------------------------------
// descriptors
// ---------------------------------------------------------------------------
// Instruction descriptor for kind::f16: float32 accumulator, A/B of type
// `ab_format` (0 = f16, 1 = bf16), M x N tile, operand majors (0 = K-major,
// 1 = MN-major).
__host__ __device__ constexpr uint32_t make_idesc(uint32_t ab_format, uint32_t m, uint32_t n, uint32_t a_mn_major,
                                                  uint32_t b_mn_major) {
  return (1u << 4) | (ab_format << 7) | (ab_format << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle. `lbo` / `sbo` in bytes.
//   K-major operand  [rows][64 elems] tiles: sbo = 1024 (8 rows), lbo unused
//   MN-major operand [k rows][64 elems] tiles: sbo = 1024 (8 k-rows),
//                    lbo = distance between 64-element chunks along M/N
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)((lbo >> 4) & 0x3FFFu) << 16;
  d |= (uint64_t)((sbo >> 4) & 0x3FFFu) << 32;
  d |= (uint64_t)1 << 46;        // descriptor version of sm_100
  d |= (uint64_t)2 << 61;        // SWIZZLE_128B
  return d;
}

// Byte offset of element (row, 16-byte chunk `c16`) inside a [rows][128 B] tile
// stored with the 128-byte swizzle (tile base 1024-byte aligned).
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t c16) {
  return row * 128u + ((c16 ^ (row & 7u)) << 4);
}

}  // namespace sm100

// ---------------------------------------------------------------------------
// host: tensor maps (driver entry point resolved at run time, no -lcuda)
// ---------------------------------------------------------------------------
// Encodes a 3-D map over a [rows][heads][dim] tensor of 16-bit elements with a
// box of (64, 1, box_rows) and the 128-byte swizzle. Returns 0 on success.
int encode_rows_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t heads, uint64_t dim,
                    uint32_t box_rows);
// Same for a plain 2-D [rows][dim] tensor with a box of (64, box_rows).
int encode_2d_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t dim, uint32_t box_rows);

unsigned* device_error_word();   // device address of the per-device error word, or nullptr

}  // namespace moba
