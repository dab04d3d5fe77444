"""Measurement rows in the column layout of the reference's benchmark driver
(reference: bench/suite.py:37-63 `BenchRow`, filled at :525-596), so that the
reference's `bench/compare.py` and plotting scripts can ingest this engine's
numbers beside its own backends' rows.

    rows = [measure_row(B200Backend(), q, k, v, cfg, dense_latency_ms=...)]
    write_csv("ours_b200.csv", rows)

A row holds: what was run (backend, batch, heads, seq_len, head_dim, block_size,
top_k, dtype), what was measured (latency_ms, tflops over the attended pairs
only, peak_memory_mb), how sparse the pattern is (sparsity, speedup_ceiling =
1 / sparsity), the speed-up over a dense-attention latency measured elsewhere
(speedup_vs_dense, attainment = speedup / ceiling; NaN when no dense latency is
given -- dense attention is not part of this engine) and where it ran.

Latency is the median of CUDA-event timings after warm-up, with the L2 flushed
between repetitions when the inputs would fit in it.
"""

import csv
import math
import statistics

import torch

COLUMNS = (
    "backend", "batch", "heads", "seq_len", "head_dim", "block_size", "top_k", "dtype",
    "latency_ms", "tflops", "peak_memory_mb", "sparsity", "speedup_vs_dense", "speedup_ceiling",
    "attainment", "gpu_name", "capability", "total_memory_mb", "torch_version", "triton_version",
    "cuda_version", "status", "note",
)
MAX_NOTE_CHARS = 160
L2_BYTES = 126 << 20


def attended_pairs(seq_len: int, cfg) -> int:
    """(query, key) pairs one head attends: per query its causal prefix of the own block plus
    `block_size` keys for each selected past block (the closed form the reference checks
    against real masks, bench/suite.py:66-95)."""
    bs = cfg.block_size
    budget = cfg.past_blocks_selected(cfg.num_blocks(seq_len))
    own = 1 if cfg.always_select_current else 0
    total = 0
    for lo in range(0, seq_len, bs):
        rows = min(bs, seq_len - lo)
        past = min(lo // bs, budget)
        total += own * rows * (rows + 1) // 2 + rows * past * bs
    return total


def sparsity_ratio(seq_len: int, cfg) -> float:
    """Attended pairs over causally visible pairs, in (0, 1]."""
    return attended_pairs(seq_len, cfg) / (seq_len * (seq_len + 1) / 2)


def effective_tflops(batch: int, heads: int, seq_len: int, head_dim: int, cfg, ms: float) -> float:
    """TFLOP/s over the attended pairs only: QK^T and PV, two FLOPs per multiply-add."""
    return 4.0 * batch * heads * attended_pairs(seq_len, cfg) * head_dim / (ms * 1e-3) / 1e12


def device_columns(device=None) -> dict:
    """The where-it-ran columns of a row."""
    if not torch.cuda.is_available():
        return dict(gpu_name="none", capability="", total_memory_mb=0, torch_version=torch.__version__,
                    triton_version="none", cuda_version=str(torch.version.cuda))
    prop = torch.cuda.get_device_properties(device)
    return dict(gpu_name=prop.name, capability=f"{prop.major}.{prop.minor}",
                total_memory_mb=int(prop.total_memory // (1 << 20)), torch_version=torch.__version__,
                triton_version="none (hand-written sm_100a CUDA)", cuda_version=str(torch.version.cuda))


def time_ms(fn, warmup: int = 3, reps: int = 10, flush_l2: bool = False) -> float:
    """Median CUDA-event time of `fn` on the current stream."""
    scrub = torch.empty(2 * L2_BYTES, dtype=torch.uint8, device="cuda") if flush_l2 else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(reps):
        if scrub is not None:
            scrub.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return statistics.median(times)


def make_row(backend: str, shape, cfg, latency_ms: float, peak_memory_mb: float, computes_moba: bool = True,
             dense_latency_ms=None, status: str = "ok", note: str = "", device=None) -> dict:
    """One row from numbers already measured; `shape` is (batch, seq_len, heads, head_dim)."""
    batch, seq_len, heads, head_dim = shape
    sparsity = sparsity_ratio(seq_len, cfg)
    ceiling = 1.0 / sparsity
    ok = status == "ok" and latency_ms == latency_ms and latency_ms > 0
    speedup = dense_latency_ms / latency_ms if (ok and dense_latency_ms) else math.nan
    if ok and computes_moba:
        tflops = effective_tflops(batch, heads, seq_len, head_dim, cfg, latency_ms)
    elif ok:                                              # a dense backend attends every causal pair
        tflops = 4.0 * batch * heads * (seq_len * (seq_len + 1) / 2) * head_dim / (latency_ms * 1e-3) / 1e12
    else:
        tflops = math.nan
    row = dict(backend=backend, batch=batch, heads=heads, seq_len=seq_len, head_dim=head_dim,
               block_size=cfg.block_size, top_k=cfg.top_k, dtype=str(cfg.dtype).replace("torch.", ""),
               latency_ms=latency_ms if ok else math.nan, tflops=tflops, peak_memory_mb=peak_memory_mb,
               sparsity=sparsity, speedup_vs_dense=speedup, speedup_ceiling=ceiling,
               attainment=speedup / ceiling, status=status, note=note[:MAX_NOTE_CHARS], **device_columns(device))
    assert tuple(row) == COLUMNS or set(row) == set(COLUMNS)
    return {c: row[c] for c in COLUMNS}


def measure_row(backend, q, k, v, cfg, dense_latency_ms=None, warmup: int = 3, reps: int = 10) -> dict:
    """Times `backend.forward(q, k, v, cfg)` (the call the reference's driver times,
    bench/suite.py:401-416) and returns its row; a backend that raises gives an "error" row."""
    shape = (q.shape[0], q.shape[1], q.shape[2], q.shape[3])
    name = getattr(backend, "name", type(backend).__name__)
    try:
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats(q.device)
        small = sum(t.numel() * t.element_size() for t in (q, k, v)) < L2_BYTES
        with torch.no_grad():
            ms = time_ms(lambda: backend.forward(q, k, v, cfg), warmup, reps, flush_l2=small)
        peak = torch.cuda.max_memory_allocated(q.device) / (1 << 20)
    except (RuntimeError, ValueError, NotImplementedError) as exc:
        return make_row(name, shape, cfg, math.nan, math.nan, status="error", note=str(exc), device=q.device)
    return make_row(name, shape, cfg, ms, peak, computes_moba=getattr(backend, "computes_moba", True),
                    dense_latency_ms=dense_latency_ms, device=q.device)


def write_csv(path: str, rows) -> None:
    """Writes rows with the reference's header line, in its column order."""
    with open(path, "w", newline="") as fh:
        w = csv.DictWriter(fh, fieldnames=list(COLUMNS))
        w.writeheader()
        for r in rows:
            w.writerow(r)
