#!/usr/bin/env python
"""Benchmark of the MoBA attention path: one step = forward + backward of
`moba_attention` over one batch of seeded synthetic input.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

Prints ONE JSON line (rank 0). With N > 1 it is launched by torchrun, one
process per GPU; the units (heads / sequences) are sharded across ranks and no
collective runs inside the op. Workloads:

  target   q,k,v [1,131072,4,64] bf16, block 128, top_k 8 per GPU  (default; weak scaling:
           a global [1,131072,4N,64] problem with 4 heads per GPU)
  cfg2     [1,65536,4,64] per GPU
  gqa      q [1,131072,32,128], k/v 8 heads, KV heads sharded over the GPUs (strong scaling)
  gqa1     one KV head of gqa with its four query heads (the shard of an 8-GPU run; for profiling)
  varlen   262144 packed tokens, 32 sequences, H=16, D=128, sequences sharded (strong scaling)
  skewed   q [1,524288,32,128], k/v 8 heads, selections concentrated on early blocks (strong)
  small    [1,8192,4,64], for quick checks and profiler captures

`--impl reference` times the reference algorithm's CPU restatement (oracle/) on
the host cores for the same workload, on a bounded sample per step.

Every line also carries a `strong` record: the grouped-query and the skewed-load
configurations with their 8 KV heads sharded over the N GPUs of this run (device-timed,
max over ranks, per-rank times listed) next to the same whole problem timed on one GPU in
the same run (rank 0), and the resulting speed-up. `--rows PATH` additionally writes the
forward measurement as a CSV row in the column layout of the reference's bench driver.
"""

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "MoBA fwd+bwd useful TFLOP/s (S=128K bf16, block 128, top_k 8; ms in ms_per_step)"
H100_REFERENCE_FWD_BWD_MS = 6.181   # results/sm90-h100/data/moba-bwd.csv:9 of the reference (H100, its Triton kernels)

BLOCK, TOPK = 128, 8


# ----------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------

def varlen_lengths():
    """32 lengths, log-uniform in [1024, 32768] from seed 1, rounded to 128, sum 262144."""
    g = torch.Generator().manual_seed(1)
    u = torch.rand(32, generator=g, dtype=torch.float64)
    raw = torch.exp(math.log(1024.0) + u * math.log(32.0))
    scaled = raw * (262144.0 / float(raw.sum()))
    lens = (torch.round(scaled / 128.0) * 128).to(torch.int64).clamp(min=128)
    lens[int(lens.argmax())] += 262144 - int(lens.sum())
    return [int(x) for x in lens]


def lpt_partition(costs, parts):
    """Longest-processing-time assignment; returns a list of index lists."""
    bins = [[] for _ in range(parts)]
    load = [0] * parts
    for i in sorted(range(len(costs)), key=lambda i: -costs[i]):
        j = load.index(min(load))
        bins[j].append(i)
        load[j] += costs[i]
    return [sorted(b) for b in bins]


def describe(name, rank, world):
    """Per-rank shard of the workload."""
    if name in ("target", "cfg2", "small"):
        s = {"target": 131072, "cfg2": 65536, "small": 8192}[name]
        return dict(name=name, seqlens=[s], hq=4, hkv=4, d=64, packed=False, scaling="weak",
                    seed=1000 * rank, skew=False,
                    text=f"[1,{s},4,64] bf16 per GPU (global [1,{s},{4 * world},64], heads sharded), "
                         f"block {BLOCK}, top_k {TOPK}, fwd+bwd")
    if name == "gqa1":
        # one KV head of cfg3 with its four query heads: what each GPU holds when cfg3 is sharded
        # over eight (small enough for a full ncu capture of the head_dim 128 kernels)
        return dict(name=name, seqlens=[131072], hq=4, hkv=1, d=128, packed=False, scaling="weak",
                    seed=1000 * rank, skew=False,
                    text=f"q [1,131072,4,128] k/v 1 head bf16 per GPU (an eighth of cfg3), "
                         f"block {BLOCK}, top_k {TOPK}, fwd+bwd")
    if name in ("gqa", "skewed"):
        s = 131072 if name == "gqa" else 524288
        if 8 % world:
            raise SystemExit(f"{name}: 8 KV heads do not shard over {world} GPUs")
        hkv = 8 // world
        return dict(name=name, seqlens=[s], hq=4 * hkv, hkv=hkv, d=128, packed=False,
                    scaling="strong", seed=1000 * rank, skew=(name == "skewed"),
                    text=f"q [1,{s},32,128] k/v 8 heads bf16, KV heads sharded {hkv}/GPU, "
                         f"block {BLOCK}, top_k {TOPK}, fwd+bwd")
    if name == "varlen":
        lens = varlen_lengths()
        mine = lpt_partition(lens, world)[rank]
        return dict(name=name, seqlens=[lens[i] for i in mine], hq=16, hkv=16, d=128, packed=True,
                    scaling="strong", seed=1000 * rank, skew=False,
                    text=f"262144 packed tokens, 32 sequences (log-uniform 1024..32768, seed 1), H=16, D=128 "
                         f"bf16, sequences sharded by token count, block {BLOCK}, top_k {TOPK}, fwd+bwd")
    raise SystemExit(f"unknown workload {name}")


def attended_pairs(seq_len):
    total = 0
    for pos0 in range(0, seq_len, BLOCK):
        j, rows = pos0 // BLOCK, min(BLOCK, seq_len - pos0)
        total += rows * (rows + 1) // 2 + rows * min(j, TOPK - 1) * BLOCK
    return total


def selected_pairs(seq_len):
    return sum(min(BLOCK, seq_len - p) * (1 + min(p // BLOCK, TOPK - 1)) for p in range(0, seq_len, BLOCK))


def gate_candidates(seq_len):
    return sum(min(BLOCK, seq_len - p) * (p // BLOCK) for p in range(0, seq_len, BLOCK))


def accounting(wl):
    """Algorithmic work of one step on this rank (useful FLOPs, compulsory bytes)."""
    t = sum(wl["seqlens"])
    hq, hkv, d = wl["hq"], wl["hkv"], wl["d"]
    att = sum(attended_pairs(s) for s in wl["seqlens"]) * hq
    pairs = sum(selected_pairs(s) for s in wl["seqlens"]) * hq
    cand = sum(gate_candidates(s) for s in wl["seqlens"]) * hq
    f_fwd = 4.0 * d * att
    e = 2                                               # bf16
    qb, kvb = t * hq * d * e, t * hkv * d * e
    nb_total = sum(-(-s // BLOCK) for s in wl["seqlens"])
    rows = t * hq
    return dict(
        tokens=t, pairs=pairs, f_fwd=f_fwd, f_step=3.5 * f_fwd,
        bytes_step=(qb + 2 * kvb + qb + rows * 4) + (qb + 2 * kvb + 2 * qb + rows * 4 + qb + 2 * kvb),
        kernels={
            "pool_kernel": ("hbm", kvb + nb_total * hkv * d * e),
            "gate_portable_kernel": ("tensor", 2.0 * d * cand),
            "gate_sm100_kernel": ("tensor", 2.0 * d * cand),
            "count_kernel": ("hbm", rows * TOPK * 4),
            "colscan_kernel": ("hbm", 0),
            "offsets_order_kernel": ("hbm", nb_total * hkv * 12),
            "scatter_kernel": ("hbm", rows * TOPK * 4 + pairs * 12),
            "fill_kernel": ("hbm", rows * TOPK * 4),
            "fwd_portable_kernel": ("tensor", f_fwd),
            "fwd_sm100_kernel": ("tensor", f_fwd),
            "merge_kernel": ("hbm", pairs * (d * e + 4) + rows * TOPK * 4 + qb + rows * 4),
            "delta_kernel": ("hbm", 2 * qb + rows * 4),
            "bwd_portable_kernel": ("tensor", 2.5 * f_fwd),
            "bwd_sm100_kernel": ("tensor", 2.5 * f_fwd),
            "dq_reduce_kernel": ("hbm", pairs * d * e + rows * TOPK * 4 + qb),
        })


def make_inputs(wl, pinned):
    """Seeded N(0,1) bf16 tensors from a CPU generator: q, k, v, dO (+cu_seqlens)."""
    g = torch.Generator().manual_seed(wl["seed"])
    t, hq, hkv, d = sum(wl["seqlens"]), wl["hq"], wl["hkv"], wl["d"]
    q = torch.randn((1, t, hq, d), generator=g)
    k = torch.randn((1, t, hkv, d), generator=g)
    v = torch.randn((1, t, hkv, d), generator=g)
    do = torch.randn((1, t, hq, d), generator=g)
    if wl["skew"]:
        g2 = torch.Generator().manual_seed(2 + wl["seed"])
        n = torch.randn((hkv, d), generator=g2)
        u = 2.0 * n / n.norm(dim=-1, keepdim=True)
        q += u.repeat_interleave(hq // hkv, dim=0)[None, None]
        k[:, : t // 10] += u[None, None]
    out = [x.to(torch.bfloat16) for x in (q, k, v, do)]
    if pinned:
        out = [x.pin_memory() for x in out]
    cu = None
    if wl["packed"]:
        cu = torch.tensor([0] + list(torch.tensor(wl["seqlens"]).cumsum(0)), dtype=torch.int32)
    return out, cu


L2_NOTE = "inputs per step (q,k,v,dO >= 268 MB) exceed the 126 MB L2; no flush"


def base_config(wl, total_tokens):
    """The `config` object, identical for both arms of the benchmark."""
    return {"workload": wl["text"], "tokens_all_gpus": int(total_tokens), "l2": L2_NOTE}


# dram__bytes_read.sum + dram__bytes_write.sum per (query head, block) pair and launch, from ncu
# captures of one launch at [1,65536,4,64] (2 082 816 pairs). The traffic of these kernels is
# per-pair partial rows, so a launch's traffic is this figure times the pairs it processes.
DRAM_BYTES_PER_PAIR = {
    "bwd_sm100_kernel": (295.4e6 + 291.0e6) / 2082816,
    "fwd_sm100_kernel": (167.6e6 + 225.0e6) / 2082816,
    "gate_sm100_kernel": 33.8e6 / 2082816,
}


def bind_to_gpu_numa_node(gpu_index):
    """Pins this process to the CPUs NVML reports as local to the GPU, before any pinned
    buffer is allocated: pinned pages then sit on the GPU's NUMA node and the copy threads
    run beside them. Reads a property, sets nothing on the GPU. Returns the CPU count or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        handle = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(handle, words)
        cpus = {64 * w + b for w, bits in enumerate(mask) for b in range(64) if (bits >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        return None
    return None


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm=float(p["hbm_gbs"]), tensor=float(p["bf16_tflops_sustained"]),
                    tensor_burst=float(p["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


# ----------------------------------------------------------------------------
# clocks
# ----------------------------------------------------------------------------

class ClockSampler:
    """One nvidia-smi process sampling the given GPUs every 100 ms (rank 0 runs it for the
    whole job: eight samplers beside eight ranks would compete with the copy threads)."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_indices):
        self.gpus, self.proc = list(gpu_indices), None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--id=" + ",".join(str(g) for g in self.gpus), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            text, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            text, _ = self.proc.communicate()
        sm, mx, reasons, per_gpu = [], [], set(), {}
        for line in text.splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not f[1].isdigit():
                continue
            sm.append(int(f[1])); mx.append(int(f[2]))
            per_gpu.setdefault(f[0], []).append(int(f[1]))
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        out = {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
               "samples": len(sm), "reasons": sorted(reasons)}
        if len(per_gpu) > 1:
            out["sm_mhz_per_gpu"] = {g: statistics.median(v) for g, v in sorted(per_gpu.items())}
        return out


# ----------------------------------------------------------------------------
# CPU baseline (oracle) -- the only place this file touches oracle/
# ----------------------------------------------------------------------------

def cpu_sample(wl, sample_tokens):
    """One pass of the oracle over the first `sample_tokens` tokens of head 0 of the
    first sequence: gate + sparse forward + backward in float32 on all host threads."""
    from oracle import moba_oracle as orc
    torch.set_num_threads(max(1, os.cpu_count() or 1))     # torchrun pins OMP_NUM_THREADS to 1
    s = min(sample_tokens, wl["seqlens"][0])
    g = torch.Generator().manual_seed(wl["seed"])
    d = wl["d"]
    q, k, v, do = (torch.randn((1, s, 1, d), generator=g).to(torch.bfloat16) for _ in range(4))
    t0 = time.perf_counter()
    mask = orc.selection_mask(q, k, BLOCK, TOPK)
    idx = orc.mask_to_block_idx(mask, TOPK)
    orc.attention_sparse(q, k, v, BLOCK, idx, dout=do, compute_dtype=torch.float32, row_chunk=1024)
    dt = time.perf_counter() - t0
    flops = 3.5 * 4.0 * d * attended_pairs(s)
    return flops, dt, f"first {s} tokens of one head ([1,{s},1,{d}]), gate + fwd + bwd, float32"


def run_reference(args, wl, rank, world):
    if rank != 0:
        return
    flops = secs = 0.0
    what = ""
    for i in range(args.warmup + args.steps):
        f, dt, what = cpu_sample(wl, 16384)
        if i >= args.warmup:
            flops += f; secs += dt
    val = flops / secs / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * secs / args.steps,
        "higher_is_better": True, "scaling": wl["scaling"], "vs_baseline": None, "dtype": "f32",
        "data": "synthetic",
        "config": base_config(wl, sum(sum(describe(args.workload, r, world)["seqlens"]) for r in range(world))),
        "sample_per_step": what,
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                         "kind": "port", "sample": what},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference checkout is not present on the GPU machine; oracle/ is its CPU restatement, "
                "pinned to the reference's own oracle by tests/golden",
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------
# our arm
# ----------------------------------------------------------------------------

def device_inputs(wl, dev):
    """Seeded N(0,1) bf16 q, k, v, dO generated on the device (used by the strong-scaling
    record only; the headline and end-to-end numbers use host-generated pinned inputs)."""
    g = torch.Generator(device=dev).manual_seed(77 + wl["seed"])
    t, hq, hkv, d = sum(wl["seqlens"]), wl["hq"], wl["hkv"], wl["d"]
    mk = lambda h: torch.randn((1, t, h, d), generator=g, device=dev, dtype=torch.float32)
    q, k, v, do = mk(hq), mk(hkv), mk(hkv), mk(hq)
    if wl["skew"]:
        n = torch.randn((hkv, d), generator=g, device=dev)
        u = 2.0 * n / n.norm(dim=-1, keepdim=True)
        q += u.repeat_interleave(hq // hkv, dim=0)[None, None]
        k[:, : t // 10] += u[None, None]
    return [x.to(torch.bfloat16) for x in (q, k, v, do)]


def run_ours(args, wl, rank, world, local_rank):
    import moba_triton_b200 as moba
    from moba_triton_b200 import _lib

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    local_cpus = bind_to_gpu_numa_node(local_rank)          # before any pinned allocation
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)
    if args.path:
        _lib.set_kernel_path({"portable": _lib.PATH_PORTABLE, "tcgen05": _lib.PATH_TCGEN05}[args.path])

    cfg = moba.MoBAConfig(block_size=BLOCK, top_k=TOPK)
    acct = accounting(wl)
    host, cu = make_inputs(wl, pinned=True)
    cu_dev = None if cu is None else cu.to(dev)
    max_seqlen = max(wl["seqlens"]) if wl["packed"] else None
    kw = dict(cu_seqlens=cu_dev, max_seqlen=max_seqlen) if wl["packed"] else {}

    q, k, v, do = (x.to(dev) for x in host)
    q.requires_grad_(True); k.requires_grad_(True); v.requires_grad_(True)

    def step():
        q.grad = k.grad = v.grad = None
        out = moba.moba_attention(q, k, v, cfg, **kw)
        out.backward(do)
        return out

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, n, ranks=None):
        """Device time of n calls of fn, bracketed by barriers: (max over ranks, per-rank list)."""
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n):
            fn()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        if dist is None:
            return ms, [ms]
        mine = torch.tensor([ms], device=dev)
        every = torch.empty(world, device=dev)
        dist.all_gather_into_tensor(every, mine)
        return float(every.max()), [float(x) for x in every.tolist()]

    # nvidia-smi needs a few hundred ms to deliver its first sample, so the sampler runs from
    # the warm-up on, and the same step keeps running (untimed) after the timed region until
    # the sampler has had about a second under this load.
    clocks = ClockSampler(range(world)) if rank == 0 else None
    if clocks is not None:
        clocks.start()
    t_load = time.perf_counter()
    for _ in range(args.warmup):
        step()
    launches0 = _lib.launch_count()
    ms_total, per_rank_total = timed(step, args.steps)
    launches = _lib.launch_count() - launches0
    while time.perf_counter() - t_load < 1.2:
        step()
    torch.cuda.synchronize()
    barrier()
    clock_info = clocks.stop() if clocks is not None else None
    ms_step = ms_total / args.steps

    # forward only (inference entry point)
    with torch.no_grad():
        fwd = lambda: moba.moba_forward(q, k, v, cfg, **kw)
        for _ in range(2):
            fwd()
        torch.cuda.reset_peak_memory_stats(dev)
        n_fwd = max(2, args.steps // 2)
        ms_fwd = timed(fwd, n_fwd)[0] / n_fwd
        fwd_peak_mb = torch.cuda.max_memory_allocated(dev) / (1 << 20)

    # end to end: host buffers in, host buffers out, through the public API. Every step copies
    # its q, k, v, dO from pinned host memory and its O, dQ, dK, dV back. The copies run on two
    # streams of their own, ordered against the op by events: dO goes up while the forward runs,
    # O comes down while the backward runs, and a step's uploads start while the previous
    # step's gradients are still on their way down (PCIe carries both directions at once).
    outs_host = [torch.empty_like(h).pin_memory() for h in (host[0], host[0], host[1], host[2])]
    main_s = torch.cuda.current_stream()
    h2d_s, d2h_s = torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_step():
        with torch.cuda.stream(h2d_s):
            qd, kd, vd = (h.to(dev, non_blocking=True) for h in host[:3])
            ev_qkv = h2d_s.record_event()
            dod = host[3].to(dev, non_blocking=True)
            ev_do = h2d_s.record_event()
        for t in (qd, kd, vd, dod):
            t.record_stream(main_s)                          # allocated on the copy stream, used here
        main_s.wait_event(ev_qkv)
        qd.requires_grad_(True); kd.requires_grad_(True); vd.requires_grad_(True)
        out = moba.moba_attention(qd, kd, vd, cfg, **kw)
        ev_fwd = main_s.record_event()
        main_s.wait_event(ev_do)
        out.backward(dod)
        ev_bwd = main_s.record_event()
        results = (out.detach(), qd.grad, kd.grad, vd.grad)
        with torch.cuda.stream(d2h_s):
            d2h_s.wait_event(ev_fwd)
            outs_host[0].copy_(results[0], non_blocking=True)
            d2h_s.wait_event(ev_bwd)
            for dst, src in zip(outs_host[1:], results[1:]):
                dst.copy_(src, non_blocking=True)
        for t in results:
            t.record_stream(d2h_s)

    def e2e_run(n):                                          # the timed region ends when the last copy has landed
        for _ in range(n):
            e2e_step()
        main_s.wait_stream(d2h_s)

    # enough steps for the steady state to show: the first upload and the last download of the
    # timed region overlap nothing, and with few steps they dominate the average
    e2e_steps = max(2, min(args.steps, 20))
    e2e_run(1)
    ms_e2e_total, per_rank_e2e = timed(lambda: e2e_run(e2e_steps), 1)
    ms_e2e = ms_e2e_total / e2e_steps
    # the overlapped path must deliver what the plain call computes (the op is deterministic)
    e2e_ok = bool(torch.equal(outs_host[0], step().detach().cpu()) and
                  torch.equal(outs_host[1], q.grad.cpu()))
    h2d = sum(h.numel() * h.element_size() for h in host)
    d2h = sum(h.numel() * h.element_size() for h in outs_host)
    # the copies alone, one direction at a time: what the host side of the step can deliver
    dev_in = [torch.empty_like(h, device=dev) for h in host]
    dev_out = [torch.empty_like(h, device=dev) for h in outs_host]

    def h2d_only():
        for d_, h_ in zip(dev_in, host):
            d_.copy_(h_, non_blocking=True)

    def d2h_only():
        for h_, d_ in zip(outs_host, dev_out):
            h_.copy_(d_, non_blocking=True)

    ms_h2d, per_rank_h2d = timed(h2d_only, 3)
    ms_d2h, per_rank_d2h = timed(d2h_only, 3)
    del dev_in, dev_out

    # per-kernel durations (CUDA events on the launching stream, inside the library)
    _lib.profile(True)
    prof_steps = 3
    for _ in range(prof_steps):
        step()
    torch.cuda.synchronize()
    _lib.profile(False)
    table = _lib.profile_read()

    total_f = acct["f_step"]
    total_tokens = acct["tokens"]
    if dist is not None:
        t = torch.tensor([total_f, float(total_tokens)], device=dev, dtype=torch.float64)
        dist.all_reduce(t)
        total_f, total_tokens = float(t[0]), int(t[1])
    pk = peaks()

    # ---- strong scaling of the sharded configurations, on every line ----
    del q, k, v, do
    torch.cuda.empty_cache()

    def strong_case(name):
        if 8 % world:
            return {"workload": name, "skipped": f"8 KV heads do not shard over {world} GPUs"}
        def run(swl, active):
            if not active:
                return None
            qq, kk, vv, dd = device_inputs(swl, dev)
            qq.requires_grad_(True); kk.requires_grad_(True); vv.requires_grad_(True)
            def one():
                qq.grad = kk.grad = vv.grad = None
                moba.moba_attention(qq, kk, vv, cfg).backward(dd)
            return one
        sharded = run(describe(name, rank, world), True)
        for _ in range(2):
            sharded()
        ms, per_rank = timed(sharded, 3)
        del sharded
        torch.cuda.empty_cache()
        rec = {"workload": describe(name, 0, world)["text"], "n_gpus": world, "ms_sharded": ms / 3,
               "per_rank_ms": [x / 3 for x in per_rank], "inputs": "seeded N(0,1), generated on the device"}
        if world == 1:
            rec["ms_one_gpu"], rec["speedup"] = rec["ms_sharded"], 1.0
            return rec
        whole = run(describe(name, 0, 1), rank == 0)           # rank 0 alone times the whole problem
        if whole is not None:
            for _ in range(2):
                whole()
        ms_one, _ = timed((whole if whole is not None else (lambda: None)), 3)
        one = torch.tensor([ms_one / 3 if rank == 0 else 0.0], device=dev)
        dist.all_reduce(one, op=dist.ReduceOp.MAX)
        del whole
        torch.cuda.empty_cache()
        rec["ms_one_gpu"] = float(one)
        rec["speedup"] = rec["ms_one_gpu"] / rec["ms_sharded"]
        return rec

    strong = [] if args.no_strong else [strong_case("gqa"), strong_case("skewed")]

    if rank == 0:
        kernels = {n: {"launches_per_step": c / prof_steps, "ms_per_launch": ms / c,
                       "share": ms / max(1e-9, sum(m for _, m in table.values()))}
                   for n, (c, ms) in sorted(table.items(), key=lambda kv: -kv[1][1])}
        top = next(iter(kernels))
        kind, amount = acct["kernels"].get(top, ("tensor", 0.0))
        dur_s = kernels[top]["ms_per_launch"] * 1e-3
        if kind == "tensor":
            achieved, peak, unit = amount / dur_s / 1e12, pk["tensor"], "TFLOP/s"
        else:
            achieved, peak, unit = amount / dur_s / 1e9, pk["hbm"], "GB/s"
        traffic = DRAM_BYTES_PER_PAIR[top] * acct["pairs"] if top in DRAM_BYTES_PER_PAIR else None
        t_roof = max(acct["f_step"] / (pk["tensor_burst"] * 1e12), acct["bytes_step"] / (pk["hbm"] * 1e9))
        roofline = {"kernel": top, "bound": kind, "achieved": achieved, "peak": peak, "unit": unit,
                    "frac": achieved / peak, "traffic": traffic,
                    "peak_source": f"{pk['source']} ({'sustained' if kind == 'tensor' else 'copy'})"}
        if kind == "tensor":
            roofline["frac_burst"] = achieved / pk["tensor_burst"]
            roofline["peak_burst"] = pk["tensor_burst"]
        config = base_config(wl, total_tokens)
        line = {
            "metric": METRIC, "value": total_f / (ms_step * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "per_rank_ms_per_step": [x / args.steps for x in per_rank_total],
            "higher_is_better": True, "scaling": wl["scaling"],
            "vs_baseline": (H100_REFERENCE_FWD_BWD_MS / ms_step) if wl["name"] == "target" else None,
            "vs_baseline_note": "reference Triton kernels on H100, fwd+bwd at [1,131072,4,64]: 6.181 ms; "
                                "the reference publishes no B200 number",
            "dtype": "bf16", "data": "synthetic", "config": config, "kernel_path": args.path or "auto",
            "fwd_ms": ms_fwd, "fwd_tflops": acct["f_fwd"] / (ms_fwd * 1e-3) / 1e12,
            "op_roofline": {"t_roof_ms": t_roof * 1e3, "frac": t_roof * 1e3 / ms_step,
                            "peak": f"{pk['tensor_burst']} TFLOP/s burst, {pk['hbm']} GB/s ({pk['source']})"},
            "e2e": {"value": total_f / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "per_rank_ms_per_step": [x / e2e_steps for x in per_rank_e2e],
                    "outputs_match_resident_run": e2e_ok,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "h2d_only_ms": ms_h2d / 3, "d2h_only_ms": ms_d2h / 3,
                    "per_rank_h2d_only_ms": [x / 3 for x in per_rank_h2d],
                    "per_rank_d2h_only_ms": [x / 3 for x in per_rank_d2h],
                    "cpus_bound_to_gpu_numa_node": local_cpus},
            "gpu_launches": launches,
            "clocks": clock_info,
            "roofline": roofline,
            "kernels": kernels,
            "strong": strong,
        }
        if world == 1 and not args.no_cpu_baseline:
            f, dt, what = cpu_sample(wl, 65536)
            line["cpu_baseline"] = {"value": f / dt / 1e12, "unit": "TFLOP/s", "cores": torch.get_num_threads(),
                                    "kind": "port", "sample": what, "seconds": dt}
        if args.rows and not wl["packed"]:
            from moba_triton_b200 import bench_rows
            shape = (1, sum(wl["seqlens"]), wl["hq"], wl["d"])
            bench_rows.write_csv(args.rows, [bench_rows.make_row("ours_b200", shape, cfg, ms_fwd, fwd_peak_mb, device=dev)])
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="target")
    ap.add_argument("--path", default="", choices=["", "portable", "tcgen05"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="skip the strong-scaling record")
    ap.add_argument("--rows", default="", help="write the forward measurement as a CSV row here")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torchrun --nproc-per-node N for --gpus N")
    wl = describe(args.workload, rank, world)
    if args.impl == "reference":
        run_reference(args, wl, rank, world)
    else:
        run_ours(args, wl, rank, world, local_rank)


if __name__ == "__main__":
    main()
