"""Host-side checks that need no GPU: configuration, validators, the C ABI."""

import ctypes
import os
import re

import pytest
import torch

import moba_triton_b200 as moba
from moba_triton_b200 import _lib
from moba_triton_b200.kernels.moba_fwd import _validate
from moba_triton_b200.varlen import from_nested, pack, unpack, validate_cu_seqlens

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_config_defaults_and_budget():
    cfg = moba.MoBAConfig(block_size=128, top_k=8)
    assert cfg.dtype is torch.bfloat16 and cfg.always_select_current and cfg.top_k_includes_current
    assert cfg.past_blocks_selected(1024) == 7 and cfg.past_blocks_selected(3) == 3
    assert cfg.num_blocks(200) == 2 and cfg.slots_per_query == 8
    assert moba.MoBAConfig(32, 2, top_k_includes_current=False).slots_per_query == 3
    assert moba.MoBAConfig(32, 2, always_select_current=False).slots_per_query == 2
    with pytest.raises(ValueError):
        moba.MoBAConfig(block_size=0, top_k=1)
    with pytest.raises(Exception):
        cfg.top_k = 3                                   # frozen


def test_validate_messages_match_the_reference_keys():
    cfg = moba.MoBAConfig(32, 4)
    q = torch.zeros(1, 64, 4, 64)
    with pytest.raises(ValueError, match="key/value"):
        _validate(q, q, torch.zeros(1, 64, 2, 64), cfg)
    with pytest.raises(ValueError, match="shape mismatch"):
        _validate(q, torch.zeros(1, 32, 4, 64), torch.zeros(1, 32, 4, 64), cfg)
    with pytest.raises(ValueError, match="divisible"):
        _validate(q, torch.zeros(1, 64, 3, 64), torch.zeros(1, 64, 3, 64), cfg)
    cu = torch.tensor([0, 64], dtype=torch.int32)
    with pytest.raises(ValueError, match="batch 1"):
        _validate(torch.zeros(2, 64, 4, 64), torch.zeros(2, 64, 4, 64), torch.zeros(2, 64, 4, 64), cfg, cu, 64)
    with pytest.raises(ValueError, match="max_seqlen"):
        _validate(q, q, q, cfg, cu, None)
    with pytest.raises(ValueError, match="below the tl.dot minimum"):
        _validate(q, q, q, moba.MoBAConfig(8, 2))
    with pytest.raises(ValueError, match="power of two"):
        _validate(torch.zeros(1, 64, 4, 48), torch.zeros(1, 64, 4, 48), torch.zeros(1, 64, 4, 48), cfg)
    with pytest.raises(ValueError, match="cache line"):
        _validate(torch.zeros(1, 64, 4, 16), torch.zeros(1, 64, 4, 16), torch.zeros(1, 64, 4, 16), cfg)


def test_cu_seqlens_validation():
    ok = torch.tensor([0, 80, 128], dtype=torch.int32)
    assert validate_cu_seqlens(ok, 128, 80) == 2
    for bad, msg in [(torch.tensor([[0, 1]], dtype=torch.int32), "1-D"),
                     (torch.tensor([0], dtype=torch.int32), "two entries"),
                     (torch.tensor([0, 128]), "int32"),
                     (torch.tensor([1, 128], dtype=torch.int32), "start at 0"),
                     (torch.tensor([0, 64, 64, 128], dtype=torch.int32), "strictly increasing"),
                     (torch.tensor([0, 100], dtype=torch.int32), "total token count")]:
        with pytest.raises(ValueError, match=msg):
            validate_cu_seqlens(bad, 128, 128)
    with pytest.raises(ValueError, match="below the longest"):
        validate_cu_seqlens(ok, 128, 64)


def test_pack_and_unpack_check_shapes_and_refuse_cpu_tensors():
    x = torch.zeros(3, 10, 2, 4)
    mask = torch.ones(3, 10, dtype=torch.bool)
    with pytest.raises(ValueError, match=r"\[B, S, H, D\]"):
        pack(x[0], mask)
    with pytest.raises(ValueError, match="attention_mask"):
        pack(x, mask[:, :5])
    with pytest.raises(ValueError, match=r"\[1, T, H, D\]"):
        unpack(x, torch.tensor([0, 10], dtype=torch.int32), 1, 10)
    with pytest.raises(ValueError, match="entries"):
        unpack(x[:1], torch.tensor([0, 10], dtype=torch.int32), 3, 10)
    with pytest.raises(ValueError, match="nested"):
        from_nested(x)
    with pytest.raises(RuntimeError, match="no CPU path"):          # the row gathers are CUDA kernels
        pack(x, mask)
    with pytest.raises(RuntimeError, match="no CPU path"):
        unpack(x[:1], torch.tensor([0, 10], dtype=torch.int32), 1, 10)


def test_product_refuses_cpu_tensors_instead_of_falling_back():
    cfg = moba.MoBAConfig(32, 4)
    q = torch.zeros(1, 64, 2, 64)
    with pytest.raises(RuntimeError, match="no CPU path"):
        moba.moba_forward(q, q, q, cfg)
    with pytest.raises(RuntimeError, match="no CPU path"):
        moba.moba_attention(q, q, q, cfg)


def test_library_loads_and_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "moba_b200.h")).read()
    declared = set(re.findall(r"\b(moba_b200_[a-z_0-9]+)\s*\(", header))
    assert declared == set(_lib.EXPORTS)
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in declared:
        assert hasattr(lib, name), name
    assert _lib.load().moba_b200_abi_version() == _lib.ABI_VERSION


def test_c_abi_rejects_bad_problems_without_touching_a_gpu():
    lib = _lib.load()
    cfg = moba.MoBAConfig(32, 4)
    prob = _lib.make_problem((1, 64, 3, 64), 2, torch.bfloat16, cfg)
    assert lib.moba_b200_path_for(prob, _lib.STAGE_FWD) == -1
    assert b"divisible" in lib.moba_b200_last_error()
    prob = _lib.make_problem((1, 64, 2, 64), 2, torch.bfloat16, cfg)
    assert lib.moba_b200_pool(prob, None, None, None, None) == -1
    assert b"NULL" in lib.moba_b200_last_error()
    assert lib.moba_b200_transpose_scratch_bytes(prob) == 1 * 2 * 2 * 1 * 1 * 4 + 16   # histograms + slot counter
    # scheduling sizes are functions of the problem record alone
    assert lib.moba_b200_chunk_tiles(prob) == 8                       # small problems: the floor
    pairs = 1 * 64 * 2 * 4
    assert lib.moba_b200_work_items_per_row(prob) == 2 + pairs // (128 * 8) + 1
    assert lib.moba_b200_dkv_scratch_bytes(prob) == (2 * (pairs // (128 * 8) + 1) + 1) * 2 * 128 * 64 * 4
    big = _lib.make_problem((1, 524288, 32, 128), 8, torch.bfloat16, moba.MoBAConfig(128, 8))
    assert lib.moba_b200_chunk_tiles(big) == -(-(524288 * 32 * 8 // 128) // (4 * 148))
    assert lib.moba_b200_work_items_per_row(big) <= 4096 + 4 * 148 + 1
    assert _lib.make_problem((1, 64, 2, 64), 2, torch.bfloat16, cfg, chunk_tiles=3).chunk_tiles == 3


def test_product_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "moba_triton_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                assert "oracle" not in open(os.path.join(base, f)).read().replace("the oracle uses", ""), f


def test_backend_adapter_follows_the_reference_protocol_and_never_raises():
    from moba_triton_b200.adapter import B200Backend
    b = B200Backend()
    assert b.name and b.vendored is False and b.computes_moba is True
    for m in ("is_available", "forward", "forward_grad", "selection"):
        assert callable(getattr(b, m))
    ok, reason = b.is_available(moba.MoBAConfig(128, 8))
    assert isinstance(ok, bool) and isinstance(reason, str)
    if not torch.cuda.is_available():
        assert not ok and reason                       # says why instead of raising


def test_kv_heads_per_pass_arguments_are_checked_before_any_device_work():
    q = torch.zeros(1, 256, 4, 64, dtype=torch.bfloat16)
    k = v = torch.zeros(1, 256, 2, 64, dtype=torch.bfloat16)
    cfg = moba.MoBAConfig(block_size=128, top_k=2, dtype=torch.bfloat16)
    for fn in (moba.moba_attention, moba.moba_forward):
        with pytest.raises(ValueError, match="kv_heads_per_pass must be positive"):
            fn(q, k, v, cfg, kv_heads_per_pass=0)
        with pytest.raises(ValueError, match="cannot be combined with index"):
            fn(q, k, v, cfg, index=object(), kv_heads_per_pass=1)


def test_a_swapped_exact_tie_is_not_accepted_as_a_near_tie():
    from helpers import near_tie_report
    scores = torch.tensor([[[[1.0, 1.0, 0.5, 0.0]]]], dtype=torch.float64)
    oracle = torch.tensor([[[[True, False, True, False]]]])
    engine = torch.tensor([[[[False, True, True, False]]]])
    assert near_tie_report(engine, oracle, scores, 8) == (1, 1)
    scores[..., 1] = 1.0 - 2.0 ** -8                         # one rounding step apart: a near tie
    assert near_tie_report(engine, oracle, scores, 8) == (1, 0)


def test_bench_rows_have_the_reference_columns_and_closed_form_sparsity(tmp_path):
    """Column names and order of the reference's BenchRow (bench/suite.py:37-63); pair counts
    against real selection masks (as tests/test_bench.py:66-92 does there)."""
    import csv
    from moba_triton_b200 import bench_rows as br
    from oracle import moba_oracle as orc
    assert br.COLUMNS == (
        "backend", "batch", "heads", "seq_len", "head_dim", "block_size", "top_k", "dtype", "latency_ms", "tflops",
        "peak_memory_mb", "sparsity", "speedup_vs_dense", "speedup_ceiling", "attainment", "gpu_name", "capability",
        "total_memory_mb", "torch_version", "triton_version", "cuda_version", "status", "note")
    for s, bs, top_k in ((512, 64, 3), (200, 32, 4), (4096, 128, 8)):
        cfg = moba.MoBAConfig(bs, top_k)
        assert br.attended_pairs(s, cfg) == orc.attended_pairs(s, bs, top_k)
    g = torch.Generator().manual_seed(0)
    q = torch.randn(1, 200, 1, 64, generator=g)
    cfg = moba.MoBAConfig(32, 3)
    mask = orc.selection_mask(q, q, 32, 3)[0, 0]                             # [S, nb]
    pos = torch.arange(200)
    visible = mask[:, pos // 32] & (pos[None, :] <= pos[:, None])
    assert int(visible.sum()) == br.attended_pairs(200, cfg)
    row = br.make_row("ours_b200", (1, 4096, 4, 64), moba.MoBAConfig(128, 8), 0.05, 12.0, dense_latency_ms=0.2)
    assert tuple(row) == br.COLUMNS and row["status"] == "ok"
    assert abs(row["speedup_vs_dense"] - 4.0) < 1e-12 and abs(row["attainment"] - 4.0 * row["sparsity"]) < 1e-12
    assert abs(row["tflops"] - 4.0 * 4 * br.attended_pairs(4096, moba.MoBAConfig(128, 8)) * 64 / 0.05e-3 / 1e12) < 1e-9
    bad = br.make_row("ours_b200", (1, 4096, 4, 64), moba.MoBAConfig(128, 8), float("nan"), float("nan"),
                      status="error", note="x" * 500)
    assert bad["latency_ms"] != bad["latency_ms"] and len(bad["note"]) == 160
    path = tmp_path / "rows.csv"
    br.write_csv(str(path), [row, bad])
    got = list(csv.DictReader(open(path)))
    assert list(got[0]) == list(br.COLUMNS) and got[1]["status"] == "error"


def test_launch_plan_is_a_table_lookup_on_the_problem_record():
    from moba_triton_b200.tuning import launch_plan
    cfg = moba.MoBAConfig(128, 8)
    target = launch_plan((1, 131072, 4, 64), 4, torch.bfloat16, cfg)
    assert target["gate_path"] == target["fwd_path"] == target["bwd_path"] == "tcgen05"
    assert (target["fwd_tiles_in_flight"], target["fwd_q_stages"]) == (4, 4)
    assert (target["bwd_kv_buffers"], target["bwd_gather_stages"]) == (2, 2)
    assert (target["gate_slots"], target["gate_step"]) == (16, 8)
    assert (target["transpose_chunk_rows"], target["transpose_chunks"], target["scatter_warps"]) == (512, 256, 8)
    assert target["chunk_tiles"] == -(-(131072 * 4 * 8 // 128) // (4 * 148))
    gqa = launch_plan((1, 524288, 32, 128), 8, torch.bfloat16, cfg)
    assert (gqa["fwd_tiles_in_flight"], gqa["fwd_q_stages"], gqa["bwd_kv_buffers"], gqa["gate_slots"]) == (2, 2, 1, 7)
    assert gqa["scatter_warps"] == 4 and gqa["transpose_chunk_rows"] == 2048
    # float32 and odd block sizes run the portable kernels; the tile plan is then empty
    slow = launch_plan((1, 4096, 4, 64), 4, torch.float32, moba.MoBAConfig(128, 8, dtype=torch.float32))
    assert slow["fwd_path"] == "portable" and slow["fwd_tiles_in_flight"] == 0
    assert launch_plan((1, 4096, 4, 64), 4, torch.bfloat16, moba.MoBAConfig(64, 4))["gate_path"] == "portable"
    # packed or padded, the same sequence length gets the same kernels (bitwise packed == alone)
    cu = torch.tensor([0, 1000, 2024], dtype=torch.int32)
    packed = launch_plan((1, 2024, 4, 64), 2, torch.bfloat16, cfg, cu_seqlens=cu, max_seqlen=1024)
    alone = launch_plan((1, 1024, 4, 64), 2, torch.bfloat16, cfg)
    for key in ("gate_path", "fwd_path", "bwd_path", "fwd_tiles_in_flight", "fwd_q_stages", "bwd_kv_buffers",
                "bwd_gather_stages", "gate_slots", "gate_step"):
        assert packed[key] == alone[key]
    with pytest.raises(ValueError):
        launch_plan((1, 64, 3, 64), 2, torch.bfloat16, cfg)


def test_reference_arm_of_the_bench_prints_the_contract_line():
    """`bench.py --impl reference` needs no GPU: it times the oracle on the host cores and
    prints one JSON line whose `config` is the object our arm prints for the same workload."""
    import json
    import subprocess
    import sys
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                          "--warmup", "0", "--workload", "small"], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    line = json.loads(out.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "TFLOP/s" and line["higher_is_better"] is True
    assert line["value"] > 0 and line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"] == {"value": line["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}
    import bench
    wl = bench.describe("small", 0, 1)
    assert line["config"] == bench.base_config(wl, 8192)
    assert set(line["config"]) == {"workload", "tokens_all_gpus", "l2"}


def test_candidate_window_rule_of_the_restatement_and_the_config():
    from oracle import moba_oracle as orc
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, 512, 1, 64, generator=g)
    k = torch.randn(1, 512, 1, 64, generator=g)
    full = orc.selection_mask(q, k, 32, 4)
    assert torch.equal(orc.selection_mask(q, k, 32, 4, gate_window=64), full)       # wider than the sequence
    win = orc.selection_mask(q, k, 32, 4, gate_window=2, gate_sinks=1)[0, 0]        # [S, nb]
    own = torch.arange(512) // 32
    for s in (100, 300, 511):
        chosen = set(win[s].nonzero().flatten().tolist())
        allowed = {0, own[s].item() - 2, own[s].item() - 1, own[s].item()}
        assert chosen <= allowed and own[s].item() in chosen and len(chosen) == min(4, len(allowed))
    with pytest.raises(ValueError):
        moba.MoBAConfig(32, 4, gate_window=0)
    with pytest.raises(ValueError):
        moba.MoBAConfig(32, 4, gate_sinks=2)
    prob = _lib.make_problem((1, 512, 2, 64), 2, torch.bfloat16, moba.MoBAConfig(32, 4, gate_window=7, gate_sinks=3))
    assert (prob.gate_window, prob.gate_sinks) == (7, 3)
    assert _lib.make_problem((1, 512, 2, 64), 2, torch.bfloat16, moba.MoBAConfig(32, 4)).gate_window == 0
