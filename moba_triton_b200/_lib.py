"""ctypes binding of libmoba_b200.so (the C ABI in include/moba_b200.h).

There is no CPU or PyTorch fallback: if the library is missing, or a call
fails, the error is raised to the caller.
"""

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_int, c_int32, c_int64, c_size_t, c_void_p

import torch

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("MOBA_B200_LIBRARY", os.path.join(PKG, "libmoba_b200.so"))

F32, BF16, F16 = 0, 1, 2
PATH_AUTO, PATH_PORTABLE, PATH_TCGEN05 = 0, 1, 2
STAGE_GATE, STAGE_FWD, STAGE_BWD = 0, 1, 2
ABI_VERSION = 2

_DTYPE_CODE = {torch.float32: F32, torch.bfloat16: BF16, torch.float16: F16}

EXPORTS = (
    "moba_b200_abi_version", "moba_b200_last_error", "moba_b200_path_for",
    "moba_b200_transpose_scratch_bytes", "moba_b200_pool", "moba_b200_gate",
    "moba_b200_transpose", "moba_b200_fwd", "moba_b200_merge", "moba_b200_bwd",
    "moba_b200_launch_count", "moba_b200_profile_enable", "moba_b200_profile_read",
    "moba_b200_device_status", "moba_b200_transpose_noalloc",
    "moba_b200_pack_index", "moba_b200_pack_rows", "moba_b200_unpack_rows", "moba_b200_seq_meta",
    "moba_b200_chunk_tiles", "moba_b200_work_items_per_row", "moba_b200_dkv_scratch_bytes",
    "moba_b200_launch_plan",
)


class Problem(Structure):
    _fields_ = [(n, c_int32) for n in (
        "dtype", "batch", "tokens", "n_seq", "max_seqlen", "q_heads", "kv_heads", "head_dim",
        "block_size", "top_k", "slots", "take", "always_current", "num_blocks", "causal",
        "packed", "path", "part_f32", "chunk_tiles", "gate_window", "gate_sinks", "win_begin", "win_rows")]


class Index(Structure):
    _fields_ = [("col_nnz", c_void_p), ("col_offsets", c_void_p), ("order", c_void_p),
                ("row_indices", c_void_p), ("head_indices", c_void_p),
                ("slot_of_pair", c_void_p), ("capacity", c_int64),
                ("work_items", c_void_p), ("items_per_row", c_int32), ("chunk_tiles", c_int32)]


class Plan(Structure):
    _fields_ = [(n, c_int32) for n in (
        "gate_path", "fwd_path", "bwd_path", "fwd_tiles_in_flight", "fwd_q_stages", "bwd_kv_buffers",
        "bwd_gather_stages", "gate_slots", "gate_step", "transpose_chunk_rows", "transpose_chunks",
        "scatter_warps", "chunk_tiles", "work_items_per_row")]


_lib = None


def load():
    """Loads the shared library once; raises if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m moba_triton_b200.build` "
            "(there is no fallback path)")
    lib = ctypes.CDLL(LIB_PATH)
    P, I, vp = POINTER(Problem), POINTER(Index), c_void_p
    lib.moba_b200_abi_version.restype = c_int
    lib.moba_b200_last_error.restype = c_char_p
    lib.moba_b200_path_for.argtypes = [P, c_int]
    lib.moba_b200_transpose_scratch_bytes.argtypes = [P]
    lib.moba_b200_transpose_scratch_bytes.restype = c_size_t
    lib.moba_b200_pool.argtypes = [P, vp, vp, vp, vp]
    lib.moba_b200_gate.argtypes = [P, vp, vp, vp, vp, vp]
    lib.moba_b200_transpose.argtypes = [P, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp, c_size_t, vp]
    lib.moba_b200_transpose_noalloc.argtypes = [P, vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.moba_b200_launch_plan.argtypes = [P, POINTER(Plan)]
    lib.moba_b200_chunk_tiles.argtypes = [P]
    lib.moba_b200_work_items_per_row.argtypes = [P]
    lib.moba_b200_dkv_scratch_bytes.argtypes = [P]
    lib.moba_b200_dkv_scratch_bytes.restype = c_size_t
    lib.moba_b200_fwd.argtypes = [P, vp, vp, vp, I, vp, vp, vp, vp]
    lib.moba_b200_merge.argtypes = [P, vp, vp, vp, vp, vp]
    lib.moba_b200_bwd.argtypes = [P, vp, vp, vp, vp, vp, vp, vp, I, vp, vp, vp, vp, vp, vp, vp, vp]
    lib.moba_b200_pack_index.argtypes = [vp, c_int, c_int, c_int, vp, vp, vp, vp, vp]
    lib.moba_b200_pack_rows.argtypes = [vp, vp, vp, vp, c_int, c_int, c_size_t, vp]
    lib.moba_b200_unpack_rows.argtypes = [vp, vp, vp, c_int, c_int, c_size_t, vp]
    lib.moba_b200_seq_meta.argtypes = [vp, c_int, vp, vp]
    lib.moba_b200_device_status.argtypes = [POINTER(ctypes.c_uint), vp]
    lib.moba_b200_launch_count.restype = ctypes.c_longlong
    lib.moba_b200_profile_enable.argtypes = [c_int]
    lib.moba_b200_profile_read.argtypes = [ctypes.c_char_p, c_size_t]
    if lib.moba_b200_abi_version() != ABI_VERSION:
        raise RuntimeError("libmoba_b200.so was built from a different ABI version; rebuild it")
    _lib = lib
    return lib


def check(rc: int, what: str) -> None:
    """Maps a status code to the exception the reference raises for the same
    condition: ValueError for rejected arguments, RuntimeError otherwise."""
    if rc >= 0:
        return
    msg = load().moba_b200_last_error().decode()
    if rc in (-1, -2):
        raise ValueError(f"{what}: {msg}")
    raise RuntimeError(f"{what}: {msg}")


def call(name: str, device, what: str, *args) -> None:
    """Runs entry point `name` with `device` made current for the call (the library
    launches on the calling thread's current device) and that device's current
    stream appended as the last argument; raises on a failure status."""
    with torch.cuda.device(device):
        check(getattr(load(), name)(*args, stream_ptr(device)), what)


def device_status(device=None) -> int:
    """Synchronises the current stream of `device` (default: the current device) and
    returns (and clears) its error word: 0 when every tensor-core kernel ran to
    completion."""
    word = ctypes.c_uint(0)
    with torch.cuda.device(device):
        check(load().moba_b200_device_status(ctypes.byref(word), stream_ptr(device)), "device_status")
    return int(word.value)


def launch_count() -> int:
    """Kernels the library has launched so far in this process."""
    return int(load().moba_b200_launch_count())


def profile(on: bool) -> None:
    load().moba_b200_profile_enable(int(on))


def profile_read() -> dict:
    """{kernel name: (launches, total ms)} of the launches recorded while
    profiling was on; waits for them and clears the record."""
    lib = load()
    buf = ctypes.create_string_buffer(8192)
    lib.moba_b200_profile_read(buf, 8192)
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms = line.split()
        out[name] = (int(n), float(ms))
    return out


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return _DTYPE_CODE[dtype]
    except KeyError:
        raise ValueError(f"unsupported dtype {dtype}; the kernels take float32, bfloat16 or float16")


def ptr(t):
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr(device) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(device).cuda_stream)


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError(
                "moba_triton_b200 runs on CUDA tensors only; there is no CPU path "
                f"(got a tensor on {t.device})")


_force_path = [PATH_AUTO]
_chunk_tiles = [0]


def set_chunk_tiles(tiles: int) -> int:
    """Overrides the scheduling chunk size (work items of at most `tiles` 128-query tiles;
    0 = the library's policy) for indices built from now on; returns the previous setting.
    Meant for tests: a small value makes small problems take the split-column paths."""
    old = _chunk_tiles[0]
    _chunk_tiles[0] = int(tiles)
    return old


def set_kernel_path(path: int) -> int:
    """Selects the kernel family for later calls (PATH_AUTO / PATH_PORTABLE /
    PATH_TCGEN05); returns the previous setting. Meant for tests and benchmarks."""
    old = _force_path[0]
    _force_path[0] = path
    return old


def make_problem(q_shape, kv_heads: int, dtype: torch.dtype, cfg, cu_seqlens=None,
                 max_seqlen=None, causal: bool = True, part_f32: bool = False,
                 chunk_tiles=None, window=None) -> Problem:
    """The problem record of a call. `window` = (first query row, rows) restricts the call to
    those query rows of every batch row (see `moba_b200_problem.win_begin`)."""
    b, s, hq, d = q_shape
    packed = cu_seqlens is not None
    n_seq = cu_seqlens.numel() - 1 if packed else b
    longest = max_seqlen if packed else s
    nb = cfg.num_blocks(longest)
    return Problem(
        dtype=dtype_code(dtype), batch=b, tokens=s, n_seq=n_seq, max_seqlen=longest,
        q_heads=hq, kv_heads=kv_heads, head_dim=d, block_size=cfg.block_size, top_k=cfg.top_k,
        slots=cfg.slots_per_query, take=cfg.past_blocks_selected(nb),
        always_current=int(cfg.always_select_current), num_blocks=nb, causal=int(causal),
        packed=int(packed), path=_force_path[0], part_f32=int(part_f32),
        chunk_tiles=_chunk_tiles[0] if chunk_tiles is None else int(chunk_tiles),
        gate_window=int(getattr(cfg, "gate_window", None) or 0), gate_sinks=int(getattr(cfg, "gate_sinks", 0)),
        win_begin=0 if window is None else int(window[0]), win_rows=0 if window is None else int(window[1]))
