"""ctypes binding of libfftopk.so (declarations: include/fftopk.h).

There is no CPU or PyTorch fallback: if the library cannot be loaded the op raises.
"""
from __future__ import annotations

import ctypes
import functools
import importlib.util
from pathlib import Path

import os

_PKG_ROOT = Path(__file__).resolve().parent.parent
#: the library next to the package, or another build of it named by FFTOPK_LIBRARY
LIB_PATH = Path(os.environ["FFTOPK_LIBRARY"]) if os.environ.get("FFTOPK_LIBRARY") else _PKG_ROOT / "lib" / "libfftopk.so"

K = 2048

ST_STAGE_TIMEOUT = 1
ST_INTERNAL = 2
ST_PEER_TIMEOUT = 4
ST_GUESS_MISSED = 8
ST_CHECK = 16

E_RANGE = -4

#: every symbol include/fftopk.h declares
EXPORTS = (
    "fftopk_version",
    "fftopk_strerror",
    "fftopk_last_cuda_error",
    "fftopk_select2048",
    "fftopk_select_topk",
    "fftopk_select2048_warm",
    "fftopk_widen_workspace_bytes",
    "fftopk_select_topk_16bit",
    "fftopk_select2048_page_table",
    "fftopk_select2048_ragged",
    "fftopk_merge2048",
    "fftopk_comm_bytes",
    "fftopk_comm_create",
    "fftopk_comm_open",
    "fftopk_comm_close",
    "fftopk_comm_destroy",
    "fftopk_select2048_cp",
    "fftopk_merge2048_cp",
    "fftopk_topk2048_cp",
    "fftopk_topk2048_sliced_noalloc",
    "fftopk_host_workspace_bytes",
    "fftopk_select2048_host",
    "fftopk_indexer_workspace_bytes",
    "fftopk_indexer_topk2048",
    "fftopk_indexer_topk2048_fp8",
    "fftopk_probe_read_bandwidth",
    "fftopk_key_of",
    "fftopk_plan",
    "fftopk_set_tuning",
    "fftopk_set_overlap",
)


class FFTopkError(RuntimeError):
    pass


def _build_if_needed() -> None:
    spec = importlib.util.spec_from_file_location("_fftopk_build", _PKG_ROOT / "build.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    if mod.is_stale():
        if mod.find_nvcc() is None:
            if LIB_PATH.exists():
                return  # prebuilt library, no compiler on this machine: use it
            raise FFTopkError(
                f"{LIB_PATH} is missing and nvcc was not found; build it with "
                f"`python {_PKG_ROOT / 'build.py'}` on a machine with the CUDA toolkit")
        mod.build_library()


@functools.cache
def lib() -> ctypes.CDLL:
    """Load (building first if the sources are newer) the native library."""
    if not os.environ.get("FFTOPK_LIBRARY"):
        _build_if_needed()
    try:
        L = ctypes.CDLL(str(LIB_PATH))
    except OSError as e:  # pragma: no cover - depends on the machine
        raise FFTopkError(f"cannot load {LIB_PATH}: {e}") from e
    c = ctypes
    L.fftopk_version.restype = c.c_int
    L.fftopk_version.argtypes = []
    L.fftopk_strerror.restype = c.c_char_p
    L.fftopk_strerror.argtypes = [c.c_int]
    L.fftopk_last_cuda_error.restype = c.c_int
    L.fftopk_last_cuda_error.argtypes = []
    L.fftopk_select2048.restype = c.c_int
    L.fftopk_select2048.argtypes = [
        c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_void_p,
        c.c_void_p, c.c_void_p, c.c_int32, c.c_void_p, c.c_void_p]
    L.fftopk_select2048_warm.restype = c.c_int
    L.fftopk_select2048_warm.argtypes = [c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_void_p, c.c_void_p,
                                         c.c_uint32, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p]
    L.fftopk_select2048_page_table.restype = c.c_int
    L.fftopk_select2048_page_table.argtypes = [
        c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_int64,
        c.c_void_p, c.c_int32, c.c_void_p, c.c_void_p]
    L.fftopk_select2048_ragged.restype = c.c_int
    L.fftopk_select2048_ragged.argtypes = [
        c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p,
        c.c_void_p]
    L.fftopk_merge2048.restype = c.c_int
    L.fftopk_merge2048.argtypes = [
        c.c_void_p, c.c_void_p, c.c_int64, c.c_int32, c.c_int32, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p]
    L.fftopk_comm_bytes.restype = c.c_int
    L.fftopk_comm_bytes.argtypes = [c.c_int32, c.POINTER(c.c_size_t)]
    L.fftopk_comm_create.restype = c.c_int
    L.fftopk_comm_create.argtypes = [c.c_int32, c.POINTER(c.c_void_p), c.c_char_p]
    L.fftopk_comm_open.restype = c.c_int
    L.fftopk_comm_open.argtypes = [c.c_char_p, c.POINTER(c.c_void_p)]
    L.fftopk_comm_close.restype = c.c_int
    L.fftopk_comm_close.argtypes = [c.c_void_p]
    L.fftopk_comm_destroy.restype = c.c_int
    L.fftopk_comm_destroy.argtypes = [c.c_void_p]
    L.fftopk_select2048_cp.restype = c.c_int
    L.fftopk_select2048_cp.argtypes = [c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_int32,
                                       c.c_void_p, c.c_int32, c.c_uint32, c.c_void_p, c.c_void_p]
    L.fftopk_merge2048_cp.restype = c.c_int
    L.fftopk_merge2048_cp.argtypes = [c.POINTER(c.c_void_p), c.c_int32, c.c_int32, c.c_int32, c.c_int32, c.c_uint32,
                                      c.c_int32, c.c_void_p, c.c_void_p, c.c_void_p, c.c_void_p]
    L.fftopk_topk2048_cp.restype = c.c_int
    L.fftopk_topk2048_cp.argtypes = [c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_int32,
                                     c.POINTER(c.c_void_p), c.c_int32, c.c_int32, c.c_int32, c.c_uint32, c.c_int32,
                                     c.c_void_p, c.c_void_p, c.c_void_p]
    L.fftopk_topk2048_sliced_noalloc.restype = c.c_int
    L.fftopk_topk2048_sliced_noalloc.argtypes = [c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_int32,
                                                 c.c_void_p, c.c_void_p, c.c_void_p]
    L.fftopk_select_topk.restype = c.c_int
    L.fftopk_select_topk.argtypes = [c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_void_p, c.c_int32,
                                     c.c_void_p, c.c_void_p, c.c_int32, c.c_void_p, c.c_void_p]
    L.fftopk_widen_workspace_bytes.restype = c.c_size_t
    L.fftopk_widen_workspace_bytes.argtypes = [c.c_int32, c.c_int64]
    L.fftopk_select_topk_16bit.restype = c.c_int
    L.fftopk_select_topk_16bit.argtypes = [c.c_void_p, c.c_int32, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_void_p,
                                           c.c_int32, c.c_void_p, c.c_void_p, c.c_size_t, c.c_void_p, c.c_void_p]
    L.fftopk_host_workspace_bytes.restype = c.c_size_t
    L.fftopk_host_workspace_bytes.argtypes = [c.c_int32, c.c_int64]
    L.fftopk_select2048_host.restype = c.c_int
    L.fftopk_select2048_host.argtypes = [c.c_void_p, c.c_int64, c.c_int32, c.c_int64, c.c_void_p, c.c_void_p,
                                         c.c_void_p, c.c_size_t, c.c_void_p, c.c_void_p]
    L.fftopk_indexer_workspace_bytes.restype = c.c_size_t
    L.fftopk_indexer_workspace_bytes.argtypes = [c.c_int32]
    L.fftopk_indexer_topk2048.restype = c.c_int
    L.fftopk_indexer_topk2048.argtypes = [c.c_void_p, c.c_void_p, c.c_int64, c.c_void_p, c.c_int32, c.c_int64, c.c_void_p,
                                          c.c_void_p, c.c_uint32, c.c_void_p, c.c_int64, c.c_void_p, c.c_void_p, c.c_size_t,
                                          c.c_void_p, c.c_void_p]
    L.fftopk_indexer_topk2048_fp8.restype = c.c_int
    L.fftopk_indexer_topk2048_fp8.argtypes = [c.c_void_p, c.c_void_p, c.c_int64, c.c_void_p, c.c_int64, c.c_void_p, c.c_int32,
                                              c.c_int64, c.c_void_p, c.c_void_p, c.c_uint32, c.c_void_p, c.c_int64,
                                              c.c_void_p, c.c_void_p, c.c_size_t, c.c_void_p, c.c_void_p]
    L.fftopk_probe_read_bandwidth.restype = c.c_int
    L.fftopk_probe_read_bandwidth.argtypes = [c.c_void_p, c.c_size_t, c.c_size_t, c.c_void_p, c.POINTER(c.c_size_t),
                                              c.c_void_p]
    L.fftopk_key_of.restype = c.c_uint32
    L.fftopk_key_of.argtypes = [c.c_float]
    L.fftopk_plan.restype = c.c_int
    L.fftopk_plan.argtypes = [c.c_int32, c.c_int64, c.POINTER(c.c_int32)]
    L.fftopk_set_tuning.restype = c.c_int
    L.fftopk_set_tuning.argtypes = [c.c_int32, c.c_int32, c.c_int32, c.c_int32, c.c_int32]
    L.fftopk_set_overlap.restype = c.c_int
    L.fftopk_set_overlap.argtypes = [c.c_int32]
    return L


def check(rc: int, what: str) -> None:
    if rc != 0:
        L = lib()
        msg = L.fftopk_strerror(rc).decode()
        if rc == -2:
            msg += f" (cudaError {L.fftopk_last_cuda_error()})"
        raise FFTopkError(f"{what}: {msg}")


def plan(B: int, L: int) -> dict:
    """Launch plan fftopk_select2048 would use for (B, L) on the current device."""
    arr = (ctypes.c_int32 * 6)()
    check(lib().fftopk_plan(B, L, arr), "fftopk_plan")
    keys = ("cluster_ctas", "threads", "smem_bytes", "list_cap", "cand_cap", "sm_count")
    return dict(zip(keys, list(arr)))


def set_tuning(cluster_ctas: int = -1, threads: int = -1, list_cap: int = -1, cand_cap: int = -1,
               force_full_histogram: bool = False) -> None:
    check(lib().fftopk_set_tuning(cluster_ctas, threads, list_cap, cand_cap, int(force_full_histogram)),
          "fftopk_set_tuning")


def set_overlap(enable: bool) -> None:
    """Allow back-to-back selection calls on a stream to overlap (see include/fftopk.h)."""
    check(lib().fftopk_set_overlap(int(bool(enable))), "fftopk_set_overlap")
