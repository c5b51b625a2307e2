"""ctypes binding of the in-tree sm_100a library (``_lib/libpithb200.so``).

The library has a plain C ABI (raw device pointers + a CUDA stream handle), so it is loaded with
ctypes rather than through torch's extension machinery: builds take seconds and the shared object
travels with the source tree. :func:`lib` raises if the library is missing, so a GPU run can never
silently fall back to eager PyTorch.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p, c_float
from functools import lru_cache
from pathlib import Path

import torch

# PITHTRAIN_CHECKED_LIB=1 loads the bounds-checking build (python -m pithtrain_b200.build --bounds-check): a
# diagnostic like a sanitizer run, slower, same entry points.
_LIB_PATH = Path(__file__).resolve().parent / "_lib" / (
    "libpithb200_checked.so" if __import__("os").environ.get("PITHTRAIN_CHECKED_LIB") == "1" else "libpithb200.so")


class NativeLibraryMissing(RuntimeError):
    pass


class KernelStatusError(RuntimeError):
    """A kernel reported a bounded-wait timeout or a capacity overflow through the status word."""


STATUS_NAMES = {
    1: "timeout in TMA producer",
    2: "timeout in MMA issuer",
    3: "timeout in epilogue",
    4: "timeout waiting for a peer",
    5: "receive-buffer capacity exceeded",
    6: "timeout draining in-flight copies",
    7: "dynamic shared memory not 1024-byte aligned",
    8: "index out of bounds (bounds-checking build)",
}


def available() -> bool:
    return _LIB_PATH.exists()


@lru_cache(maxsize=1)
def lib() -> ctypes.CDLL:
    if not _LIB_PATH.exists():
        raise NativeLibraryMissing(
            f"{_LIB_PATH} not found: run `python -m pithtrain_b200.build` (or __graft_entry__.build())"
        )
    L = ctypes.CDLL(str(_LIB_PATH))
    _declare(L)
    return L


SIGS = {
    "pt_status_fetch_and_clear": "",
    "pt_sm_count": "",
    "pt_set_peer_wait_limit_ns": "L",
    "pt_gemm_bf16": "PPPIIIIIILLLLLLLLPIILIIIIIIPILP",
    "pt_gemm_bf16_kgroup2": "PPPLPPPLPIILLLLIIP",
    "pt_merge_partial": "PPPIPPIIIILP",
    "pt_rmsnorm_fwd": "PPPPPPIIFIP",
    "pt_rmsnorm_bwd_grid": "I",
    "pt_rmsnorm_bwd": "PPPPPPPIIIP",
    "pt_colsum_accumulate": "PIIIPIP",
    "pt_qk_norm_rope_fwd": "PPPPPPPPPPIIIIILFIP",
    "pt_qk_norm_rope_bwd_grid": "",
    "pt_qk_norm_rope_bwd": "PPPPPPPPPPPPIIIIILIP",
    "pt_router_topk_fwd": "PIPPPIIIIIFP",
    "pt_router_topk_bwd": "PPPPPPIIIIIIFP",
    "pt_route_sort": "PPIIIPLPPPIP",
    "pt_route_sort_noalloc": "PIIIPPPIP",
    "pt_gather_rows": "PPIPPIILP",
    "pt_indexed_bias_add": "PPPIPPIIP",
    "pt_segment_sum": "PIPPIPIP",
    "pt_combine": "PPPPPPIIIP",
    "pt_swiglu_fwd": "PPPIIIFFP",
    "pt_swiglu_bwd": "PPPPPPPIIIFFPP",
    "pt_cross_entropy": "PPPIILIP",
    "pt_scale_bf16": "PPLP",
    "pt_sumsq_grid": "",
    "pt_sumsq": "PILPP",
    "pt_adamw": "PIPIPPLPFFFFFFFP",
    "pt_muon_momentum": "PIPIPLFPP",
    "pt_symm_malloc": "PL",
    "pt_symm_free": "P",
    "pt_ipc_export": "PP",
    "pt_ipc_import": "PP",
    "pt_ipc_close": "P",
    "pt_ipc_handle_size": "",
    "pt_can_access_peer": "II",
    "pt_symm_signal": "PIIIP",
    "pt_symm_wait": "PIIIP",
    "pt_symm_copy": "PPLIP",
    "pt_ep_chan_struct_size": "",
    "pt_ep_plan": "PIIIIIPPPPP",
    "pt_ep_push": "PIIPLPPPPPP",
    "pt_ep_receive": "PIIPPPPIP",
    "pt_ep_return": "PIIPPPPP",
    "pt_ep_wait_returned": "PIIP",
    "pt_ep_ack": "PIIP",
    "pt_axpby_bf16": "PPLFFP",
    "pt_fsdp_chan_struct_size": "",
    "pt_fsdp_ctl_bytes": "",
    "pt_fsdp_reduce_grid": "",
    "pt_fsdp_signal_ready": "PIP",
    "pt_fsdp_reduce_scatter": "PIFPP",
    "pt_fsdp_wait_acks": "PIP",
    "pt_fsdp_push_params": "PIP",
    "pt_fsdp_wait_params": "PIP",
    "pt_quant_rows": "PLPIPIIPPLP",
    "pt_quant_blocks": "PIIIPPPPP",
    "pt_gemm_fp8": "PPPIIIILLLLPLPPIIIIP",
    "pt_attn_fwd": "PPPPPPP" + "IIIIIII" + "LLLL" + "F" + "II" + "P",
    "pt_attn_bwd": "PPPPPPPPPPPPPPP" + "IIIIII" + "LLLLL" + "F" + "II" + "P",
    "pt_gemm2cta_nt": "PPPIIILLLP",
    "pt_gdr_state_fwd": "PPPPPPPPIIIIP",
    "pt_gdr_state_bwd": "PPPPPPPPPPPPPIIIIP",
}

_CT = {"P": c_void_p, "I": c_int, "L": c_longlong, "F": c_float}


def _declare(L: ctypes.CDLL) -> None:
    for name, args in SIGS.items():
        if hasattr(L, name):
            fn = getattr(L, name)
            fn.argtypes = [_CT[a] for a in args]
            fn.restype = c_int


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


# Number of kernel launches issued through this module since it was last reset (bench bookkeeping).
LAUNCHES = 0
_LAUNCHES_PER_CALL = {"pt_route_sort": 4, "pt_attn_bwd": 5, "pt_merge_partial": 2}


def check(rc: int, what: str) -> None:
    global LAUNCHES
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
    LAUNCHES += _LAUNCHES_PER_CALL.get(what, 1)


def set_peer_wait_limit(seconds: float) -> None:
    """Limit of every in-kernel wait on another GPU's flag (current device). Bounded waits that run out set the status
    word, which the train step reads once per step; the default of 2 s suits tests, production jobs pass a longer one
    through ``DistributedCfg.peer_wait_timeout``."""
    rc = lib().pt_set_peer_wait_limit_ns(int(seconds * 1e9))
    if rc != 0:
        raise RuntimeError(f"pt_set_peer_wait_limit_ns failed with code {rc}")


def fetch_status() -> int:
    """Synchronise, read and clear the status word; returns the code (0 = no kernel reported anything)."""
    v = lib().pt_status_fetch_and_clear()
    if v < 0:
        raise RuntimeError(f"status word unavailable ({v})")
    return v


def check_status() -> None:
    """Synchronise and raise if any kernel recorded a timeout / overflow since the last check."""
    v = lib().pt_status_fetch_and_clear()
    if v > 0:
        raise KernelStatusError(STATUS_NAMES.get(v, f"status {v}"))
    if v < 0:
        raise RuntimeError(f"status word unavailable ({v})")
