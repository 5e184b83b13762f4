"""ctypes binding of libb2g.so (the C ABI declared in include/b2g.h)."""
from __future__ import annotations

import ctypes as C
import os
import threading
from pathlib import Path

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE.parent / "csrc" / "libb2g.so"

_vp, _i32, _i64, _f32 = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> (restype, argtypes); mirrors include/b2g.h one to one
SIGNATURES = {
    "b2g_last_error": (C.c_char_p, []),
    "b2g_abi_version": (_i32, []),
    "b2g_set_iq2xxs_grid": (_i32, [_vp]),
    "b2g_set_iq2s_grid": (_i32, [_vp]),
    "b2g_dequant": (_i32, [_i32, _vp, _i64, _i64, _vp, _vp]),
    "b2g_qlinear_fwd": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "b2g_debug_stalled_qlinear_fwd": (_i32, [_i32, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp, _vp]),
    "b2g_qlinear_dgrad": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "b2g_fixed_grouped_fwd": (_i32, [_i32, _vp, _vp, _vp, _i64, _i32, _i64, _i64, _vp, _vp]),
    "b2g_fixed_grouped_dgrad": (_i32, [_i32, _vp, _vp, _vp, _i64, _i32, _i64, _i64, _vp, _vp]),
    "b2g_cross_entropy_inplace": (_i32, [_vp, _i64, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _vp, _i32, _vp, _vp]),
    "b2g_lora_down": (_i32, [_vp, _vp, _i32, _f32, _vp, _vp, _i64, _i64, _i32, _vp]),
    "b2g_lora_wgrad_workspace_bytes": (_i64, [_i64, _i64]),
    "b2g_lora_wgrad": (_i32, [_vp, _vp, _f32, _vp, _i32, _vp, _i64, _i64, _i64, _i32, _vp]),
    "b2g_lora_wgrad_static_max_bytes": (_i64, []),
    "b2g_lora_wgrad_static": (_i32, [_vp, _vp, _f32, _vp, _i32, _i64, _i64, _i32, _vp]),
    "b2g_router_topk": (_i32, [_vp, _i32, _vp, _i32, _vp, _i64, _i32, _i32, _vp]),
    "b2g_route_plan_workspace_bytes": (_i64, [_i64, _i32]),
    "b2g_route_plan": (_i32, [_vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "b2g_route_gather": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "b2g_route_gather_bwd": (_i32, [_vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "b2g_route_combine": (_i32, [_vp, _vp, _i32, _vp, _vp, _i64, _i32, _i32, _vp]),
    "b2g_route_combine_bwd": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _i64, _i32, _i32, _vp]),
    "b2g_grouped_tiles_bytes": (_i64, [_i64, _i32]),
    "b2g_grouped_schedule": (_i32, [_vp, _vp, _vp, _i32, _i64, _vp, _vp, _vp]),
    "b2g_grouped_fwd": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _i64, _i32, _vp, _vp]),
    "b2g_grouped_dgrad": (_i32, [_i32, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _i64, _i64, _i32, _vp, _vp]),
    "b2g_grouped_lora_down": (_i32, [_vp, _vp, _vp, _i32, _f32, _vp, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b2g_grouped_lora_wgrad": (_i32, [_vp, _vp, _f32, _vp, _vp, _vp, _i32, _i64, _i64, _i32, _i32, _i64, _i64, _vp]),
    "b2g_grouped_lora_up": (_i32, [_vp, _i64, _vp, _i32, _vp, _vp, _i64, _i64, _i32, _i32, _vp]),
    "b2g_ep_scatter_rows": (_i32, [_vp, _vp, _i32, _vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i32, _i64, _i32, _i64, _i32, _vp, _vp]),
    "b2g_ep_return_rows": (_i32, [_vp, _vp, _vp, _vp, _i32, _i32, _i32, _i32, _i64, _i32, _vp]),
    "b2g_set_gemm_sm_margin": (_i32, [_i32]),
    "b2g_ep_peer_plan": (_i32, [_vp, _i64, _i32, _i32, _i32, _vp, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp]),
    "b2g_swiglu_fwd": (_i32, [_vp, _vp, _vp, _i64, _f32, _vp, _vp, _i64, _vp]),
    "b2g_swiglu_bwd": (_i32, [_vp, _vp, _vp, _vp, _vp, _i64, _f32, _vp, _vp, _i64, _vp]),
}

_lib = None
_lock = threading.Lock()


class B2GError(RuntimeError):
    """A libb2g call returned an error code."""


def load() -> C.CDLL:
    """Load the library once.  Raises (never falls back) when it has not been built."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = Path(os.environ.get("B2G_LIB", LIB_PATH))
                if not path.exists():
                    raise B2GError(
                        f"{path} is missing: build it with `python {LIB_PATH.parent / 'build.py'}`. "
                        "This package has no CPU or PyTorch fallback."
                    )
                lib = C.CDLL(str(path))
                for name, (res, args) in SIGNATURES.items():
                    fn = getattr(lib, name)
                    fn.restype, fn.argtypes = res, args
                _lib = lib
    return _lib


# Kernels launched by one call of each entry point (the benchmark reports the total it issued).
KERNELS_PER_CALL = {
    "b2g_dequant": 1, "b2g_qlinear_fwd": 1, "b2g_qlinear_dgrad": 1, "b2g_lora_down": 1, "b2g_lora_wgrad": 2, "b2g_lora_wgrad_static": 2,
    "b2g_router_topk": 1, "b2g_route_plan": 4, "b2g_route_gather": 1, "b2g_route_gather_bwd": 1, "b2g_route_combine": 1,
    "b2g_route_combine_bwd": 1, "b2g_grouped_schedule": 1, "b2g_grouped_fwd": 1, "b2g_grouped_dgrad": 1,
    "b2g_grouped_lora_down": 1, "b2g_grouped_lora_wgrad": 1, "b2g_grouped_lora_up": 1, "b2g_ep_scatter_rows": 1, "b2g_ep_return_rows": 1, "b2g_ep_peer_plan": 1, "b2g_swiglu_fwd": 1, "b2g_swiglu_bwd": 1,
    "b2g_cross_entropy_inplace": 1, "b2g_fixed_grouped_fwd": 8, "b2g_fixed_grouped_dgrad": 8,      # one launch per group (eight in the DeepSeek layout)
}
COUNT_LAUNCHES = False
LAUNCHES = 0
TIMED: set = set()      # entry points to bracket with CUDA events on the launching stream
EVENTS: list = []       # (name, (int args...), start_event, end_event)


def call(name: str, *args):
    """Invoke an int-returning entry point; raise B2GError with the library's message on failure."""
    global LAUNCHES
    lib = load()
    if COUNT_LAUNCHES:
        LAUNCHES += KERNELS_PER_CALL.get(name, 0)
    if name in TIMED:
        import torch

        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = getattr(lib, name)(*args)
        b.record()
        EVENTS.append((name, tuple(v for v in args if isinstance(v, int))[-3:], a, b))
    else:
        rc = getattr(lib, name)(*args)
    if rc != 0:
        msg = lib.b2g_last_error().decode("utf-8", "replace")
        kind = ValueError if rc == -1 else B2GError
        raise kind(f"{name}: {msg} (code {rc})")


def query(name: str, *args) -> int:
    return int(getattr(load(), name)(*args))
