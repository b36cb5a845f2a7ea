"""Loader of the in-tree sm_100a extension (``_C.so``).

The library registers its kernels as ``torch.ops.b200.*``. CPU code paths never need it;
anything that touches a CUDA tensor does, and fails loudly if the library is absent instead
of falling back to eager PyTorch.
"""
from __future__ import annotations

import os
import threading

import torch

_LOCK = threading.Lock()
_LOADED = False
DEBUG = os.environ.get("B200_DEBUG", "") not in ("", "0")   # range-checked build of the same kernels
LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_C_debug.so" if DEBUG else "_C.so")

STATUS_NAMES = {
    0: "ok", 1: "wait_full_timeout", 2: "wait_empty_timeout", 3: "wait_tmem_full_timeout",
    4: "wait_tmem_empty_timeout", 5: "wait_flag_timeout", 6: "bad_argument", 7: "wait_attn_timeout",
    8: "bounds_violation",
}


class KernelStatusError(RuntimeError):
    """A kernel's bounded wait expired (or it rejected its arguments) and it exited early."""


def load(build_if_missing: bool = True) -> None:
    """Loads ``_C.so`` (building it first when absent and nvcc is available)."""
    global _LOADED
    if _LOADED:
        return
    with _LOCK:
        if _LOADED:
            return
        if not os.path.exists(LIB_PATH):
            if not build_if_missing:
                raise RuntimeError(f"{LIB_PATH} is missing; run `python -m jax_gpt_b200.build`")
            from . import build as _build
            _build.build(debug=DEBUG)
        torch.ops.load_library(LIB_PATH)
        _LOADED = True


def ops():
    """Returns the ``torch.ops.b200`` namespace, loading the library on first use."""
    load()
    return torch.ops.b200


def is_loaded() -> bool:
    return _LOADED


def check_status(device=None, reset: bool = True) -> None:
    """Synchronises ``device`` and raises :class:`KernelStatusError` if any kernel recorded an error."""
    load()
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    st = torch.ops.b200.status(idx)
    vals = st.cpu().tolist()
    if vals[0] != 0:
        if reset:
            st.zero_()
        raise KernelStatusError(
            f"kernel status {vals[0]} ({STATUS_NAMES.get(vals[0], '?')}), detail={vals[1:]} on {dev}")
