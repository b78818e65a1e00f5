"""Reads the timeline that a library built with ``-DSLB_TIMELINE`` records (``csrc/common.cuh``: one record
per block with the time it entered, up to three marks, and the time it left, in nanoseconds of the GPU's
global timer). The ordinary build records nothing and ``start`` says so.

    SLEUTH_B200_NVCC_FLAGS=-DSLB_TIMELINE SLEUTH_B200_BUILD_DIR=/tmp/slb_timeline python my_script.py

    from sleuth_b200.kernels import timeline
    timeline.start(1 << 20); ...run steps...; records = timeline.read()
"""

from __future__ import annotations

import torch

from . import library

FILES = ("gemm_skinny", "attention_flash", "elementwise", "sampling")
KINDS = {1: "embed", 2: "rmsnorm", 3: "gemm_skinny", 4: "attention_decode", 5: "argmax_partial", 6: "argmax_final",
         7: "sample", 8: "other"}
_buffer = None


def start(records: int = 1 << 20, device="cuda:0") -> None:
    """Give every instrumented file a fresh buffer for ``records`` records."""
    global _buffer
    lib = library.load()
    _buffer = torch.zeros(1 + 6 * records, dtype=torch.int64, device=device)
    for f in FILES:
        try:
            fn = getattr(lib.dll, f"slb_timeline_set_{f}")
        except AttributeError:
            raise RuntimeError("this build of the kernel library records no timeline: build one with "
                               "SLEUTH_B200_NVCC_FLAGS=-DSLB_TIMELINE (and SLEUTH_B200_BUILD_DIR set to a folder of its own)") from None
        fn.argtypes = [library.P, library.ctypes.c_uint]
        fn.restype = library.ctypes.c_int
        if fn(_buffer.data_ptr(), records) != 0:
            raise RuntimeError(f"could not hand the timeline buffer to {f}")


def read() -> list[dict]:
    """The records so far, sorted by the time their block entered: ``kind, block, sm, enter, marks (3), leave``."""
    torch.cuda.synchronize()
    host = _buffer.cpu()
    n = min(int(host[0]) & 0xFFFFFFFF, (host.numel() - 1) // 6)
    out = []
    for r in host[1:1 + 6 * n].view(n, 6).tolist():
        head = r[0] & 0xFFFFFFFFFFFFFFFF
        out.append({"kind": KINDS.get(head & 0xFFFF, "?"), "block": (head >> 16) & 0xFFFFFFFF, "sm": head >> 48,
                    "enter": r[1], "marks": r[2:5], "leave": r[5]})
    out.sort(key=lambda d: d["enter"])
    return out


def clear() -> None:
    _buffer[0] = 0
