"""The matrix product y = h @ W^T that every projection uses, chosen by dtype and row count.

* float32 run: the package's own FMA kernel (``csrc/gemm_f32.cu``); no tensor-core mode, and every
  output element sums over k in one fixed order whatever the number of rows.
* bfloat16 run, up to 32 rows (decode steps): the package's weight-streaming tensor-core kernel
  (``csrc/gemm_skinny.cu``), with the residual add or the float32 store in its epilogue.
* bfloat16 run, 128 rows or more: the package's tcgen05/TMA kernel (``csrc/gemm_tc.cu``: operands by TMA into
  swizzled shared memory, accumulation in tensor memory, the same epilogues).
* bfloat16 run, between those, or an inner dimension that is no multiple of 8 (TMA needs 16-byte rows): a library
  product (cuBLAS through ``torch.mm``, float32 accumulation), as the reference's ``nn.Linear`` always is
  (sleuth/forge/model/attention.py:106-108). The thresholds and what they were measured on stand below.

``into`` adds the product to a float32 tensor (the residual stream) instead of returning it.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Normed


import os

# Which kernel multiplies how many rows (bfloat16), as measured on a B200 with the Qwen3-0.6B shapes:
#   up to SKINNY_ROWS rows   the weight-streaming kernel (equal to the library at 32 rows, behind it at 64)
#   from TC_ROWS rows on     this package's tcgen05 kernel (level with the library at 2,048 rows product by product,
#                            ahead with its fused epilogues: a 128-token prompt takes 2.4 ms against 3.6 ms, a
#                            1,024-token one 3.2 ms either way)
#   between                  the library product (cuBLAS through torch.mm): fewer than 128 rows leave most of the
#                            tcgen05 kernel's 128-row tiles empty
# SLEUTH_B200_GEMM=own sends everything the own kernels take to them, =library everything above SKINNY_ROWS to cuBLAS.
_CHOICE = os.environ.get("SLEUTH_B200_GEMM", "auto")
USE_TC = _CHOICE != "library"
SKINNY_ROWS = 64 if _CHOICE == "own" else 32
TC_ROWS = 1 if _CHOICE == "own" else 128


# The norm fused into the weight-streaming kernel pays as long as normalising all rows again in every block is short
# beside the block's weight stream: measured against the norm kernel plus the plain product (us, q/k/v shapes):
#   K 1,024: 1 row 3.5 / 4.1, 8 rows 4.2 / 5.0, 16 rows 5.7 / 5.3    K 2,048: 1 row 6.4 / 6.8, 8 rows 7.3 / 7.1
#   K 2,560: 1 row 12.7 / 11.7, 8 rows 14.6 / 12.5                    K 4,096: 1 row 18.7 / 15.1, 8 rows 22.1 / 16.7
# Inside a step the fused form saves a kernel boundary on top of that: at K 2,048 with 8 rows the step is 4 % faster
# with it (1.660 against 1.726 ms), at K 4,096 6 % slower (1.626 against 1.528 ms with one row).
NORM_FUSE_MAX_K = 2048
NORM_FUSE_MAX_ELEMENTS = 16384


def use_skinny(M: int, N: int, K: int, norm: bool = False) -> bool:
    if norm and (K > NORM_FUSE_MAX_K or M * K > NORM_FUSE_MAX_ELEMENTS):
        return False
    return M <= SKINNY_ROWS and ops.skinny_supported(M, N, K, norm)


def use_tc(M: int, N: int, K: int) -> bool:
    return USE_TC and M >= TC_ROWS and ops.tc_supported(M, N, K)

# How many output features a block of the weight-streaming kernel takes (8, 16 or 32) decides how many blocks there
# are and how many fit an SM; which is fastest depends on the matrix (measured on a B200, 16 rows: a 2,560 x 9,728
# down projection 19.1 us with 8, 15.9 us with 16; a gated 9,728 x 2,560 product 26.1 us with 16, 22.3 us with 8; the
# 0.6B shapes are fastest with the launcher's own rule). So the first time a shape is met outside a graph recording,
# the choices are timed on it (cold: the L2 cache is swept between runs) and the fastest is kept for the process.
# The choice changes which block computes which feature, never a sum's order: results are the same bits for all.
_FEATURES: dict = {}
TUNE = os.environ.get("SLEUTH_B200_TUNE", "1") != "0"


def _bucket(M: int) -> int:
    return 1 if M <= 1 else (8 if M <= 8 else 16)


def tuned_features(kind: str, M: int, N: int, K: int, launch) -> int:
    """The features-per-block choice for this product; ``launch(features)`` runs it once on the current stream."""
    if M > 16 or not TUNE:
        return 0
    key = (kind, _bucket(M), N, K)
    best = _FEATURES.get(key)
    if best is not None:
        return best
    if torch.cuda.is_current_stream_capturing():
        return 0            # timed another time; the rule serves meanwhile
    candidates = [0, 8, 16] + ([32] if kind != "swiglu" and N >= 1024 else [])
    device = torch.cuda.current_device()
    sweep = torch.empty(160 << 20, dtype=torch.uint8, device=f"cuda:{device}")        # larger than the L2 cache
    times = {}
    for f in candidates:
        launch(f)
        t = []
        for _ in range(3):
            sweep.zero_()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            launch(f)
            b.record()
            b.synchronize()
            t.append(a.elapsed_time(b))
        times[f] = min(t)
    del sweep
    # the rule's own choice stays unless something else is clearly faster (3 %: timing noise must not flip it)
    best = 0
    for f in candidates[1:]:
        if times[f] < 0.97 * times[best]:
            best = f
    _FEATURES[key] = best
    return best


_MODE: dict = {}


def _accumulate_mode(device) -> str:
    """How the bfloat16 library product adds into the float32 stream on this torch build, found once
    per device by running each form on a 8x8 case: "addmm" (one call, float32 output and addend),
    "mm32" (float32 output, then the add kernel) or "mm16" (bfloat16 output, then the add kernel)."""
    key = str(device)
    if key not in _MODE:
        a = torch.ones((8, 8), dtype=torch.bfloat16, device=device)
        c = torch.zeros((8, 8), dtype=torch.float32, device=device)
        mode = "mm16"
        try:
            torch.addmm(c, a, a.t(), out_dtype=torch.float32, out=c)
            if float(c[0, 0]) == 8.0:
                mode = "addmm"
        except (RuntimeError, TypeError):
            try:
                torch.mm(a, a.t(), out_dtype=torch.float32, out=c)
                mode = "mm32"
            except (RuntimeError, TypeError):
                pass
        _MODE[key] = mode
    return _MODE[key]


class Linear:
    def __init__(self, weight: torch.Tensor, dtype: torch.dtype):
        """weight [out, in]: float32 for the 32-bit run, bfloat16 otherwise."""
        if weight.dtype != dtype:
            weight = weight.to(dtype)
        self.weight = weight.contiguous()
        self.dtype = dtype
        self.out_features, self.in_features = self.weight.shape
        self._wt = self.weight.t()      # a view; the library product reads W^T without a copy

    def forward(self, h: torch.Tensor, out: torch.Tensor | None = None, into: torch.Tensor | None = None,
                ws=None, stream=None, out_dtype: torch.dtype | None = None, next_read: torch.Tensor | None = None,
                next_pages=None):
        """``next_read``: the weight matrix of the product that follows this one; the weight-streaming kernel asks
        the L2 cache for it while it runs (the other kernels ignore it). ``next_pages``: the same for the cache pages
        that a single-token attention kernel right behind this product reads first (``ops.next_pages``)."""
        M = h.shape[0]
        if isinstance(h, Normed):
            if (self.dtype == torch.bfloat16 and h.gain is not None and into is None
                    and use_skinny(M, self.out_features, self.in_features, norm=True)):
                want = out_dtype or (out.dtype if out is not None else self.dtype)
                if out is None:
                    out = ws.take((M, self.out_features), want)
                mode = "f32" if want == torch.float32 else "bf16"
                f = tuned_features("norm-" + mode, M, self.out_features, self.in_features,
                                   lambda f: ops.gemm_skinny_norm(h.x, h.gain, h.eps, self.weight, out, mode, stream, features=f))
                ops.gemm_skinny_norm(h.x, h.gain, h.eps, self.weight, out, mode, stream, next_read, next_pages, features=f)
                return out
            h = h.tensor()
        if self.dtype == torch.float32:
            if into is not None:
                ops.gemm_f32(h, self.weight, into, accumulate=True, stream=stream)
                return into
            if out is None:
                out = ws.take((M, self.out_features), torch.float32)
            ops.gemm_f32(h, self.weight, out, stream=stream)
            return out
        if use_skinny(M, self.out_features, self.in_features):
            if into is not None:
                # (timing runs add into a scratch copy of the stream's shape, not into the stream)
                f = tuned_features("add", M, self.out_features, self.in_features,
                                   lambda f: ops.gemm_skinny(h, self.weight, torch.empty_like(into), "add", stream, features=f))
                ops.gemm_skinny(h, self.weight, into, "add", stream, next_read, features=f)
                return into
            want = out_dtype or (out.dtype if out is not None else self.dtype)
            if out is None:
                out = ws.take((M, self.out_features), want)
            mode = "f32" if want == torch.float32 else "bf16"
            f = tuned_features(mode, M, self.out_features, self.in_features,
                               lambda f: ops.gemm_skinny(h, self.weight, out, mode, stream, features=f))
            ops.gemm_skinny(h, self.weight, out, mode, stream, next_read, next_pages, features=f)
            return out
        if use_tc(M, self.out_features, self.in_features):
            if into is not None:
                ops.gemm_tc(h, self.weight, into, "add", stream)
                return into
            want = out_dtype or (out.dtype if out is not None else self.dtype)
            if out is None:
                out = ws.take((M, self.out_features), want)
            ops.gemm_tc(h, self.weight, out, "f32" if want == torch.float32 else "bf16", stream)
            return out
        if into is not None:
            mode = _accumulate_mode(h.device)
            if mode == "addmm":
                torch.addmm(into, h, self._wt, out_dtype=torch.float32, out=into)
            else:
                mark = ws.mark()
                tmp = ws.take((M, self.out_features), torch.float32 if mode == "mm32" else self.dtype)
                if mode == "mm32":
                    torch.mm(h, self._wt, out_dtype=torch.float32, out=tmp)
                else:
                    torch.mm(h, self._wt, out=tmp)
                ops.add(into, tmp, stream=stream)
                ws.release(mark)
            return into
        want = out_dtype or (out.dtype if out is not None else self.dtype)
        if out is None:
            out = ws.take((M, self.out_features), want)
        if want == self.dtype:
            torch.mm(h, self._wt, out=out)
        else:
            torch.mm(h, self._wt, out_dtype=want, out=out)
        return out
