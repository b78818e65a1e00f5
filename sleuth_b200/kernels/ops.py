"""Thin, checked Python fronts of the CUDA launchers.

Every function takes CUDA tensors, checks device, dtype, contiguity and the sizes that tie the
arguments together, and launches on the stream it is given (an integer handle, the current torch
stream by default). Nothing here computes with torch operations, with one exception that the
architecture's own engine makes too: the bfloat16 matrix product of more rows than the skinny
kernel takes is a library product (cuBLAS through ``torch.mm``), as the reference's ``nn.Linear``
is (sleuth/forge/model/attention.py:106-108,157; mlp.py:38-41; transformer.py:302).
"""

from __future__ import annotations

import ctypes
import os

import torch

from . import library

DT = {torch.float32: 0, torch.bfloat16: 1}


def lib() -> library.KernelLibrary:
    return library.load()


def current_stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def _cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            _need(t.is_cuda, "the kernels of sleuth_b200 run on CUDA tensors only")
            _need(False, f"tensor of shape {tuple(t.shape)} must be contiguous")


def embed(ids: torch.Tensor, table: torch.Tensor, x: torch.Tensor, scale: float = 1.0, stream=None,
          ids_map: torch.Tensor | None = None) -> None:
    """x[t] = table[ids[t]] * scale, or table[ids[ids_map[t]]] with a map. Ids outside the table are clamped
    (the caller checks host ids; ids that a sampler left on the device lie inside by construction)."""
    _cuda(ids, table, x, ids_map)
    T, d = x.shape
    _need(ids.dtype == torch.int32 and (ids_map is not None or ids.numel() >= T), "embed: ids must be int32, one per row of x")
    _need(ids_map is None or (ids_map.dtype == torch.int32 and ids_map.numel() >= T), "embed: the map is int32, one per row")
    _need(table.shape[1] == d and x.dtype == torch.float32 and table.dtype in DT, "embed: shapes or dtypes disagree")
    lib().call("slb_embed", _p(ids), _p(ids_map), _p(table), DT[table.dtype], _p(x), T, d, table.shape[0], float(scale),
               stream if stream is not None else current_stream())


def rmsnorm(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, eps: float, rows: torch.Tensor | None = None,
            stream=None) -> None:
    _cuda(x, w, out, rows)
    R, d = out.shape
    _need(x.dtype == torch.float32 and w.dtype == torch.float32 and out.dtype in DT, "rmsnorm: dtypes")
    _need(x.shape[1] == d and w.numel() == d, "rmsnorm: widths disagree")
    if rows is None:
        _need(x.shape[0] >= R, "rmsnorm: fewer input rows than output rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() >= R, "rmsnorm: rows must be int32, one per output row")
    lib().call("slb_rmsnorm", _p(x), _p(w), _p(out), DT[out.dtype], _p(rows), R, d, float(eps),
               stream if stream is not None else current_stream())


def add(x: torch.Tensor, delta: torch.Tensor, stream=None) -> None:
    _cuda(x, delta)
    _need(x.dtype == torch.float32 and delta.dtype in DT and x.numel() == delta.numel(), "add: shapes or dtypes")
    lib().call("slb_add", _p(x), _p(delta), DT[delta.dtype], x.numel(),
               stream if stream is not None else current_stream())


def swiglu(gu: torch.Tensor, act: torch.Tensor, stream=None) -> None:
    _cuda(gu, act)
    T, inter = act.shape
    _need(gu.shape == (T, 2 * inter) and gu.dtype == act.dtype and act.dtype in DT, "swiglu: shapes or dtypes")
    lib().call("slb_swiglu", _p(gu), _p(act), DT[act.dtype], T, inter,
               stream if stream is not None else current_stream())


def qkv_post(qkv, bias, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table,
             heads: int, kv_heads: int, head_dim: int, rot_dim: int, eps: float, stream=None) -> None:
    _cuda(qkv, bias, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table)
    T = q_out.shape[0]
    rows = heads + 2 * kv_heads
    _need(qkv.shape == (T, rows * head_dim) and q_out.shape[1:] == (heads, head_dim), "qkv_post: shapes disagree")
    _need(qkv.dtype == q_out.dtype and qkv.dtype in DT, "qkv_post: dtypes")
    for v in (bias, q_gain, k_gain, cos, sin):
        _need(v is None or v.dtype == torch.float32, "qkv_post: gains, biases and tables are float32")
    _need(bias is None or bias.numel() == rows * head_dim, "qkv_post: bias length")
    _need(q_gain is None or (q_gain.numel() == head_dim and k_gain.numel() == head_dim), "qkv_post: gain length")
    if rot_dim:
        _need(cos is not None and cos.shape[1] == rot_dim // 2 and sin.shape == cos.shape, "qkv_post: rotation tables")
    stride = 0
    if kv_heads and k_pool is not None:
        _need(k_pool.dtype == qkv.dtype and k_pool.shape == v_pool.shape and
              tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim), "qkv_post: cache pool shape or dtype")
        _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "qkv_post: block table")
        stride = block_table.shape[1]
    _need(tok_seq.dtype == torch.int32 and tok_pos.dtype == torch.int32, "qkv_post: token tables are int32")
    lib().call("slb_qkv_post", _p(qkv), _p(bias), _p(q_gain), _p(k_gain), _p(cos), _p(sin), _p(q_out), _p(k_pool),
               _p(v_pool), _p(tok_seq), _p(tok_pos), _p(block_table), stride, T, heads, kv_heads, head_dim, rot_dim,
               float(eps), DT[qkv.dtype], stream if stream is not None else current_stream())


def attention(q, k_pool, v_pool, out, tok_seq, tok_pos, block_table, heads: int, kv_heads: int, head_dim: int,
              window: int, scale: float, stream=None) -> None:
    _cuda(q, k_pool, v_pool, out, tok_seq, tok_pos, block_table)
    T = q.shape[0]
    _need(q.shape == (T, heads, head_dim) and out.shape == (T, heads * head_dim), "attention: shapes disagree")
    _need(q.dtype == out.dtype == k_pool.dtype == v_pool.dtype and q.dtype in DT, "attention: dtypes")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape, "attention: pool shape")
    _need(block_table.dtype == torch.int32 and block_table.dim() == 2, "attention: block table")
    lib().call("slb_attention_generic", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(tok_seq), _p(tok_pos),
               _p(block_table), block_table.shape[1], T, heads, kv_heads, head_dim, int(window), float(scale),
               DT[q.dtype], stream if stream is not None else current_stream())


def flash_supported(head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tensor-core attention kernels take this head size and dtype."""
    return dtype == torch.bfloat16 and head_dim in (64, 128)


_SMS: dict = {}


def sm_count(device=None) -> int:
    """Streaming multiprocessors of the device, asked of the library once (148 on a B200). The launch choices made
    in Python count with the same number as those made in the launchers."""
    key = torch.cuda.current_device() if device is None else torch.device(device).index
    if key not in _SMS:
        fn = lib().dll.slb_sm_count
        fn.restype = ctypes.c_int
        with torch.cuda.device(key):
            _SMS[key] = int(fn())
    return _SMS[key]


def decode_splits(n_seqs: int, kv_heads: int, group: int, table_stride: int, sms: int | None = None) -> int:
    """Slices of the key range per (sequence, kv head) in a decode step: enough blocks to fill the
    GPU a few times over, never more than a sequence can have pages. It depends on the batch size
    only, not on the lengths, so a captured step stays valid as sequences grow. ``sms``: the device's
    multiprocessors (asked of the library when not given)."""
    if sms is None:
        sms = sm_count()
    blocks = max(1, n_seqs * kv_heads * ((group + 15) // 16))
    # Two blocks of this kernel fit an SM with its three page buffers (100 KB of shared memory at head size 128),
    # three with two buffers, which the launcher picks when that makes all blocks run at once: 2 or 3 per SM.
    # All slices should run in one wave.
    resident = sms * 2
    if blocks >= resident:
        return 1
    if 2 * blocks > resident and 2 * blocks <= sms * 3 and table_stride >= 8:
        return 2          # one slice each would leave half the GPU idle; two fit with two page buffers
    # merging the slices costs a few microseconds that grow with their number: a slice should hold at least
    # four pages of the longest sequence
    most = max(1, table_stride // 4)
    three_buffers = max(1, min(resident // blocks, 64, most))
    # with two page buffers three blocks fit an SM: more, shorter slices in the same single round (measured at
    # batch 8: 18.7 us with 6 slices against 19.5 us with 4 at 2,112 keys; 7 slices, a second round, take 24.2 us)
    two_buffers = max(1, min((sms * 3) // blocks, 64, most))
    # only where that is half as many slices again: batch 8, 6 for 4 slices, 0.982 against 1.010 ms a step; batch 16,
    # 3 for 2, 1.395 against 1.412 ms; batch 12, 4 for 3, is slower, 1.197 against 1.171 ms
    if 2 * two_buffers >= 3 * three_buffers and two_buffers * blocks > resident:
        return two_buffers
    return three_buffers


def attention_prefill(q, k_pool, v_pool, out, seq_start, past, counts, block_table, max_count: int, heads: int,
                      kv_heads: int, head_dim: int, window: int, scale: float, stream=None) -> None:
    """Tensor-core attention for a step in which sequences bring any number of tokens."""
    _cuda(q, k_pool, v_pool, out, seq_start, past, counts, block_table)
    T, n = q.shape[0], block_table.shape[0]
    _need(q.shape == (T, heads, head_dim) and out.shape == (T, heads * head_dim), "attention: shapes disagree")
    _need(q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16, "attention (tensor cores): bfloat16 only")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape, "attention: pool shape")
    _need(seq_start.numel() >= n + 1 and past.numel() >= n and counts.numel() >= n, "attention: per-sequence tables")
    lib().call("slb_attention_prefill", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past), _p(counts),
               _p(block_table), block_table.shape[1], n, int(max_count), heads, kv_heads, head_dim, int(window),
               float(scale), stream if stream is not None else current_stream())


def attention_tc_supported(heads: int, kv_heads: int, head_dim: int, dtype: torch.dtype) -> bool:
    """Whether the tcgen05 attention kernel takes this shape (bfloat16, head size 64 or 128, group size dividing 128)."""
    if dtype != torch.bfloat16 or heads <= 0 or kv_heads <= 0 or heads % kv_heads:
        return False
    group = heads // kv_heads
    return head_dim in (64, 128) and group <= 128 and 128 % group == 0


def attention_tc_takes_two_pages(n_seqs: int, max_count: int, max_keys: int, heads: int, kv_heads: int, window: int = 0) -> bool:
    """Whether ``attention_tc``, left to choose, takes its kernel for long tiles (two pages a step, one block an SM)
    for a step of ``n_seqs`` sequences whose longest brings ``max_count`` tokens and then has ``max_keys`` keys."""
    fn = lib().dll.slb_attention_tc_wide_pays
    fn.argtypes = [ctypes.c_int] * 6
    fn.restype = ctypes.c_int
    return fn(int(n_seqs), int(max_count), int(max_keys), int(heads), int(kv_heads), int(window)) != 0


def attention_tc(q, k_pool, v_pool, out, seq_start, past, counts, block_table, max_count: int, heads: int,
                 kv_heads: int, head_dim: int, window: int, scale: float, stream=None, wide: bool | None = None,
                 max_keys: int = 0) -> None:
    """Attention for a step in which sequences bring many tokens, on the tcgen05 tensor cores (same contract as
    ``attention_prefill``). A bounded wait that gave up inside the kernel shows in ``tc_check``. ``wide``: the
    kernel that walks two pages a step (True), one page a step (False), or the library's choice from the step's
    shape; ``max_keys`` (the most keys a sequence has after this step, 0 = not known) helps that choice."""
    _cuda(q, k_pool, v_pool, out, seq_start, past, counts, block_table)
    T, n = q.shape[0], block_table.shape[0]
    _need(q.shape == (T, heads, head_dim) and out.shape == (T, heads * head_dim), "attention: shapes disagree")
    _need(q.dtype == out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16, "attention (tcgen05): bfloat16 only")
    _need(q.is_contiguous() and k_pool.is_contiguous() and v_pool.is_contiguous() and out.is_contiguous(),
          "attention (tcgen05): contiguous tensors")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape, "attention: pool shape")
    _need(seq_start.numel() >= n + 1 and past.numel() >= n and counts.numel() >= n, "attention: per-sequence tables")
    lib().call("slb_attention_tc", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past), _p(counts),
               _p(block_table), block_table.shape[1], n, int(max_count), T, k_pool.shape[0], heads, kv_heads, head_dim,
               int(window), float(scale), _p(_tc_status(q.device)), -1 if wide is None else int(bool(wide)),
               int(max_keys), stream if stream is not None else current_stream())


def attention_decode(q, k_pool, v_pool, out, seq_start, past, block_table, heads: int, kv_heads: int, head_dim: int,
                     window: int, scale: float, splits: int, scratch, stream=None, qkv=None, qkv_kv_heads: int = 0,
                     bias=None, q_gain=None, k_gain=None, cos=None, sin=None, eps: float = 1e-6, next_read=None) -> None:
    """Tensor-core attention for a step in which every sequence brings one token (split-KV).

    With ``qkv`` (the raw fused projection ``[n, (heads + 2 * qkv_kv_heads) * head_dim]``) the kernel also does what
    ``qkv_post`` does for that token: bias, per-head QK-norm, rotation of the whole head, and, when
    ``qkv_kv_heads == kv_heads``, the write of its key and value into the cache; ``q`` is then not read.
    ``next_read``: a tensor that the kernel after this one reads and no kernel writes (a weight matrix); the blocks
    ask the L2 cache for it once their own pages are on their way."""
    _cuda(q, k_pool, v_pool, out, seq_start, past, block_table, scratch, qkv, bias, q_gain, k_gain, cos, sin)
    n = block_table.shape[0]
    _need(out.shape == (n, heads * head_dim) and out.dtype == k_pool.dtype == v_pool.dtype == torch.bfloat16,
          "attention (tensor cores): shapes disagree or not bfloat16")
    _need(tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape, "attention: pool shape")
    _need(scratch is None or scratch.dtype == torch.float32, "attention: scratch is float32")
    if qkv is None:
        _need(q is not None and q.shape == (n, heads, head_dim) and q.dtype == torch.bfloat16, "attention: q shape or dtype")
    else:
        _need(qkv.shape == (n, (heads + 2 * qkv_kv_heads) * head_dim) and qkv.dtype == torch.bfloat16, "attention: raw projection shape")
        for v in (bias, q_gain, k_gain, cos, sin):
            _need(v is None or v.dtype == torch.float32, "attention: gains, biases and tables are float32")
        _need(cos is None or (cos.shape[1] == head_dim // 2 and sin.shape == cos.shape), "attention: rotation tables")
    counters = _decode_counters(out.device, n * kv_heads * ((heads // kv_heads + 15) // 16)) if splits > 1 else None
    lib().call("slb_attention_decode", _p(q), _p(k_pool), _p(v_pool), _p(out), _p(seq_start), _p(past),
               _p(block_table), block_table.shape[1], n, heads, kv_heads, head_dim, int(window), float(scale),
               int(splits), _p(scratch), 0 if scratch is None else scratch.numel(), _p(counters),
               0 if counters is None else counters.numel(), _p(qkv), int(qkv_kv_heads), _p(bias), _p(q_gain), _p(k_gain),
               _p(cos), _p(sin), float(eps), _p(next_read) if _nbytes(next_read) else None, _nbytes(next_read),
               stream if stream is not None else current_stream())


_COUNTERS: dict = {}


def _decode_counters(device, n: int) -> torch.Tensor:
    """Ticket counters of the split-KV decode kernel: zero when a launch starts, left at zero when it ends."""
    key = str(device)
    t = _COUNTERS.get(key)
    if t is None or t.numel() < n:
        if t is not None:
            _RETIRED.append(t)          # a captured graph may still point at the smaller one
        t = torch.zeros(max(n, 4096), dtype=torch.int32, device=device)
        _COUNTERS[key] = t
    return t


_RETIRED: list = []


def decode_scratch_floats(n_seqs: int, heads: int, head_dim: int, splits: int) -> int:
    return 0 if splits <= 1 else n_seqs * heads * splits * (head_dim + 2)


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias=None, accumulate: bool = False,
             stream=None) -> None:
    """out[M, N] (+)= a[M, K] @ w[N, K]^T (+ bias), all float32, plain FMA."""
    _cuda(a, w, out, bias)
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm_f32: shapes disagree")
    _need(a.dtype == w.dtype == out.dtype == torch.float32, "gemm_f32: float32 only")
    lib().call("slb_gemm_f32", _p(a), _p(w), _p(bias), _p(out), M, N, K, K, K, N, int(accumulate),
               stream if stream is not None else current_stream())


SKINNY_MODES = {"bf16": 0, "f32": 1, "add": 2, "swiglu": 3}


def skinny_supported(M: int, N: int, K: int, norm: bool = False) -> bool:
    """Whether the few-rows bfloat16 product kernel takes this problem (with the norm fused in: up to 16 rows of
    at most 4,096 values, which it keeps normalised in shared memory)."""
    return 1 <= M <= (16 if norm else 64) and K >= 32 and K % 32 == 0 and N >= 1 and (not norm or K <= 4096)


# SLEUTH_B200_PREFETCH=0: kernels are not told what the kernel after them reads (for comparisons; measured on a
# B200 at batch 8: 1.055 ms a step with the hints, 1.073 ms without; no difference at batch 1).
PREFETCH = os.environ.get("SLEUTH_B200_PREFETCH", "1") != "0"
# No hint for a matrix of more than a quarter of the 126 MB L2: it would push out what it is meant to keep, and a
# product that large is bound by memory bandwidth, not by latency (hidden 4,096, one row: 1.40 ms a step with this
# limit, 1.57 ms without; hidden 2,048: 1.31 against 1.27 ms).
PREFETCH_MOST = 32 << 20


def _nbytes(t) -> int:
    """Bytes of a range handed to a kernel as its ``next_read``: 0 (no hint) unless it is one aligned piece of memory."""
    if t is None or not PREFETCH or not t.is_contiguous() or t.data_ptr() % 16:
        return 0
    n = t.numel() * t.element_size()
    return n if n <= PREFETCH_MOST else 0


class _NextPages(ctypes.Structure):
    _fields_ = [("k_pool", ctypes.c_void_p), ("v_pool", ctypes.c_void_p), ("block_table", ctypes.c_void_p),
                ("past", ctypes.c_void_p), ("page_bytes", ctypes.c_longlong), ("table_stride", ctypes.c_int),
                ("n_seqs", ctypes.c_int), ("splits", ctypes.c_int), ("depth", ctypes.c_int), ("window", ctypes.c_int)]


def next_pages(k_pool, v_pool, block_table, past, splits: int, window: int, depth: int = 2):
    """What a few-rows product hands its kernel as ``next_pages`` when ``attention_decode`` with these arguments
    follows it: the product's blocks then ask the L2 cache for the first ``depth`` pages of every slice."""
    if not PREFETCH:
        return None
    _cuda(k_pool, v_pool, block_table, past)
    page_bytes = k_pool[0].numel() * k_pool.element_size()
    if page_bytes > 32 * 32768 or page_bytes % 16:
        return None
    return _NextPages(k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(), past.data_ptr(), page_bytes,
                      block_table.shape[1], block_table.shape[0], int(splits), int(depth), int(window))


def _pages_arg(pages):
    return None if pages is None else ctypes.addressof(pages)


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str, stream=None, next_read=None,
                next_pages=None, features: int = 0) -> None:
    """out = x[M, K] @ w^T for M <= 16 (bfloat16 in, float32 accumulation). mode: "bf16" / "f32" store,
    "add" adds into a float32 ``out``, "swiglu" takes w = [gate rows; up rows] and stores silu(gate) * up.
    ``next_read``: a weight tensor that the kernel after this one reads; the blocks ask the L2 cache for it.
    ``features``: output features a block takes (8, 16, 32; 0 = the launcher's rule)."""
    _cuda(x, w, out)
    M, K = x.shape
    N = out.shape[1]
    _need(x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K and out.shape[0] == M, "gemm_skinny: shapes or dtypes")
    _need(w.shape[0] == (2 * N if mode == "swiglu" else N), "gemm_skinny: weight rows")
    _need(out.dtype == (torch.bfloat16 if mode in ("bf16", "swiglu") else torch.float32), "gemm_skinny: output dtype")
    lib().call("slb_gemm_skinny", _p(x), _p(w), _p(out), M, N, K, N, SKINNY_MODES[mode], _p(next_read) if _nbytes(next_read) else None, _nbytes(next_read),
               _pages_arg(next_pages), int(features), stream if stream is not None else current_stream())


def gemm_skinny_norm(x: torch.Tensor, gain: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor, mode: str,
                     stream=None, next_read=None, next_pages=None, features: int = 0) -> None:
    """``gemm_skinny`` on rmsnorm(x; gain, eps): x is the float32 stream [M, K], normalised inside the kernel."""
    _cuda(x, gain, w, out)
    M, K = x.shape
    N = out.shape[1]
    _need(x.dtype == torch.float32 and gain.dtype == torch.float32 and gain.numel() == K, "gemm_skinny_norm: x and gain are float32")
    _need(w.dtype == torch.bfloat16 and w.shape[1] == K and out.shape[0] == M, "gemm_skinny_norm: shapes or dtypes")
    _need(w.shape[0] == (2 * N if mode == "swiglu" else N), "gemm_skinny_norm: weight rows")
    _need(out.dtype == (torch.bfloat16 if mode in ("bf16", "swiglu") else torch.float32), "gemm_skinny_norm: output dtype")
    lib().call("slb_gemm_skinny_norm", _p(x), _p(gain), float(eps), _p(w), _p(out), M, N, K, N, SKINNY_MODES[mode],
               _p(next_read) if _nbytes(next_read) else None, _nbytes(next_read), _pages_arg(next_pages), int(features),
               stream if stream is not None else current_stream())


def tc_supported(M: int, N: int, K: int) -> bool:
    """Whether the tcgen05/TMA product kernel takes this problem."""
    return M >= 1 and N >= 1 and K >= 8 and K % 8 == 0


_TC_STATUS: dict = {}


def _tc_status(device) -> torch.Tensor:
    st = _TC_STATUS.get(device)
    if st is None:
        st = _TC_STATUS.get(str(device))
        if st is None:
            st = torch.zeros(1, dtype=torch.int32, device=device)
            _TC_STATUS[str(device)] = st
        _TC_STATUS[device] = st
    return st


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, mode: str, stream=None) -> None:
    """out = x[M, K] @ w^T on the tcgen05 tensor cores (bfloat16 in, float32 accumulation in tensor memory).
    mode as for ``gemm_skinny``: "bf16" / "f32" store, "add" into a float32 ``out``, "swiglu" with w = [gate; up]."""
    _cuda(x, w, out)
    M, K = x.shape
    N = out.shape[1]
    _need(x.dtype == w.dtype == torch.bfloat16 and w.shape[1] == K and out.shape[0] == M, "gemm_tc: shapes or dtypes")
    _need(w.shape[0] == (2 * N if mode == "swiglu" else N), "gemm_tc: weight rows")
    _need(out.dtype == (torch.bfloat16 if mode in ("bf16", "swiglu") else torch.float32), "gemm_tc: output dtype")
    lib().call("slb_gemm_tc", _p(x), _p(w), _p(out), M, N, K, N, SKINNY_MODES[mode], _p(_tc_status(x.device)),
               stream if stream is not None else current_stream())


def gemm_tc_qkv(x, w, heads: int, kv_heads: int, head_dim: int, bias, q_gain, k_gain, cos, sin, eps: float, q_out,
                k_pool, v_pool, tok_seq, tok_pos, block_table, stream=None) -> None:
    """The fused q/k/v projection of many tokens with everything ``qkv_post`` does in its epilogue, on the float32
    accumulators: bias, per-head RMSNorm of q and k, rotation of the whole head, q into ``q_out [T, H, hd]``, k and v
    into each token's cache page. ``kv_heads == 0``: ``w`` holds only q heads and nothing is written to the cache."""
    _cuda(x, w, bias, q_gain, k_gain, cos, sin, q_out, k_pool, v_pool, tok_seq, tok_pos, block_table)
    M, K = x.shape
    _need(x.dtype == w.dtype == q_out.dtype == torch.bfloat16, "gemm_tc_qkv: bfloat16 only")
    _need(w.shape == ((heads + 2 * kv_heads) * head_dim, K) and w.is_contiguous() and x.is_contiguous(), "gemm_tc_qkv: weight shape")
    _need(q_out.shape == (M, heads, head_dim) and q_out.is_contiguous(), "gemm_tc_qkv: q_out shape")
    for v in (bias, q_gain, k_gain, cos, sin):
        _need(v is None or (v.dtype == torch.float32 and v.is_contiguous()), "gemm_tc_qkv: gains, biases and tables are float32")
    _need(cos is None or (cos.shape[1] == head_dim // 2 and sin.shape == cos.shape), "gemm_tc_qkv: rotation tables [positions, hd / 2]")
    _need(tok_pos.numel() >= M and (kv_heads == 0 or tok_seq.numel() >= M), "gemm_tc_qkv: per-token tables")
    if kv_heads:
        _need(k_pool is not None and tuple(k_pool.shape[1:]) == (kv_heads, 64, head_dim) and k_pool.shape == v_pool.shape
              and k_pool.dtype == v_pool.dtype == torch.bfloat16, "gemm_tc_qkv: pool shape")
    lib().call("slb_gemm_tc_qkv", _p(x), _p(w), M, K, heads, kv_heads, head_dim, _p(bias), _p(q_gain), _p(k_gain), _p(cos),
               _p(sin), float(eps), _p(q_out), _p(k_pool) if kv_heads else None, _p(v_pool) if kv_heads else None,
               _p(tok_seq), _p(tok_pos), _p(block_table), 0 if block_table is None else block_table.shape[1],
               _p(_tc_status(x.device)), stream if stream is not None else current_stream())


def tc_wait_probe(device, polls: int = 1000, code: int = 99, stream=None) -> None:
    """Run the give-up path of the tensor-memory kernels on purpose and harmlessly: a one-block kernel takes tensor
    memory, waits ``polls`` times on a barrier that nothing completes, records ``code`` in the status word, frees its
    tensor memory and returns. ``gemm_tc_check`` then raises. For tests of that path; nothing faults or hangs."""
    with torch.cuda.device(torch.device(device)):
        lib().call("slb_tc_wait_probe", _p(_tc_status(torch.device(device))), int(polls), int(code),
                   stream if stream is not None else current_stream())


def tc_status(device):
    """The status word of the tcgen05 kernels on ``device`` (an int32 CUDA tensor), or None if none has run there."""
    return _TC_STATUS.get(str(torch.device(device)))


def gemm_tc_check(device) -> None:
    """Raise if a tcgen05 product kernel gave up one of its bounded waits since the last check (synchronises)."""
    st = _TC_STATUS.get(str(torch.device(device)))
    if st is None:
        return
    code = int(st.item())
    if code:
        st.zero_()
        raise RuntimeError(f"a wait inside a tcgen05 kernel gave up (code {code}; product: 1 = free stage, 2 = loaded "
                           f"stage, 3 = finished accumulator, 4 = drained accumulator; attention: 20 = shared memory "
                           f"misaligned, 21-27 = producer and MMA waits, 28-32 = softmax waits; persistent single-token kernel: 40 = grid "
                           f"barrier, 41 = a ring slot that did not fill, 42 = a ring slot that did not empty; 99 = the wait "
                           f"probe of the tests); "
                           f"its results are not valid")


# ---------------------------------------------------------------- the persistent single-token kernel ----
_VP, _LL, _CI, _CF = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
DL_MAX_PLANS, DL_MAX_ROWS, DL_MAX_UNITS, DL_MAX_GROUP, DL_MAX_COMBOS = 4, 16, 256, 8, 4


class _DlLayer(ctypes.Structure):          # mirrors DlLayer in csrc/decode_layers.cu
    _fields_ = [(n, _VP) for n in ("w_qkv", "w_o", "w_gu", "w_down", "norm1", "norm2", "bias", "q_gain", "k_gain", "cos_table",
                                   "sin_table", "k_pool", "v_pool")] + \
               [("k_row0", _LL), ("v_row0", _LL), ("eps1", _CF), ("eps2", _CF), ("qk_eps", _CF), ("scale_log2", _CF),
                ("heads", _CI), ("kv_heads", _CI), ("inter", _CI), ("window", _CI), ("group", _CI), ("plan", _CI),
                ("combo", _CI), ("pad1", _CI)]


class _DlArgs(ctypes.Structure):           # mirrors DlArgs
    _fields_ = [(n, _VP) for n in ("layers", "x", "qkv", "y", "act", "parts", "tickets", "barrier", "status", "past", "trace")] + \
               [("tables", _VP * 2), ("table_stride", _CI * 2), ("plan_window", _CI * DL_MAX_PLANS),
                ("plan_kv_heads", _CI * DL_MAX_PLANS), ("combo_plan", _CI * DL_MAX_COMBOS), ("combo_group", _CI * DL_MAX_COMBOS),
                ("n_plans", _CI), ("n_combos", _CI), ("n_layers", _CI), ("B", _CI), ("d", _CI), ("n_slots", _CI),
                ("stage_bytes", _CI), ("pad", _CI)]


class _DlHost(ctypes.Structure):           # mirrors DlHost
    _fields_ = [("args", _DlArgs), ("pool_base", _VP * 2), ("pool_rows", _LL * 2), ("head_dim", _CI), ("n_groups", _CI)]


class DecodeProgram:
    """A run of layers prepared for ``decode_layers``: the layers' descriptions in device memory and what is the same
    for every launch. Built by ``decode_program`` from what the layers' parts offer (``Part.fused_decode``)."""

    def __init__(self, layers_dev, n_layers, head_dim, hidden, kmax, max_qkv, max_heads, max_inter, plans, groups, combos, keep):
        self.layers_dev, self.n_layers, self.head_dim, self.hidden, self.kmax = layers_dev, n_layers, head_dim, hidden, kmax
        self.max_qkv, self.max_heads, self.max_inter = max_qkv, max_heads, max_inter
        self.plans, self.groups, self.combos, self.keep = plans, groups, combos, keep
        device = layers_dev.device
        self.tickets = torch.zeros(DL_MAX_UNITS, dtype=torch.int32, device=device)
        self.barrier = torch.zeros(4, dtype=torch.int32, device=device)
        self._slots: dict = {}

    def slots_for(self, rows: int) -> tuple[int, int]:
        """(ring slots, bytes of the staging area) for a step of ``rows`` sequences; fewer than 4 slots: do not fuse."""
        if rows not in self._slots:
            dll = lib().dll
            dll.slb_decode_layers_stage_bytes.restype = ctypes.c_int
            dll.slb_decode_layers_slots.restype = ctypes.c_int
            stage = int(dll.slb_decode_layers_stage_bytes(int(rows), int(self.kmax), int(self.head_dim)))
            self._slots[rows] = (int(dll.slb_decode_layers_slots(stage, int(rows))), stage)
        return self._slots[rows]


def decode_program(shares: list, views: list, pools: list) -> DecodeProgram | None:
    """Prepare a run of layers for the persistent single-token kernel. ``shares``: per layer what its parts offer
    (``PreNormLayer.fused_decode``); ``views``: per layer the ``KVView`` of its cache entry; ``pools``: the cache's
    pool tensor of each group. None when the run does not fit the kernel (mixed head sizes or widths, more than two
    cache groups or four page plans)."""
    if not shares:
        return None
    hd = shares[0]["mixer"]["head_dim"]
    d = shares[0]["mixer"]["hidden"]
    group_ids, plans, combos, keep = [], [], [], []
    arr = (_DlLayer * len(shares))()
    kmax = max_qkv = max_heads = max_inter = 0
    for i, (sh, view) in enumerate(zip(shares, views)):
        m, f = sh["mixer"], sh["ffn"]
        if m["head_dim"] != hd or m["hidden"] != d or view is None or not getattr(view, "writes", False):
            return None
        if view.group not in group_ids:
            group_ids.append(view.group)
        plan = (int(m["window"]), int(m["kv_heads"]))
        if plan not in plans:
            plans.append(plan)
        combo = (plans.index(plan), group_ids.index(view.group))
        if combo not in combos:
            combos.append(combo)
        if len(group_ids) > 2 or len(plans) > DL_MAX_PLANS or len(combos) > DL_MAX_COMBOS:
            return None
        pool = pools[view.group]
        L = arr[i]
        for name, t in (("w_qkv", m["w_qkv"]), ("w_o", m["w_o"]), ("w_gu", f["w_gu"]), ("w_down", f["w_down"]),
                        ("norm1", sh["norm1"]["gain"]), ("norm2", sh["norm2"]["gain"]), ("bias", m["bias"]),
                        ("q_gain", m["q_gain"]), ("k_gain", m["k_gain"]), ("cos_table", m["cos"]), ("sin_table", m["sin"]),
                        ("k_pool", view.k_pool), ("v_pool", view.v_pool)):
            if t is not None:
                _need(t.is_cuda and t.is_contiguous() and t.data_ptr() % 16 == 0, f"decode_program: {name} must be a contiguous, aligned CUDA tensor")
                keep.append(t)
            setattr(L, name, _p(t))
        for t in (m["w_qkv"], m["w_o"], f["w_gu"], f["w_down"], view.k_pool):
            _need(t.dtype == torch.bfloat16, "decode_program: matrices and the cache are bfloat16")
        for t in (sh["norm1"]["gain"], sh["norm2"]["gain"], m["bias"], m["q_gain"], m["k_gain"], m["cos"], m["sin"]):
            _need(t is None or t.dtype == torch.float32, "decode_program: gains, biases and tables are float32")
        row_bytes = hd * 2
        L.k_row0 = (view.k_pool.data_ptr() - pool.data_ptr()) // row_bytes
        L.v_row0 = (view.v_pool.data_ptr() - pool.data_ptr()) // row_bytes
        L.eps1, L.eps2, L.qk_eps = float(sh["norm1"]["eps"]), float(sh["norm2"]["eps"]), float(m["qk_eps"])
        L.scale_log2 = float(m["scale"]) * 1.4426950408889634
        L.heads, L.kv_heads, L.inter, L.window = int(m["heads"]), int(m["kv_heads"]), int(f["inter"]), int(m["window"])
        L.group, L.plan, L.combo = group_ids.index(view.group), plans.index(plan), combos.index(combo)
        n_qkv = (L.heads + 2 * L.kv_heads) * hd
        _need(tuple(m["w_qkv"].shape) == (n_qkv, d) and tuple(m["w_o"].shape) == (d, L.heads * hd) and
              tuple(f["w_gu"].shape) == (2 * L.inter, d) and tuple(f["w_down"].shape) == (d, L.inter),
              "decode_program: weight shapes disagree with the sizes")
        kmax = max(kmax, d, L.heads * hd, L.inter)
        max_qkv, max_heads, max_inter = max(max_qkv, n_qkv), max(max_heads, L.heads * hd), max(max_inter, L.inter)
    device = shares[0]["mixer"]["w_qkv"].device
    raw = torch.frombuffer(bytearray(bytes(arr)), dtype=torch.uint8).to(device)
    groups = [(pools[g], pools[g].numel() // hd) for g in group_ids]
    keep.extend(p for p, _ in groups)
    return DecodeProgram(raw, len(shares), hd, d, kmax, max_qkv, max_heads, max_inter, plans,
                         [(gid, *g) for gid, g in zip(group_ids, groups)], combos, keep)


def decode_layers_scratch_floats(prog: DecodeProgram, rows: int, blocks: int) -> int:
    return (blocks + DL_MAX_UNITS) * (DL_MAX_GROUP * prog.head_dim + 2 * DL_MAX_GROUP)


def decode_layers(prog: DecodeProgram, x: torch.Tensor, past: torch.Tensor, tables: list, qkv, y, act, parts, stream=None,
                  trace: torch.Tensor | None = None) -> None:
    """Run the program's layers on the float32 stream ``x [B, hidden]`` of a step in which each of the B sequences
    brings one token: ``past [B]`` their positions, ``tables`` the step's block table of every cache group
    (indexed as the cache indexes its groups). ``qkv``, ``y``, ``act`` (bfloat16) and ``parts`` (float32) are scratch.
    ``trace``: None, or an int64 tensor [blocks, layers, 24] that receives every block's nanosecond stamps at the phase
    boundaries of every layer (entries 0-14) and the clock cycles each phase waited for its data (15-19): a diagnostic."""
    _cuda(x, past, qkv, y, act, parts)
    B, d = x.shape
    _need(x.dtype == torch.float32 and d == prog.hidden and 1 <= B <= DL_MAX_ROWS, "decode_layers: x is float32 [1..16, hidden]")
    n_slots, stage = prog.slots_for(B)
    _need(n_slots >= 4, "decode_layers: the token rows leave no room for the ring in shared memory")
    blocks = sm_count(x.device)
    _need(qkv.numel() >= B * prog.max_qkv and y.numel() >= B * prog.max_heads and act.numel() >= B * prog.max_inter and
          parts.numel() >= decode_layers_scratch_floats(prog, B, blocks) and qkv.dtype == y.dtype == act.dtype == torch.bfloat16
          and parts.dtype == torch.float32, "decode_layers: scratch buffers are too small or of the wrong dtype")
    h = _DlHost()
    a = h.args
    a.layers, a.x, a.qkv, a.y, a.act, a.parts = prog.layers_dev.data_ptr(), x.data_ptr(), qkv.data_ptr(), y.data_ptr(), act.data_ptr(), parts.data_ptr()
    a.tickets, a.barrier, a.status, a.past = prog.tickets.data_ptr(), prog.barrier.data_ptr(), _tc_status(x.device).data_ptr(), past.data_ptr()
    if trace is not None:
        _need(trace.is_cuda and trace.dtype == torch.int64 and trace.numel() >= blocks * prog.n_layers * 24, "decode_layers: trace is int64 [blocks, layers, 24]")
    a.trace = _p(trace)
    for i, (gid, pool, rows) in enumerate(prog.groups):
        t = tables[gid]
        _need(t.dtype == torch.int32 and t.dim() == 2 and t.shape[0] >= B and t.is_contiguous(), "decode_layers: block tables are int32 [B, stride]")
        a.tables[i], a.table_stride[i] = t.data_ptr(), t.shape[1]
        h.pool_base[i], h.pool_rows[i] = pool.data_ptr(), rows
    for i, (window, kvh) in enumerate(prog.plans):
        a.plan_window[i], a.plan_kv_heads[i] = window, kvh
    for i, (plan, group) in enumerate(prog.combos):
        a.combo_plan[i], a.combo_group[i] = plan, group
    a.n_plans, a.n_combos, a.n_layers, a.B, a.d, a.n_slots, a.stage_bytes = len(prog.plans), len(prog.combos), prog.n_layers, B, d, n_slots, stage
    h.head_dim, h.n_groups = prog.head_dim, len(prog.groups)
    lib().call("slb_decode_layers", ctypes.addressof(h), stream if stream is not None else current_stream())


def penalize(logits, limit: int, recent, n_recent, penalty: float, banned, n_banned, stream=None) -> None:
    _cuda(logits, recent, n_recent, banned, n_banned)
    R = logits.shape[0]
    lib().call("slb_penalize", _p(logits), logits.stride(0), R, limit, _p(recent), _p(n_recent),
               0 if recent is None else recent.shape[1], float(penalty), _p(banned), _p(n_banned),
               0 if banned is None else banned.shape[1], stream if stream is not None else current_stream())


def argmax_scratch_words(rows: int) -> int:
    return 2 * rows * 64


def argmax(logits: torch.Tensor, limit: int, out: torch.Tensor, scratch: torch.Tensor, stream=None) -> None:
    """out[r] = first index of the largest of logits[r, :limit]. ``scratch``: int32, ``argmax_scratch_words(rows)`` long."""
    _need(logits.is_cuda and out.is_cuda and logits.dtype == torch.float32 and out.dtype == torch.int32, "argmax: dtypes")
    _need(logits.stride(1) == 1 and out.numel() >= logits.shape[0] and 0 < limit <= logits.shape[1], "argmax: shapes")
    _need(scratch.is_cuda and scratch.dtype == torch.int32, "argmax: scratch is an int32 CUDA tensor")
    lib().call("slb_argmax", _p(logits), logits.stride(0), logits.shape[0], limit, _p(out), _p(scratch), scratch.numel(),
               stream if stream is not None else current_stream())


def sample(logits: torch.Tensor, limit: int, temperature: float, top_k: int, top_p: float, min_p: float,
           uniform: torch.Tensor, out: torch.Tensor, stream=None) -> None:
    _need(logits.is_cuda and logits.dtype == torch.float32 and uniform.dtype == torch.float32 and
          out.dtype == torch.int32, "sample: dtypes")
    _need(logits.stride(1) == 1 and uniform.numel() >= logits.shape[0] and out.numel() >= logits.shape[0] and
          0 < limit <= logits.shape[1], "sample: shapes")
    lib().call("slb_sample", _p(logits), logits.stride(0), logits.shape[0], limit, float(temperature), int(top_k),
               float(top_p), float(min_p), _p(uniform), _p(out), stream if stream is not None else current_stream())
