"""What every part of a model is: its interface, the build context, and the registries by kind.

A part is built from its spec (sizes and constants as parameters) and a ``BuildContext`` (device,
run dtype, longest position). It then

* ``declare()``s the tensors it needs, by local name, with shape and role;
* is ``bind()``-ed to those tensors once the loader has put them on the device;
* says through ``cache_request()`` what its cache entry must hold (mixers only);
* runs in ``forward``; the signatures per kind are below.

Interfaces (``b`` is the step's ``StepBatch``; tensors are CUDA tensors; the residual stream ``x``
is float32 ``[tokens, hidden]``; ``h`` is in the run dtype):

* norm:      ``forward(x, out=None, rows=None) -> h``          normalises rows of the float32 stream
* position:  ``tables() -> (cos, sin) | None``                 what the attention kernels read
* mixer:     ``forward(h, x, b, view, ws)``                    adds its output into ``x`` in place
* ffn:       ``forward(h, x, b, ws)``                          adds its output into ``x`` in place
             (a mixer or ffn with ``accepts_normed = True`` gets a ``Normed`` for ``h``, see below)
* layer:     ``forward(x, b, view, ws)``                       one whole layer on the stream, in place
* embedding: ``forward(b, x)``                                 fills ``x`` from the batch's token ids (and, if it
                                                               wants, their positions ``b.tok_pos``); a part whose
                                                               table a tied head may use exposes it as ``table``
* head:      ``forward(x, b, logits, ws)``                     final norm + output matrix on the rows ``b.rows``;
                                                               ``bind(tensors, embedding_table=...)``

Roles decide the dtype a tensor is kept in on the device: ``"matrix"`` in the run dtype (bfloat16
on the fast path), ``"vector"`` (gains, biases) in float32, ``"table"`` (integer tables) in int32.
A tensor that the file stores in 32-bit is never narrowed on the way in; a matrix product that
runs in bfloat16 makes its own bfloat16 copy of such a matrix.

A part whose ``forward`` must run afresh every step (it reads the step's host-side values, or its launches
depend on the data) sets ``capturable = False``; single-token steps are then not recorded as CUDA graphs.

New kinds are added with ``register_norm``, ``register_position``, ``register_mixer``,
``register_ffn``, ``register_layer``, ``register_embedding``, ``register_head``; a spec's ``kind``
selects the class.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass(frozen=True)
class ParamDecl:
    shape: tuple
    role: str = "matrix"        # "matrix" | "vector" | "table"
    optional: bool = False
    init: str = "normal"        # how random weights draw it: "normal" = N(0, std), "gain" = 1 + N(0, std)


@dataclass
class BuildContext:
    device: torch.device
    dtype: torch.dtype          # run dtype: torch.bfloat16 or torch.float32
    max_positions: int          # longest sequence the engine will hold
    shared: dict = field(default_factory=dict)   # parts that several layers share (position tables)


class Normed:
    """The normalised rows of the stream, handed to a mixer or feed-forward that set ``accepts_normed``.

    Such a part may either ask for the tensor (``tensor()`` runs the norm kernel once and keeps the result)
    or, when its first product can normalise on the fly, read ``x``, ``gain`` and ``eps`` and skip the
    norm kernel altogether. ``gain`` is None when the norm is not a plain RMSNorm."""

    def __init__(self, norm, x: torch.Tensor, ws, stream, dtype):
        self.norm, self.x, self.ws, self.stream, self.dtype = norm, x, ws, stream, dtype
        self.gain = getattr(norm, "weight", None) if getattr(norm, "fusable", False) else None
        self.eps = getattr(norm, "eps", 0.0)
        self.shape = x.shape
        self._h = None

    def tensor(self) -> torch.Tensor:
        if self._h is None:
            self._h = self.ws.take(self.x.shape, self.dtype)
            self.norm.forward(self.x, self._h, stream=self.stream)
        return self._h


class Part:
    accepts_normed = False      # True: ``forward`` takes a ``Normed`` instead of the normalised tensor
    # False: ``forward`` cannot be recorded once and replayed, because it reads host-side values of the step
    # (``b.host_slots``, ``b.host_counts``), waits for the device, or launches work whose shape depends on the data
    # (routing). A model with such a part runs its single-token steps launch by launch instead of as a CUDA graph.
    capturable = True

    def declare(self) -> dict[str, ParamDecl]:
        return {}

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        pass

    def cache_request(self):
        return None

    def fused_decode(self):
        """What the persistent single-token kernel (``csrc/decode_layers.cu``) needs of this part, as a dictionary of
        tensors and constants, or None when the part cannot take part in it (the layer then runs launch by launch).
        The built-in RMSNorm, grouped-query attention, gated feed-forward and pre-norm layer answer; a part that
        says nothing is simply not fused."""
        return None

    def lead_weight(self):
        """The weight matrix that this part's first product reads, or None. The part that runs before this one may
        hand it to its last kernel, which then asks the L2 cache for it (``StepBatch.next_read``)."""
        return None


def lead_weight_of(part):
    """``part.lead_weight()`` for anything that has one, else None."""
    f = getattr(part, "lead_weight", None)
    return f() if callable(f) else None


_REGISTRIES: dict[str, dict[str, type]] = {"norm": {}, "position": {}, "mixer": {}, "ffn": {}, "layer": {},
                                           "embedding": {}, "head": {}}


def _register(family: str, kind: str, cls: type) -> None:
    _REGISTRIES[family][kind] = cls


def _build(family: str, spec, ctx: BuildContext, **extra):
    kind = getattr(spec, "kind", None)
    try:
        cls = _REGISTRIES[family][kind]
    except KeyError:
        raise KeyError(f"no {family} of kind {kind!r} is registered (known: {sorted(_REGISTRIES[family])})") from None
    return cls(spec, ctx, **extra)


def register_norm(kind, cls): _register("norm", kind, cls)
def register_position(kind, cls): _register("position", kind, cls)
def register_mixer(kind, cls): _register("mixer", kind, cls)
def register_ffn(kind, cls): _register("ffn", kind, cls)
def register_layer(kind, cls): _register("layer", kind, cls)
def register_embedding(kind, cls): _register("embedding", kind, cls)
def register_head(kind, cls): _register("head", kind, cls)


def build_norm(spec, ctx): return _build("norm", spec, ctx)
def build_position(spec, ctx):
    """Layers with equal position specs share one part (one pair of tables)."""
    key = ("position", spec)
    if key not in ctx.shared:
        ctx.shared[key] = _build("position", spec, ctx)
    return ctx.shared[key]
def build_mixer(spec, ctx): return _build("mixer", spec, ctx)
def build_ffn(spec, ctx): return _build("ffn", spec, ctx)
def build_layer(spec, ctx): return _build("layer", spec, ctx)
def build_embedding(spec, ctx): return _build("embedding", spec, ctx)
def build_head(spec, ctx): return _build("head", spec, ctx)


def unregister(family: str, kind: str) -> None:
    _REGISTRIES[family].pop(kind, None)


class Workspace:
    """Scratch memory of a step: a bump allocator over one device buffer.

    ``take`` hands out aligned views; ``mark``/``release`` free in stack order. The same sequence of
    requests always yields the same addresses, which a captured CUDA graph relies on. When the
    buffer is too small it is replaced by a larger one (``generation`` then changes, and graphs
    captured against the old one must be dropped)."""

    ALIGN = 256

    def __init__(self, device, nbytes: int = 1 << 24):
        self.device = torch.device(device)
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.top = 0
        self.high = 0
        self.generation = 0
        self.frozen = False
        self._views: dict = {}

    def mark(self) -> int:
        return self.top

    def release(self, mark: int) -> None:
        self.top = mark

    _ITEM = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int32: 4, torch.int64: 8, torch.uint8: 1,
             torch.int8: 1, torch.float64: 8, torch.int16: 2, torch.bool: 1}

    def take(self, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * self._ITEM[dtype]
        start = (self.top + self.ALIGN - 1) // self.ALIGN * self.ALIGN
        if start + nbytes > self.buf.numel():
            if self.frozen:
                raise RuntimeError("the step workspace would have to grow while a CUDA graph is being captured")
            grown = max(2 * self.buf.numel(), start + nbytes + (1 << 20))
            self.buf = torch.empty(grown, dtype=torch.uint8, device=self.device)   # earlier views keep the old buffer
            self.generation += 1
            self.top = 0
            start = 0
            self._views.clear()
        self.top = start + nbytes
        if self.top > self.high:
            self.high = self.top
        # the same requests come back step after step at the same places: the views are kept
        key = (start, dtype, tuple(shape))
        view = self._views.get(key)
        if view is None:
            if len(self._views) > 4096:
                self._views.clear()
            view = self.buf[start:start + nbytes].view(dtype).view(*shape)
            self._views[key] = view
        return view
