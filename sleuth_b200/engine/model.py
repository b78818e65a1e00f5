"""A model as the engine sees it: an embedding, layers built from a description, a schedule, a head.

``Model`` knows nothing about any architecture. It builds each layer from its ``LayerSpec`` through
the part registries, collects the tensors the parts declare under the names the description gives
them, asks the parts what their cache entries must hold, and runs ``ModelSpec.schedule``: a list of
layer applications that may name a layer twice (its weights are then shared and each application has
a cache entry of its own, as the reference's ``shared_layers``, sleuth/forge/model/config.py:80-86)
or let an application read the cache entry an earlier one wrote.

One forward pass is the reference's ``Transformer.forward`` (sleuth/forge/model/transformer.py:257-313)
for a ragged batch: embed, run the layers on the float32 stream, final norm and output matrix on the
rows whose logits are wanted only.
"""

from __future__ import annotations

import os

import torch

from ..parts import ends as _ends   # noqa: F401  (registers the token embedding and the output head)
from ..parts.base import BuildContext, ParamDecl, build_embedding, build_head, build_layer, lead_weight_of
from ..parts.spec import ModelSpec


# How a step in which every sequence brings one token runs: "fused" = runs of layers whose parts offer it go through
# the persistent kernel (csrc/decode_layers.cu), up to FUSED_DECODE_ROWS sequences; "kernels" = every layer launch
# by launch, as steps of many tokens always run.
DECODE_CHOICE = os.environ.get("SLEUTH_B200_DECODE", "kernels")
FUSED_DECODE_ROWS = 16
FUSED_DECODE_MIN_SLOTS = 5      # ring slots the kernel must have left beside the token rows in shared memory


class Model:
    def __init__(self, spec: ModelSpec, ctx: BuildContext):
        self.spec, self.ctx = spec, ctx
        self.embedding = build_embedding(spec.embedding, ctx)      # by ``spec.kind``, like every other part
        self.layers = [build_layer(ls, ctx) for ls in spec.layers]
        self.head = build_head(spec.head, ctx)
        self.hidden = spec.embedding.dim
        self.vocab = spec.head.vocab
        # single-token steps are recorded as CUDA graphs only if every layer allows it
        self.capturable = all(getattr(part, "capturable", True) for part in (self.embedding, *self.layers, self.head))
        # cache entries: the first application that names an entry owns it
        self.entry_owner: dict[int, int] = {}
        for i, e in enumerate(spec.schedule):
            self.entry_owner.setdefault(e.cache, i)
        self.cache_requests = [self.layers[spec.schedule[self.entry_owner[c]].layer].cache_request()
                               for c in range(len(self.entry_owner))]
        self._programs: dict = {}       # per cache: the runs of the schedule prepared for the persistent kernel

    # ---- weights ----
    def _end_names(self, which: str) -> dict[str, str]:
        """Checkpoint names of the tensors an end part declares: ``weight`` (and the head's ``norm.weight``) from the
        spec's own fields, anything else from the spec's ``names``."""
        spec = getattr(self.spec, which)
        part = getattr(self, which)
        given = dict(getattr(spec, "names", {}) or {})
        given.setdefault("weight", spec.name)
        if which == "head":
            given.setdefault("norm.weight", spec.norm_name)
        out = {}
        for local in part.declare():
            if local not in given:
                raise KeyError(f"{which}: its description gives no checkpoint name for tensor {local!r}")
            out[local] = given[local]
        return out

    def expected(self) -> dict[str, ParamDecl]:
        out = {}
        emb = self.embedding.declare()
        for local, name in self._end_names("embedding").items():
            out[name] = emb[local]
        for i, (layer, ls) in enumerate(zip(self.layers, self.spec.layers)):
            for local, decl in layer.declare().items():
                if local not in ls.names:
                    raise KeyError(f"layer {i}: its description gives no checkpoint name for tensor {local!r}")
                out[ls.names[local]] = decl
        hd = self.head.declare()
        for local, name in self._end_names("head").items():
            out[name] = hd[local]
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.embedding.bind({local: tensors[name] for local, name in self._end_names("embedding").items() if name in tensors})
        for layer, ls in zip(self.layers, self.spec.layers):
            layer.bind({local: tensors[ls.names[local]] for local in layer.declare() if ls.names[local] in tensors})
        head = {local: tensors[name] for local, name in self._end_names("head").items() if name in tensors}
        self.head.bind(head, embedding_table=getattr(self.embedding, "table", None))

    # ---- one step ----
    def forward(self, b, cache, ws, logits: torch.Tensor) -> torch.Tensor:
        """Run the tokens of batch ``b``; fill ``logits`` [len(b.rows), vocab] (float32)."""
        b.stream = torch.cuda.current_stream().cuda_stream   # inside a graph capture this is the capture stream
        mark = ws.mark()
        x = ws.take((b.T, self.hidden), torch.float32)
        self.embedding.forward(b, x)
        schedule = self.spec.schedule
        fused = self._fused_runs(b, cache)
        i = 0
        while i < len(schedule):
            if i in fused:
                i = self._run_fused(fused[i], x, b, ws)
                continue
            e = schedule[i]
            view = cache.view(e.cache, writes=self.entry_owner[e.cache] == i)
            following = self.layers[schedule[i + 1].layer] if i + 1 < len(schedule) and (i + 1) not in fused else None
            b.next_read = lead_weight_of(following)
            self.layers[e.layer].forward(x, b, view, ws)
            i += 1
        b.next_read = None
        if logits.shape[0]:
            self.head.forward(x, b, logits, ws)
        ws.release(mark)
        return logits

    # ---- single-token steps through the persistent kernel ----
    def _fused_runs(self, b, cache) -> dict:
        """{first schedule index: (index after the run, program)} for this step, or {} when it does not qualify: every
        sequence brings one token, at most FUSED_DECODE_ROWS of them, in bfloat16."""
        if (DECODE_CHOICE != "fused" or self.ctx.dtype != torch.bfloat16 or b.max_count != 1 or b.T != b.n
                or not 1 <= b.n <= FUSED_DECODE_ROWS):
            return {}
        runs = self._programs.get(id(cache))
        if runs is None:
            runs = self._programs[id(cache)] = self._prepare_runs(cache)
        return {start: (end, prog) for start, end, prog in runs if prog.slots_for(b.n)[0] >= FUSED_DECODE_MIN_SLOTS}

    def _prepare_runs(self, cache) -> list:
        """Maximal runs of consecutive layer applications whose layers offer ``fused_decode`` and own their cache entry."""
        from ..kernels import ops
        runs, cur = [], []
        schedule = self.spec.schedule

        def close():
            if cur:
                prog = ops.decode_program([s for _, s, _ in cur], [v for _, _, v in cur], cache.pools)
                if prog is not None:
                    runs.append((cur[0][0], cur[-1][0] + 1, prog))
                cur.clear()

        for i, e in enumerate(schedule):
            offer = getattr(self.layers[e.layer], "fused_decode", lambda: None)()
            view = cache.view(e.cache, writes=True) if offer is not None and self.entry_owner[e.cache] == i else None
            if offer is None or view is None or not hasattr(view, "k_pool"):
                close()
                continue
            if cur and (offer["mixer"]["head_dim"] != cur[0][1]["mixer"]["head_dim"]):
                close()
            cur.append((i, offer, view))
        close()
        return runs

    def _run_fused(self, run, x, b, ws) -> int:
        from ..kernels import ops
        end, prog = run
        mark = ws.mark()
        qkv = ws.take((b.n, prog.max_qkv), torch.bfloat16)
        y = ws.take((b.n, prog.max_heads), torch.bfloat16)
        act = ws.take((b.n, prog.max_inter), torch.bfloat16)
        parts = ws.take((ops.decode_layers_scratch_floats(prog, b.n, ops.sm_count(x.device)),), torch.float32)
        ops.decode_layers(prog, x, b.past, b.tables, qkv, y, act, parts, b.stream, trace=getattr(self, "decode_trace", None))
        ws.release(mark)
        return end

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self._all_tensors():
            if t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                total += t.numel() * t.element_size()
        return total

    def _all_tensors(self):
        """The tensors the parts hold: attributes that are tensors, or objects with a tensor ``weight`` (a product,
        a norm), looked for in the end parts and in each layer's ``children``."""
        parts = [self.embedding, self.head]
        for layer in self.layers:
            parts.extend(getattr(layer, "children", {}).values())
        for part in parts:
            for v in vars(part).values():
                if isinstance(v, torch.Tensor):
                    yield v
                elif isinstance(getattr(v, "weight", None), torch.Tensor):
                    yield v.weight


def declare_model(spec: ModelSpec) -> dict[str, ParamDecl]:
    """The tensors a model description expects, found without a GPU."""
    ctx = BuildContext(device=torch.device("cpu"), dtype=torch.float32, max_positions=1)
    return Model(spec, ctx).expected()
