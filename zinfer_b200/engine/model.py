"""A decoder assembled from a :class:`ModelSpec`: embedding, the scheduled runs of
its layers, final norm, output head.  The model knows nothing of Qwen3; the family
function decided the parts and their parameters
(the reference's stack: src/model/layers/decoder_only_stack.zig:48-93).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from .. import ops
from ..cache.storage import CacheStorage
from ..config.spec import ModelSpec
from ..parts.base import BuildContext, KVCacheNeed, StateNeed, TensorSpec, make_part, prefixed, take


EMBEDDING_STATE = "embedding"      # name of the state an embedding keeps per request (its last token)


@dataclass(frozen=True)
class Run:
    """One scheduled execution of a layer with the cache it uses."""

    layer: int
    cache: str
    writes: bool
    pre_add: Optional[tuple[str, int]] = None
    pre_add_input: bool = False


def _plan_runs(spec: ModelSpec) -> list[Run]:
    runs, seen = [], set()
    for i, e in enumerate(spec.schedule):
        name = e.cache if e.cache is not None else f"run{i}"
        runs.append(Run(e.layer, name, writes=name not in seen, pre_add=e.pre_add, pre_add_input=e.pre_add_input))
        seen.add(name)
    return runs


class DecoderModel:
    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device, max_positions: Optional[int] = None):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise ValueError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        self.max_positions = min(spec.max_positions, max_positions) if max_positions else spec.max_positions
        self.ctx = BuildContext(device=self.device, dtype=dtype, max_positions=self.max_positions)
        self.embedding = make_part(spec.embedding, self.ctx)
        self.blocks = [make_part(layer.block, self.ctx) for layer in spec.layers]
        self.final_norm = make_part(spec.final_norm, self.ctx)
        self.head = make_part(spec.head, self.ctx)
        self.runs = _plan_runs(spec)
        self._views: list = []
        self._embedding_view = None
        self.tables: dict[str, torch.Tensor] = {}

    # ----------------------------------------------------------------- weights
    def _final_norm_prefix(self) -> str:
        params = self.spec.final_norm.params
        return params["prefix"] if "prefix" in params else params.get("name", "norm") + "."

    def tensor_specs(self) -> dict[str, TensorSpec]:
        out = dict(self.embedding.tensor_specs())
        for layer, block in zip(self.spec.layers, self.blocks):
            out.update(prefixed(layer.prefix, block.tensor_specs()))
        out.update(prefixed(self._final_norm_prefix(), self.final_norm.tensor_specs()))
        out.update(self.head.tensor_specs())
        for name, shape in self.spec.tables:
            out[name] = TensorSpec(tuple(shape))
        return out

    def bind(self, tensors: dict[str, torch.Tensor]) -> None:
        self.embedding.bind(tensors)
        for layer, block in zip(self.spec.layers, self.blocks):
            block.bind(take(tensors, layer.prefix))
        self.final_norm.bind(take(tensors, self._final_norm_prefix()))
        self.head.bind(tensors)
        if getattr(self.head, "tied_to", None) is not None:
            self.head.tie(self.embedding.weight)
        # vectors added to the 32-bit residual stream are kept in 32-bit
        self.tables = {name: tensors[name].to(torch.float32).contiguous() for name, _ in self.spec.tables}

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        for t in self.tables.values():
            seen.add(t.data_ptr())
            total += t.numel() * t.element_size()
        for part in [self.embedding, self.final_norm, self.head, *self.blocks]:
            stack = [part]
            while stack:
                p = stack.pop()
                for v in vars(p).values():
                    if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                        seen.add(v.data_ptr())
                        total += v.numel() * v.element_size()
                    elif hasattr(v, "tensor_specs"):
                        stack.append(v)
        return total

    # ------------------------------------------------------------------- caches
    def cache_needs(self) -> tuple[dict[str, KVCacheNeed], dict[str, StateNeed]]:
        kv, state = {}, {}
        emb = self._embedding_need()
        if emb is not None:
            state[EMBEDDING_STATE] = emb
        for run in self.runs:
            for name, need in self._needs_of(run).items():
                prev = kv.get(name, state.get(name))
                if isinstance(prev, KVCacheNeed) and isinstance(need, KVCacheNeed) and prev.same_pages(need):
                    need = prev.merged(need)     # runs that share pages may look back differently far: keep the most
                elif prev is not None and prev != need:
                    raise ValueError(f"cache {name!r} is shared by layers with different needs: {prev} and {need}")
                if isinstance(need, KVCacheNeed):
                    kv[name] = need
                elif isinstance(need, StateNeed):
                    state[name] = need
                else:
                    raise TypeError(f"layer {run.layer}: unknown cache need {need!r}")
        return kv, state

    def _embedding_need(self) -> Optional[StateNeed]:
        """An embedding that looks at the token before keeps per-request state of its own."""
        need = getattr(self.embedding, "cache_need", None)
        return need() if need is not None else None

    def _needs_of(self, run: Run) -> dict:
        """The caches and states a run uses, by name.  A mixer needs one (named like the run's cache), none, or
        several (a dictionary part -> need: a mixer of several branches; named ``<run's cache>.<part>``)."""
        need = self.blocks[run.layer].mixer.cache_need()
        if need is None:
            return {}
        if isinstance(need, dict):
            return {f"{run.cache}.{part}": n for part, n in need.items() if n is not None}
        return {run.cache: need}

    def _view(self, storage: CacheStorage, name: str, writes: bool, kv: dict, state: dict):
        if name in kv:
            return storage.kv_view(name, writes)
        if name in state:
            return storage.state_view(name, writes)
        return None

    def attach(self, storage: CacheStorage) -> None:
        """Binds every run to its view of the cache storage."""
        kv, state = self.cache_needs()
        self._embedding_view = storage.state_view(EMBEDDING_STATE) if EMBEDDING_STATE in state else None
        self._views = []
        for run in self.runs:
            need = self.blocks[run.layer].mixer.cache_need()
            if isinstance(need, dict):     # a mixer of several branches gets its views by the branches' names
                self._views.append({part: self._view(storage, f"{run.cache}.{part}", run.writes, kv, state) for part in need})
            else:
                self._views.append(self._view(storage, run.cache, run.writes, kv, state))

    # ------------------------------------------------------------------ forward
    def forward(self, step, argmax: bool = False):
        """Runs the step's tokens through every scheduled layer (filling the caches)
        and returns 32-bit logits [wanted rows, vocab], or None if none are wanted.
        With ``argmax`` it returns the pair (logits, first maximum of every row as int32)."""
        if self._embedding_view is not None:
            h = self.embedding.forward(step.token_ids, step, self._embedding_view)
        else:
            h = self.embedding.forward(step.token_ids)
        # the stream is updated in place: a stack that feeds its input in again keeps a copy of it
        h0 = h.clone() if any(run.pre_add_input for run in self.runs) else None
        pending = None
        for run, view in zip(self.runs, self._views):
            if run.pre_add_input:        # one more update that the run's norm adds with the others
                pending = ops.Several([pending, h0])
            if run.pre_add is None:
                pending = self.blocks[run.layer].forward(h, pending, step, view)
            else:
                name, row = run.pre_add
                pending = self.blocks[run.layer].forward(h, pending, step, view, bias=self.tables[name][row])
        if step.logit_rows is None or step.logit_rows.numel() == 0:
            return (None, None) if argmax else None
        x = self.final_norm.forward(h, pending, rows=step.logit_rows)
        if not argmax:
            return self.head.forward(x)
        if hasattr(self.head, "forward_argmax"):     # a head may find the maxima while it makes the logits
            return self.head.forward_argmax(x)
        logits = self.head.forward(x)
        return logits, ops.argmax(logits)


def declared_tensors(spec: ModelSpec) -> dict[str, TensorSpec]:
    """The tensors a model of this spec needs; builds no device memory."""
    return DecoderModel(spec, torch.float32, "cpu").tensor_specs()
