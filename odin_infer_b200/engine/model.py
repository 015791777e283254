"""A running model put together from a ModelSpec: embedding, blocks in schedule
order, final norm, head.  Architecture-independent."""
from __future__ import annotations

import torch

from ..parts.base import ParamSpec, build_part, split_update, update_factor
from ..parts.spec import ModelSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.embedding = build_part("embedding", spec.embedding)
        self.position_encodings = {n: build_part("position_encoding", s) for n, s in spec.position_encodings.items()}
        self.layers = [build_part("block", s) for s in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.head = build_part("head", spec.head)
        for e in spec.schedule:
            if not (0 <= e.layer < len(self.layers)):
                raise ValueError(f"the schedule names layer {e.layer}; there are {len(self.layers)}")
        for blk in self.layers:
            name = getattr(blk.mixer, "pe_name", None)
            if name is not None:
                if name not in self.position_encodings:
                    raise ValueError(f"a mixer asks for position encoding '{name}', which the model does not define")
                pe = self.position_encodings[name]
                layout = getattr(pe, "layout", "halves")
                if layout not in getattr(blk.mixer, "rope_layouts", ("halves",)):
                    raise ValueError(f"{type(blk.mixer).__name__} does not rotate in the '{layout}' layout of encoding '{name}'")
                blk.mixer.pe = pe

    def _all_parts(self):
        return [self.embedding, *self.position_encodings.values(), *self.layers, self.final_norm, self.head]

    def params(self) -> list[ParamSpec]:
        seen, out = set(), []
        for part in self._all_parts():
            for p in part.params():
                if p.name not in seen:
                    seen.add(p.name)
                    out.append(p)
        out += [ParamSpec(n, (), optional=True) for n in self.spec.tolerated_tensors if n not in seen]
        return out

    def kernel_groups(self) -> set[str]:
        return set().union(*(p.kernel_groups() for p in self._all_parts()))

    @property
    def graph_safe(self) -> bool:
        """May a step of this model be captured in a CUDA graph and replayed (see Part.graph_safe)?"""
        return all(p.graph_safe for p in self._all_parts())

    def parts_not_graph_safe(self) -> list[str]:
        out = []
        for p in self._all_parts():
            inner = getattr(p, "_parts", None)
            for q in (inner() if inner is not None else [p]):
                if not q.graph_safe:
                    out.append(type(q).__name__)
        return sorted(set(out))

    def notes(self, rt) -> list[str]:
        """Every part's notes, each once."""
        out: list[str] = []
        for part in self._all_parts():
            for n in part.notes(rt):
                if n not in out:
                    out.append(n)
        return out

    def bind(self, tensors: dict[str, torch.Tensor], rt, n_positions: int) -> None:
        for part in self._all_parts():
            part.bind(tensors, rt)
        for pe in self.position_encodings.values():
            pe.prepare(rt, n_positions)

    def register_cache(self, cache) -> None:
        """Tell the cache what every schedule entry keeps."""
        writes = []
        requests = [self.layers[e.layer].mixer.cache_request() for e in self.spec.schedule]
        for idx, e in enumerate(self.spec.schedule):
            mixer = self.layers[e.layer].mixer
            kv = requests[idx]
            if kv is not None and e.reads_cache_of is None:
                # a line keeps what its writer and every entry that reads it can see
                readers = [requests[j] for j, o in enumerate(self.spec.schedule)
                           if o.reads_cache_of == idx and requests[j] is not None]
                kv = type(kv).keeping_for_all([kv] + readers)
            cache.add_entry(kv, mixer.state_bytes(), e.reads_cache_of)
            writes.append(e.reads_cache_of is None)
        # an embedding that keeps something per sequence (the token before) gets a state entry after the layers'
        own = getattr(self.embedding, "state_bytes", lambda: 0)()
        if own > 0:
            self.embedding.state_entry = cache.add_entry(None, own)
            writes.append(False)
        cache.entry_writes = writes

    def forward(self, rt, step) -> torch.Tensor | None:
        """Runs the step's tokens; returns 32-bit logits [wanted rows, vocab] (None if none wanted)."""
        x = self.embedding.forward(rt, step)
        for pe in self.position_encodings.values():
            pe.on_embedding(rt, step, x)
        pending = None
        for idx, e in enumerate(self.spec.schedule):
            x, pending = self.layers[e.layer].forward(rt, step, x, pending, idx)
        if step.n_logit_rows == 0:
            return None
        delta, bias = split_update(pending)
        more = {}
        if update_factor(pending) != 1.0:
            if not self.final_norm.takes_scale:
                raise TypeError(f"{type(self.final_norm).__name__} follows a block whose update carries a factor, and takes none")
            more["scale"] = update_factor(pending)
        if bias is not None:
            more["bias"] = bias
        h = self.final_norm.forward(rt, x, delta, rows=step.logit_rows, **more)
        return self.head.forward(rt, step, h)
