"""The decoder: embedding part, the layers in their order, final norm, head part.

Built from a :class:`ModelSpec` alone: every layer's parts are looked up by kind, and the
order in which layers run is the spec's ``order`` list (an entry may repeat a layer; a
mixer may read the storage of an earlier layer). The step itself follows
AntoineBut/TileInfer.jl's ``run_step!`` (src/model/decoder.jl:165-196): embed, first norm,
per layer mixer / add+norm / feed-forward / add+norm, and the LM head on the wanted rows
only, with 32-bit logits.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.spec import ModelSpec, TensorDecl
from ..kernels import ops
from ..parts import Linear, Runtime, lookup


def tensor_declarations(spec: ModelSpec) -> List[TensorDecl]:
    """Every checkpoint tensor a model of this spec reads."""
    decls = list(lookup("embedding", spec.embedding_kind).tensors(spec)) + list(lookup("head", spec.head_kind).tensors(spec))
    decls += lookup("norm", spec.final_norm.kind).tensors(spec.final_norm)
    for layer in spec.layers:
        decls += lookup("norm", layer.mixer_norm.kind).tensors(layer.mixer_norm)
        decls += lookup("mixer", layer.mixer.kind).tensors(layer.mixer)
        decls += lookup("norm", layer.feed_forward_norm.kind).tensors(layer.feed_forward_norm)
        decls += lookup("feed_forward", layer.feed_forward.kind).tensors(layer.feed_forward)
    seen, out = set(), []
    for d in decls:
        if d.name not in seen:
            seen.add(d.name)
            out.append(d)
    return out


def ignorable_tensors(spec: ModelSpec) -> List[str]:
    # A tied checkpoint may still store a copy of the head (src/hub/loader.jl:157-163).
    return ["lm_head.weight"] if spec.lm_head_name is None else []


class DecoderModel:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], rt: Runtime, max_positions: int):
        self.spec, self.rt = spec, rt
        self.max_positions = int(min(max_positions, spec.max_positions))
        self.embedding = lookup("embedding", spec.embedding_kind)(spec, tensors, rt)
        self.head = lookup("head", spec.head_kind)(spec, tensors, rt, self.embedding)
        self.final_norm = lookup("norm", spec.final_norm.kind)(spec.final_norm, tensors, rt)
        self._positions: Dict[tuple, object] = {}
        self.blocks = []
        for layer in spec.layers:
            position = self._position(layer.mixer.position)
            mixer = lookup("mixer", layer.mixer.kind)(layer.mixer, tensors, rt, position)
            ffn = lookup("feed_forward", layer.feed_forward.kind)(layer.feed_forward, tensors, rt)
            n1 = lookup("norm", layer.mixer_norm.kind)(layer.mixer_norm, tensors, rt)
            n2 = lookup("norm", layer.feed_forward_norm.kind)(layer.feed_forward_norm, tensors, rt)
            self.blocks.append(lookup("block", layer.block)(layer, mixer, ffn, n1, n2))
        self.status = torch.zeros(1, dtype=torch.int32, device=rt.device)

    def _position(self, pspec):
        key = (pspec.kind, pspec.head_dim, pspec.theta, pspec.scaling, pspec.max_positions, tuple(sorted(pspec.options.items())))
        if key not in self._positions:
            self._positions[key] = lookup("position", pspec.kind)(pspec, self.rt, self.max_positions)
        return self._positions[key]

    # ---- what the cache has to hold, one entry per position of ``order``
    def cache_requests(self):
        return [self.blocks[li].mixer.cache_request() for li in self.spec.order]

    def cache_shares(self) -> Dict[int, int]:
        """occurrence -> the earlier occurrence whose storage it reads."""
        shares, last = {}, {}
        for occ, li in enumerate(self.spec.order):
            src = self.spec.layers[li].mixer.kv_source
            if src is not None:
                if src not in last:
                    raise ValueError(f"layer {li} reads the cache of layer {src}, which has not run before it")
                shares[occ] = last[src]
            last[li] = occ
        return shares

    def weight_bytes(self) -> int:
        """Bytes of every weight a step reads once: the parts' matrices and vectors and the head (a tied
        head counts once). The embedding table is not among them: a step reads one row of it per token.
        Parts are walked through their attributes, lists and dicts included (experts kept in a list
        count); position encodings hold tables, not weights, and are left out."""
        from ..parts.base import Part, PositionEncoding
        seen, total = set(), 0

        def visit(obj):
            nonlocal total
            if isinstance(obj, torch.Tensor):
                if obj.is_floating_point() and obj.numel() > 1 and obj.data_ptr() not in seen:
                    seen.add(obj.data_ptr())
                    total += obj.numel() * obj.element_size()
            elif isinstance(obj, (list, tuple)):
                for v in obj:
                    visit(v)
            elif isinstance(obj, dict):
                for v in obj.values():
                    visit(v)
            elif isinstance(obj, (Part, Linear)) and not isinstance(obj, PositionEncoding) and id(obj) not in seen:
                seen.add(id(obj))
                for v in vars(obj).values():
                    visit(v)

        for b in self.blocks:
            visit([b.mixer, b.feed_forward, b.mixer_norm, b.feed_forward_norm])
        visit([self.final_norm, self.head])
        return total

    def forward(self, step, cache, logits: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        """Run the step's tokens; write the logits of ``step.want_idx`` rows to ``logits``."""
        from ..kernels.library import stream_scope
        with stream_scope():
            return self._forward(step, cache, logits)

    def _forward(self, step, cache, logits: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        rt, spec = self.rt, self.spec
        n = step.n_tokens
        x = rt.buffer("model.x", (n, spec.hidden_size))
        h = rt.buffer("model.h", (n, spec.hidden_size))
        self.embedding.forward(step.token_ids, x, self.status)
        order = spec.order
        self.blocks[order[0]].input_norm.forward(x, h) if order else self.final_norm.forward(x, h)
        for occ, li in enumerate(order):
            nxt = self.blocks[order[occ + 1]].input_norm if occ + 1 < len(order) else self.final_norm
            self.blocks[li].forward(x, h, step, cache.layer(occ), nxt, h)
        if logits is None or step.n_want == 0:
            return None
        hw = rt.buffer("model.h_wanted", (step.n_want, spec.hidden_size))
        ops.gather_rows(hw, h, step.want_idx)
        self.head.forward(hw, logits)
        return logits
