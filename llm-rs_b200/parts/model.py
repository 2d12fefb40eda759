"""A decoder model assembled from a ``ModelSpec``: embedding, blocks in run order, final
norm, output head. It knows parts and their interfaces, not architectures."""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .base import Runtime
from .registry import build
from .spec import CacheNeed, ModelSpec, StateNeed, WeightSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        spec.validate()
        self.spec = spec
        self.embedding = build("embedding", spec.embedding)
        self.blocks = [build("block", layer.block, layer=layer) for layer in spec.layers]
        self.final_norm = build("norm", spec.final_norm)
        self.lm_head = build("lm_head", spec.lm_head)

    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.lm_head]

    def weight_specs(self) -> List[WeightSpec]:
        seen: Dict[str, WeightSpec] = {}
        for part in self.parts():
            for s in part.weight_specs():
                if s.name in seen and seen[s.name].shape != s.shape:
                    raise ValueError(f"two parts want {s.name} with shapes {seen[s.name].shape} and {s.shape}")
                seen.setdefault(s.name, s)
        return list(seen.values())

    def bind(self, tensors: Dict[str, torch.Tensor], runtime: Runtime) -> None:
        self.runtime = runtime
        for part in self.parts():
            part.bind(tensors, runtime)
        # Every product learns which weights are streamed after its own (see ``Part.chain``).
        order = [lin for step in self.spec.run_order for lin in getattr(self.blocks[step.layer], "chain", list)()]
        order += getattr(self.lm_head, "chain", list)()
        for lin, after in zip(order, order[1:]):
            lin.next_weight = after.weight if lin.warms_next and after.weight.dtype == torch.bfloat16 else None

    def cache_needs(self) -> List[Tuple[Optional[CacheNeed], Optional[StateNeed]]]:
        """Per run-order entry: the pages and the state its mixer wants. An entry that
        reads another entry's cache wants nothing of its own."""
        needs = []
        for step in self.spec.run_order:
            if step.cache_of is not None:
                needs.append((None, None))
            else:
                mixer = self.blocks[step.layer].mixer
                needs.append((mixer.cache_need(), mixer.state_need()))
        return needs

    def forward(self, ctx) -> Optional[torch.Tensor]:
        """Run the step's tokens through every run-order entry; float32 logits of the
        wanted rows ([wanted, vocab]), or None when nothing is wanted."""
        h = self.embedding.forward(ctx.token_ids)
        pending = None
        order = self.spec.run_order
        for s, step in enumerate(order):
            block = self.blocks[step.layer]
            after = self.blocks[order[s + 1].layer] if s + 1 < len(order) else None
            if (getattr(block, "links_norms", False) and getattr(after, "links_norms", False)
                    and after.accepts_prenormed(ctx.n_tokens)):
                # The norm between the two blocks is spread over this block's last product and the next one's first.
                h, pending = block.forward(h, pending, ctx, ctx.layer_cache(s), next_norm=after.mixer_norm.link())
            else:
                h, pending = block.forward(h, pending, ctx, ctx.layer_cache(s))
        if ctx.n_want == 0:
            return None
        x = self.final_norm.forward(h, pending, rows=ctx.want_rows)
        return self.lm_head.forward(x)
