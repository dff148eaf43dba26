"""A decoder put together from a `ModelSpec`: embedding, the layers in schedule order, final
norm, head. It knows parts only through their interfaces and checkpoint tensors only through
the names the spec gives; which architecture the spec came from is not visible here.

Forward = one step over the tokens it is given (src/model.py:145-185 of the reference is the
same walk for one dense batch): gather embeddings into a float32 residual stream, run each
schedule entry's block on its cache unit, normalise only the rows whose logits are wanted, and
multiply by the head; logits are float32.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import torch

from ..config.spec import ModelSpec
from ..kernels import ops, trace
from ..parts.base import Block, ParamSpec, Part, Runtime, build_part, lookup
from ..parts.linear import Linear


class DecoderModel:
    def __init__(self, spec: ModelSpec, runtime: Runtime):
        spec.validate()
        self.spec = spec
        self.runtime = runtime
        self.hidden_size = spec.hidden_size
        self.vocab_size = spec.vocab_size
        self.blocks: List[Block] = []
        for i, layer in enumerate(spec.layers):
            block_cls = lookup("block", layer.block)
            roles = block_cls.ROLES
            if set(roles) != set(layer.parts):
                raise ValueError(f"layer {i}: block {layer.block!r} has the roles {sorted(roles)}, the layer names "
                                 f"{sorted(layer.parts)}")
            self.blocks.append(block_cls({role: build_part(group, layer.parts[role], runtime)
                                          for role, group in roles.items()}, runtime))
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.after_embedding = build_part("pointwise", spec.after_embedding, runtime) if spec.after_embedding else None
        self.after_head = build_part("pointwise", spec.after_head, runtime) if spec.after_head else None
        self.embedding: torch.Tensor = None
        self.head: Linear = None

        # cache units: one per schedule entry that owns its cache
        self.unit_requests: List[List[object]] = []
        self.unit_of_entry: List[int] = []
        for pos, call in enumerate(spec.schedule):
            if call.cache_of is None:
                self.unit_of_entry.append(len(self.unit_requests))
                self.unit_requests.append(list(self.blocks[call.layer].cache_requests()))
            else:
                self.unit_of_entry.append(self.unit_of_entry[call.cache_of])

    # ------------------------------------------------------------------ checkpoint tensors
    def _named_parts(self) -> List[Tuple[str, Part]]:
        out = []
        for i, (layer, block) in enumerate(zip(self.spec.layers, self.blocks)):
            prefix = self.spec.layer_prefix.format(i=i)
            for role, part in block.parts().items():
                out.append((prefix + layer.names[role] + ".", part))
        out.append((self.spec.final_norm_name + ".", self.final_norm))
        if self.after_embedding is not None:
            out.append((self.spec.after_embedding_name + ".", self.after_embedding))
        if self.after_head is not None:
            out.append((self.spec.after_head_name + ".", self.after_head))
        return out

    def param_specs(self) -> Dict[str, ParamSpec]:
        """Every checkpoint tensor this model reads, by full name."""
        specs = {self.spec.embedding_name: ParamSpec((self.vocab_size, self.hidden_size))}
        for prefix, part in self._named_parts():
            for local, ps in part.param_specs().items():
                specs[prefix + local] = ps
        if not self.spec.tie_head:
            specs[self.spec.head_name] = ParamSpec((self.vocab_size, self.hidden_size))
        return specs

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """tensors: full name -> device tensor, for exactly the names of param_specs()."""
        self.embedding = tensors[self.spec.embedding_name].contiguous()
        for prefix, part in self._named_parts():
            part.load({local: tensors[prefix + local] for local in part.param_specs()})
        self.head = Linear(self.embedding if self.spec.tie_head else tensors[self.spec.head_name])

    def weight_bytes_per_step(self) -> int:
        """Bytes of weights a decode step has to read once: every layer the schedule runs, the
        final norm and the head (the embedding rows gathered are negligible)."""
        total = self.head.nbytes() + self.final_norm.weight_bytes()
        for call in self.spec.schedule:
            total += sum(p.weight_bytes() for p in self.blocks[call.layer].parts().values())
        return total

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, cache) -> torch.Tensor:
        h = torch.empty((ctx.n_tokens, self.hidden_size), dtype=torch.float32, device=self.runtime.device)
        trace.push("Embed")
        ops.embedding(ctx.tokens, self.embedding, h)
        if self.after_embedding is not None:
            h = self.after_embedding.forward(h, ctx)
        trace.pop()
        pending = None
        trace.push("Layers")
        for pos, call in enumerate(self.spec.schedule):
            unit = cache.unit(self.unit_of_entry[pos])
            ctx.entry = pos
            h, pending = self.blocks[call.layer].forward(h, pending, ctx, unit, call.cache_of is None)
        trace.pop()
        trace.push("Output")
        logits = None
        if pending is None and ctx.all_rows and self.head.weight.dtype == torch.bfloat16 \
                and self.vocab_size % 16 == 0:
            x = self.final_norm.defer(h)
            if x is not None and x.kind == "rmsnorm":
                # one-token steps: final norm and head in one kernel
                logits = torch.empty((h.shape[0], self.vocab_size), dtype=torch.float32, device=h.device)
                ops.norm_gemm_f32(x.h, x.weight, x.eps, self.head.weight, logits)
        if logits is None:
            x = self.final_norm.forward(h, pending, rows=ctx.logit_rows)
            logits = self.head(x, out_dtype=torch.float32)
        if self.after_head is not None:
            logits = self.after_head.forward(logits, ctx, rows=ctx.logit_rows)
        trace.pop()
        return logits
