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
from ..kernels import ops
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
        for layer in spec.layers:
            block_cls = lookup("block", layer.block)
            self.blocks.append(block_cls(
                build_part("mixer", layer.mixer, runtime), build_part("feed_forward", layer.feed_forward, runtime),
                build_part("norm", layer.mixer_norm, runtime), build_part("norm", layer.feed_forward_norm, runtime),
                runtime))
        self.final_norm = build_part("norm", spec.final_norm, runtime)
        self.embedding: torch.Tensor = None
        self.head: Linear = None

        # cache units: one per schedule entry that owns its cache
        self.unit_requests: List[List[object]] = []
        self.unit_of_entry: List[int] = []
        for pos, call in enumerate(spec.schedule):
            if call.cache_of is None:
                self.unit_of_entry.append(len(self.unit_requests))
                self.unit_requests.append(list(self.blocks[call.layer].mixer.cache_requests()))
            else:
                self.unit_of_entry.append(self.unit_of_entry[call.cache_of])

    # ------------------------------------------------------------------ checkpoint tensors
    def _layer_parts(self) -> List[Tuple[str, Part]]:
        out = []
        for i, (layer, block) in enumerate(zip(self.spec.layers, self.blocks)):
            prefix = self.spec.layer_prefix.format(i=i)
            for role, part in block.parts().items():
                out.append((prefix + layer.names[role] + ".", part))
        return out

    def param_specs(self) -> Dict[str, ParamSpec]:
        """Every checkpoint tensor this model reads, by full name."""
        specs = {self.spec.embedding_name: ParamSpec((self.vocab_size, self.hidden_size))}
        for prefix, part in self._layer_parts():
            for local, ps in part.param_specs().items():
                specs[prefix + local] = ps
        for local, ps in self.final_norm.param_specs().items():
            specs[self.spec.final_norm_name + "." + local] = ps
        if not self.spec.tie_head:
            specs[self.spec.head_name] = ParamSpec((self.vocab_size, self.hidden_size))
        return specs

    def load_tensors(self, tensors: Dict[str, torch.Tensor]) -> None:
        """tensors: full name -> device tensor, for exactly the names of param_specs()."""
        self.embedding = tensors[self.spec.embedding_name].contiguous()
        for prefix, part in self._layer_parts():
            part.load({local: tensors[prefix + local] for local in part.param_specs()})
        self.final_norm.load({local: tensors[self.spec.final_norm_name + "." + local]
                              for local in self.final_norm.param_specs()})
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
        ops.embedding(ctx.tokens, self.embedding, h)
        pending = None
        for pos, call in enumerate(self.spec.schedule):
            unit = cache.unit(self.unit_of_entry[pos])
            h, pending = self.blocks[call.layer].forward(h, pending, ctx, unit, call.cache_of is None)
        if pending is None and ctx.all_rows and self.head.weight.dtype == torch.bfloat16 \
                and self.vocab_size % 16 == 0:
            x = self.final_norm.defer(h)
            if x is not None and x.kind == "rmsnorm":
                # one-token steps: final norm and head in one kernel
                logits = torch.empty((h.shape[0], self.vocab_size), dtype=torch.float32, device=h.device)
                return ops.norm_gemm_f32(x.h, x.weight, x.eps, self.head.weight, logits)
        x = self.final_norm.forward(h, pending, rows=ctx.logit_rows)
        return self.head(x, out_dtype=torch.float32)
