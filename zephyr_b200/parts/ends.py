"""What lies before the first layer and after the last one, as parts.

``embedding``: h[t, :] = E[id[t], :], no scaling (reference: src/layer/embedding.cpp:17-31,
src/model/causal_lm/qwen3.cpp:122-123,169).

``norm_head``: the final norm and the vocabulary projection without bias, for the wanted tokens only
(reference: src/model/causal_lm/qwen3.cpp:133-136,173-180).  The norm is row-wise, so it runs on
the wanted rows alone (the reference norms every token and selects after); the logits come out in
float32 whatever the model's type (the reference stores them in the model's type).  A tied head
names the embedding's tensor and so reads the very same memory.
"""

from __future__ import annotations

from typing import Mapping

import torch

from ..config.spec import InputSpec, OutputSpec
from ..kernels import ops
from ..weights.loader import ROLE_EMBEDDING, ROLE_LINEAR, WeightDecl
from .base import NORMS, InputPart, OutputPart, ResidualStream, StepContext, lookup, register_input, register_output


class Embedding(InputPart):
    graph_safe = True

    def __init__(self, spec: InputSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        self.table = weights[spec.params["weight"]]

    @staticmethod
    def weight_decls(spec: InputSpec) -> dict[str, WeightDecl]:
        p = spec.params
        return {p["weight"]: WeightDecl((int(p["vocab_size"]), int(p["hidden_size"])), ROLE_EMBEDDING)}

    def weights_read(self) -> list[torch.Tensor]:
        return []          # a step gathers a few rows of the table; it does not stream it

    def forward(self, ctx: StepContext) -> torch.Tensor:
        return ops.embedding(self.table, ctx.token_ids, ctx.status)


class NormHead(OutputPart):
    graph_safe = True

    def __init__(self, spec: OutputSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype):
        p = spec.params
        self.vocab_size = int(p["vocab_size"])
        self.norm = lookup(NORMS, "norm", p["norm"].kind)(p["norm"], weights, dtype)
        self.weight = weights[p["weight"]]

    @staticmethod
    def weight_decls(spec: OutputSpec) -> dict[str, WeightDecl]:
        p = spec.params
        decls = dict(lookup(NORMS, "norm", p["norm"].kind).weight_decls(p["norm"]))
        # A name the input part declares too (a tied head) keeps the role it was given first.
        decls[p["weight"]] = WeightDecl((int(p["vocab_size"]), int(p["hidden_size"])), ROLE_LINEAR)
        return decls

    def weights_read(self) -> list[torch.Tensor]:
        return [self.weight, *self.norm.weights_read()]

    def forward(self, stream: ResidualStream, ctx: StepContext) -> torch.Tensor:
        wanted = ctx.logit_tokens
        if wanted.numel() == 0:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=stream.hidden.device)
        rows = ops.gather_rows(stream.hidden, wanted, ctx.status)
        if stream.pending is not None:
            normed = self.norm.add_forward(rows, ops.gather_rows(stream.pending, wanted, ctx.status))
        else:
            normed = self.norm.forward(rows)
        return ops.linear(normed, self.weight, out_dtype=torch.float32)


register_input("embedding", Embedding)
register_output("norm_head", NormHead)
