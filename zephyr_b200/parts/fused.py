"""Decode steps of a few tokens as fused chains of small products.

A pre-norm residual layer whose mixer is  out(core(in(x)))  and whose feed-forward is
down(silu(gate(x)) * up(x))  is, between two calls of ``core``, a chain of four products with
residual sums and RMS norms between them:

    o     = core_out  W_out^T
    act   = silu * up of  rmsnorm(residual + o) W_gate_up^T          (the sum becomes the residual)
    down  = act  W_down^T
    proj' = rmsnorm(residual + down)  W_in'^T                        (the next layer's mixer input)

``kernels.ops.fused_chain`` runs such a chain in one cooperative launch.  This module only plans:
it asks each block what it is made of (``Block.chain_plan``, built from what the parts themselves
offer) and, if every layer of the run order answers, runs a step as

    proj_0 = rmsnorm(embedding) W_in^T;  for each call:  core;  the chain above

No part learns anything about the model; a model with a block, mixer, feed-forward or norm that
does not offer its pieces simply takes the general path.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch

from ..config.spec import LayerCall
from ..kernels import ops


@dataclass
class BlockPlan:
    """What a pre-norm residual block is made of, as the chain needs it."""

    mixer: object                              # offers projections(call) and core(projected, ctx, call)
    mixer_norm: tuple[torch.Tensor, float]     # (scale, eps)
    feed_forward_norm: tuple[torch.Tensor, float]
    w_gate_up: torch.Tensor                    # blocks of 8 gate rows and their 8 up rows
    w_down: torch.Tensor


def run_stages(stages: list, tokens: int, status: torch.Tensor) -> None:
    """The stages in order: runs of stages the chain kernel takes as one launch each, the others
    as kernels of their own (norm, product, activation) that leave the same tensors behind."""
    run: list = []
    for stage in stages:
        if ops.fused_chain_stage_supported(tokens, stage.w, stage.norm_w is not None, stage.swiglu):
            run.append(stage)
            continue
        if run:
            ops.fused_chain(run, tokens, status)
            run = []
        if stage.norm_w is None:
            x = stage.x
        elif stage.delta is None:
            x = ops.rmsnorm(stage.residual_in, stage.norm_w, stage.eps)
        else:
            stage.residual_out.copy_(stage.residual_in)
            x = ops.add_rmsnorm(stage.residual_out, stage.delta, stage.norm_w, stage.eps)
        stage.y.copy_(ops.gemm_small(x, stage.w, swiglu=stage.swiglu))
    if run:
        ops.fused_chain(run, tokens, status)


class DecodeChains:
    """The fused path of a whole model for steps of up to ``ops.FUSED_CHAIN_MAX_TOKENS`` tokens."""

    def __init__(self, plans: Sequence[BlockPlan], run_order: Sequence[LayerCall], hidden: int):
        self.plans = list(plans)
        self.run_order = list(run_order)
        self.hidden = hidden
        self._supported: dict[int, bool] = {}       # tokens -> whether steps of that size take this path

    @classmethod
    def build(cls, layers: Sequence[object], run_order: Sequence[LayerCall], hidden: int,
              dtype: torch.dtype) -> "DecodeChains | None":
        if dtype != torch.bfloat16 or not run_order:
            return None
        plans = []
        for block in layers:
            plan = block.chain_plan() if hasattr(block, "chain_plan") else None
            if plan is None:
                return None
            plans.append(plan)
        for call in run_order:
            if plans[call.layer].mixer.projections(call) is None:
                return None
        return cls(plans, run_order, hidden)

    def supports(self, tokens: int) -> bool:
        """True if a step of this many tokens takes this path: every product of every layer can be a
        stage of a chain, or at least run as a product of its own beside the chains (a stage whose
        input does not fit beside the weight ring in shared memory: K = 12288 at 8 tokens)."""
        if not 1 <= tokens <= ops.FUSED_CHAIN_MAX_TOKENS:
            return False
        known = self._supported.get(tokens)
        if known is None:
            known = True
            some_chain = False
            probe = torch.empty((tokens, 8), dtype=torch.bfloat16, device=self.plans[0].w_down.device)
            for call in self.run_order:
                plan = self.plans[call.layer]
                w_in, w_out = plan.mixer.projections(call)
                for w, normed, swiglu in ((w_in, True, False), (w_out, False, False), (plan.w_gate_up, True, True),
                                          (plan.w_down, False, False)):
                    if ops.fused_chain_stage_supported(tokens, w, normed, swiglu):
                        some_chain = True
                    elif not ops.gemm_small_supported(probe.new_empty((tokens, w.shape[1])), w):
                        known = False
            known = known and some_chain
            self._supported[tokens] = known
        return known

    def forward(self, hidden: torch.Tensor, ctx) -> tuple[torch.Tensor, torch.Tensor]:
        """Runs all layers on ``hidden`` [T, H] (the embeddings).  Returns (residual, pending): the
        stream before the last feed-forward's output has been added, and that output."""
        T, H = hidden.shape
        device, dtype = hidden.device, hidden.dtype
        new = lambda n: torch.empty((T, n), dtype=dtype, device=device)
        # Three residual buffers take turns, so that no stage writes what another CTA may still read.
        residuals, current = [hidden, new(H), new(H)], 0
        first = self.run_order[0]
        plan = self.plans[first.layer]
        w_in, _ = plan.mixer.projections(first)
        projected = new(w_in.shape[0])
        run_stages([ops.ChainStage(w=w_in, y=projected, residual_in=hidden, norm_w=plan.mixer_norm[0],
                                  eps=plan.mixer_norm[1])], T, ctx.status)
        for index, call in enumerate(self.run_order):
            plan = self.plans[call.layer]
            _, w_out = plan.mixer.projections(call)
            mixed = plan.mixer.core(projected, ctx, call)
            o, act, down = new(w_out.shape[0]), new(plan.w_down.shape[1]), new(plan.w_down.shape[0])
            after_mixer, after_ffn = (i for i in range(3) if i != current)
            stages = [
                ops.ChainStage(w=w_out, y=o, x=mixed),
                ops.ChainStage(w=plan.w_gate_up, y=act, residual_in=residuals[current], residual_out=residuals[after_mixer],
                               delta=o, norm_w=plan.feed_forward_norm[0], eps=plan.feed_forward_norm[1], swiglu=True),
                ops.ChainStage(w=plan.w_down, y=down, x=act),
            ]
            if index + 1 == len(self.run_order):
                run_stages(stages, T, ctx.status)
                return residuals[after_mixer], down
            following = self.run_order[index + 1]
            next_plan = self.plans[following.layer]
            w_next, _ = next_plan.mixer.projections(following)
            projected = new(w_next.shape[0])
            stages.append(ops.ChainStage(w=w_next, y=projected, residual_in=residuals[after_mixer],
                                         residual_out=residuals[after_ffn], delta=down, norm_w=next_plan.mixer_norm[0],
                                         eps=next_plan.mixer_norm[1]))
            run_stages(stages, T, ctx.status)
            current = after_ffn
        raise AssertionError("unreachable: the run order is not empty")
