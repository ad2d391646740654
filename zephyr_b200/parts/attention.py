"""Grouped-query causal attention over the paged cache, as a mixer.

q = x Wq^T, k = x Wk^T, v = x Wv^T without bias; q and k are RMS-normalised per head (one scale
vector each, shared by the heads) before the position encoding; query head j reads key/value head
j // (heads / kv_heads); scale 1/sqrt(head_dim); causal, with an optional window; the heads are
concatenated in order and projected by Wo (reference: src/model/causal_lm/qwen3.cpp:17-69).

The three projections run as one product over the row-concatenated weight.  Per-head norm, rotation
and the cache write are one kernel when the position encoding offers rotation tables
(``PositionEncoding.as_rotation_tables``: the NeoX rotation, or no encoding at all); any other
encoding goes through its own ``apply`` and separate norm and write kernels.
"""

from __future__ import annotations

import math
from typing import Mapping

import torch

from ..cache import PagedCacheSpec
from ..config.errors import ConfigError
from ..config.spec import LayerCall, MixerSpec
from ..kernels import ops
from ..weights.loader import ROLE_LINEAR, ROLE_NORM, WeightDecl
from .base import POSITION_ENCODINGS, Mixer, StepContext, lookup, register_mixer


class Attention(Mixer):
    graph_safe = True

    def __init__(self, spec: MixerSpec, weights: Mapping[str, torch.Tensor], dtype: torch.dtype,
                 device: torch.device | str):
        p = spec.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.nkv = int(p["num_kv_heads"])
        self.hd = int(p["head_dim"])
        self.window = int(p.get("window", 0))
        self.eps = float(p["qk_norm_eps"]) if p.get("q_norm") else 0.0
        self.dtype = dtype
        if self.nh <= 0 or self.nkv <= 0 or self.nh % self.nkv != 0:
            raise ConfigError("attention needs positive head counts with heads divisible by kv_heads")
        if self.hd % 16 != 0 or not 16 <= self.hd <= 256:
            raise ConfigError(f"attention kernels take head sizes 16..256 in steps of 16, not {self.hd}")
        self.scale = 1.0 / math.sqrt(float(self.hd))
        self.w_qkv = torch.cat([weights[p["q_proj"]], weights[p["k_proj"]], weights[p["v_proj"]]], dim=0).contiguous()
        self.w_q = self.w_qkv[: self.nh * self.hd]
        self.w_o = weights[p["o_proj"]]
        self.q_norm = weights[p["q_norm"]] if p.get("q_norm") else None
        self.k_norm = weights[p["k_norm"]] if p.get("k_norm") else None
        if (self.q_norm is None) != (self.k_norm is None):
            raise ConfigError("q_norm and k_norm come together")
        if spec.position is not None:
            self.position = lookup(POSITION_ENCODINGS, "position encoding", spec.position.kind)(
                spec.position, dtype, device)
        else:
            self.position = None
        # The fused kernels (norm + rotation + cache write, and the decode attention that does all of it
        # itself) rotate NeoX pairs by per-position angles from float32 tables; an encoding says whether
        # it is one of those, and any other goes through its own ``apply``.
        tables = self.position.as_rotation_tables() if self.position is not None else (None, None)
        self.fused_position = tables is not None
        self.cos, self.sin = tables if tables is not None else (None, None)
        # An encoding that is a bias on the scores: only the general kernel adds one.
        self.score_slopes = self.position.as_score_slopes() if self.position is not None else None
        self.group = self.nh // self.nkv
        self.tile_tokens = ops.attention_tile_tokens(self.group)
        self.fast_decode = self.score_slopes is None and ops.paged_decode_supported(self.nh, self.nkv, self.hd, dtype)
        # Decode-only steps of this many requests or more: position encoding inside the attention kernel.
        # With few requests the kernel's own chain (the projection's arrival, a head's loads, its norm
        # and rotation, then the first tile) is as long as the separate kernel's: 4467 against 4620
        # tokens a second at 8 requests, 11305 against 11143 at 64.
        self.fuse_decode_rows = 32
        self.fast_prefill = self.score_slopes is None and ops.paged_prefill_supported(self.nh, self.nkv, self.hd, dtype)
        self.prefill_tile_tokens = ops.paged_prefill_tile_tokens()

    @staticmethod
    def weight_decls(spec: MixerSpec) -> dict[str, WeightDecl]:
        p = spec.params
        hidden, nh, nkv, hd = int(p["hidden_size"]), int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        decls = {
            p["q_proj"]: WeightDecl((nh * hd, hidden), ROLE_LINEAR),
            p["k_proj"]: WeightDecl((nkv * hd, hidden), ROLE_LINEAR),
            p["v_proj"]: WeightDecl((nkv * hd, hidden), ROLE_LINEAR),
            p["o_proj"]: WeightDecl((hidden, nh * hd), ROLE_LINEAR),
        }
        if p.get("q_norm"):
            decls[p["q_norm"]] = WeightDecl((hd,), ROLE_NORM)
            decls[p["k_norm"]] = WeightDecl((hd,), ROLE_NORM)
        return decls

    def weights_read(self) -> list[torch.Tensor]:
        return [t for t in (self.w_qkv, self.w_o, self.q_norm, self.k_norm) if t is not None]

    @staticmethod
    def cache_spec(spec: MixerSpec) -> PagedCacheSpec:
        p = spec.params
        return PagedCacheSpec(int(p["num_kv_heads"]), key_dim=int(p["head_dim"]), value_dim=int(p["head_dim"]),
                              window=int(p.get("window", 0)))

    @staticmethod
    def tile_requests(spec: MixerSpec) -> list[tuple[int, str]]:
        p = spec.params
        tokens = ops.attention_tile_tokens(int(p["num_heads"]) // int(p["num_kv_heads"]))
        return [(tokens, "all"), (tokens, "multi"), (tokens, "single"), (ops.paged_prefill_tile_tokens(), "multi")]

    # ------------------------------------------------------------------ forward
    def _store_projected(self, projected: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        """Per-head norm, rotation and cache write in one kernel; returns the queries."""
        nh, nkv, hd = self.nh, self.nkv, self.hd
        table = ctx.block_table(call.cache)
        cos, sin = self.cos, self.sin
        if call.writes_cache:
            return ops.qk_norm_rope_cache(projected, nh, nkv, hd, self.q_norm, self.k_norm, self.eps, cos, sin,
                                          ctx.positions, ctx.token_row, ctx.caches[call.cache], table, ctx.status)
        return ops.qk_norm_rope_cache(projected, nh, 1, hd, self.q_norm, self.k_norm, self.eps, cos, sin,
                                      ctx.positions, ctx.token_row, None, table, ctx.status)

    def _project_and_store(self, x: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        nh, nkv, hd = self.nh, self.nkv, self.hd
        cache = ctx.caches[call.cache]
        table = ctx.block_table(call.cache)
        if self.fused_position:
            # A layer that reads another layer's cache needs no k and v.
            return self._store_projected(ops.linear(x, self.w_qkv if call.writes_cache else self.w_q), ctx, call)
        # Any other position encoding: the parts one after the other.
        T = x.shape[0]
        if not call.writes_cache:
            q = ops.linear(x, self.w_q)
            if self.q_norm is not None:
                q = ops.rmsnorm(q.view(T, nh, hd), self.q_norm, self.eps).view(T, nh * hd)
            return self.position.apply(q, nh, ctx.positions, ctx.status)
        qkv = ops.linear(x, self.w_qkv)
        q = qkv[:, : nh * hd].contiguous()
        k = qkv[:, nh * hd: (nh + nkv) * hd].contiguous()
        v = qkv[:, (nh + nkv) * hd:]
        if self.q_norm is not None:
            q = ops.rmsnorm(q.view(T, nh, hd), self.q_norm, self.eps).view(T, nh * hd)
            k = ops.rmsnorm(k.view(T, nkv, hd), self.k_norm, self.eps).view(T, nkv * hd)
        q = self.position.apply(q, nh, ctx.positions, ctx.status)
        k = self.position.apply(k, nkv, ctx.positions, ctx.status)
        ops.kv_write(k, v, nkv, hd, ctx.positions, ctx.token_row, cache, table, ctx.status)
        return q

    def attend(self, q: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        """Rows with one new token go to the split-context decode kernel, rows with several to the
        tensor-core prompt kernel, where those kernels take this shape and type; whatever is left
        goes to the general kernel."""
        cache = ctx.caches[call.cache]
        table = ctx.block_table(call.cache)
        out = torch.empty_like(q)
        common = (self.nh, self.nkv, self.hd, self.window, self.scale, ctx.status)
        decode_done = self.fast_decode and ctx.num_decode_rows > 0
        if decode_done:
            ops.paged_decode(q, cache, table, ctx.decode_rows, ctx.row_q_start, ctx.row_ctx, ctx.max_decode_context,
                             *common, out=out)
        prefill_done = False
        if self.fast_prefill:
            tile_row, tile_q0 = ctx.tiles[(self.prefill_tile_tokens, "multi")]
            prefill_done = True
            if tile_row.numel() > 0:
                ops.paged_prefill(q, cache, table, tile_row, tile_q0, ctx.row_q_start, ctx.row_q_len, ctx.row_ctx,
                                  *common, out=out)
        if decode_done and prefill_done:
            return out
        which = "multi" if decode_done else ("single" if prefill_done else "all")
        tile_row, tile_q0 = ctx.tiles[(self.tile_tokens, which)]
        if tile_row.numel() > 0:
            ops.paged_attention(q, cache, table, tile_row, tile_q0, self.tile_tokens, ctx.row_q_start, ctx.row_q_len,
                                ctx.row_ctx, *common, out=out, head_slopes=self.score_slopes)
        return out

    def forward(self, x: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        if self.fused_position and call.writes_cache:
            return ops.linear(self.core(ops.linear(x, self.w_qkv), ctx, call), self.w_o)
        q = self._project_and_store(x, ctx, call)
        return ops.linear(self.attend(q, ctx, call), self.w_o)

    def projections(self, call: LayerCall) -> tuple[torch.Tensor, torch.Tensor] | None:
        if not self.fused_position:
            return None
        return (self.w_qkv if call.writes_cache else self.w_q), self.w_o

    def core(self, projected: torch.Tensor, ctx: StepContext, call: LayerCall) -> torch.Tensor:
        if self._decodes_in_one(projected, ctx, call):
            # Every request brings one token: norms, rotation, the cache write of the new key and value
            # and the attention are one kernel, and nothing stands between the projection and it.
            out = torch.empty((projected.shape[0], self.nh * self.hd), dtype=projected.dtype, device=projected.device)
            return ops.paged_decode_fused(
                projected, ctx.caches[call.cache], ctx.block_table(call.cache), ctx.decode_rows, ctx.row_q_start,
                ctx.row_ctx, ctx.max_decode_context, self.nh, self.nkv, self.hd, self.window, self.scale, self.q_norm,
                self.k_norm, self.eps, self.cos, self.sin, ctx.status, out)
        return self.attend(self._store_projected(projected, ctx, call), ctx, call)

    def _decodes_in_one(self, projected: torch.Tensor, ctx: StepContext, call: LayerCall) -> bool:
        return (self.fast_decode and self.fused_position and call.writes_cache and projected.dtype == torch.bfloat16
                and ctx.num_decode_rows == ctx.num_rows == ctx.num_tokens and ctx.num_rows >= self.fuse_decode_rows)


register_mixer("attention", Attention)
