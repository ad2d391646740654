"""The step function: one batch of (request, its next tokens) through the model, from the cache.

``ModelRunner.step`` takes portions of prompts beside single decoded tokens, cut anywhere, runs
exactly the tokens it is given as one batch, writes their cache entries and returns float32 logits
at the wanted places.  It is what generation, trace replay and the bench all call.

The reference's executor (src/executor/causal_lm.cpp:111-295,551-624) builds per-phase batches
(padded prompt, packed prompt, prefix gather, decode) and never mixes phases; here every batch
is one flat token stream with per-row metadata, and the attention kernels sort out which rows
are long and which are single tokens.
"""

from __future__ import annotations

from collections import OrderedDict
from dataclasses import dataclass, field
from typing import Hashable, Sequence

import numpy as np
import torch

from ..cache import CacheManager, CacheStorage, bytes_per_page
from ..config.errors import InvalidArgumentError, OutOfPagesError
from ..kernels import ops
from ..parts import Model, StepContext


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, and the places among them whose logits are wanted."""

    request_id: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=tuple)


@dataclass
class PreparedStep:
    """A decode-only step whose description is already written, all but its tokens (``ModelRunner.prepare``)."""

    key: tuple
    turn: int
    info: dict
    request_ids: tuple


class ModelRunner:
    def __init__(self, model: Model, page_size: int, num_pages: int, max_requests: int,
                 max_seq_len: int | None = None, use_cuda_graphs: bool = True):
        self.model = model
        self.device = model.device
        self.dtype = model.dtype
        self.max_seq_len = min(max_seq_len or model.spec.max_seq_len, model.spec.max_seq_len)
        self.manager = CacheManager(model.cache_specs, page_size, num_pages, max_requests)
        self.storage = CacheStorage(self.manager, model.dtype, model.device)
        self.status = ops.device_status(model.device)
        self.poison_freed_pages = False      # tests: NaN into every page that is given back
        self.steps = 0
        self.use_cuda_graphs = use_cuda_graphs
        self._graphs: OrderedDict = OrderedDict()      # graph key -> captured step
        self._shapes_seen: dict = {}                   # graph key -> times seen before its capture
        self._graph_pool = None                        # one memory pool for all captured steps (made at the first capture)
        self.last_step_h2d_bytes = 0     # bytes of the last step's description copied to the device

    # ------------------------------------------------------------------ sizing
    @staticmethod
    def pages_for_memory(model: Model, page_size: int, memory_bytes: int) -> int:
        per_page = bytes_per_page(model.cache_specs, page_size, model.dtype)
        return max(0, memory_bytes // max(per_page, 1))

    def cache_bytes_per_token(self) -> int:
        return bytes_per_page(self.model.cache_specs, self.manager.page_size, self.dtype) // self.manager.page_size

    # --------------------------------------------------------------- lifecycle
    def add_request(self, request_id: Hashable, reserve_tokens: int = 0, step_tokens: int = 1) -> bool:
        """Admit a request (state slot, page reservation).  False if there is no room."""
        if not self.manager.add_request(request_id, reserve_tokens, step_tokens):
            return False
        if self.manager.state_cache_ids:
            self.storage.reset_state_slot(self.manager, self.manager.state_slot(request_id))
        return True

    def free_request(self, request_id: Hashable) -> None:
        if self.poison_freed_pages:
            for group in range(len(self.manager.groups)):
                self.storage.poison_pages(self.manager, group, list(self.manager.block_table(request_id, group)))
        self.manager.free_request(request_id)

    def num_computed(self, request_id: Hashable) -> int:
        return self.manager.computed(request_id)

    # -------------------------------------------------------------------- step
    def _validate(self, entries: Sequence[StepEntry], tokens_known: bool = True) -> None:
        if not entries:
            raise InvalidArgumentError("a step needs at least one entry")
        seen = set()
        vocab = self.model.spec.vocab_size
        for entry in entries:
            if entry.request_id not in self.manager:
                raise InvalidArgumentError(f"request {entry.request_id!r} is unknown to the runner")
            if entry.request_id in seen:
                raise InvalidArgumentError(f"request {entry.request_id!r} appears twice in one step")
            seen.add(entry.request_id)
            n = len(entry.tokens)
            if n == 0:
                raise InvalidArgumentError(f"request {entry.request_id!r} brings no tokens")
            if self.manager.computed(entry.request_id) + n > self.max_seq_len:
                raise InvalidArgumentError(
                    f"request {entry.request_id!r} would exceed the maximum sequence length {self.max_seq_len}")
            for token in entry.tokens if tokens_known else ():
                if not 0 <= int(token) < vocab:
                    raise InvalidArgumentError(f"token id {token} lies outside the vocabulary of {vocab}")
            for place in entry.want:
                if not 0 <= int(place) < n:
                    raise InvalidArgumentError(f"wanted place {place} lies outside the {n} tokens brought")

    def _describe(self, entries: Sequence[StepEntry], table_width: int | None = None):
        """The step as host arrays (all int32), in the order they are packed for the device."""
        manager = self.manager
        q_len = [len(e.tokens) for e in entries]
        ctx_before = [manager.computed(e.request_id) for e in entries]
        for entry, ctx, n in zip(entries, ctx_before, q_len):
            if not manager.ensure_capacity(entry.request_id, ctx + n):
                raise OutOfPagesError(
                    f"no pages left for request {entry.request_id!r} ({ctx} cached + {n} new tokens); "
                    f"free pages per group: {[g.pool.num_free for g in manager.groups]}")
        R = len(entries)
        q_start = np.zeros(R, dtype=np.int32)
        np.cumsum(q_len[:-1], out=q_start[1:])
        token_ids = np.concatenate([np.asarray(e.tokens, dtype=np.int32) for e in entries])
        positions = np.concatenate([np.arange(c, c + n, dtype=np.int32) for c, n in zip(ctx_before, q_len)])
        token_row = np.repeat(np.arange(R, dtype=np.int32), q_len)
        slots = np.asarray([manager.state_slot(e.request_id) for e in entries], dtype=np.int32)
        tables = []
        for group in range(len(manager.groups)):
            rows = [manager.block_table_array(e.request_id, group) for e in entries]
            width = table_width or max(1, max(r.size for r in rows))
            table = np.zeros((R, width), dtype=np.int32)
            for i, r in enumerate(rows):
                table[i, :r.size] = r
            tables.append(table)
        logit_tokens = np.asarray([q_start[i] + int(p) for i, e in enumerate(entries) for p in e.want], dtype=np.int32)
        decode_rows = np.asarray([i for i, n in enumerate(q_len) if n == 1], dtype=np.int32)
        max_decode_context = max([ctx_before[i] + 1 for i in decode_rows], default=0)
        tiles = {}
        for tile_tokens, which in self.model.tile_requests:
            tile_row, tile_q0 = [], []
            for i, n in enumerate(q_len):
                if (which == "multi" and n == 1) or (which == "single" and n != 1):
                    continue
                for q0 in range(0, n, tile_tokens):
                    tile_row.append(i)
                    tile_q0.append(q0)
            # By the number of keys a tile sees, fewest first (the kernels start at the far end of the
            # list, so the longest tiles of the whole step run first).
            order = sorted(range(len(tile_row)), key=lambda t: ctx_before[tile_row[t]] + tile_q0[t])
            tiles[(tile_tokens, which)] = (np.asarray([tile_row[t] for t in order], dtype=np.int32),
                                           np.asarray([tile_q0[t] for t in order], dtype=np.int32))
        arrays = [token_ids, positions, token_row, q_start, np.asarray(q_len, dtype=np.int32),
                  np.asarray(ctx_before, dtype=np.int32), slots, logit_tokens, decode_rows]
        arrays += [t.reshape(-1) for t in tables]
        for pair in tiles.values():
            arrays += list(pair)
        info = dict(R=R, T=sum(q_len), q_len=q_len, ctx_before=ctx_before, slots=slots.tolist(),
                    table_widths=[t.shape[1] for t in tables], tile_keys=list(tiles),
                    num_decode_rows=int(decode_rows.size), max_decode_context=int(max_decode_context))
        return arrays, info

    def _context_from(self, device: torch.Tensor, sizes: list[int], info: dict) -> StepContext:
        """A StepContext whose index tensors are views of the packed device buffer."""
        views, offset = [], 0
        for size in sizes:
            views.append(device[offset:offset + size])
            offset += size
        (d_tokens, d_pos, d_row, d_qstart, d_qlen, d_ctx, d_slots, d_logit, d_decode), rest = views[:9], views[9:]
        widths = info["table_widths"]
        d_tables = [rest[g].view(info["R"], widths[g]) for g in range(len(widths))]
        rest = rest[len(widths):]
        d_tiles = {key: (rest[2 * i], rest[2 * i + 1]) for i, key in enumerate(info["tile_keys"])}
        return StepContext(
            num_tokens=info["T"], num_rows=info["R"], token_ids=d_tokens, positions=d_pos, token_row=d_row,
            row_q_start=d_qstart, row_q_len=d_qlen, row_ctx=d_ctx, state_slots=d_slots, block_tables=d_tables,
            group_of_cache=self.manager.group_of_cache, logit_tokens=d_logit, decode_rows=d_decode,
            num_decode_rows=info["num_decode_rows"], max_decode_context=info["max_decode_context"], tiles=d_tiles,
            caches=self.storage, status=self.status, dtype=self.dtype, host_q_len=list(info["q_len"]),
            host_ctx=list(info["ctx_before"]), host_slots=list(info["slots"]))

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Describe the step and bring the description to the device: one pinned buffer, one copy."""
        arrays, info = self._describe(entries)
        sizes = [a.size for a in arrays]
        # A ring of pinned buffers, grown when a step needs more: a buffer is written again only after
        # the copy that last read it is done.
        total = max(1, sum(sizes))
        turn = self._eager_turn = (getattr(self, "_eager_turn", -1) + 1) % 4
        ring = self.__dict__.setdefault("_eager_ring", [None] * 4)
        if ring[turn] is None or ring[turn][0].numel() < total:
            ring[turn] = (torch.empty(max(total, 4096), dtype=torch.int32, pin_memory=True), None)
        host, copied = ring[turn]
        if copied is not None:
            copied.synchronize()
        if sum(sizes):
            np.concatenate(arrays, out=host.numpy()[:sum(sizes)])
        device = host[:total].to(self.device, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        ring[turn] = (host, event)
        self.last_step_h2d_bytes = 4 * sum(sizes)
        return self._context_from(device, sizes, info)

    # ------------------------------------------------------------------ graphs
    MAX_SHAPE_GRAPHS = 16         # captured graphs of steps other than decode-only ones, least recently used first out
    MAX_SHAPES_COUNTED = 4096
    MAX_GRAPH_LOGIT_ROWS = 64     # a graph keeps its logits; steps that want more places run launch by launch

    def _graph_key(self, entries: Sequence[StepEntry]):
        """A step whose shape comes again replays a captured CUDA graph: the launches of a whole step
        become one.  The key fixes everything a launch bakes in: the number of new tokens of every row
        and the wanted places (they size every grid and buffer), and a power-of-two bound on the
        context of the rows with one new token, if the model keeps a paged cache at all (it sizes the
        decode attention's grid).  What a step
        reads beyond that (tokens, positions, contexts, block tables) it reads from the device.
        Decode-only steps are captured at once; any other shape when it is seen a second time."""
        if not self.use_cuda_graphs or not self.model.graph_safe:
            return None
        singles = [self.manager.computed(e.request_id) + 1 for e in entries if len(e.tokens) == 1]
        bound = 0
        if singles and self.manager.groups:       # a model without a paged cache has no context to bound
            bound = max(ops.DECODE_SPLIT_SIZE, 1 << (max(singles) - 1).bit_length())
            bound = min(bound, max(self.max_seq_len, ops.DECODE_SPLIT_SIZE))
        if len(singles) == len(entries) and all(tuple(e.want) == (0,) for e in entries):
            return (len(entries), bound)
        if sum(len(e.want) for e in entries) > self.MAX_GRAPH_LOGIT_ROWS:
            return None
        key = (tuple((len(e.tokens), tuple(e.want)) for e in entries), bound)
        if key in self._graphs:
            self._graphs.move_to_end(key)
            return key
        if len(self._shapes_seen) >= self.MAX_SHAPES_COUNTED:
            self._shapes_seen.clear()
        self._shapes_seen[key] = self._shapes_seen.get(key, 0) + 1
        if self._shapes_seen[key] < 2:
            return None
        del self._shapes_seen[key]
        shaped = [k for k in self._graphs if not isinstance(k[0], int)]
        if len(shaped) >= self.MAX_SHAPE_GRAPHS:
            del self._graphs[shaped[0]]
        return key

    def _rewrite_decode(self, record: dict, host: np.ndarray, entries: Sequence[StepEntry], width: int) -> dict:
        """A decode-only step's values, written into their places of the pinned buffer (the order of
        ``_describe``: 0 tokens, 1 positions, 5 contexts, 6 slots, 9.. one block table per group)."""
        manager, R, offsets = self.manager, len(entries), record["offsets"]
        ctx_before = [manager.computed(e.request_id) for e in entries]
        for entry, ctx in zip(entries, ctx_before):
            if not manager.ensure_capacity(entry.request_id, ctx + 1):
                raise OutOfPagesError(
                    f"no pages left for request {entry.request_id!r} ({ctx} cached + 1 new token); "
                    f"free pages per group: {[g.pool.num_free for g in manager.groups]}")
        host[offsets[0]:offsets[0] + R] = [e.tokens[0] for e in entries]
        host[offsets[1]:offsets[1] + R] = ctx_before
        host[offsets[5]:offsets[5] + R] = ctx_before
        slots = [manager.state_slot(e.request_id) for e in entries]
        host[offsets[6]:offsets[6] + R] = slots
        for group in range(len(manager.groups)):
            table = host[offsets[9 + group]:offsets[10 + group]].reshape(R, width)
            table[:] = 0
            for i, entry in enumerate(entries):
                row = manager.block_table_array(entry.request_id, group)
                table[i, :row.size] = row
        return dict(record["info"], ctx_before=ctx_before, slots=slots)

    def _step_with_graph(self, key, entries: Sequence[StepEntry]) -> tuple[torch.Tensor, dict]:
        width = self.manager.blocks_for(self.max_seq_len)
        decode_only = isinstance(key[0], int)
        record = self._graphs.get(key)
        described = None
        if record is None or not decode_only:
            described = self._describe(entries, table_width=width)
            described[1]["max_decode_context"] = key[1]
        if record is None:
            arrays, info = described
            sizes = [a.size for a in arrays]
            total = sum(sizes)
            # A small ring of pinned buffers: the host may run ahead of the device, and a buffer must not
            # be refilled before the copy that reads it has been done.  For decode-only steps every buffer
            # starts as a copy of the first step's description: what depends only on the number of rows
            # stays as it is, and later steps rewrite the rest in place (tokens, positions, contexts,
            # slots, block tables).  Steps of other shapes write the whole description every time.
            template = np.concatenate(arrays)
            offsets = np.concatenate([[0], np.cumsum(sizes)]).tolist()
            record = {"host": [torch.empty(total, dtype=torch.int32, pin_memory=True) for _ in range(4)],
                      "copied": [None] * 4, "turn": 0, "sizes": sizes, "info": info, "offsets": offsets,
                      "device": torch.empty(total, dtype=torch.int32, device=self.device), "graph": None}
            for buffer in record["host"]:
                buffer.numpy()[:] = template
            self._graphs[key] = record
        sizes = record["sizes"]
        turn = self._claim_buffer(record)
        if decode_only:
            info = self._rewrite_decode(record, record["host"][turn].numpy(), entries, width)
        else:
            arrays, info = described
            if [a.size for a in arrays] != sizes:
                raise RuntimeError("a step's description changed size under one graph key")
            np.concatenate(arrays, out=record["host"][turn].numpy())
        return self._launch_graph(record, turn, info, decode_only)

    @staticmethod
    def _claim_buffer(record: dict) -> int:
        """The next pinned buffer of the record's ring, once the copy that last read it is done."""
        turn = record["turn"]
        record["turn"] = (turn + 1) % len(record["host"])
        if record["copied"][turn] is not None:
            record["copied"][turn].synchronize()
        return turn

    def _launch_graph(self, record: dict, turn: int, info: dict, decode_only: bool,
                      device_tokens: torch.Tensor | None = None) -> tuple[torch.Tensor, dict]:
        """Copy the written description to the device and run the record's graph (captured at its first run)."""
        sizes, total = record["sizes"], record["offsets"][-1]
        record["device"].copy_(record["host"][turn], non_blocking=True)
        if device_tokens is not None:       # the tokens come from the device, over what the host wrote in their place
            at, rows = record["offsets"][0], info["R"]
            record["device"][at:at + rows].copy_(device_tokens[:rows], non_blocking=True)
        event = record["copied"][turn] or torch.cuda.Event()
        event.record()
        record["copied"][turn] = event
        self.last_step_h2d_bytes = 4 * total
        if record["graph"] is None:
            ctx = self._context_from(record["device"], sizes, info)
            # One ordinary run first (libraries pick their algorithms and allocate workspaces outside the
            # capture), then the capture, which records the launches without running them.
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self.model.forward(ctx)
            torch.cuda.current_stream(self.device).wait_stream(side)
            graph = torch.cuda.CUDAGraph()
            launched = ops.LAUNCHES
            # All graphs of this runner draw from one pool: they replay one after the other on one stream,
            # so a graph's intermediate buffers may lie where another graph's lay, and the pool grows to
            # the largest step, not to the sum of all captured steps.  A graph's logits stay its own for as
            # long as the record holds them.
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            with ops.capture(graph, pool=self._graph_pool):
                record["logits"] = self.model.forward(ctx)
            record["kernels"] = ops.LAUNCHES - launched     # this package's kernels inside the graph
            record["graph"] = graph
        record["graph"].replay()
        ops.LAUNCHES += record["kernels"]
        # A decode-only step hands out its graph's own tensor (the caller samples from it at once);
        # steps of other shapes hand out a copy, which the next step of that shape leaves alone.
        return (record["logits"] if decode_only else record["logits"].clone()), info

    def prepare(self, entries: Sequence[StepEntry]) -> PreparedStep | None:
        """Write a decode-only step's description before its tokens are known (each entry's token is
        a placeholder): positions, contexts, slots and block tables go into the graph's next pinned
        buffer, pages are made sure of.  The host does this while the device still runs the step
        before; ``step(entries, prepared)`` then only adds the tokens.  None if the step is not one
        that replays an existing decode graph, or if pages are missing (``step`` will say so)."""
        if any(len(e.tokens) != 1 or tuple(e.want) != (0,) for e in entries):
            return None
        self._validate(entries, tokens_known=False)
        key = self._graph_key(entries)
        record = self._graphs.get(key) if key is not None else None
        if record is None or record["graph"] is None:
            return None
        turn = self._claim_buffer(record)
        try:
            info = self._rewrite_decode(record, record["host"][turn].numpy(), entries,
                                        self.manager.blocks_for(self.max_seq_len))
        except OutOfPagesError:
            return None
        return PreparedStep(key, turn, info, tuple(e.request_id for e in entries))

    def holds(self, prepared: PreparedStep | None, entries: Sequence[StepEntry]) -> bool:
        """True if ``step(entries, prepared)`` would use ``prepared`` as it is."""
        return prepared is not None and self._still_holds(prepared, entries)

    def _still_holds(self, prepared: PreparedStep, entries: Sequence[StepEntry]) -> bool:
        """True if ``prepared`` was made for these entries and nothing has moved since."""
        if len(entries) != len(prepared.request_ids) or prepared.key not in self._graphs:
            return False
        manager = self.manager
        for entry, request_id, before in zip(entries, prepared.request_ids, prepared.info["ctx_before"]):
            if (entry.request_id != request_id or len(entry.tokens) != 1 or tuple(entry.want) != (0,)
                    or request_id not in manager or manager.computed(request_id) != before):
                return False
        return True

    @torch.no_grad()
    def step(self, entries: Sequence[StepEntry], prepared: PreparedStep | None = None,
             device_tokens: torch.Tensor | None = None) -> torch.Tensor:
        """Run the entries as one batch.  Returns float32 logits [sum of wanted places, vocab] on the
        device, in the order of the entries and of each entry's ``want``.  The call does not wait for
        the GPU; ``check()`` (or reading the logits on the host and then ``check()``) does.  The tensor
        returned by a decode-only step belongs to that step's graph and is overwritten by the next
        step of the same shape: use it (sample from it, copy it) before stepping again.
        ``prepared``: what ``prepare`` returned for these very entries, nothing else having touched the
        runner in between; anything else is ignored and the step is described afresh.
        ``device_tokens`` (with a ``prepared`` that ``holds``): int32 on the device, the entries' tokens
        in their order, for example a selection's output that has not reached the host yet; the
        entries' own tokens are then not looked at."""
        if device_tokens is not None and not self.holds(prepared, entries):
            raise InvalidArgumentError("tokens on the device need a prepared step that still holds")
        if prepared is not None and self._still_holds(prepared, entries):
            # Everything but the tokens was checked and written by ``prepare``.
            record = self._graphs[prepared.key]
            if device_tokens is None:
                tokens = [int(e.tokens[0]) for e in entries]
                if not 0 <= min(tokens) <= max(tokens) < self.model.spec.vocab_size:
                    raise InvalidArgumentError(f"a token id among {tokens} lies outside the vocabulary")
                at = record["offsets"][0]
                record["host"][prepared.turn].numpy()[at:at + len(entries)] = tokens
            elif device_tokens.dtype != torch.int32 or device_tokens.numel() < len(entries) or not device_tokens.is_cuda:
                raise InvalidArgumentError("device_tokens must be int32 on the device, one per entry")
            logits, info = self._launch_graph(record, prepared.turn, prepared.info, True, device_tokens)
            before_all = info["ctx_before"]
        else:
            self._validate(entries)
            key = self._graph_key(entries)
            if key is not None:
                logits, info = self._step_with_graph(key, entries)
                before_all = info["ctx_before"]
            else:
                ctx = self.build_context(entries)
                logits = self.model.forward(ctx)
                before_all = ctx.host_ctx
        for entry, before in zip(entries, before_all):
            if self.poison_freed_pages:
                old = [list(self.manager.block_table(entry.request_id, g)) for g in range(len(self.manager.groups))]
            self.manager.commit(entry.request_id, before + len(entry.tokens))
            if self.poison_freed_pages:
                for g, pages in enumerate(old):
                    now = self.manager.block_table(entry.request_id, g)
                    self.storage.poison_pages(self.manager, g, [p for p, q in zip(pages, now) if p != q])
        self.steps += 1
        return logits

    def check(self) -> None:
        """Wait for the device and raise if a kernel of an earlier step reported an error."""
        ops.check_status(self.status, "model step")
