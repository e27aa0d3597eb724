"""The step function: one ragged batch in, logits at the wanted places out.

``ModelRunner.step`` is the single host -> GPU boundary of the engine. It flattens the batch to
one token axis, ships every integer array of the step in one copy, writes the keys and values of
every token it is given, runs the model's layer calls in their listed order and returns float32
logits for the wanted places only. Nothing here knows about prompts versus decoding: a portion
of a prompt, a single decoded token and a recomputation are the same operation
(reference: src/paged_kv_serving/engine/runner.py:161-227).

The runner also owns the bytes behind page numbers (``CacheStorage``), which is what
copy-on-write and state-slot copies act on (reference: src/paged_kv_serving/engine/runner.py:128-133).
"""

from __future__ import annotations

import gc
import hashlib
from dataclasses import dataclass

import numpy as np
import torch

from paged_kv_serving_b200 import ops
from paged_kv_serving_b200.cache.manager import GroupSpec, plan_groups
from paged_kv_serving_b200.cache.pages import NULL_PAGE
from paged_kv_serving_b200.engine.batch import BatchEntry, ExecutionBatch
from paged_kv_serving_b200.engine.sequence import TableSnapshot
from paged_kv_serving_b200.models.decoder import DecoderModel
from paged_kv_serving_b200.ops import arena, gemm
from paged_kv_serving_b200.parts.base import CacheBinding, GroupView, IntArena, StepContext

__all__ = ["CacheStorage", "ModelRunner", "StepResult"]


class CacheStorage:
    """Device memory of the cache: per page group one key pool and one value pool shaped
    ``[layers of the group, pages, kv heads, page_size, head_dim]``, and per state entry a
    tensor ``[slots, *shape]``."""

    def __init__(self, groups: list[GroupSpec], state_entries: list, *, num_blocks: int, block_size: int,
                 dtype: torch.dtype, device: torch.device, num_state_slots: int) -> None:
        self.groups = groups
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.k_pools: list[torch.Tensor] = []
        self.v_pools: list[torch.Tensor] = []
        self.location: dict[int, tuple[int, int]] = {}
        for g, spec in enumerate(groups):
            shape = (len(spec.entries), num_blocks, spec.n_kv_heads, block_size, spec.head_dim)
            self.k_pools.append(torch.zeros(shape, dtype=dtype, device=device))
            self.v_pools.append(torch.zeros(shape, dtype=dtype, device=device))
            for index, entry in enumerate(spec.entries):
                self.location[entry] = (g, index)
        self.states: list[torch.Tensor] = []
        self.state_index: dict[int, int] = {}
        for entry, request in state_entries:
            state_dtype = {"float32": torch.float32, "bfloat16": torch.bfloat16}[request.dtype]
            self.state_index[entry] = len(self.states)
            self.states.append(torch.zeros((max(1, num_state_slots), *request.shape), dtype=state_dtype, device=device))

    @property
    def cache_bytes(self) -> int:
        pools = sum(t.numel() * t.element_size() for t in (*self.k_pools, *self.v_pools))
        return pools + sum(t.numel() * t.element_size() for t in self.states)

    def copy_page(self, group: int, source: int, destination: int) -> None:
        if source == destination:
            raise ValueError("a page is never copied onto itself")
        ops.copy_page(self.k_pools[group], self.v_pools[group], source, destination)

    def copy_state(self, source_slot: int, destination_slot: int) -> None:
        for state in self.states:
            state[destination_slot].copy_(state[source_slot])

    def clear_state(self, slots: list[int]) -> None:
        if slots and self.states:
            index = torch.tensor(slots, dtype=torch.long, device=self.states[0].device)
            for state in self.states:
                state.index_fill_(0, index, 0)

    def reset(self) -> None:
        for tensor in (*self.k_pools, *self.v_pools, *self.states):
            tensor.zero_()

    def fill(self, value: float) -> None:
        """Overwrite every page with ``value`` (tests poison the pool with it)."""
        for tensor in (*self.k_pools, *self.v_pools):
            tensor.fill_(value)

    def page_fingerprint(self, group: int, page: int) -> bytes:
        digest = hashlib.blake2b(digest_size=16)
        for pool in (self.k_pools[group], self.v_pools[group]):
            digest.update(pool[:, page].contiguous().view(torch.uint8).cpu().numpy().tobytes())
        return digest.digest()


@dataclass(slots=True)
class StepResult:
    """Logits of one step: ``logits[i]`` belongs to ``rows[i] = (seq_id, place in its entry)``."""

    logits: torch.Tensor | None        # float32 [R, vocab] on the device, or None when R == 0
    rows: list[tuple[str, int]]
    num_tokens: int
    h2d_bytes: int

    def by_sequence(self) -> dict[str, np.ndarray]:
        """Host rows keyed by sequence id (the last wanted place of each entry)."""
        if self.logits is None:
            return {}
        host = self.logits.cpu().numpy()
        return {seq_id: host[i] for i, (seq_id, _) in enumerate(self.rows)}


class ModelRunner:
    """Owns the cache storage of one model and runs ragged batches against it."""

    def __init__(self, model: DecoderModel, *, num_blocks: int, block_size: int, max_running_seqs: int = 64,
                 use_graphs: bool = True) -> None:
        if num_blocks < 1 or block_size < 1:
            raise ValueError("num_blocks and block_size must be >= 1")
        if not torch.cuda.is_available():
            raise RuntimeError("paged_kv_serving_b200 runs on a CUDA GPU only; there is no CPU path")
        self.model = model
        self.num_blocks = num_blocks
        self.block_size = block_size
        self.order = model.layout.resolved_order()
        self.groups, self.state_entries = plan_groups(model.layout.cache_entries())
        self.num_state_slots = max_running_seqs if self.state_entries else 0
        self.storage = CacheStorage(self.groups, self.state_entries, num_blocks=num_blocks, block_size=block_size,
                                    dtype=model.dtype, device=model.device, num_state_slots=self.num_state_slots)
        self.bindings: list[CacheBinding | None] = []
        for call in self.order:
            if call.cache is None:
                self.bindings.append(None)
            elif call.cache in self.storage.location:
                g, index = self.storage.location[call.cache]
                self.bindings.append(CacheBinding(call.cache, group=g, index=index, write=call.write))
            else:
                self.bindings.append(CacheBinding(call.cache, state=self.storage.state_index[call.cache], write=call.write))
        self._status = ops.status_word(model.device)
        # Where a sampler leaves the ids of a step (and, behind them, the status word) so that the
        # next step's embedding lookup can read a decoded token without a trip through the host.
        # Its address is fixed: captured graphs read it.
        self.sampled_ids = torch.zeros((max(1, max_running_seqs) + 1,), dtype=torch.int32, device=model.device)
        self.steps_run = 0
        self.use_graphs = use_graphs
        layout = model.layout
        self._graph_safe = all(part.graph_safe for part in (*layout.blocks, layout.final_norm, layout.embedding, layout.head))
        self._graphs: dict[tuple[int, int], dict] = {}
        self._last_graph_step: tuple[ExecutionBatch, tuple[int, int]] | None = None
        self._ahead: dict | None = None
        self._graph_pool = torch.cuda.graph_pool_handle() if use_graphs else None
        self._capture_stream = None
        # memory for the outputs of a step's kernels (steps that are not graph replays); it grows to
        # what the largest step needed and is reused by every step after it
        self._arena = arena.StepArena(model.device)

    # --- storage behind the cache manager -------------------------------------------------

    @property
    def num_groups(self) -> int:
        return len(self.groups)

    @property
    def cache_bytes(self) -> int:
        return self.storage.cache_bytes

    @property
    def capacity_tokens(self) -> int:
        return self.num_blocks * self.block_size

    def copy_page(self, group: int, source: int, destination: int) -> None:
        self.storage.copy_page(group, source, destination)

    def copy_state(self, source_slot: int, destination_slot: int) -> None:
        self.storage.copy_state(source_slot, destination_slot)

    def reset_cache(self) -> None:
        self.storage.reset()

    # --- the step ------------------------------------------------------------------------

    def _validate(self, batch: ExecutionBatch) -> None:
        config = self.model.layout
        for entry in batch.entries:
            ids = entry.token_ids
            if min(ids) < 0 or max(ids) >= config.vocab_size:
                raise ValueError(f"sequence {entry.seq_id}: token id outside the vocabulary")
            if entry.context_len > config.max_positions:
                raise ValueError(f"sequence {entry.seq_id}: position beyond max_seq_len")
            if len(entry.block_tables) != len(self.groups):
                raise ValueError(f"sequence {entry.seq_id}: {len(entry.block_tables)} page tables for "
                                 f"{len(self.groups)} page groups")
            first_page = entry.first_position // self.block_size
            last_page = (entry.context_len - 1) // self.block_size
            for table in entry.block_tables:
                if last_page >= len(table):
                    raise ValueError(f"sequence {entry.seq_id}: position {entry.context_len - 1} has no page in the table")
                for page in table[first_page:last_page + 1]:
                    if page == NULL_PAGE or not 0 <= page < self.num_blocks:
                        raise ValueError(f"sequence {entry.seq_id}: a written position has no valid page")
            if self.state_entries and entry.state_slot is None:
                raise ValueError(f"sequence {entry.seq_id}: the model keeps per-request state but no slot was given")

    def _feedback_array(self, entries, feedback: dict[str, int] | None, starts) -> np.ndarray:
        """Per token -1, or (for a one-token entry named in ``feedback``) the place of its id in
        ``sampled_ids``."""
        array = np.full(int(starts[-1]), -1, dtype=np.int32)
        if feedback:
            for e, start in zip(entries, starts[:-1]):
                place = feedback.get(e.seq_id) if e.num_tokens == 1 else None
                if place is not None:
                    if not 0 <= place < self.sampled_ids.numel() - 1:
                        raise ValueError(f"sequence {e.seq_id}: fed-back id outside the sampler's buffer")
                    array[int(start)] = place
        return array

    def _context(self, batch: ExecutionBatch, table_width: int | None = None, pad_to: int | None = None,
                 feedback: dict[str, int] | None = None) -> tuple[StepContext, list[tuple[str, int]]]:
        """Flatten a batch into the step's integer arrays. ``pad_to`` appends stand-in entries of
        one token (no page, no store, token 0) up to that many entries and ``table_width`` fixes
        the width of the block tables, so that a captured graph keeps its shapes. ``feedback``
        maps sequence ids of one-token entries to the place in ``sampled_ids`` where the token's
        id lies (the entry's own ``token_ids`` is then a stand-in)."""
        entries = batch.entries
        if pad_to is not None and len(entries) < pad_to:
            filler = BatchEntry("", (0,), 0, tuple((NULL_PAGE,) for _ in self.groups), (0,), 0)
            entries = entries + (filler,) * (pad_to - len(entries))
        lens = [e.num_tokens for e in entries]
        total = sum(lens)
        arena = IntArena()
        tokens = np.fromiter((t for e in entries for t in e.token_ids), dtype=np.int32, count=total)
        starts = np.zeros(len(entries) + 1, dtype=np.int64)
        np.cumsum(lens, out=starts[1:])
        first = np.asarray([e.first_position for e in entries], dtype=np.int64)
        seq_of_token = np.repeat(np.arange(len(entries)), lens)
        positions = np.arange(total, dtype=np.int64) - starts[seq_of_token] + first[seq_of_token]
        arena.add(StepContext.TOKEN_IDS, tokens)
        arena.add(StepContext.TOKEN_FEEDBACK, self._feedback_array(entries, feedback, starts))
        arena.add(StepContext.POSITIONS, positions)
        arena.add(StepContext.SEQ_STARTS, starts)
        arena.add(StepContext.FIRST_POS, first)
        arena.add(StepContext.CONTEXT_LENS, first + np.asarray(lens))
        arena.add(StepContext.STATE_SLOTS, [e.state_slot if e.state_slot is not None else 0 for e in entries])
        rows: list[tuple[str, int]] = []
        row_index: list[int] = []
        for e, start in zip(entries, starts[:-1]):
            for place in e.logits_at:
                rows.append((e.seq_id, place))
                row_index.append(int(start) + place)
        arena.add(StepContext.LOGITS_ROWS, row_index if row_index else [0])
        views = []
        for g in range(len(self.groups)):
            width = max(len(e.block_tables[g]) for e in entries)
            if table_width is not None:
                if width > table_width:
                    raise ValueError("a block table is wider than the captured graph allows")
                width = table_width
            table = np.full((len(entries), width), NULL_PAGE, dtype=np.int32)
            for i, e in enumerate(entries):
                pages = e.block_tables[g]
                table[i, :len(pages)] = pages.array if isinstance(pages, TableSnapshot) else pages
            page_of_token = table[seq_of_token, positions // self.block_size].astype(np.int64)
            slots = np.where(page_of_token >= 0, page_of_token * self.block_size + positions % self.block_size, -1)
            table_name, slots_name = f"group{g}/block_table", f"group{g}/slots"
            arena.add(table_name, table)
            arena.add(slots_name, slots)
            views.append(GroupView(self.storage.k_pools[g], self.storage.v_pools[g], self.block_size,
                                   self.groups[g].window, table_name, slots_name))
        ctx = StepContext(dtype=self.model.dtype, device=self.model.device, num_tokens=total, num_seqs=len(entries),
                          seq_lens=lens, first_positions=[e.first_position for e in entries], arena=arena,
                          groups=views, states=self.storage.states, status=self._status, fed_back_ids=self.sampled_ids)
        return ctx, rows

    def _plan(self, ctx: StepContext) -> None:
        for call, binding in zip(self.order, self.bindings):
            self.model.layout.blocks[call.layer].plan_step(ctx, binding)

    def _forward(self, ctx: StepContext, want_logits: bool) -> torch.Tensor | None:
        """The kernels of one step, launched on the current stream; nothing here reads device
        data on the host, so the whole sequence can be captured in a CUDA graph."""
        model = self.model
        hidden = model.layout.embedding.forward(ctx)
        blocks = model.layout.blocks
        delta = None
        step_arena = arena.active()
        for i, (call, binding) in enumerate(zip(self.order, self.bindings)):
            if step_arena is not None:
                step_arena.next_layer()
            # the block may carry the next block's first norm in the tail of its last kernel; the
            # last block hands on its plain update (the final norm takes only the wanted rows)
            following = blocks[self.order[i + 1].layer] if i + 1 < len(self.order) else None
            if following is not None and getattr(following, "first_norm", None) is not None:
                delta = blocks[call.layer].forward(hidden, delta, ctx, binding, next_norm=following.first_norm)
            else:
                delta = blocks[call.layer].forward(hidden, delta, ctx, binding)
        if step_arena is not None:
            step_arena.end_layers()
        if not want_logits:
            return None
        normed = model.layout.final_norm.add_norm(hidden, delta, model.dtype, rows=ctx.ints(StepContext.LOGITS_ROWS))
        return model.layout.head.forward(normed, ctx)

    def step(self, batch: ExecutionBatch, clear_state_slots: list[int] | None = None,
             feedback: dict[str, int] | None = None) -> StepResult:
        """Run one batch: writes the cache for every token given, returns logits where wanted.

        A batch of single decoded tokens (every entry one token whose logits are wanted) replays
        a CUDA graph captured for its size class. The memory of a step's logits is used again by
        the next step (a graph's static output, or the step's arena), so the caller reads or
        samples from them before stepping again; work already queued on the stream is safe.

        ``feedback``: sequence id -> place in ``sampled_ids``, for one-token entries whose token
        was sampled by the step before and has not left the device: the embedding lookup reads
        the id there (the entry's ``token_ids`` is a stand-in and is not looked at).
        """
        if not batch.entries:
            return StepResult(None, [], 0, 0)
        self._validate(batch)
        self.steps_run += 1
        self._last_graph_step = None
        if self.use_graphs and self._graph_safe and not clear_state_slots and \
                all(e.num_tokens == 1 and e.logits_at == (0,) for e in batch.entries):
            return self._step_graph(batch, feedback)
        ctx, rows = self._context(batch, feedback=feedback)
        self._plan(ctx)
        ctx.arena.upload(self.model.device)
        if clear_state_slots:
            self.storage.clear_state(clear_state_slots)
        self._arena.begin_step()
        before = arena.activate(self._arena)
        try:
            logits = self._forward(ctx, bool(rows))
        finally:
            arena.activate(before)
        return StepResult(logits, rows, ctx.num_tokens, ctx.arena.bytes_uploaded)

    # --- decode steps as CUDA graphs -----------------------------------------------------

    GRAPH_BATCH_SIZES = (1, 2, 4, 8, 16, 32, 64, 128, 256)
    GRAPH_TABLE_STEP = 32     # block tables of a graph are this many pages wide, or a multiple
    MAX_GRAPHS = 96           # captured graphs kept; the least recently replayed one goes first

    def _step_graph(self, batch: ExecutionBatch, feedback: dict[str, int] | None = None) -> StepResult:
        count = len(batch.entries)
        size = next((b for b in self.GRAPH_BATCH_SIZES if b >= count), None)
        if size is None:
            size = -(-count // 256) * 256
        widest = max(len(t) for e in batch.entries for t in e.block_tables) if self.groups else 1
        width = -(-widest // self.GRAPH_TABLE_STEP) * self.GRAPH_TABLE_STEP
        key = (size, width)
        ahead, self._ahead = self._ahead, None
        if ahead is not None and ahead["key"] == key and self._as_expected(batch, ahead["batch"]):
            # prepared while the GPU ran the step before: only the token ids were not known then
            ctx, rows = ahead["ctx"], ahead["rows"]
            tokens = [e.token_ids[0] for e in batch.entries] + [0] * (size - count)
            ctx.arena.patch(StepContext.TOKEN_IDS, tokens)
            places = [(feedback or {}).get(e.seq_id, -1) for e in batch.entries] + [-1] * (size - count)
            ctx.arena.patch(StepContext.TOKEN_FEEDBACK, places)
        else:
            ctx, rows = self._context(batch, table_width=width, pad_to=size, feedback=feedback)
            ctx.planning_context_len = width * self.block_size
            self._plan(ctx)
        self._last_graph_step = (batch, key)
        rows = rows[:count]
        entry = self._graphs.get(key)
        if entry is not None:
            self._graphs[key] = self._graphs.pop(key)          # most recently used last
        if entry is not None and entry["signature"] == ctx.arena.signature():
            ctx.arena.upload(self.model.device, into=entry["ints"], views=False)
            entry["graph"].replay()
            ops.LAUNCHES["count"] += entry["launches"]     # the kernels of this module that the graph holds
            return StepResult(entry["logits"][:count], rows, count, ctx.arena.bytes_uploaded)
        # first step of this size class: run it eagerly on a buffer that stays, then capture the
        # same launches (a capture records, it does not run) for the steps that follow
        ints = torch.empty((ctx.arena.total_ints(),), dtype=torch.int32, device=self.model.device)
        ctx.arena.upload(self.model.device, into=ints)
        logits = self._forward(ctx, True)
        torch.cuda.synchronize(self.model.device)
        graph = torch.cuda.CUDAGraph()
        ctx.scratch = {k: v for k, v in ctx.scratch.items() if not isinstance(v, torch.Tensor)}
        before = ops.launch_count()
        # The cyclic garbage collector stays off while the capture runs: were it to free, in the
        # middle of it, an object that owns CUDA resources (the graphs and memory pool of a runner
        # that died in a reference cycle), the driver would refuse the call during capture and the
        # capture would be void. (Entering the capture collects garbage first.)
        # The capture runs on a stream of its own between capture_begin and capture_end; the
        # library's context manager would also collect garbage and empty the allocator's cache
        # first, which costs tens of milliseconds with a few hundred live requests and is not
        # needed with a memory pool of the graphs' own.
        collecting = gc.isenabled()
        gc.disable()
        main = torch.cuda.current_stream(self.model.device)
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.model.device)
        self._capture_stream.wait_stream(main)
        try:
            with torch.cuda.stream(self._capture_stream):
                graph.capture_begin(pool=self._graph_pool)
                try:
                    captured = self._forward(ctx, True)
                finally:
                    graph.capture_end()
        finally:
            if collecting:
                gc.enable()
        main.wait_stream(self._capture_stream)
        launches = ops.launch_count() - before
        ops.LAUNCHES["count"] = before                     # a capture records launches, it runs none
        self._graphs.pop(key, None)
        self._graphs[key] = {"graph": graph, "ints": ints, "logits": captured, "signature": ctx.arena.signature(),
                             "launches": launches}
        while len(self._graphs) > self.MAX_GRAPHS:             # a long-lived server meets many (rows, width) classes
            self._graphs.pop(next(iter(self._graphs)))
        return StepResult(logits[:count], rows, count, ctx.arena.bytes_uploaded)

    def prepare_next(self) -> None:
        """Call after a step was launched and before its results are waited for: if that step
        was a captured decode step, the integer arrays of the step that most likely follows (the
        same requests, each one position on, the same pages) are built and packed now, while the
        GPU is busy. The next ``step`` uses them if its batch is the expected one and builds its
        own otherwise; the arrays are the same either way, only earlier."""
        last, self._last_graph_step = self._last_graph_step, None
        self._ahead = None
        if last is None:
            return
        batch, key = last
        size, width = key
        entries = []
        for e in batch.entries:
            position = e.first_position + 1
            if position >= self.model.layout.max_positions or \
                    any(position // self.block_size >= len(t) or t[position // self.block_size] == NULL_PAGE
                        for t in e.block_tables):
                return                      # a request ends or needs a page the table does not have yet
            entries.append(BatchEntry(e.seq_id, (0,), position, e.block_tables, (0,), e.state_slot))
        expected = ExecutionBatch(tuple(entries))
        ctx, rows = self._context(expected, table_width=width, pad_to=size)
        ctx.planning_context_len = width * self.block_size
        self._plan(ctx)
        ctx.arena.stage()
        self._ahead = {"key": key, "batch": expected, "ctx": ctx, "rows": rows}

    @staticmethod
    def _as_expected(batch: ExecutionBatch, expected: ExecutionBatch) -> bool:
        """Whether ``batch`` differs from ``expected`` in nothing but its token ids."""
        if len(batch.entries) != len(expected.entries):
            return False
        for e, x in zip(batch.entries, expected.entries):
            if e.seq_id != x.seq_id or e.first_position != x.first_position or e.state_slot != x.state_slot \
                    or e.block_tables != x.block_tables or e.logits_at != x.logits_at or len(e.token_ids) != 1:
                return False
        return True

    @property
    def status(self) -> torch.Tensor:
        """The device's status word (int32 [1]): zero unless a kernel recorded a fault. Callers
        that copy results to the host anyway read it in the same copy and hand the value to
        ``ops.raise_for_status``; ``check_status`` is the stand-alone form."""
        return self._status

    def check_status(self) -> None:
        """Raise if a kernel recorded a fault since the last check (this synchronises)."""
        ops.raise_for_status(int(self._status.item()), self.model.device)

    def execute(self, batch: ExecutionBatch) -> dict[str, np.ndarray]:
        """The reference's executor interface (src/paged_kv_serving/engine/engine.py:64-73):
        host float32 rows keyed by sequence id."""
        result = self.step(batch).by_sequence()
        self.check_status()
        return result
