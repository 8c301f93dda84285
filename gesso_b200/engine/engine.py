"""The step function and the device side of the cache.

:class:`Engine` ties a bound :class:`~gesso_b200.engine.model.Model` to a
:class:`~gesso_b200.cache.manager.CacheManager` and the device memory the manager's indices
point into.  Its one operation is :meth:`Engine.step`: a batch of (request, next tokens,
wanted places) runs as one flat batch from the cache that earlier steps left, and the logits
at the wanted places come back as float32 ``[wanted, vocab]``.  Admission, portioning and
sampling live above it (scheduler); nothing below it knows about requests.

Reference counterparts: the per-sequence prefill pass and decode step
(src/Inference/Inference.jl:2272-2530, 3270-3383) and the Session's page manager
(src/Inference/session.jl:687-828); the reference never batches sequences
(src/Inference/session.jl:18), so the mixed batch is this engine's own.
"""
from __future__ import annotations

import gc
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import numpy as np
import torch

from ..cache.manager import CacheManager
from .. import ops
from ..csrc.lib import launch_count
from ..errors import ErrorCode, GessoError, invalid, resource
from .batch import QUERY_TILE, StepContext, StepEntry, StepLayout, count_tiles, prepare_step
from .model import Model, PagedView, StateView


@dataclass
class StagedStep:
    """A decoding step prepared before its tokens are known: pages reserved, metadata packed in pinned
    host memory with the token ids left open (:meth:`Engine.stage_single_tokens`)."""

    req_ids: tuple
    layout: StepLayout
    slot_i: int
    host: torch.Tensor
    max_kv: int
    all_rows: bool


_ZERO_TOKEN = (0,)      # a stand-in's single token, and the place it wants


class DeviceCache:
    """Device memory for the manager's pages and slots."""

    def __init__(self, model: Model, page_size: int, num_pages: Sequence[int], num_slots: int):
        plan = model.cache_plan
        dev, dt = model.rt.device, model.dtype
        self.kv: List[torch.Tensor] = []
        for (need, owners), pages in zip(plan.paged_groups, num_pages):
            # Pages go from request to request as they are.  The tensor-core attention kernels multiply
            # masked probabilities (exact zeros) with the V slots of the 16-slot block that holds a
            # request's last position; the cache writer keeps those slots zero (qk_rope_store.cu), and
            # wholly masked pages are never read.  Zero-filled here only so that fresh memory is defined.
            # One page more than the manager hands out: the scratch page of padded steps.
            self.kv.append(torch.zeros((len(owners), 2, max(pages, 1) + 1, need.n_kv_heads, page_size,
                                        need.head_dim), dtype=dt, device=dev))
        self.scratch_pages = [max(pages, 1) for pages in num_pages]
        self.scratch_slot = max(num_slots, 1)
        # One buffer for all fixed-size state, a slot's entries side by side (each padded to 128 bytes),
        # so that a fresh slot is zeroed by one fill; entry i is the view [slots, *shape] into it, in the
        # dtype its need names.
        dtypes = [getattr(torch, need.dtype, None) for need, _ in plan.state_entries]
        for (need, _), t in zip(plan.state_entries, dtypes):
            if not isinstance(t, torch.dtype):
                raise invalid(f"state need: {need.dtype!r} is not a torch dtype")
        nbytes = [int(np.prod(need.shape)) * t.itemsize for (need, _), t in zip(plan.state_entries, dtypes)]
        offsets = np.concatenate([[0], np.cumsum([-(-n // 128) * 128 for n in nbytes])]).astype(int)
        self._state_flat = torch.zeros((max(num_slots, 1) + 1, max(int(offsets[-1]), 128)), dtype=torch.uint8,
                                       device=dev)       # the last slot is the scratch slot of padded steps
        self.state: List[torch.Tensor] = [
            self._state_flat[:, off:off + n].view(t).view((self._state_flat.shape[0],) + tuple(need.shape))
            for (need, _), t, off, n in zip(plan.state_entries, dtypes, offsets, nbytes)]

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv + [self._state_flat])

    def zero_slot(self, slot: int) -> None:
        if self.state:
            self._state_flat[slot].zero_()


class Engine:
    accepts_device_tokens = True      # step(entries, device_tokens=...): token ids the host has not read yet

    def __init__(self, model: Model, *, max_positions: Optional[int] = None, page_size: int = 16,
                 num_pages: Optional[int] = None, max_requests: int = 8, use_graphs: bool = True):
        self.model = model
        self.max_positions = int(max_positions or model.rt.max_positions)
        if self.max_positions > model.rt.max_positions:
            raise invalid(f"context {self.max_positions} exceeds the model's position limit "
                          f"{model.rt.max_positions}")
        self.page_size = int(page_size)
        plan = model.cache_plan
        per_req = (self.max_positions + self.page_size - 1) // self.page_size
        if num_pages is None:
            num_pages = per_req * max_requests
        self.num_pages = int(num_pages)
        groups = plan.group_specs()
        self.cache = CacheManager(groups, self.page_size, [self.num_pages] * len(groups),
                                  max_requests, self.max_positions)
        self.device_cache = DeviceCache(model, self.page_size, [self.num_pages] * len(groups), max_requests)
        # What kernels report instead of trapping: [0] a position without a cache page, [1] a tcgen05
        # pipeline wait that ran out.  Read back after steps (status_read_launch / status_read_finish,
        # or check_status); a word that is set fails the requests of the steps since the last read.
        self.status_words = torch.zeros((2,), dtype=torch.int32, device=model.rt.device)
        self.status = self.status_words[0:1]
        self._tc_status = self.status_words[1:2]
        self._unchecked: set = set()          # requests of steps whose status has not been read yet
        self._broken: Dict[Hashable, str] = {}     # requests that took part in a failed step: release only
        self._status_host = [torch.zeros((2,), dtype=torch.int32, pin_memory=True) for _ in range(4)]
        self._status_turn = 0
        self.steps_run = 0
        self.staged_steps_run = 0
        self.tokens_run = 0
        self.launches = 0            # kernels of this library launched by steps (graph nodes included)
        self.h2d_bytes = 0           # metadata bytes copied to the device by steps
        self.use_graphs = use_graphs and getattr(model, "graph_safe", True)
        self.max_graph_batch = 256
        self._graphs: Dict = {}
        self._portion_shapes: Dict = {}           # how often a single-portion step of a shape has come
        self._graph_pool = None
        self._capture_stream = None
        self._padded_rows = None      # set by _prepare for a step that was filled up to a padded shape
        self.padded_steps_run = 0
        # ring of pinned staging buffers; an event per buffer says when its copy has left it
        self._pinned: List[Optional[torch.Tensor]] = [None] * 4
        self._pinned_events: List[Optional[torch.cuda.Event]] = [None] * 4
        self._pinned_next = 0

    # ---- requests --------------------------------------------------------------------------
    def admit(self, req_id: Hashable) -> None:
        self.cache.admit(req_id)

    def release(self, req_id: Hashable) -> None:
        self.cache.release(req_id)
        self._broken.pop(req_id, None)
        self._unchecked.discard(req_id)

    def is_live(self, req_id: Hashable) -> bool:
        return self.cache.is_live(req_id)

    def length(self, req_id: Hashable) -> int:
        return self.cache.length(req_id)

    # ---- the step ----------------------------------------------------------------------------
    def _pinned_buffer(self, n: int):
        i = self._pinned_next
        self._pinned_next = (i + 1) % len(self._pinned)
        if self._pinned_events[i] is not None:
            self._pinned_events[i].synchronize()
        if self._pinned[i] is None or self._pinned[i].numel() < n:
            self._pinned[i] = torch.empty((max(n, 4096),), dtype=torch.int32, pin_memory=True)
        return i, self._pinned[i]

    def _prepare(self, entries: Sequence[StepEntry], tokens_known: bool = True):
        """Check the entries, reserve pages (for all the step's requests or for none), zero fresh slots and
        pack the step's metadata into pinned host memory: one call of the native step packer.  A mixed
        step whose padded shape has a graph (or is due one) is filled up with stand-ins first."""
        self._padded_rows = None
        if not entries:
            raise invalid("step: no entries")
        if self._broken:
            for e in entries:
                if e.req_id in self._broken:
                    raise self._broken_error(e.req_id)
        S = len(entries)
        lens = [len(e.tokens) for e in entries]
        T, R = sum(lens), sum(len(e.want) for e in entries)
        max_seg = max(lens) if lens else 0
        n_groups, max_pages = len(self.cache.groups), self.cache.max_pages_per_request
        padded = self._padded_shape(entries, S, T) if T > S else None
        if padded is not None:
            T_b, S_b = padded
            k = S_b - S                                   # stand-ins: k - 1 single tokens and one portion
            portion = T_b - T - (k - 1)                   # >= 1
            pad = [StepEntry(None, _ZERO_TOKEN, _ZERO_TOKEN) for _ in range(k - 1)]
            # the portion wants what is left of the S_b rows (the same place over and over)
            pad.append(StepEntry(None, [0] * portion, [0] * (S_b - R - (k - 1))))
            packed = list(entries) + pad
            layout = StepLayout(n_tokens=T_b, n_segs=S_b, n_rows=S_b, n_groups=n_groups, max_pages=max_pages,
                                n_tiles=T_b // QUERY_TILE + S_b)
            max_seg = max(max_seg, portion)
        else:
            packed = entries
            layout = StepLayout(n_tokens=T, n_segs=S, n_rows=R, n_groups=n_groups, max_pages=max_pages,
                                n_tiles=S if max_seg == 1 else count_tiles(lens))
        size = layout.offsets()["_end"]
        slot_i, host = self._pinned_buffer(size)
        dc = self.device_cache
        fresh, max_kv = prepare_step(self.cache, packed, layout, host.numpy()[:size], self.model.vocab_size,
                                     dc.scratch_slot, dc.scratch_pages, tokens_known)
        for slot in fresh:
            dc.zero_slot(slot)
        if padded is not None:
            self._all_rows = False
            self._padded_rows = R
            return layout, slot_i, host[:size], layout.n_tokens, max_kv
        if max_seg == 1:
            self._all_rows = R == S
        else:
            self._all_rows = R == T and all(len(e.want) == len(e.tokens) and list(e.want) == list(range(len(e.tokens)))
                                            for e in entries)
        return layout, slot_i, host[:size], max_seg, max_kv

    # ---- mixed steps in a few padded shapes, so that they replay graphs -------------------------------
    # A mixed step's kernels are launched one by one from the host unless its shape has a graph (some 140
    # launches, 2 ms of host time where the device needs 1.5), and the shapes of mixed steps hardly ever
    # repeat.  So a mixed step is filled up to one of a few shapes with stand-in requests: single tokens and
    # one portion of token id 0 at position 0, all on a scratch state slot and a scratch cache page that no
    # request owns.  They are ordinary entries to every kernel (what they compute is never read), so no kernel
    # knows of padding.  Segments go up to a multiple of 8 (at least one stand-in); tokens to the next of a
    # ladder of sizes whose steps grow with the size (64 up to 512 tokens, then an eighth of the size, so at
    # most an eighth of a step is padding); the wanted rows to the number of segments; the attention tiles
    # to the most that shape can have.  A shape's graph is captured the first time the shape comes.
    MAX_PADDED_SHAPES = 128

    @staticmethod
    def _padded_tokens(n: int) -> int:
        if n <= 512:
            return -(-n // 64) * 64
        step = 64
        while step * 16 < n:          # the step is between a sixteenth and an eighth of the size
            step *= 2
        return -(-n // step) * step

    def _padded_shape(self, entries, S: int, T: int):
        if (not self.use_graphs or S < 2 or T > 8192 or any(len(e.want) > 1 for e in entries)):
            return None
        S_b = -(-(S + 1) // 8) * 8
        T_b = self._padded_tokens(T + S_b - S)
        # The stand-in portion sits at positions 0 .. portion - 1 of a block table whose every entry is the
        # scratch page, and reads the rotary table at those positions: it has to fit both (an engine with
        # a context shorter than the padding runs its mixed steps unpadded).
        portion = T_b - T - (S_b - S - 1)
        if portion > min(self.cache.max_pages_per_request * self.page_size, self.max_positions):
            return None
        key = (T_b, S_b, S_b, False)
        if key not in self._graphs and sum(1 for k in self._graphs if k[0] > k[1] > 1) >= self.MAX_PADDED_SHAPES:
            return None              # too many shapes already: as it is, launched one by one
        return T_b, S_b

    def _upload(self, buf: torch.Tensor, slot_i: int, host: torch.Tensor, layout: Optional[StepLayout] = None,
                device_tokens=None) -> None:
        """The step's metadata from pinned host memory into ``buf``, and the token ids that are still on the
        device behind it.  Small buffers go by one kernel that reads the pinned memory itself (no change to
        the copy engine and back between two steps); where the device-sourced tokens are the first tokens of
        the step (as the scheduler puts them) the same launch copies them, and the host's place-holders for
        them are left out of the upload."""
        n = host.numel()
        if ops.KERNEL_COPIES and n <= ops.KERNEL_COPY_MAX_WORDS:
            skip, segs = 0, []
            if device_tokens is not None:
                ids, runs = device_tokens
                at = layout.offsets()["token_ids"]
                covered = sorted((dst, cnt) for _, dst, cnt in runs)
                prefix = 0
                for dst, cnt in covered:
                    if dst != prefix:
                        prefix = -1
                        break
                    prefix += cnt
                if at == 0 and prefix > 0 and len(runs) <= 5:
                    skip = prefix
                    segs = [((buf, dst), (ids, src), cnt) for src, dst, cnt in runs]
                    device_tokens = None
            ops.copy_words([((buf, skip), (host, skip), n - skip)] + segs)
        else:
            buf.copy_(host, non_blocking=True)
        if self._pinned_events[slot_i] is None:
            self._pinned_events[slot_i] = torch.cuda.Event()
        self._pinned_events[slot_i].record()
        self.h2d_bytes += n * 4
        self._fill_device_tokens(buf, layout, device_tokens)

    def build_context(self, entries: Sequence[StepEntry]) -> StepContext:
        """Reserve pages, zero fresh slots and upload the step's metadata (one transfer)."""
        layout, slot_i, host, max_seg, max_kv = self._prepare(entries)
        buf = torch.empty((host.numel(),), dtype=torch.int32, device=self.model.rt.device)
        self._upload(buf, slot_i, host)
        return StepContext(layout, buf, self.status, max_seg, max_kv, self._all_rows)

    def views(self, ctx: StepContext):
        """Per schedule entry what its mixer declared: ``None``, one view, or a tuple of views."""
        plan, dc = self.model.cache_plan, self.device_cache
        out = []
        for e, plans in enumerate(plan.entries):
            views = []
            for p in plans:
                if p.kind == "paged":
                    kv = dc.kv[p.group][p.index]
                    # K pages are [page, kv head, slot, feature]; V pages hold the same bytes as
                    # [page, kv head, feature, slot]
                    v = kv[1].view(kv.shape[1], kv.shape[2], kv.shape[4], kv.shape[3])
                    views.append(PagedView(kv[0], v, ctx.block_tables[p.group], writes=(p.owner == e)))
                else:
                    views.append(StateView(dc.state[p.index], ctx.slots, writes=(p.owner == e)))
            out.append(None if not views else views[0] if plan.single[e] else tuple(views))
        return out

    def step(self, entries: Sequence[StepEntry], device_tokens=None) -> Optional[torch.Tensor]:
        """Run one batch; returns float32 logits ``[wanted, vocab]`` (``None`` if nothing is wanted).

        ``device_tokens``: ``(ids, runs)`` for a step some of whose token ids the host has not seen yet:
        ``ids`` is an int32 tensor on the device (what an earlier selection left there), ``runs`` a list of
        ``(first id, first token of the step, count)``; those tokens (whatever the entries say) are copied
        from ``ids`` on the device, in stream order, before the step's kernels run.

        A step of single tokens only (decoding) replays a CUDA graph captured for its batch size:
        the metadata goes into the graph's fixed buffer and the whole layer loop is one launch.
        So does a step that is one prompt portion of a length seen before (the portions of a chunked
        prompt) with few wanted rows, and a mixed step whose padded shape has come before (see
        ``_padded_shape``).  The logits of such a step live in the graph's output buffer and are valid
        until the next step of the same shape.

        A step that raises after its kernels have started has written part of its keys, values and
        state: its requests can only be released (a later step with one of them is refused).
        """
        # a refusal here (bad entries, no pages: all requests' pages are reserved or none) leaves every
        # request as it was
        if device_tokens is not None:
            ids, runs = device_tokens
            n_given = sum(len(e.tokens) for e in entries)
            if (ids.dtype != torch.int32 or not ids.is_cuda
                    or any(n < 1 or src < 0 or dst < 0 or src + n > ids.numel() or dst + n > n_given for src, dst, n in runs)):
                raise invalid("step: device tokens must be int32 ids on the device and runs inside them and the step")
        layout, slot_i, host, max_seg, max_kv = self._prepare(entries)
        req_ids = [e.req_id for e in entries]
        self._unchecked.update(req_ids)
        try:
            with ops.tc_status_scope(self._tc_status):
                if self._padded_rows is not None:
                    # a mixed step filled up to a shape that has a graph (or gets one now)
                    logits = self._step_graph(layout, slot_i, host, max_kv, max_seg=max_seg, device_tokens=device_tokens)
                    logits = logits[:self._padded_rows] if self._padded_rows else None
                    self.padded_steps_run += 1
                elif self.use_graphs and max_seg == 1 and layout.n_segs <= self.max_graph_batch:
                    logits = self._step_graph(layout, slot_i, host, max_kv, device_tokens=device_tokens)
                elif self.use_graphs and self._portion_graph_wanted(layout):
                    logits = self._step_graph(layout, slot_i, host, max_kv, max_seg=max_seg, device_tokens=device_tokens)
                else:
                    buf = torch.empty((host.numel(),), dtype=torch.int32, device=self.model.rt.device)
                    self._upload(buf, slot_i, host, layout, device_tokens)
                    ctx = StepContext(layout, buf, self.status, max_seg, max_kv, self._all_rows)
                    before = launch_count()
                    logits = self.model.forward(ctx, self.views(ctx))
                    self.launches += launch_count() - before
            if max_seg == 1:
                self.cache.commit_single_tokens(req_ids)
            else:
                self.cache.commit_step(req_ids, [len(e.tokens) for e in entries])
        except Exception as e:
            self._mark_broken(req_ids, f"a step it took part in failed ({type(e).__name__}: {e})")
            raise
        self.steps_run += 1
        self.tokens_run += sum(len(e.tokens) for e in entries)
        return logits

    def stage_single_tokens(self, req_ids: Sequence[Hashable]) -> Optional[StagedStep]:
        """Prepare the decoding step that gives every request of ``req_ids`` one more token, while the
        device still runs the step before it: everything but the token ids (pages, positions, block
        tables) is settled on the host now, so that once the ids are sampled only they have to be
        filled in before the launch.  Returns ``None`` where steps are not replayed from graphs.  A
        staged step that is never run costs nothing but its page reservations, which the requests keep."""
        if not self.use_graphs or not req_ids or len(req_ids) > self.max_graph_batch:
            return None
        entries = [StepEntry(rid, _ZERO_TOKEN, _ZERO_TOKEN) for rid in req_ids]
        layout, slot_i, host, _, max_kv = self._prepare(entries, tokens_known=False)
        return StagedStep(tuple(req_ids), layout, slot_i, host, max_kv, self._all_rows)

    def step_staged(self, staged: StagedStep, tokens: Optional[Sequence[int]] = None,
                    device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run a staged step with its tokens (one per request, in the staged order); logits of every
        request.  The tokens come from the host (``tokens``) or straight from the device
        (``device_tokens``: int32 ids that an earlier selection left there), in which case the step
        starts without the host ever having seen them."""
        n = len(staged.req_ids)
        at = staged.layout.offsets()["token_ids"]
        if device_tokens is None:
            V = self.model.vocab_size
            if tokens is None or len(tokens) != n:
                raise invalid("step: a staged step takes one token per request")
            for rid, tok in zip(staged.req_ids, tokens):
                if not (0 <= tok < V):
                    raise invalid(f"step: token id {tok} of request {rid!r} is outside the vocabulary (0..{V - 1})")
            staged.host.numpy()[at:at + n] = tokens
        elif device_tokens.dtype != torch.int32 or device_tokens.numel() != n or not device_tokens.is_cuda:
            raise invalid("step: device tokens must be one int32 id per request on the device")
        self._all_rows = staged.all_rows
        self._unchecked.update(staged.req_ids)
        try:
            with ops.tc_status_scope(self._tc_status):
                logits = self._step_graph(staged.layout, staged.slot_i, staged.host, staged.max_kv,
                                          device_tokens=None if device_tokens is None else (device_tokens, [(0, 0, n)]))
            self.cache.commit_single_tokens(staged.req_ids)
        except Exception as e:
            self._mark_broken(staged.req_ids, f"a step it took part in failed ({type(e).__name__}: {e})")
            raise
        self.steps_run += 1
        self.staged_steps_run += 1
        self.tokens_run += staged.layout.n_tokens
        return logits

    def _portion_graph_wanted(self, layout: StepLayout) -> bool:
        """One prompt portion of at least 64 tokens with at most 16 wanted rows, of a length that has come
        before (a graph is captured at the second step of a shape, and for at most 8 shapes)."""
        if layout.n_segs != 1 or layout.n_tokens < 64 or layout.n_rows > 16:
            return False
        key = (layout.n_tokens, layout.n_segs, layout.n_rows, self._all_rows)
        if key in self._graphs:
            return True
        seen = self._portion_shapes.get(key, 0)
        self._portion_shapes[key] = seen + 1
        return seen >= 1 and sum(1 for k in self._graphs if k[0] > k[1] == 1) < 8

    @staticmethod
    def _fill_device_tokens(buf: torch.Tensor, layout: StepLayout, device_tokens) -> None:
        """Token ids that are still on the device go into the step's metadata there (device to device, in
        stream order, behind the upload of the rest)."""
        if device_tokens is None:
            return
        ids, runs = device_tokens
        at = layout.offsets()["token_ids"]
        for src, dst, n in runs:
            buf[at + dst:at + dst + n].copy_(ids[src:src + n])

    def _step_graph(self, layout: StepLayout, slot_i: int, host: torch.Tensor, max_kv: int,
                    device_tokens=None, max_seg: int = 1):
        key = (layout.n_tokens, layout.n_segs, layout.n_rows, self._all_rows)
        g = self._graphs.get(key)
        if g is None:
            buf = torch.zeros((host.numel(),), dtype=torch.int32, device=self.model.rt.device)
            self._upload(buf, slot_i, host, layout, device_tokens)
            ctx = StepContext(layout, buf, self.status, max_seg, self.max_positions, self._all_rows)
            views = self.views(ctx)
            # One eager run first: libraries initialise lazily, and capture records rather than runs,
            # so this run is also the one that produces the step's result.
            before = launch_count()
            logits = self.model.forward(ctx, views)
            n_launch = launch_count() - before
            self.launches += n_launch
            if self._capture_stream is None:
                self._capture_stream = torch.cuda.Stream(self.model.rt.device)
            ops.ensure_workspaces(self.model.rt.device, self._capture_stream)
            torch.cuda.synchronize(self.model.rt.device)
            graph = torch.cuda.CUDAGraph()
            # No garbage collection while the stream records: a collected object that owns device
            # resources (an older engine's graphs, for one) would free them in the middle of the
            # capture, which CUDA forbids and which invalidates the capture.
            gc_was_on = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool, stream=self._capture_stream):
                    out = self.model.forward(ctx, views)
            finally:
                if gc_was_on:
                    gc.enable()
            if self._graph_pool is None:
                self._graph_pool = graph.pool()
            self._graphs[key] = (graph, buf, out, n_launch)
            return logits
        graph, buf, out, n_launch = g
        self._upload(buf, slot_i, host, layout, device_tokens)
        graph.replay()
        self.launches += n_launch
        return out

    # ---- what the kernels reported ----------------------------------------------------------------
    def _mark_broken(self, req_ids, why: str) -> None:
        for rid in req_ids:
            if self.cache.is_live(rid):
                self._broken[rid] = why

    def _broken_error(self, req_id) -> GessoError:
        return GessoError(ErrorCode.RUNTIME, f"step: request {req_id!r} cannot go on: {self._broken[req_id]}; "
                          "what it holds in the cache is not valid any more, release it")

    def _status_error(self, words) -> Optional[GessoError]:
        if int(words[0]) != 0:
            return GessoError(ErrorCode.RUNTIME, "a kernel met a position without a cache page; the step's results "
                              "are not valid")
        if int(words[1]) != 0:
            return ops.tc_wait_error(int(words[1]))
        return None

    def status_read_launch(self):
        """Start the copy of the status words to pinned host memory, behind everything launched so far,
        without waiting.  Returns a ticket for :meth:`status_read_finish`."""
        self._status_turn = (self._status_turn + 1) % len(self._status_host)
        host = self._status_host[self._status_turn]
        if ops.KERNEL_COPIES:
            ops.copy_words([((host, 0), (self.status_words, 0), host.numel())])
        else:
            host.copy_(self.status_words, non_blocking=True)
        covered, self._unchecked = self._unchecked, set()
        return host, covered

    def status_read_finish(self, ticket, synchronize: bool = False):
        """Look at a launched read.  The caller has waited for something that was put on the stream after
        the read (the sampled ids' copy), or asks for ``synchronize``.  ``None`` if all is well; else
        ``(error, requests)``: the live requests of the steps the read covers, which are now marked and can
        only be released; the words are cleared for the steps to come."""
        host, covered = ticket
        if synchronize:
            torch.cuda.current_stream(self.model.rt.device).synchronize()
        error = self._status_error(host.numpy())
        if error is None:
            return None
        self.status_words.zero_()
        hit = [rid for rid in covered if self.cache.is_live(rid)]
        self._mark_broken(hit, str(error))
        return error, hit

    def check_status(self) -> None:
        """Raise if a kernel reported a position without a page or an exhausted wait since the last read
        (synchronises).  The requests of the steps since then are marked: they can only be released."""
        res = self.status_read_finish(self.status_read_launch(), synchronize=True)
        if res is not None:
            raise res[0]

    def stats(self) -> Dict[str, object]:
        return {
            "steps": self.steps_run, "staged_steps": self.staged_steps_run, "padded_steps": self.padded_steps_run,
            "tokens": self.tokens_run,
            "pages_in_use": self.cache.pages_in_use(), "pages_free": self.cache.free_pages(),
            "slots_in_use": self.cache.slots_in_use(), "cache_bytes": self.device_cache.bytes(),
            "live_requests": len(self.cache.live_requests()),
        }
