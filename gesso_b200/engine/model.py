"""A model put together from its spec: embedding, blocks in schedule order, final norm, head.

The model owns the bound parts and the *cache plan*: for every schedule entry, which cache it
owns or reads and which group that cache belongs to.  It knows nothing about requests; the
engine hands it a :class:`~gesso_b200.engine.batch.StepContext` and per-entry cache views.

Forward of one step (src/Inference/Inference.jl:2358-2521 is the reference's per-pass loop)::

    h = embedding[token_ids]                      (float32 residual stream)
    for entry in schedule:  pending = block(h, pending, ctx, cache_view(entry))
    logits = lm_head( final_norm(h + pending)[wanted rows] )      (then the spec's logit scale / soft cap, if any)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .. import ops
from ..cache.manager import PagedGroupSpec
from ..config.spec import ModelSpec
from ..errors import invalid
from ..parts.base import PagedNeed, ParamDecl, StateNeed
from ..parts.registry import build_block, build_norm
from ..weights.loader import model_param_decls, place_tensor


class Runtime:
    """What parts may ask of their surroundings: device, run dtype, position limit, shared tables."""

    def __init__(self, device, dtype: torch.dtype, max_positions: int):
        if dtype not in (torch.float32, torch.bfloat16):
            raise invalid(f"run dtype must be float32 or bfloat16, got {dtype}")
        self.device = torch.device(device)
        self.dtype = dtype
        self.max_positions = int(max_positions)
        self.shared: Dict = {}

    def attention(self, q, cache, ctx, window, scale):
        """Attention of the step's queries over the paged cache (kernel choice lives here)."""
        from . import attention_dispatch
        return attention_dispatch.paged_attention(self, q, cache, ctx, window, scale)


@dataclass
class PagedView:
    k_pages: torch.Tensor        # [pages, kv heads, page size, head size]
    v_pages: torch.Tensor
    block_table: torch.Tensor    # [segments, max pages] int32, -1 where no page is held
    writes: bool                 # False: this entry reads a cache another entry writes


@dataclass
class StateView:
    state: torch.Tensor          # [slots, *shape], the need's dtype
    slots: torch.Tensor          # [segments] int32
    writes: bool = True


@dataclass
class CacheSlotPlan:
    kind: str                    # "paged" | "state"
    owner: int                   # schedule entry that owns the cache
    group: int = -1              # paged group index
    index: int = -1              # index inside the group / among the state tensors
    need: object = None


class CachePlan:
    """Which caches every schedule entry uses, and the groups those caches form.

    A mixer declares no need, one, or a list of page and state needs (``Mixer.cache_need``);
    ``entries[e]`` lists the plans of schedule entry e in the order of its needs, and ``single[e]`` says
    that the mixer declared one bare need (its ``forward`` then gets the view itself, not a tuple)."""

    def __init__(self, spec: ModelSpec, blocks):
        self.entries: List[List[CacheSlotPlan]] = []
        self.single: List[bool] = []
        self.paged_groups: List[Tuple[PagedNeed, List[Tuple[int, int]]]] = []     # need, owning (entry, need index)
        self.state_entries: List[Tuple[StateNeed, int]] = []                      # need, owning entry
        group_of: Dict[PagedNeed, int] = {}
        for e, entry in enumerate(spec.schedule):
            if not (0 <= entry.layer < len(blocks)):
                raise invalid(f"schedule entry {e}: layer {entry.layer} does not exist")
            declared = blocks[entry.layer].cache_need()
            needs = [] if declared is None else (list(declared) if isinstance(declared, (list, tuple)) else [declared])
            self.single.append(declared is not None and not isinstance(declared, (list, tuple)))
            for need in needs:
                if not isinstance(need, (PagedNeed, StateNeed)):
                    raise invalid(f"schedule entry {e}: unknown cache need {need!r}")
            if entry.cache_of is not None and needs:
                o = entry.cache_of
                if not (0 <= o < e) or spec.schedule[o].cache_of is not None or not self.entries[o]:
                    raise invalid(f"schedule entry {e}: cache_of must name an earlier entry that owns a cache")
                theirs = self.entries[o]
                if len(theirs) != len(needs):
                    raise invalid(f"schedule entry {e}: the cache of entry {o} has another geometry")
                plans = []
                for need, op in zip(needs, theirs):
                    same = (isinstance(need, PagedNeed) and op.kind == "paged"
                            and (need.n_kv_heads, need.head_dim) == (op.need.n_kv_heads, op.need.head_dim)) or \
                           (isinstance(need, StateNeed) and op.kind == "state"
                            and (need.shape, need.dtype) == (op.need.shape, op.need.dtype))
                    if not same:
                        raise invalid(f"schedule entry {e}: the cache of entry {o} has another geometry")
                    if isinstance(need, PagedNeed) and op.need.window is not None and \
                            (need.window is None or need.window > op.need.window):
                        # the owner's window decides when pages are given back: a reader that looks further
                        # back would find them gone (and silently attend to fewer keys)
                        raise invalid(f"schedule entry {e}: reads the cache of entry {o} with a window of "
                                      f"{need.window or 'all'} keys, but that cache keeps only {op.need.window}")
                    plans.append(CacheSlotPlan(op.kind, o, op.group, op.index, need))
                self.entries.append(plans)
                continue
            plans = []
            for k, need in enumerate(needs):
                if isinstance(need, PagedNeed):
                    if need not in group_of:
                        group_of[need] = len(self.paged_groups)
                        self.paged_groups.append((need, []))
                    g = group_of[need]
                    self.paged_groups[g][1].append((e, k))
                    plans.append(CacheSlotPlan("paged", e, g, len(self.paged_groups[g][1]) - 1, need))
                else:
                    self.state_entries.append((need, e))
                    plans.append(CacheSlotPlan("state", e, -1, len(self.state_entries) - 1, need))
            self.entries.append(plans)

    def group_specs(self) -> List[PagedGroupSpec]:
        return [PagedGroupSpec(f"kv{n.n_kv_heads}x{n.head_dim}" + (f"w{n.window}" if n.window else ""), n.window)
                for n, _ in self.paged_groups]


class Model:
    def __init__(self, spec: ModelSpec, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
                 device="cuda", max_positions: int = 4096):
        self.spec = spec
        self.rt = Runtime(device, dtype, max_positions)
        self.dtype = dtype
        decls = model_param_decls(spec)
        missing = [n for n in decls if n not in tensors]
        if missing:
            raise invalid(f"model tensors missing: {missing[:8]}")
        dev: Dict[str, torch.Tensor] = {n: place_tensor(tensors[n], decls[n], dtype, self.rt.device)
                                        for n in decls}
        self.blocks = [build_block(b) for b in spec.blocks]
        for b, blk in zip(spec.blocks, self.blocks):
            blk.bind({k[len(b.prefix):]: v for k, v in dev.items() if k.startswith(b.prefix)}, self.rt)
        self.final_norm = build_norm(spec.final_norm)
        self.final_norm.bind({"weight": dev["final_norm.weight"]}, self.rt)
        self.embedding = dev["embedding.weight"]
        self.lm_head = self.embedding if spec.tie_embedding else dev["lm_head.weight"]
        self.cache_plan = CachePlan(spec, self.blocks)
        self.graph_safe = all(getattr(part, "graph_safe", True) for blk in self.blocks
                              for _, part in getattr(blk, "parts", lambda: [])())
        self.param_bytes = sum(t.numel() * t.element_size() for t in dev.values())

    @property
    def vocab_size(self) -> int:
        return self.spec.vocab_size

    def forward(self, ctx, views) -> Optional[torch.Tensor]:
        """Run the step's tokens; ``views[e]`` is the cache view of schedule entry e."""
        h = ops.embed_gather(ctx.token_ids, self.embedding, self.spec.embedding_scale)
        pending = (None, None)
        for e, entry in enumerate(self.spec.schedule):
            pending = self.blocks[entry.layer].forward(h, pending, ctx, views[e])
        if ctx.n_rows == 0:
            # the last sublayer's output is only needed by the head; nothing to return
            return None
        if ctx.rows_are_all_tokens and pending[0] is None:
            # every token's logits are wanted, in order: no gather, and the norm can ride in the
            # prologue of the head's matrix product
            if getattr(self.final_norm, "supports_lazy", False):
                x = self.final_norm.add_norm(h, None, None, lazy=True)
            else:
                x = self.final_norm.add_norm(h, None, None)
        else:
            x = self.final_norm.add_norm(h, pending[0], pending[1], rows=ctx.logit_rows)
        logits = ops.linear(x, self.lm_head, out_dtype=torch.float32)
        if self.spec.logit_scale != 1.0 or self.spec.logit_softcap is not None:
            ops.logit_transform(logits, self.spec.logit_scale, self.spec.logit_softcap)
        return logits
