"""The native step packer on the CPU: what it writes into a step's metadata against a plain restatement, its
refusals (which must leave every request as it was), stand-in segments, and a field added to the layout
table from outside."""
import numpy as np
import pytest

from gesso_b200.cache import CacheManager, PagedGroupSpec
from gesso_b200.engine import batch
from gesso_b200.engine.batch import QUERY_TILE, StepEntry, StepLayout, count_tiles, prepare_step
from gesso_b200.errors import ErrorCode, GessoError

VOCAB = 1000


def manager(pages=64, page_size=4, slots=6, ctx=128, groups=2):
    specs = [PagedGroupSpec("kv")] + [PagedGroupSpec(f"win{g}", window=9) for g in range(1, groups)]
    return CacheManager(specs, page_size, pages, slots, ctx)


def layout_for(entries, cm, tiles=None, rows=None):
    lens = [len(e.tokens) for e in entries]
    return StepLayout(n_tokens=sum(lens), n_segs=len(entries), n_rows=sum(len(e.want) for e in entries) if rows is None else rows,
                      n_groups=len(cm.groups), max_pages=cm.max_pages_per_request,
                      n_tiles=count_tiles(lens) if tiles is None else tiles)


def plain_pack(entries, starts, slots, tables, layout, scratch_slot, scratch_pages):
    """The same buffer, field by field, from the layout's offsets."""
    o = layout.offsets()
    out = np.full(o["_end"], -99, dtype=np.int32)
    cur, row, tile = 0, 0, 0
    for i, e in enumerate(entries):
        n = len(e.tokens)
        p0 = starts[i]
        out[o["seg_start"] + i] = cur
        out[o["seg_pos0"] + i] = p0
        out[o["slots"] + i] = slots[i]
        for t in range(n):
            out[o["token_ids"] + cur + t] = e.tokens[t]
            out[o["positions"] + cur + t] = p0 + t
            out[o["seg_of_token"] + cur + t] = i
        for w in e.want:
            out[o["logit_rows"] + row] = cur + w
            row += 1
        for q0 in range(0, n, QUERY_TILE):
            out[o["tile_seg"] + tile] = i
            out[o["tile_q0"] + tile] = q0
            tile += 1
        for g in range(layout.n_groups):
            at = o[f"block_table{g}"] + i * layout.max_pages
            out[at:at + layout.max_pages] = tables[g][i]
        cur += n
    out[o["seg_start"] + len(entries)] = cur
    ends = [starts[i] + len(e.tokens) for i, e in enumerate(entries) if e.req_id is not None]
    out[o["kv_span"]] = max(ends, default=0)                 # the longest sequence after the step and the
    out[o["kv_span"] + 1] = -(-sum(ends) // len(ends)) if ends else 0      # average one, over the real requests
    while tile < layout.n_tiles:
        out[o["tile_seg"] + tile] = len(entries) - 1
        out[o["tile_q0"] + tile] = 0
        tile += 1
    return out


@pytest.mark.parametrize("seed", range(6))
def test_packed_steps_equal_the_plain_packing(seed):
    rng = np.random.default_rng(seed)
    cm = manager()
    live = {}
    for step in range(12):
        while len(live) < 4:
            rid = f"r{step}_{len(live)}_{rng.integers(1 << 30)}"
            cm.admit(rid)
            live[rid] = 0
        chosen = [r for r in live if rng.random() < 0.8] or list(live)[:1]
        rng.shuffle(chosen)
        entries = []
        for rid in chosen:
            n = int(rng.choice([1, 1, 2, 3, 7, 70])) if live[rid] + 70 <= 110 else 1
            toks = rng.integers(0, VOCAB, n).tolist()
            want = sorted(rng.choice(n, size=int(rng.integers(0, min(n, 3) + 1)), replace=False).tolist())
            entries.append(StepEntry(rid, toks, want))
        n_standins = int(rng.integers(0, 3))
        packed = entries + [StepEntry(None, [0] * int(rng.integers(1, 5)), [0]) for _ in range(n_standins)]
        spare_tiles = int(rng.integers(0, 3)) if n_standins else 0
        layout = layout_for(packed, cm, tiles=count_tiles(len(e.tokens) for e in packed) + spare_tiles)
        out = np.full(layout.offsets()["_end"], -99, dtype=np.int32)
        scratch_slot, scratch_pages = 6, [64, 64]
        before = {rid: cm.length(rid) for rid in live}
        fresh, max_kv = prepare_step(cm, packed, layout, out, VOCAB, scratch_slot, scratch_pages)
        starts = [before[e.req_id] if e.req_id is not None else 0 for e in packed]
        slots = [cm.slot(e.req_id) if e.req_id is not None else scratch_slot for e in packed]
        tables = [[cm.block_table_row(e.req_id, g) if e.req_id is not None else np.full(cm.max_pages_per_request, scratch_pages[g])
                   for e in packed] for g in range(2)]
        want = plain_pack(packed, starts, slots, tables, layout, scratch_slot, scratch_pages)
        assert np.array_equal(out, want)
        assert sorted(fresh) == sorted(cm.slot(e.req_id) for e in entries if before[e.req_id] == 0)
        assert max_kv == max([before[e.req_id] + len(e.tokens) for e in entries]
                             + [len(e.tokens) for e in packed if e.req_id is None])
        cm.commit_step([e.req_id for e in entries], [len(e.tokens) for e in entries])
        for e in entries:
            live[e.req_id] += len(e.tokens)
        cm.check_invariants()
        for rid in [r for r in live if live[r] > 100 or rng.random() < 0.15]:
            cm.release(rid)
            del live[rid]


def test_refusals_name_the_request_and_reserve_nothing():
    cm = manager(pages=4, groups=1)
    for rid in ("x", "y"):
        cm.admit(rid)

    def attempt(entries, **kw):
        layout = layout_for(entries, cm, **kw)
        out = np.zeros(layout.offsets()["_end"], dtype=np.int32)
        return prepare_step(cm, entries, layout, out, VOCAB, 6, [4])

    cases = [
        ([StepEntry("x", [1], [0]), StepEntry("x", [2], [])], "twice", ErrorCode.INVALID_PLAN),
        ([StepEntry("nobody", [1], [0])], "not live", ErrorCode.INVALID_PLAN),
        ([StepEntry("x", [], [])], "no tokens", ErrorCode.INVALID_PLAN),
        ([StepEntry("x", [1, VOCAB], [])], f"token id {VOCAB}", ErrorCode.INVALID_PLAN),
        ([StepEntry("x", [1, -1], [])], "token id -1", ErrorCode.INVALID_PLAN),
        ([StepEntry("x", [1, 1 << 40], [])], "token id", ErrorCode.INVALID_PLAN),       # must not wrap to a valid id
        ([StepEntry("x", [1, 2], [2])], "wanted place 2", ErrorCode.INVALID_PLAN),
        ([StepEntry("x", [1.5], [])], "integers", ErrorCode.INVALID_PLAN),
        ([StepEntry("x", [1] * 9, []), StepEntry("y", [1] * 9, [])], "pages", ErrorCode.RESOURCE_LIMIT),   # 3 + 3 > 4
        ([StepEntry("x", [1] * 129, [])], "context", ErrorCode.RESOURCE_LIMIT),
    ]
    for entries, text, code in cases:
        with pytest.raises(GessoError, match=text) as ei:
            attempt(entries)
        assert ei.value.code == code
        assert cm.pages_in_use() == [0] and cm.length("x") == 0 and cm.length("y") == 0
        cm.check_invariants()
    # a layout that does not match the entries is a bug of the caller, not a silent overrun
    with pytest.raises(GessoError, match="layout"):
        attempt([StepEntry("x", [1, 2, 3], [0])], rows=2)
    assert cm.pages_in_use() == [0]
    fresh, max_kv = attempt([StepEntry("x", [1] * 9, [8]), StepEntry("y", [7], [0])])
    assert sorted(fresh) == [cm.slot("x"), cm.slot("y")] and max_kv == 9 and cm.pages_in_use() == [4]


def test_token_ids_may_be_left_open():
    cm = manager(groups=1)
    cm.admit("x")
    entries = [StepEntry("x", [0], [0])]
    layout = layout_for(entries, cm)
    out = np.full(layout.offsets()["_end"], 5, dtype=np.int32)
    prepare_step(cm, entries, layout, out, VOCAB, 6, [64], tokens_known=False)
    assert out[layout.offsets()["token_ids"]] == 0 and out[layout.offsets()["positions"]] == 0


def test_a_field_added_to_the_table_is_laid_out_filled_and_found():
    """One line in the layout table and a filler: the packer, the offsets and the context follow."""
    def fill(entries, view):
        view[:] = [len(e.tokens) * 10 + (0 if e.req_id is None else 1) for e in entries]
    batch.register_step_field("toy_per_segment", "seg", fill)
    try:
        cm = manager(groups=1)
        cm.admit("x")
        entries = [StepEntry("x", [3, 4, 5], [2]), StepEntry(None, [0], [0])]
        layout = layout_for(entries, cm)
        o = layout.offsets()
        assert o["toy_per_segment"] == o["block_table0"] + 2 * layout.max_pages and o["_end"] == o["toy_per_segment"] + 2
        out = np.zeros(o["_end"], dtype=np.int32)
        prepare_step(cm, entries, layout, out, VOCAB, 6, [64])
        assert out[o["toy_per_segment"]:].tolist() == [31, 10]
        with pytest.raises(GessoError):
            batch.register_step_field("toy_per_segment", "seg", fill)
        with pytest.raises(GessoError):
            batch.register_step_field("positions", "token", fill)
    finally:
        batch.unregister_step_field("toy_per_segment")
    assert "toy_per_segment" not in layout_for([StepEntry("x", [1], [])], cm).offsets()
