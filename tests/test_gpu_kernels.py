"""Each kernel alone against a plain PyTorch float32/float64 reference of the same operation, at
sizes other than the engine's (ragged widths, odd vocabularies, several head sizes)."""
import math

import numpy as np
import pytest
import torch

import plain_lfm2 as P

pytestmark = pytest.mark.gpu

DEV = "cuda"
BF16_EPS = 2.0 ** -8          # spacing of bfloat16 relative to the value (one rounding is half of it)


def rel_err(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / max(1e-30, float(b.abs().max())))


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ---- embedding, norms ------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H", [48, 1000, 2048])
def test_embed_and_add_rmsnorm(dtype, H):
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(H)
    V, N = 301, 37
    table = torch.randn(V, H, generator=g).to(dtype).to(DEV)
    toks = torch.randint(0, V, (N,), generator=g)
    h = ops.embed_gather(i32(toks.tolist()), table, 1.0)
    assert torch.equal(h.cpu(), table.float().cpu()[toks])
    delta = torch.randn(N, H, generator=g).to(dtype).to(DEV)
    bias = torch.randn(H, generator=g).to(DEV)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(DEV)
    h0 = h.clone()
    out = ops.add_rmsnorm(h, delta, bias, w, 1e-5, dtype)
    want_h = h0.double() + delta.double() + bias.double()
    assert rel_err(h, want_h) < 1e-6
    want = P.rmsnorm(want_h.cpu(), w.double().cpu(), 1e-5)
    assert rel_err(out, want) < (2e-6 if dtype == torch.float32 else BF16_EPS)
    # row selection: only the chosen rows, h untouched
    rows = i32([5, 0, 36])
    h1 = h.clone()
    sel = ops.add_rmsnorm(h, delta, None, w, 1e-6, torch.float32, rows=rows)
    assert torch.equal(h, h1)
    want = P.rmsnorm((h1.double() + delta.double()).cpu()[[5, 0, 36]], w.double().cpu(), 1e-6)
    assert rel_err(sel, want) < 2e-6
    # no delta: plain norm
    out = ops.add_rmsnorm(h, None, None, w, 1e-5, torch.float32)
    assert rel_err(out, P.rmsnorm(h1.double().cpu(), w.double().cpu(), 1e-5)) < 2e-6


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,N", [(512, 257), (1024, 300), (1536, 1001), (2048, 2040), (2560, 256), (2048, 255), (640, 400)])
def test_add_rmsnorm_many_rows(dtype, H, N):
    """Steps of 256 rows and more use a warp per row at the widths that kernel is compiled for (a number
    of rows that is no multiple of four; 255 rows and width 640 take the other kernels)."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(H + N)
    h = torch.randn(N, H, generator=g).to(DEV)
    h[N // 2] *= 100.0                                   # one row far larger than the others
    delta = torch.randn(N, H, generator=g).to(dtype).to(DEV)
    bias = torch.randn(H, generator=g).to(DEV)
    w = (1 + 0.1 * torch.randn(H, generator=g)).to(DEV)
    h0 = h.clone()
    out = ops.add_rmsnorm(h, delta, bias, w, 1e-5, dtype)
    want_h = h0.double() + delta.double() + bias.double()
    assert rel_err(h, want_h) < 1e-6
    want = P.rmsnorm(want_h.cpu(), w.double().cpu(), 1e-5)
    err = ((out.double().cpu() - want).abs() / want.abs().clamp_min(1.0)).max()
    assert float(err) < (2e-6 if dtype == torch.float32 else BF16_EPS)
    rows = i32(list(range(N - 1, -1, -1)))               # every row, backwards; h untouched
    h1 = h.clone()
    sel = ops.add_rmsnorm(h, delta, None, w, 1e-6, torch.float32, rows=rows)
    assert torch.equal(h, h1)
    want = P.rmsnorm((h1.double() + delta.double()).cpu().flip(0), w.double().cpu(), 1e-6)
    assert rel_err(sel, want) < 2e-6
    out = ops.add_rmsnorm(h, None, None, w, 1e-5, torch.float32)
    assert rel_err(out, P.rmsnorm(h1.double().cpu(), w.double().cpu(), 1e-5)) < 2e-6


def test_rmsnorm_rows_per_head():
    from gesso_b200 import ops
    x = torch.randn(11, 5, 24, device=DEV)
    w = torch.rand(24, device=DEV) + 0.5
    assert rel_err(ops.rmsnorm_rows(x, w, 1e-6), P.rmsnorm(x.double().cpu(), w.double().cpu(), 1e-6)) < 2e-6


# ---- matrix product, SwiGLU ---------------------------------------------------------------------------
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (7, 130, 33), (65, 64, 16), (200, 503, 96), (3, 2048, 700)])
def test_gemm_f32_is_true_fp32(M, N, K):
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(M * 1000 + K)
    a = torch.randn(M, K, generator=g).to(DEV)
    w = torch.randn(N, K, generator=g).to(DEV)
    got = ops.gemm_f32(a, w)
    want = a.double() @ w.double().T
    assert rel_err(got, want) < 5e-6        # FP32 sums of up to 700 terms; TF32 would be ~1e-3
    # rows do not depend on the batch they are in
    if M > 2:
        assert torch.equal(ops.gemm_f32(a[1:2].contiguous(), w), got[1:2])
    # mixed operands: bfloat16 activations with a matrix that stays float32
    ab = a.to(torch.bfloat16)
    assert rel_err(ops.gemm_f32(ab, w), ab.double() @ w.double().T) < 5e-6       # the same FP32 sums


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    from gesso_b200 import ops
    gu = (3 * torch.randn(19, 2 * 77, device=DEV)).to(dtype)
    g, u = gu[:, :77].double(), gu[:, 77:].double()
    want = (g / (1 + torch.exp(-g))) * u
    assert rel_err(ops.swiglu(gu), want) < (2e-6 if dtype == torch.float32 else BF16_EPS)


def test_linear_bf16_and_fp32_logits():
    from gesso_b200 import ops
    x = torch.randn(9, 160, device=DEV).to(torch.bfloat16)
    w = torch.randn(333, 160, device=DEV).to(torch.bfloat16)
    want = x.double() @ w.double().T
    assert rel_err(ops.linear(x, w, out_dtype=torch.float32), want) < 1e-5
    assert rel_err(ops.linear(x, w), want) < BF16_EPS


# ---- short convolution -----------------------------------------------------------------------------
def conv_reference(bcx, in_bias, taps, conv_bias):
    b = bcx.double().cpu()
    if in_bias is not None:
        b = b + in_bias.double().cpu()
    return P.short_conv_fir(b, taps.double().cpu(), None if conv_bias is None else conv_bias.double().cpu())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,L,bias", [(1, 2, False), (13, 4, True), (200, 3, False), (333, 4, True)])
def test_short_conv_carried_state(dtype, H, L, bias):
    """A sequence fed in calls of 5, 1, 1, 4, 2, 30 tokens equals one call (the reference's device
    parity test feeds (5, 1, 1, 4), test/test_lava_lfm25.jl:44-53); two requests share the batch and
    a reused slot starts from zero."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(H * 10 + L)
    cuts = [5, 1, 1, 4, 2, 30]
    T = sum(cuts)
    taps = torch.randn(H, L, generator=g).to(DEV)
    in_b = torch.randn(3 * H, generator=g).to(DEV) if bias else None
    cv_b = torch.randn(H, generator=g).to(DEV) if bias else None
    seqs = [torch.randn(T, 3 * H, generator=g).to(dtype).to(DEV) for _ in range(2)]
    want = [conv_reference(s, in_b, taps, cv_b) for s in seqs]
    state = torch.full((3, L - 1, H), 7.0, device=DEV)         # garbage: position 0 must ignore it
    state[1].zero_()
    state[2].zero_()
    pos = 0
    outs = [[], []]
    for n in cuts:
        # batch: request 0 (slot 2) and request 1 (slot 1), the second one token behind at first
        bcx = torch.cat([seqs[0][pos:pos + n], seqs[1][pos:pos + n]])
        out = ops.short_conv(bcx, in_b, taps, cv_b, state, i32([0] * n + [1] * n), i32([0, n, 2 * n]),
                             i32([pos, pos]), i32([2, 1]), 2, n)
        outs[0].append(out[:n])
        outs[1].append(out[n:])
        pos += n
    tol = 2e-6 if dtype == torch.float32 else BF16_EPS
    for k in range(2):
        assert rel_err(torch.cat(outs[k]), want[k]) < tol
    # slot 0 still holds garbage; a request starting there at position 0 must not read it
    fresh = ops.short_conv(seqs[0][:9].contiguous(), in_b, taps, cv_b, state, i32([0] * 9), i32([0, 9]),
                           i32([0]), i32([0]), 1, 9)
    assert rel_err(fresh, want[0][:9]) < tol
    # the two code paths (portion kernel + state update, and the short-portion kernel) leave the same state
    st_a = torch.zeros((1, L - 1, H), device=DEV)
    st_b = torch.zeros((1, L - 1, H), device=DEV)
    ops.short_conv(seqs[0][:12].contiguous(), in_b, taps, cv_b, st_a, i32([0] * 12), i32([0, 12]), i32([0]), i32([0]), 1, 12)
    for p in range(0, 12, 3):
        ops.short_conv(seqs[0][p:p + 3].contiguous(), in_b, taps, cv_b, st_b, i32([0] * 3), i32([0, 3]), i32([p]),
                       i32([0]), 1, 3)
    assert torch.equal(st_a, st_b)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,L,bias,packed", [(64, 3, False, True), (200, 4, True, False), (8, 2, False, True),
                                             (328, 3, True, True)])
def test_short_conv_long_portions(dtype, H, L, bias, packed):
    """Steps of hundreds of tokens (each thread walks runs of 8 tokens with the history in registers):
    three requests in one step whose borders fall inside a run, one of them starting at position 0 and
    the others carrying state from an earlier step; then a second long step.  Against the formulas."""
    from gesso_b200 import ops
    if packed and dtype != torch.bfloat16:
        pytest.skip("the packed layout belongs to bfloat16 runs")
    g = torch.Generator().manual_seed(H + 7 * L)
    lens1, lens2 = [5, 9, 0], [397, 313, 61]          # first a short step (carried state), then a long one
    T = [a + b_ for a, b_ in zip(lens1, lens2)]
    taps = torch.randn(H, L, generator=g).to(DEV)
    in_b = torch.randn(3 * H, generator=g).to(DEV) if bias else None
    cv_b = torch.randn(H, generator=g).to(DEV) if bias else None
    seqs = [torch.randn(t_, 3 * H, generator=g).to(dtype).to(DEV) for t_ in T]
    want = [conv_reference(s_, in_b, taps, cv_b) for s_ in seqs]

    def lay(x):       # rows as the (packed) projection gives them
        return x.reshape(-1, 3, H // 8, 8).permute(0, 2, 1, 3).reshape(-1, 3 * H).contiguous() if packed else x
    state = torch.full((4, L - 1, H), 3.0, device=DEV)           # stale values: position 0 must ignore them
    slots = [2, 0, 3]
    out1 = ops.short_conv(lay(torch.cat([seqs[0][:5], seqs[1][:9]])), in_b, taps, cv_b, state, i32([0] * 5 + [1] * 9),
                          i32([0, 5, 14]), i32([0, 0]), i32(slots[:2]), 2, 9, packed=packed)
    bcx = lay(torch.cat([seqs[0][5:], seqs[1][9:], seqs[2]]))
    n = lens2
    out2 = ops.short_conv(bcx, in_b, taps, cv_b, state, i32([0] * n[0] + [1] * n[1] + [2] * n[2]),
                          i32([0, n[0], n[0] + n[1], sum(n)]), i32([5, 9, 0]), i32(slots), 3, max(n), packed=packed)
    tol = 2e-6 if dtype == torch.float32 else BF16_EPS
    assert rel_err(out1[:5], want[0][:5]) < tol and rel_err(out1[5:], want[1][:9]) < tol
    assert rel_err(out2[:n[0]], want[0][5:]) < tol
    assert rel_err(out2[n[0]:n[0] + n[1]], want[1][9:]) < tol
    assert rel_err(out2[n[0] + n[1]:], want[2]) < tol
    # the state after the long step: the last L-1 products of every request
    for k, slot in enumerate(slots):
        r = seqs[k].double().cpu() + (in_b.double().cpu() if bias else 0)
        bx = (r[:, :H] * r[:, 2 * H:])[-(L - 1):]
        assert rel_err(state[slot], bx) < 1e-6


@pytest.mark.parametrize("H,L,bias", [(64, 3, False), (40, 4, True), (8, 2, False)])
def test_short_conv_packed_layout(H, L, bias):
    """The same convolution from rows of bcx laid out in groups of 24 columns (B, C, X of 8 channels)."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(H + L)
    T = 41
    taps = torch.randn(H, L, generator=g).to(DEV)
    in_b = torch.randn(3 * H, generator=g).to(DEV) if bias else None
    cv_b = torch.randn(H, generator=g).to(DEV) if bias else None
    bcx = torch.randn(T, 3 * H, generator=g).to(torch.bfloat16).to(DEV)
    packed = bcx.reshape(T, 3, H // 8, 8).permute(0, 2, 1, 3).reshape(T, 3 * H).contiguous()
    # pack_bcx permutes the rows of the projection the same way
    w = torch.arange(3 * H, dtype=torch.float32).reshape(3 * H, 1).repeat(1, 2)
    assert torch.equal(ops.pack_bcx(w)[:, 0], torch.arange(3 * H, dtype=torch.float32)
                       .reshape(3, H // 8, 8).permute(1, 0, 2).reshape(-1))
    for cuts in ([T], [9, 1, 1, 3, 27]):
        st_a = torch.zeros((1, L - 1, H), device=DEV)
        st_b = torch.zeros((1, L - 1, H), device=DEV)
        pos = 0
        for n in cuts:
            args = (i32([0] * n), i32([0, n]), i32([pos]), i32([0]), 1, n)
            a = ops.short_conv(bcx[pos:pos + n].contiguous(), in_b, taps, cv_b, st_a, *args)
            b = ops.short_conv(packed[pos:pos + n].contiguous(), in_b, taps, cv_b, st_b, *args, packed=True)
            assert torch.equal(a, b) and torch.equal(st_a, st_b)
            pos += n


@pytest.mark.parametrize("M", [1, 3, 8, 11, 16])
@pytest.mark.parametrize("H,K,L,bias", [(64, 64, 3, False), (2048, 2048, 3, False), (40, 96, 4, True),
                                        (8, 32, 2, False), (48, 8192, 3, True)])
def test_skinny_projection_with_conv_epilogue(M, H, K, L, bias):
    """Input projection + gated FIR + state shift in one kernel (a step of single tokens) against the
    projection followed by the convolution kernel, and against the formulas; fresh and running requests
    in one step, slots in any order, two steps in a row."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(M * 100 + H + K + L)
    w = (torch.randn(3 * H, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    wp = ops.pack_bcx(w)
    taps = torch.randn(H, L, generator=g).to(DEV)
    in_b = torch.randn(3 * H, generator=g).to(DEV) if bias else None
    cv_b = torch.randn(H, generator=g).to(DEV) if bias else None
    assert ops.skinny_conv_takes(M, wp, torch.bfloat16, L)
    slots = torch.randperm(M + 3, generator=g)[:M].tolist()
    st_fused = torch.randn(M + 3, L - 1, H, generator=g).to(DEV)
    st_split = st_fused.clone()
    st_ref = st_fused.double().cpu()
    pos = [0 if i % 3 == 0 else 5 + i for i in range(M)]           # every third request starts here
    for step in range(2):
        x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
        y = ops.linear_conv(x, wp, in_b, taps, cv_b, st_fused, i32(pos), i32(slots))
        bcx = ops.linear(x, w)
        y2 = ops.short_conv(bcx, in_b, taps, cv_b, st_split, i32(list(range(M))), i32(list(range(M + 1))),
                            i32(pos), i32(slots), M, 1)
        # the plain formulas on the rounded projection (src/Inference/lfm2.jl:253-271)
        r = (x.double() @ w.double().T).to(torch.bfloat16).double().cpu()
        if bias:
            r = r + in_b.double().cpu()
        B, C, X = r[:, :H], r[:, H:2 * H], r[:, 2 * H:]
        want = torch.zeros(M, H, dtype=torch.float64)
        for i in range(M):
            hist = torch.zeros(L - 1, H, dtype=torch.float64) if pos[i] == 0 else st_ref[slots[i]].clone()
            bx = B[i] * X[i]
            yv = (hist * taps.double().cpu().T[:L - 1]).sum(0) + bx * taps.double().cpu()[:, L - 1]
            if bias:
                yv = yv + cv_b.double().cpu()
            want[i] = C[i] * yv
            st_ref[slots[i]] = torch.cat([hist[1:], bx[None]])
        assert rel_err(y, want) < BF16_EPS
        assert rel_err(y2, want) < BF16_EPS
        assert rel_err(y, y2.double()) < BF16_EPS
        used = torch.tensor(slots)
        assert rel_err(st_fused[used.to(DEV)], st_ref[used]) < 1e-2 and rel_err(st_split[used.to(DEV)], st_ref[used]) < 1e-2
        assert rel_err(st_fused, st_split.double()) < 1e-2
        pos = [p + 1 for p in pos]
    # a norm in the prologue (weight folded into the matrix by the caller, or applied here)
    h = torch.randn(M, K, generator=g).to(DEV)
    nw = (1 + 0.1 * torch.randn(K, generator=g)).to(DEV)
    st1, st2 = st_fused.clone(), st_fused.clone()
    y1 = ops.linear_conv(ops.LazyNorm(h, nw, 1e-5, torch.bfloat16), wp, in_b, taps, cv_b, st1, i32(pos), i32(slots))
    y2 = ops.linear_conv(ops.add_rmsnorm(h, None, None, nw, 1e-5, torch.bfloat16), wp, in_b, taps, cv_b, st2,
                         i32(pos), i32(slots))
    assert rel_err(y1, y2.double()) < 2 * BF16_EPS


def test_short_conv_tap_order_identity():
    """All-ones B, C, X with taps [2, -1, 3] gives [3, 2, 4, 4] (the newest tap is on the current
    token; test/test_lfm25.jl:79-90 without its norm factor); reversed taps give something else."""
    from gesso_b200 import ops
    bcx = torch.ones(4, 3, device=DEV)
    state = torch.zeros(1, 2, 1, device=DEV)
    out = ops.short_conv(bcx, None, torch.tensor([[2.0, -1.0, 3.0]], device=DEV), None, state, i32([0] * 4),
                         i32([0, 4]), i32([0]), i32([0]), 1, 4)
    assert out.flatten().tolist() == [3.0, 2.0, 4.0, 4.0]
    state.zero_()
    out = ops.short_conv(bcx, None, torch.tensor([[3.0, -1.0, 2.0]], device=DEV), None, state, i32([0] * 4),
                         i32([0, 4]), i32([0]), i32([0]), 1, 4)
    assert out.flatten().tolist() == [2.0, 1.0, 4.0, 4.0]


def test_short_conv_nan_stays_in_its_channel():
    from gesso_b200 import ops
    bcx = torch.randn(6, 3 * 5, device=DEV)
    bcx[2, 3] = float("nan")                     # B of channel 3
    state = torch.zeros(1, 2, 5, device=DEV)
    out = ops.short_conv(bcx, None, torch.randn(5, 3, device=DEV), None, state, i32([0] * 6), i32([0, 6]),
                         i32([0]), i32([0]), 1, 6)
    bad = torch.isnan(out).any(dim=0).cpu()
    assert bad.tolist() == [False, False, False, True, False]


# ---- q/k norm, rotation, cache write -------------------------------------------------------------------
def build_cache(seqs_k, seqs_v, nkv, hd, page_size, dtype, shuffle_seed=0):
    """Paged K [pages, nkv, slot, hd] and V [pages, nkv, hd, slot] holding the given sequences on
    shuffled pages; returns (k_pages, v_pages, block_table).  Every slot that no sequence owns holds
    NaN, as a page may that a failed request gave back; only the V slots between a sequence's end and
    the end of that 16-slot block are zero, which is what the cache writer guarantees."""
    n_pages = sum((len(k) + page_size - 1) // page_size for k in seqs_k) + 3
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(shuffle_seed)).tolist()
    kp = torch.full((n_pages, nkv, page_size, hd), float("nan")).to(dtype)
    vp = torch.full((n_pages, nkv, hd, page_size), float("nan")).to(dtype)
    max_pages = max((len(k) + page_size - 1) // page_size for k in seqs_k) + 1
    bt = torch.full((len(seqs_k), max_pages), -1, dtype=torch.int32)
    nxt = 0
    for s, (k, v) in enumerate(zip(seqs_k, seqs_v)):
        for p in range((len(k) + page_size - 1) // page_size):
            page = perm[nxt]
            nxt += 1
            bt[s, p] = page
            rows = slice(p * page_size, min(len(k), (p + 1) * page_size))
            n = rows.stop - rows.start
            kp[page, :, :n] = k[rows].to(dtype).transpose(0, 1)
            vp[page, :, :, :n] = v[rows].to(dtype).permute(1, 2, 0)
            if rows.stop == len(k):
                vp[page, :, :, n:min(page_size, -(-n // 16) * 16)] = 0
    return kp.to(DEV), vp.to(DEV), bt.to(DEV)


def check_v_tails(vp, bt, starts, lens, page):
    """What the writer leaves behind a portion's last position: zeros up to the end of that position's
    16-slot block (the attention kernels multiply those slots with masked, zero probabilities), and
    the slots after that block, and every slot before the portion, as they were (NaN here)."""
    v = vp.float().cpu()
    for i, (s0, n) in enumerate(zip(starts, lens)):
        last = s0 + n - 1
        slot = last % page
        end = min(page, (slot // 16 + 1) * 16)
        pg = int(bt[i, last // page])
        assert torch.isfinite(v[pg, :, :, :slot + 1][..., max(0, slot + 1 - n):]).all()
        assert (v[pg, :, :, slot + 1:end] == 0).all(), "the rest of the last 16-slot block must be zero"
        assert torch.isnan(v[pg, :, :, end:]).all(), "slots behind that block are not the writer's"
        assert torch.isnan(v[int(bt[i, s0 // page]), :, :, :s0 % page]).all(), "slots before the portion stay"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 16, 16), (3, 1, 24, 8), (6, 3, 64, 16), (2, 2, 128, 32), (2, 1, 32, 48)])
def test_qk_norm_rope_store(dtype, nh, nkv, hd, page):
    from gesso_b200 import ops
    from gesso_b200.parts.rope import rope_tables
    g = torch.Generator().manual_seed(nh * 100 + hd)
    lens, starts = [5, 1, 19], [0, 40, 7]              # three portions at different positions
    N = sum(lens)
    qkv = torch.randn(N, (nh + 2 * nkv) * hd, generator=g).to(dtype)
    qw = torch.rand(hd, generator=g) + 0.5
    kw = torch.rand(hd, generator=g) + 0.5
    theta, eps = 12345.0, 1e-5
    cos, sin = rope_tables(theta, hd, 64)
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)])
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)])
    n_pages, max_pages = 16, (64 + page - 1) // page
    bt = torch.full((3, max_pages), -1, dtype=torch.int32)
    free = list(range(n_pages))[::-1]
    for i, (s, n) in enumerate(zip(starts, lens)):
        for p in range((s + n + page - 1) // page):
            bt[i, p] = free.pop()
    kp = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=dtype, device=DEV)
    vp = torch.full((n_pages, nkv, hd, page), float("nan"), dtype=dtype, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    q = ops.qk_norm_rope_store(qkv.to(DEV), qw.to(DEV), kw.to(DEV), eps, cos.to(DEV), sin.to(DEV), i32(positions.tolist()),
                               i32(seg.tolist()), bt.to(DEV), kp, vp, nh, nkv, hd, True, status)
    check_v_tails(vp, bt, starts, lens, page)
    x = qkv.double()
    qr = P.rope(P.rmsnorm(x[:, :nh * hd].reshape(N, nh, hd), qw.double(), eps), positions.tolist(), theta)
    kr = P.rope(P.rmsnorm(x[:, nh * hd:(nh + nkv) * hd].reshape(N, nkv, hd), kw.double(), eps), positions.tolist(), theta)
    vr = x[:, (nh + nkv) * hd:].reshape(N, nkv, hd)
    tol = 3e-6 if dtype == torch.float32 else BF16_EPS
    assert rel_err(q, qr) < tol
    for tkn in range(N):
        s, pos = int(seg[tkn]), int(positions[tkn])
        page_id, slot = int(bt[s, pos // page]), pos % page
        assert rel_err(kp[page_id, :, slot], kr[tkn]) < tol
        assert torch.equal(vp[page_id, :, :, slot].cpu().double(), vr[tkn].to(dtype).double())
    assert int(status.item()) == 0
    # a position without a page is recorded, nothing is written
    bt2 = bt.clone()
    bt2[1, 40 // page] = -1
    before = kp.clone()
    ops.qk_norm_rope_store(qkv.to(DEV), qw.to(DEV), kw.to(DEV), eps, cos.to(DEV), sin.to(DEV), i32(positions.tolist()),
                           i32(seg.tolist()), bt2.to(DEV), kp, vp, nh, nkv, hd, True, status)
    bits = torch.int32 if dtype == torch.float32 else torch.int16
    assert int(status.item()) == 1 and torch.equal(kp.view(bits), before.view(bits))


@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 32, 16), (6, 3, 64, 16), (2, 2, 128, 32), (32, 8, 64, 8), (3, 1, 64, 24)])
def test_qk_norm_rope_store_by_tiles(nh, nkv, hd, page):
    """The kernel for prompt portions (64-token tiles, v written along the slots of its transposed page)
    against the formulas: portions that start inside a page and inside a group of 8 positions, end
    anywhere, span several tiles, beside single tokens; stale values around the written slots stay."""
    from gesso_b200 import ops
    from gesso_b200.engine.batch import QUERY_TILE
    from gesso_b200.parts.rope import rope_tables
    g = torch.Generator().manual_seed(nh * 100 + hd + page)
    lens, starts = [150, 1, 67, 2, 9], [3, 40, 0, 250, 121]
    N, S = sum(lens), len(lens)
    ctx_len = 320
    qkv = torch.randn(N, (nh + 2 * nkv) * hd, generator=g).to(torch.bfloat16)
    qw = torch.rand(hd, generator=g) + 0.5
    kw = torch.rand(hd, generator=g) + 0.5
    theta, eps = 54321.0, 1e-6
    cos, sin = rope_tables(theta, hd, ctx_len)
    positions = torch.cat([torch.arange(s, s + n) for s, n in zip(starts, lens)])
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)])
    seg_start = [0]
    for n in lens:
        seg_start.append(seg_start[-1] + n)
    tile_seg, tile_q0 = [], []
    for i, n in enumerate(lens):
        for q0 in range(0, n, QUERY_TILE):
            tile_seg.append(i)
            tile_q0.append(q0)
    max_pages = (ctx_len + page - 1) // page
    n_pages = S * max_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    bt = torch.full((S, max_pages), -1, dtype=torch.int32)
    for i, (s0, n) in enumerate(zip(starts, lens)):
        for p in range((s0 + n + page - 1) // page):
            bt[i, p] = perm.pop()
    kp = torch.full((n_pages, nkv, page, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    vp = torch.full((n_pages, nkv, hd, page), float("nan"), dtype=torch.bfloat16, device=DEV)
    kp0, vp0 = kp.clone(), vp.clone()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert ops._lib.library().gesso_qk_rope_store_tiles_takes(hd, page, nh, nkv)
    args = (qkv.to(DEV), qw.to(DEV), kw.to(DEV), eps, cos.to(DEV), sin.to(DEV), i32(positions.tolist()),
            i32(seg.tolist()), bt.to(DEV))
    tiles = (i32(seg_start), i32(starts), i32(tile_seg), i32(tile_q0))
    q = ops.qk_norm_rope_store(*args, kp, vp, nh, nkv, hd, True, status, tiles=tiles)
    kp1, vp1 = kp0.clone(), vp0.clone()
    q1 = ops.qk_norm_rope_store(*args, kp1, vp1, nh, nkv, hd, True, status)      # one warp per (token, head)
    x = qkv.double()
    qr = P.rope(P.rmsnorm(x[:, :nh * hd].reshape(N, nh, hd), qw.double(), eps), positions.tolist(), theta)
    assert rel_err(q, qr) < BF16_EPS and rel_err(q, q1.double()) < BF16_EPS
    assert torch.equal(torch.isnan(kp), torch.isnan(kp1))                      # the same slots were written
    assert rel_err(kp.float().nan_to_num(0.0), kp1.float().nan_to_num(0.0)) < BF16_EPS
    # values are copied: identical, the cleared tails and the untouched slots (NaN) included
    assert torch.equal(vp.view(torch.int16), vp1.view(torch.int16))
    check_v_tails(vp, bt, starts, lens, page)
    written = torch.zeros(n_pages, page, dtype=torch.bool)
    for tkn in range(N):
        s0, pos = int(seg[tkn]), int(positions[tkn])
        written[int(bt[s0, pos // page]), pos % page] = True
    kc = kp.float().cpu()
    for pg in range(n_pages):
        for sl in range(page):
            assert bool(torch.isnan(kc[pg, :, sl]).all()) != bool(written[pg, sl]), "K: written slots only"
    assert int(status.item()) == 0
    bt2 = bt.clone()
    bt2[0, (3 + 70) // page] = -1                      # a page of the long portion is missing
    ops.qk_norm_rope_store(args[0], *args[1:8], bt2.to(DEV), kp, vp, nh, nkv, hd, True, status, tiles=tiles)
    assert int(status.item()) == 1


# ---- attention -----------------------------------------------------------------------------------
def attention_reference(q, ks, vs, seg_lens_new, window):
    """q [N, nh, hd]; per request: all keys/values so far (the new tokens are the last ones)."""
    outs = []
    cur = 0
    for k, v, n in zip(ks, vs, seg_lens_new):
        Lk = k.shape[0]
        qq = torch.zeros(Lk, q.shape[1], q.shape[2], dtype=torch.float64)
        qq[Lk - n:] = q[cur:cur + n].double()
        outs.append(P.causal_attention(qq, k.double(), v.double(), window)[Lk - n:])
        cur += n
    return torch.cat(outs).reshape(q.shape[0], -1)


CASES = [  # nh, nkv, hd, page
    (4, 2, 16, 16), (4, 1, 24, 8), (6, 3, 32, 16), (8, 2, 64, 16), (16, 1, 64, 32), (3, 3, 96, 16), (4, 2, 128, 16),
    (8, 2, 64, 32), (4, 2, 64, 16), (8, 1, 64, 16), (4, 1, 128, 48),
]


def make_attention_case(nh, nkv, hd, page, dtype, kv_lens, new_lens, seed):
    g = torch.Generator().manual_seed(seed)
    ks = [torch.randn(L, nkv, hd, generator=g).to(dtype) for L in kv_lens]
    vs = [torch.randn(L, nkv, hd, generator=g).to(dtype) for L in kv_lens]
    N = sum(new_lens)
    q = (2.0 * torch.randn(N, nh, hd, generator=g)).to(dtype)
    # one far key stands out: scale one (query, key) pair so that a single score dominates
    ks[0][3 % kv_lens[0]] *= 6.0
    kp, vp, bt = build_cache(ks, vs, nkv, hd, page, dtype, seed)
    positions = torch.cat([torch.arange(L - n, L) for L, n in zip(kv_lens, new_lens)])
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(new_lens)])
    starts = [0]
    for n in new_lens:
        starts.append(starts[-1] + n)
    return q, ks, vs, kp, vp, bt, positions, seg, starts


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("nh,nkv,hd,page", CASES)
def test_generic_attention(dtype, window, nh, nkv, hd, page):
    from gesso_b200 import ops
    kv_lens, new_lens = [150, 33, 1, 64], [20, 1, 1, 64]
    q, ks, vs, kp, vp, bt, positions, seg, _ = make_attention_case(nh, nkv, hd, page, dtype, kv_lens, new_lens, hd + page)
    out = ops.paged_attention_generic(q.to(DEV), kp, vp, bt, i32(positions.tolist()), i32(seg.tolist()), window,
                                      1.0 / math.sqrt(hd))
    want = attention_reference(q, ks, vs, new_lens, window)
    assert rel_err(out, want) < (5e-6 if dtype == torch.float32 else 2 * BF16_EPS)


@pytest.mark.parametrize("window", [None, 50])
@pytest.mark.parametrize("nh,nkv,hd,page", [c for c in CASES if c[2] in (32, 64, 96, 128)])
@pytest.mark.parametrize("splits", [1, 3, 8])
def test_decode_attention_split_kv(window, nh, nkv, hd, page, splits):
    from gesso_b200 import ops
    assert ops.fast_attention_takes(hd, page, nh, nkv)
    kv_lens = [500, 17, 1, 16, 129]
    new_lens = [1] * len(kv_lens)
    q, ks, vs, kp, vp, bt, positions, seg, starts = make_attention_case(nh, nkv, hd, page, torch.bfloat16, kv_lens,
                                                                         new_lens, hd + splits)
    want = attention_reference(q, ks, vs, new_lens, window)
    S = len(kv_lens)
    ws = (torch.empty(S * nh * splits * hd, device=DEV), torch.empty(S * nh * splits * 2, device=DEV),
          torch.zeros(S * nkv, dtype=torch.int32, device=DEV))
    for _ in range(2):      # twice with one workspace: the tickets of the first launch must have been reset
        out = ops.decode_attention(q.to(DEV), kp, vp, bt, i32(positions.tolist()), window,
                                   1.0 / math.sqrt(hd), splits, ws)
        assert rel_err(out, want) < 2 * BF16_EPS


def attention_reference_new_rows(q, ks, vs, new_lens, window=None):
    """The same as :func:`attention_reference` for long sequences: only the rows of the new tokens
    are computed (scores [n, keys] per head instead of [keys, keys])."""
    outs, cur = [], 0
    nh, nkv = q.shape[1], ks[0].shape[1]
    for k, v, n in zip(ks, vs, new_lens):
        Lk = k.shape[0]
        qq, kk, vv = q[cur:cur + n].double(), k.double(), v.double()
        pos = torch.arange(Lk - n, Lk)[:, None]
        key = torch.arange(Lk)[None, :]
        mask = key > pos
        if window is not None:
            mask = mask | (key < pos - window + 1)
        o = torch.zeros(n, nh, q.shape[2], dtype=torch.float64)
        for h in range(nh):
            g = h // (nh // nkv)
            sc = (qq[:, h] @ kk[:, g].T) / math.sqrt(q.shape[2])      # Inference.jl:1201-1207
            sc = sc.masked_fill(mask, float("-inf"))
            pr = torch.exp(sc - sc.max(dim=-1, keepdim=True).values)  # :1414-1430
            o[:, h] = (pr / pr.sum(dim=-1, keepdim=True)) @ vv[:, g]  # :1449-1457
        outs.append(o)
        cur += n
    return torch.cat(outs).reshape(q.shape[0], -1)


def test_new_rows_reference_is_the_plain_one():
    q, ks, vs, *_ = make_attention_case(4, 2, 32, 16, torch.float32, [70, 9], [13, 2], 5)
    for window in (None, 20):
        assert rel_err(attention_reference_new_rows(q, ks, vs, [13, 2], window),
                       attention_reference(q, ks, vs, [13, 2], window)) < 1e-12


def test_split_counts_of_the_benchmark_shapes():
    """What the decoding steps of the benchmark run with (LFM2-1.2B: 8 kv heads, context 4,096): one
    request has its keys split 16 ways, eight requests 4 ways, sixty-four not at all.  The tests below
    and the long-context replay run exactly these."""
    from gesso_b200 import ops
    assert ops.decode_splits(1, 8, 4096) == 16
    assert ops.decode_splits(8, 8, 4096) == 4
    assert ops.decode_splits(64, 8, 4096) == 1


@pytest.mark.parametrize("splits", [1, 4, 9, 16, 37])
def test_decode_attention_at_the_benchmark_context(splits):
    """Head 64, 32 query heads on 8 kv heads, 16-slot pages, up to 4,096 keys (256 pages a request):
    the split counts the benchmark's steps use (16 at batch 1, 4 at batch 8, 1 at batch 64), and odd
    ones whose parts do not divide the blocks evenly.  Lengths end at page and split borders."""
    from gesso_b200 import ops
    nh, nkv, hd, page = 32, 8, 64, 16
    kv_lens = [4096, 4095, 4081, 2049, 256, 4080, 1, 3000]
    new_lens = [1] * len(kv_lens)
    q, ks, vs, kp, vp, bt, positions, seg, starts = make_attention_case(nh, nkv, hd, page, torch.bfloat16, kv_lens,
                                                                         new_lens, 40 + splits)
    want = attention_reference_new_rows(q, ks, vs, new_lens)
    S = len(kv_lens)
    ws = (torch.empty(S * nh * splits * hd, device=DEV), torch.empty(S * nh * splits * 2, device=DEV),
          torch.zeros(S * nkv, dtype=torch.int32, device=DEV))
    for _ in range(2):
        out = ops.decode_attention(q.to(DEV), kp, vp, bt, i32(positions.tolist()), None, 1.0 / math.sqrt(hd), splits, ws)
        assert torch.isfinite(out).all()
        assert rel_err(out, want) < 2 * BF16_EPS


@pytest.mark.parametrize("window", [None, 700])
@pytest.mark.parametrize("kv_lens", [[4096, 300, 64, 1, 2047], [1500] * 3, [4000] + [40] * 44, [900, 880, 910, 870] * 10,
                                     [3000, 2900, 100, 90, 80, 3100, 17, 16, 15] * 4])
@pytest.mark.parametrize("splits", [1, 4, 8])
def test_decode_attention_cut_by_the_steps_lengths(splits, kv_lens, window):
    """The kernel is told the longest sequence of the step and the average one and decides per request how
    many of the grid's pieces it uses: one long request among short ones, even lengths that fill the device
    by themselves, few requests that do not, and a window that bounds what a request reads."""
    from gesso_b200 import ops
    nh, nkv, hd, page = 24, 8, 64, 16
    new_lens = [1] * len(kv_lens)
    q, ks, vs, kp, vp, bt, positions, seg, starts = make_attention_case(nh, nkv, hd, page, torch.bfloat16, kv_lens,
                                                                         new_lens, 77 + splits)
    want = attention_reference_new_rows(q, ks, vs, new_lens, window)
    S = len(kv_lens)
    ws = (torch.empty(S * nh * splits * hd, device=DEV), torch.empty(S * nh * splits * 2, device=DEV),
          torch.zeros(S * nkv, dtype=torch.int32, device=DEV))
    span = i32([max(kv_lens), -(-sum(kv_lens) // len(kv_lens))])
    for _ in range(2):      # twice with one workspace: the tickets must count the pieces in use, and be reset
        out = ops.decode_attention(q.to(DEV), kp, vp, bt, i32(positions.tolist()), window, 1.0 / math.sqrt(hd), splits, ws,
                                   kv_span=span)
        assert torch.isfinite(out).all()
        assert rel_err(out, want) < 2 * BF16_EPS
    # the cut changes which partial sums are merged, not what is summed
    whole = ops.decode_attention(q.to(DEV), kp, vp, bt, i32(positions.tolist()), window, 1.0 / math.sqrt(hd), splits, ws)
    assert rel_err(out, whole.double().cpu()) < BF16_EPS


@pytest.mark.parametrize("window", [None, 50])
@pytest.mark.parametrize("nh,nkv,hd,page", [c for c in CASES if c[2] in (32, 64, 96, 128)])
def test_prefill_attention_flash(window, nh, nkv, hd, page):
    from gesso_b200 import ops
    from gesso_b200.engine.batch import QUERY_TILE
    kv_lens, new_lens = [200, 70, 1, 130, 16], [200, 3, 1, 65, 2]     # whole prompt, portions, single tokens
    q, ks, vs, kp, vp, bt, positions, seg, starts = make_attention_case(nh, nkv, hd, page, torch.bfloat16, kv_lens,
                                                                         new_lens, hd + page + 1)
    tile_seg, tile_q0 = [], []
    for s, n in enumerate(new_lens):
        for q0 in range(0, n, QUERY_TILE):
            tile_seg.append(s)
            tile_q0.append(q0)
    pos0 = [L - n for L, n in zip(kv_lens, new_lens)]
    want = attention_reference(q, ks, vs, new_lens, window)
    out = ops.prefill_attention(q.to(DEV), kp, vp, bt, i32(starts), i32(pos0), i32(tile_seg), i32(tile_q0), window,
                                1.0 / math.sqrt(hd))
    assert rel_err(out, want) < 2 * BF16_EPS


def test_fast_attention_refuses_other_sizes():
    from gesso_b200 import ops
    assert not ops.fast_attention_takes(24, 16, 4, 1)
    assert not ops.fast_attention_takes(64, 8, 4, 1)
    assert not ops.fast_attention_takes(64, 16, 32, 1)      # 32 query heads per kv head


# ---- sampling ----------------------------------------------------------------------------------------
def test_argmax_ties_and_nonfinite():
    from gesso_b200 import ops
    V = 5003
    x = torch.randn(6, V)
    x[0, 4000] = x[0, 17] = 9.0                      # tie: the lowest id wins
    x[1, V - 1] = 11.0
    x[2, 3] = float("nan")
    x[3, 100] = float("inf")
    x[4] = -3.0                                      # all equal
    ids, bad = ops.argmax_rows(x.to(DEV))
    assert ids.tolist()[:2] == [17, V - 1] and ids.tolist()[4] == 0
    assert ids.tolist()[5] == int(torch.argmax(x[5]))
    assert bad.tolist() == [0, 0, 1, 1, 0, 0]


@pytest.mark.parametrize("V", [65536, 65530, 8192, 50001])
def test_argmax_wide_rows(V):
    """Rows of 8192 and more are scanned by 32 blocks each (16-byte reads where the width allows): ties
    inside one 16-byte group, across threads and across blocks go to the lowest id."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(V)
    x = torch.randn(9, V, generator=g)
    x[0, 4001] = x[0, 4002] = x[0, 17] = x[0, V - 1] = 9.0
    x[1, V - 1] = 11.0
    x[2, V // 2] = float("nan")
    x[3, 100] = float("-inf")
    x[4] = -3.0
    x[5, 2049] = x[5, 2048] = 12.0                    # neighbours in one group
    x[6, 5000] = x[6, 3000] = 12.0                    # same block, different threads
    ids, bad = ops.argmax_rows(x.to(DEV))
    assert ids.tolist()[:2] == [17, V - 1] and ids.tolist()[4:7] == [0, 2048, 3000]
    assert ids.tolist()[7:] == torch.argmax(x[7:], dim=1).tolist()
    assert bad.tolist() == [0, 0, 1, 1, 0, 0, 0, 0, 0]


@pytest.mark.parametrize("V", [503, 65536])
def test_sampler_matches_the_plain_rule(V):
    """Same seed, same ids as the plain full-sort sampler (temperature and nucleus)."""
    from gesso_b200.sampling import SamplingParams, SplitMix64, sample_host, select_tokens
    g = torch.Generator().manual_seed(V)
    rows = 12
    logits = 3.0 * torch.randn(rows, V, generator=g)
    logits[3] = 0.25                                  # flat row: every weight ties
    logits[4, 7] = 40.0                               # peaked row
    logits[5, :] = torch.round(logits[5, :])          # many ties
    params = [SamplingParams(temperature=[0.7, 1.3, 0.05][i % 3], top_p=[1.0, 0.9, 0.5, 0.999][i % 4], seed=i)
              for i in range(rows)]
    dev_rngs = [SplitMix64(p.seed) for p in params]
    host_rngs = [SplitMix64(p.seed) for p in params]
    plain = [P.PlainSampler(p.temperature, p.top_p, p.seed) for p in params]
    for _ in range(4):                                # several draws: the streams stay aligned
        got = select_tokens(logits.to(DEV), params, dev_rngs)
        want_host = [sample_host(logits[i].numpy(), params[i], host_rngs[i]) for i in range(rows)]
        want_plain = [plain[i].sample(logits[i].tolist()) for i in range(rows)] if V < 1000 else want_host
        assert got == want_host == want_plain


@pytest.mark.parametrize("V", [503, 65536, 50001])
@pytest.mark.parametrize("rows", [1, 20, 40, 100])
def test_sampler_rows_do_not_depend_on_the_batch(V, rows):
    """The kernel gives a row 8, 4, 2 or 1 blocks by the number of rows in the call; a row's id must be the
    same whichever it is: the 12 rows checked against the plain rule above, repeated to `rows` rows."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(V)
    logits = 3.0 * torch.randn(12, V, generator=g)
    logits[3] = 0.25
    logits[4, 7] = 40.0
    logits[5, :] = torch.round(logits[5, :])
    t = torch.tensor([[0.7, 1.3, 0.05][i % 3] for i in range(12)], dtype=torch.float64)
    p = torch.tensor([[1.0, 0.9, 0.5, 0.999][i % 4] for i in range(12)], dtype=torch.float64)
    u = torch.rand(12, generator=g, dtype=torch.float64)
    base, bad = ops.sample_rows(logits.to(DEV), t.to(DEV), p.to(DEV), u.to(DEV))
    assert bad.tolist() == [0] * 12
    idx = [i % 12 for i in range(rows)]
    got, bad = ops.sample_rows(logits[idx].contiguous().to(DEV), t[idx].to(DEV), p[idx].to(DEV), u[idx].to(DEV))
    assert bad.tolist() == [0] * rows
    assert got.tolist() == [base.tolist()[i] for i in idx]


def test_sampler_low_temperature_is_argmax_and_nucleus_keeps_the_top_set():
    from gesso_b200.sampling import SamplingParams, SplitMix64, select_tokens
    V = 1000
    logits = torch.randn(4, V)
    got = select_tokens(logits.to(DEV), [SamplingParams(1e-4, 1.0, s) for s in range(4)],
                        [SplitMix64(s) for s in range(4)])
    assert got == torch.argmax(logits, dim=1).tolist()
    # nucleus of mass 0.5 over three dominant ids: only they are ever drawn
    row = torch.full((1, V), -30.0)
    row[0, [5, 50, 500]] = torch.tensor([2.0, 1.5, 1.0])
    seen = set()
    for s in range(40):
        seen.add(select_tokens(row.to(DEV), [SamplingParams(1.0, 0.5, s)], [SplitMix64(s)])[0])
    assert seen <= {5, 50} and 5 in seen


# ---- copies between steps by a kernel -------------------------------------------------------------------
def test_copy_words_between_device_and_pinned_memory():
    """One launch, several segments, either way round, odd offsets and lengths (the 16-byte form and the
    word-by-word form); and the greedy selection writing ids and flags into pinned memory itself."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(5)
    host = torch.randint(0, 1 << 30, (5000,), generator=g, dtype=torch.int32).pin_memory()
    dev = torch.zeros(6000, dtype=torch.int32, device=DEV)
    ids = torch.arange(100, 164, dtype=torch.int32, device=DEV)
    back = torch.zeros(300, dtype=torch.int32).pin_memory()
    ops.copy_words([((dev, 8), (host, 8), 4000), ((dev, 0), (ids, 3), 5), ((dev, 5), (ids, 40), 3),
                    ((dev, 4101), (host, 4001), 999)])
    ops.copy_words([((back, 1), (dev, 0), 290)])
    torch.cuda.synchronize()
    want = torch.zeros(6000, dtype=torch.int32)
    want[8:4008] = host[8:4008]
    want[0:5] = torch.arange(103, 108)
    want[5:8] = torch.arange(140, 143)
    want[4101:5100] = host[4001:5000]
    assert torch.equal(dev.cpu(), want)
    assert torch.equal(back[1:291], want[:290]) and int(back[0]) == 0 and int(back[291]) == 0
    with pytest.raises(Exception):
        ops.copy_words([((dev, 5990), (host, 0), 20)])                       # leaves its tensor
    with pytest.raises(Exception):
        ops.copy_words([((dev, 0), (torch.zeros(4, dtype=torch.int32), 0), 4)])  # pageable host memory
    for V in (503, 65536):
        logits = torch.randn(7, V, generator=g).to(DEV)
        logits[3, 11] = float("nan")
        out = torch.full((2, 7), -1, dtype=torch.int32).pin_memory()
        got_ids, got_bad = ops.argmax_rows(logits, host_out=out)
        torch.cuda.synchronize()
        assert torch.equal(out[0], got_ids.cpu()) and torch.equal(out[1], got_bad.cpu())
        ref_ids, ref_bad = ops.argmax_rows(logits)
        assert torch.equal(got_ids, ref_ids) and torch.equal(got_bad, ref_bad) and int(out[1, 3]) == 1


# ---- skinny matrix product (steps of few tokens) -------------------------------------------------------
@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(16, 32), (48, 96), (2048, 2048), (160, 8192), (503 * 16, 64), (32, 352),
                                 (64, 4096), (2048, 8192), (48, 6144), (48, 6912), (32, 1728), (64, 1120)])
def test_skinny_gemm_epilogues(M, N, K):
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(M * 1000 + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    assert ops.skinny_takes(M, w, x.dtype)
    want = x.double() @ w.double().T
    assert rel_err(ops.linear(x, w, out_dtype=torch.float32), want) < 2e-6
    assert rel_err(ops.linear(x, w), want) < BF16_EPS
    # a row does not depend on the rows beside it
    if M > 1:
        assert torch.equal(ops.linear(x[M - 1:].contiguous(), w, out_dtype=torch.float32),
                           ops.linear(x, w, out_dtype=torch.float32)[M - 1:])
    # residual epilogue: h += x W^T + bias, in float32
    h = torch.randn(M, N, generator=g).to(DEV)
    bias = torch.randn(N, generator=g).to(DEV)
    h0 = h.clone()
    assert ops.linear_residual(x, w, h, bias) is None
    assert rel_err(h, h0.double() + want + bias.double()) < 2e-6
    # SwiGLU epilogue on the packed gate/up layout
    if N % 16 == 0:
        F = N // 2
        gate, up = w[:F], w[F:]
        a = ops.linear_swiglu(x, ops.pack_gate_up(gate, up), True)
        gg, uu = x.double() @ gate.double().T, x.double() @ up.double().T
        assert rel_err(a, (gg / (1 + torch.exp(-gg))) * uu) < BF16_EPS
        # the separate kernels give the same function on both layouts
        plain = ops.swiglu(torch.cat([gg, uu], dim=1).float().to(DEV))
        packed = ops.swiglu((x.double() @ ops.pack_gate_up(gate, up).double().T).float(), packed=True)
        assert rel_err(plain, packed) < 1e-6


@pytest.mark.parametrize("M", [1, 7, 8, 13, 16])
@pytest.mark.parametrize("H,F", [(2048, 8192), (1536, 6144), (2048, 4096), (256, 10240), (2560, 5120), (1536, 6912)])
def test_skinny_feed_forward_of_few_tokens(M, H, F):
    """The feed-forward of a decoding step at widths where a block walks several tiles (folded norm +
    gate/up product + SwiGLU, then the down product with its inner size split over blocks and the
    residual add) against the formulas.  An inner size of 6 chunks per warp (1536) uses six places of a
    queue of eight, 6912 splits into four shares of 54 chunks (seven per warp, the last one ragged), and
    10 chunks per warp (2560) take the path whose token-side fragments are reloaded tile after tile."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(M + H + F)
    gate = (torch.randn(F, H, generator=g) / math.sqrt(H)).to(torch.bfloat16).to(DEV)
    up = (torch.randn(F, H, generator=g) / math.sqrt(H)).to(torch.bfloat16).to(DEV)
    w1 = ops.pack_gate_up(gate, up)
    w2 = (torch.randn(H, F, generator=g) / math.sqrt(F)).to(torch.bfloat16).to(DEV)
    for rep in range(2):
        h = torch.randn(M, H, generator=g).to(DEV)
        h_two = h.clone()
        a = ops.linear_swiglu(ops.LazyNorm(h_two, None, 1e-5, torch.bfloat16), w1, True)
        assert ops.linear_residual(a, w2, h_two, None) is None
        # the kernel feeds bf16(h) to the tensor cores and divides by the root mean square afterwards
        hb = h.to(torch.bfloat16).double()
        rinv = 1.0 / torch.sqrt((h.double() ** 2).mean(dim=1, keepdim=True) + 1e-5)
        gg, uu = (hb @ gate.double().T) * rinv, (hb @ up.double().T) * rinv
        act = ((gg / (1 + torch.exp(-gg))) * uu)
        assert rel_err(a, act) < BF16_EPS
        want = h.double() + a.double() @ w2.double().T
        assert rel_err(h_two, want) < 1e-5
    x = torch.randn(M, H, generator=g).to(torch.bfloat16).to(DEV)              # plain input, no norm
    gg, uu = x.double() @ gate.double().T, x.double() @ up.double().T
    assert rel_err(ops.linear_swiglu(x, w1, True), (gg / (1 + torch.exp(-gg))) * uu) < BF16_EPS
    # the lm_head shape at those widths: many tiles per block, float32 output
    wv = (torch.randn(8192, H, generator=g) / math.sqrt(H)).to(torch.bfloat16).to(DEV)
    assert rel_err(ops.linear(x, wv, out_dtype=torch.float32), x.double() @ wv.double().T) < 2e-6


@pytest.mark.parametrize("M", [1, 5, 8, 16])
@pytest.mark.parametrize("N,K", [(64, 64), (6144, 2048), (32, 8192)])
def test_skinny_gemm_fused_norm(M, N, K):
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(M + N + K)
    h = (3 * torch.randn(M, K, generator=g)).to(DEV)
    nw = (1 + 0.1 * torch.randn(K, generator=g)).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    lazy = ops.LazyNorm(h, nw, 1e-5, torch.bfloat16)
    xn = lazy.materialize()
    want = xn.double() @ w.double().T                 # against the separate norm kernel's rounding
    got = ops.linear(lazy, w, out_dtype=torch.float32)
    assert rel_err(got, want) < 3 * BF16_EPS / math.sqrt(K) * 8 + 1e-3
    exact = P.rmsnorm(h.double().cpu(), nw.double().cpu(), 1e-5) @ w.double().cpu().T
    assert rel_err(got, exact) < BF16_EPS
    F = N // 2
    a = ops.linear_swiglu(lazy, ops.pack_gate_up(w[:F], w[F:]), True)
    gg, uu = exact[:, :F], exact[:, F:]
    assert rel_err(a, (gg / (1 + torch.exp(-gg))) * uu) < 2 * BF16_EPS


def test_skinny_gemm_refuses_other_sizes():
    from gesso_b200 import ops
    w = torch.zeros(40, 64, dtype=torch.bfloat16, device=DEV)
    assert not ops.skinny_takes(4, w, torch.bfloat16)             # 40 is not a multiple of 16
    assert not ops.skinny_takes(17, torch.zeros(64, 64, dtype=torch.bfloat16, device=DEV), torch.bfloat16)
    assert not ops.skinny_takes(4, torch.zeros(64, 200, dtype=torch.bfloat16, device=DEV), torch.bfloat16)
    # such products still work: they take the library path
    x = torch.randn(4, 200, device=DEV).to(torch.bfloat16)
    w2 = torch.randn(64, 200, device=DEV).to(torch.bfloat16)
    assert rel_err(ops.linear(x, w2), x.double() @ w2.double().T) < BF16_EPS


@pytest.mark.parametrize("M", [1, 7, 8, 13, 16])
@pytest.mark.parametrize("N,K", [(64, 64), (6144, 2048), (48, 8192), (32, 352)])
def test_skinny_gemm_folded_norm(M, N, K):
    """The norm's weight folded into the matrix: the kernel takes bf16(h), gathers sum(h^2) from the
    fragments it loads and scales in the epilogue.  Compared with the exact rmsnorm(h)*w @ W^T."""
    from gesso_b200 import ops
    g = torch.Generator().manual_seed(M * 7 + N + K)
    h = (3 * torch.randn(M, K, generator=g)).to(DEV)
    nw = (1 + 0.2 * torch.randn(K, generator=g)).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    wf = ops.fold_norm_weight(w, nw)
    exact = P.rmsnorm(h.double().cpu(), nw.double().cpu(), 1e-5) @ w.double().cpu().T
    lazy = ops.LazyNorm(h, None, 1e-5, torch.bfloat16)
    assert rel_err(ops.linear(lazy, wf, out_dtype=torch.float32), exact) < BF16_EPS
    assert rel_err(ops.linear(lazy, wf), exact) < 2 * BF16_EPS
    # the materialised form (norm kernel without a weight, then any product) agrees
    assert rel_err(lazy.materialize().double() @ wf.double().T, exact) < BF16_EPS
    if N % 16 == 0:
        F = N // 2
        a = ops.linear_swiglu(lazy, ops.pack_gate_up(wf[:F].contiguous(), wf[F:].contiguous()), True)
        gg, uu = exact[:, :F], exact[:, F:]
        assert rel_err(a, (gg / (1 + torch.exp(-gg))) * uu) < 2 * BF16_EPS
