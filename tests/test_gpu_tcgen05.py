"""The tcgen05 matrix product against a float64 reference, smallest case first."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF16_EPS = 2.0 ** -8


def rel_err(a, b):
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).abs().max() / max(1e-30, float(b.abs().max())))


def case(M, N, K, seed=0):
    g = torch.Generator().manual_seed(seed + M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).to(torch.bfloat16).to(DEV)
    return x, w, x.double() @ w.double().T


@pytest.mark.parametrize("pair", [True, False])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 64), (128, 128, 256), (256, 512, 512), (2048, 2048, 2048),
                                   (300, 384, 200), (130, 1032, 72), (1000, 6144, 2048), (128, 2048, 8192), (40, 256, 128),
                                   (17, 64, 96), (256, 256, 64), (2040, 16384, 2048), (520, 264, 8192)])
def test_tcgen05_gemm(M, N, K, pair, monkeypatch):
    """Both kernels: one block per 128 x 256 tile, and (from 256 rows and columns on) two blocks per
    256 x 256 tile; every epilogue; sizes with ragged last tiles in every direction."""
    from gesso_b200 import ops
    monkeypatch.setattr(ops, "TC_PAIR", pair)
    if pair and not ops._lib.library().gesso_gemm_tcgen05_pair_takes(M, N, K):
        pytest.skip("below the pair kernel's sizes: the single-block kernel runs either way")
    x, w, want = case(M, N, K)
    got = ops.gemm_tcgen05(x, w, ops.EPI_F32)
    ops.check_tc_status()
    assert rel_err(got, want) < 3e-5      # float32 sums of up to 8192 products
    assert rel_err(ops.gemm_tcgen05(x, w, ops.EPI_BF16), want) < BF16_EPS
    h = torch.randn(M, N, device=DEV)
    bias = torch.randn(N, device=DEV)
    h0 = h.clone()
    ops.gemm_tcgen05(x, w, ops.EPI_RESID, out=h, bias=bias)
    assert rel_err(h, h0.double() + want + bias.double()) < 3e-5
    if N % 16 == 0:
        F = N // 2
        a = ops.gemm_tcgen05(x, ops.pack_gate_up(w[:F].contiguous(), w[F:].contiguous()), ops.EPI_SWIGLU)
        gg, uu = want[:, :F], want[:, F:]
        assert rel_err(a, (gg / (1 + torch.exp(-gg))) * uu) < BF16_EPS
    ops.check_tc_status()


@pytest.mark.parametrize("M,N,K", [(17, 128, 64), (32, 128, 64), (64, 256, 256), (17, 64, 96), (64, 2048, 2048),
                                   (64, 6144, 2048), (64, 16384, 2048), (64, 2048, 8192), (100, 1536, 6912),
                                   (128, 2048, 2048), (33, 504, 200), (48, 72, 72), (128, 65536, 2048), (20, 3072, 1024),
                                   (96, 264, 8192), (1, 128, 64), (5, 2048, 512)])
def test_tcgen05_few_rows(M, N, K):
    """The few-row product (W on the MMA's M side): every epilogue, tiles that one block finishes alone
    and tiles summed from the parts of a cluster's blocks, ragged sizes in every direction."""
    from gesso_b200 import ops
    x, w, want = case(M, N, K)
    for _ in range(2):
        got = ops.gemm_tcgen05_few(x, w, ops.EPI_F32)
        ops.check_tc_status()
        assert rel_err(got, want) < 3e-5
    assert torch.equal(got, ops.gemm_tcgen05_few(x, w, ops.EPI_F32))       # the order of the sum is fixed
    assert rel_err(ops.gemm_tcgen05_few(x, w, ops.EPI_BF16), want) < BF16_EPS
    h = torch.randn(M, N, device=DEV)
    bias = torch.randn(N, device=DEV)
    h0 = h.clone()
    ops.gemm_tcgen05_few(x, w, ops.EPI_RESID, out=h, bias=bias)
    assert rel_err(h, h0.double() + want + bias.double()) < 3e-5
    if N % 16 == 0:
        F = N // 2
        a = ops.gemm_tcgen05_few(x, ops.pack_gate_up(w[:F].contiguous(), w[F:].contiguous()), ops.EPI_SWIGLU)
        gg, uu = want[:, :F], want[:, F:]
        assert rel_err(a, (gg / (1 + torch.exp(-gg))) * uu) < BF16_EPS
    ops.check_tc_status()


@pytest.mark.parametrize("cluster", [1, 2, 3, 4, 5, 6, 7, 8])
def test_tcgen05_few_rows_clusters(cluster):
    """Every cluster size on one product; one large weight far along K and one near its start must each
    be counted once, whichever block of the cluster multiplies that part of K."""
    from gesso_b200 import ops
    M, N, K = 40, 256, 8192
    x = torch.ones(M, K, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(N, K, dtype=torch.bfloat16, device=DEV)
    w[130, 8000] = 64.0
    w[3, 70] = -2.0
    got = ops.gemm_tcgen05_few(x, w, ops.EPI_F32, cluster=cluster)
    ops.check_tc_status()
    want = torch.zeros(M, N, device=DEV)
    want[:, 130], want[:, 3] = 64.0, -2.0
    assert torch.equal(got, want)
    x, w, want = case(100, 2048, 6912)
    got = ops.gemm_tcgen05_few(x, w, ops.EPI_F32, cluster=cluster)
    ops.check_tc_status()
    assert rel_err(got, want) < 3e-5


# ---- flash prefill attention on tcgen05 --------------------------------------------------------------
@pytest.mark.parametrize("window", [None, 50, 200])
@pytest.mark.parametrize("nh,nkv,page", [(8, 2, 16), (32, 8, 16), (4, 2, 32), (8, 1, 16), (16, 1, 32),
                                         (24, 8, 16), (6, 2, 32), (10, 2, 16), (12, 2, 16), (7, 1, 16), (12, 1, 48)])
def test_tcgen05_prefill_attention(window, nh, nkv, page):
    import test_gpu_kernels as K
    from gesso_b200 import ops
    from gesso_b200.engine.batch import QUERY_TILE
    hd = 64
    assert ops.attention_tcgen05_takes(hd, page, nh, nkv)
    kv_lens, new_lens = [300, 70, 1, 130, 16, 257], [300, 3, 1, 65, 2, 129]   # whole prompt, portions, single tokens
    q, ks, vs, kp, vp, bt, positions, seg, starts = K.make_attention_case(nh, nkv, hd, page, torch.bfloat16, kv_lens,
                                                                           new_lens, nh + page)
    tile_seg, tile_q0 = [], []
    for s, n in enumerate(new_lens):
        for q0 in range(0, n, QUERY_TILE):
            tile_seg.append(s)
            tile_q0.append(q0)
    pos0 = [L - n for L, n in zip(kv_lens, new_lens)]
    out = ops.prefill_attention_tcgen05(q.to(DEV), kp, vp, bt, K.i32(starts), K.i32(pos0), K.i32(tile_seg), K.i32(tile_q0),
                                        window, 1.0 / math.sqrt(hd))
    ops.check_tc_status()
    want = K.attention_reference(q, ks, vs, new_lens, window)
    assert torch.isfinite(out).all()
    assert rel_err(out, want) < 2 * BF16_EPS


def test_tcgen05_prefill_attention_late_portion():
    """The benchmark's head layout (32 query heads on 8 kv heads of 64, 16-slot pages) with portions
    that start deep inside a sequence: 2,048 tokens from position 2,048 (every query reads more than
    2,048 keys over 256 pages), a short portion that ends at key 4,096, and one beside them that
    starts at a position that is no multiple of anything."""
    import test_gpu_kernels as K
    from gesso_b200 import ops
    from gesso_b200.engine.batch import QUERY_TILE
    nh, nkv, hd, page = 32, 8, 64, 16
    kv_lens, new_lens = [4096, 4096, 2500], [2048, 33, 131]
    q, ks, vs, kp, vp, bt, positions, seg, starts = K.make_attention_case(nh, nkv, hd, page, torch.bfloat16, kv_lens,
                                                                           new_lens, 91)
    tile_seg, tile_q0 = [], []
    for s, n in enumerate(new_lens):
        for q0 in range(0, n, QUERY_TILE):
            tile_seg.append(s)
            tile_q0.append(q0)
    pos0 = [L - n for L, n in zip(kv_lens, new_lens)]
    out = ops.prefill_attention_tcgen05(q.to(DEV), kp, vp, bt, K.i32(starts), K.i32(pos0), K.i32(tile_seg), K.i32(tile_q0),
                                        None, 1.0 / math.sqrt(hd))
    ops.check_tc_status()
    want = K.attention_reference_new_rows(q, ks, vs, new_lens)
    assert torch.isfinite(out).all()
    assert rel_err(out, want) < 2 * BF16_EPS
