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


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 64), (128, 128, 256), (256, 512, 512), (2048, 2048, 2048),
                                   (300, 384, 200), (130, 1032, 72), (1000, 6144, 2048), (128, 2048, 8192), (40, 256, 128), (17, 64, 96)])
def test_tcgen05_gemm(M, N, K):
    from gesso_b200 import ops
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
