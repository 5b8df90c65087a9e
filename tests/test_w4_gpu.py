"""MXFP4 / NVFP4 weight-expanding GEMM against dequantise-then-matmul in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)


@pytest.fixture(scope="module")
def K():
    from cuteafd_b200.ops import kernels
    return kernels


def _quant(w, fmt):
    from cuteafd_b200.quant import codecs
    if fmt == "mxfp4":
        p, s = codecs.mxfp4_quant(w)
        return (p.to(DEV), s.to(DEV), None), codecs.mxfp4_dequant(p, s)
    p, s, g = codecs.nvfp4_quant(w)
    return (p.to(DEV), s.view(torch.uint8).to(DEV) if s.dtype != torch.uint8 else s.to(DEV), g.to(DEV)), codecs.nvfp4_dequant(p, s, g)


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("T,N,Kd,dual", [(1, 256, 512, False), (8, 200, 1024, True), (33, 384, 256, False), (100, 128, 2048, False),
                                         (64, 256, 384, True)])
def test_linear_w4(K, fmt, T, N, Kd, dual):
    g = torch.Generator().manual_seed(T + N)
    x = torch.randn(T, Kd, generator=g).to(torch.bfloat16)
    w = torch.randn(N, Kd, generator=g) * 0.05
    wq, wd = _quant(w, fmt)
    ref = x.float() @ wd.float().T
    wu = None
    if dual:
        wu, ud = _quant(torch.randn(N, Kd, generator=g) * 0.05, fmt)
        ref = torch.nn.functional.silu(ref) * (x.float() @ ud.float().T)
    for _ in range(2):
        out = K.linear_w4(x.to(DEV), wq, fmt, w_up=wu)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    err = (out.float().cpu() - ref).abs().max().item()
    assert err < 0.02 * max(1.0, ref.abs().max().item()), err
    dq = K.w4_dequant(wq, fmt).float().cpu()
    assert (dq - wd.float()).abs().max().item() <= 0.01 * wd.abs().max().item()


@pytest.mark.parametrize("fmt", ["mxfp4", "nvfp4"])
@pytest.mark.parametrize("T", [5, 48, 700])
def test_moe_w4(K, fmt, T):
    from cuteafd_b200.parallel.moe_exchange import ExchangeGeometry, LocalExchange
    from cuteafd_b200.quant import codecs
    H, I, E, k = 512, 256, 16, 4
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)
    logits = torch.randn(T, E, generator=g).to(DEV)
    res = torch.randn(T, H, generator=g).to(torch.bfloat16).to(DEV)

    def stack(rows, cols):
        qs = [_quant(torch.randn(rows, cols, generator=g) * 0.05, fmt) for _ in range(E)]
        packed = torch.stack([q[0][0] for q in qs]).contiguous()
        scales = torch.stack([q[0][1] for q in qs]).contiguous()
        glob = torch.cat([q[0][2] for q in qs]).contiguous() if fmt == "nvfp4" else None
        dense = torch.stack([q[1] for q in qs]).to(torch.bfloat16).to(DEV).contiguous()
        return (packed, scales, glob), dense
    (wg, dg), (wu, du), (wd, dd) = stack(I, H), stack(I, H), stack(H, I)
    ex = LocalExchange(ExchangeGeometry(H, I, E, k, 1024, 1), DEV)
    kw = dict(scoring="softmax", num_groups=1, topk_groups=1, normalize=True, routed_scale=1.0)
    out = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    ref = torch.empty(T, H, dtype=torch.bfloat16, device=DEV)
    ex.forward_w4(fmt, x, logits, kw, wg, wu, wd, out, residual=res)
    ex.forward(x, logits, kw, dg, du, dd, ref, residual=res)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    err = (out.float() - ref.float()).abs().max().item()
    assert err < 0.03 * max(1.0, ref.float().abs().max().item()), err


@pytest.mark.parametrize("bits", [2, 3, 4, 5, 8])
@pytest.mark.parametrize("T,Kd,N", [(1, 256, 128), (8, 512, 384), (70, 1024, 256)])
def test_linear_exl3(K, bits, T, Kd, N):
    from cuteafd_b200.quant import codecs
    g = torch.Generator().manual_seed(bits * 100 + T)
    trellis, suh, svh = codecs.exl3_random(Kd, N, bits, g, scale=0.02)
    x = torch.randn(T, Kd, generator=g).to(torch.bfloat16)
    w = codecs.exl3_dequant(trellis, suh, svh)                      # [K, N] float64
    ref = (x.double() @ w).float()
    for _ in range(2):
        out = K.linear_exl3(x.to(DEV), trellis.to(DEV), suh.to(DEV), svh.to(DEV))
    torch.cuda.synchronize()
    assert K.read_status() == 0
    err = (out.float().cpu() - ref).abs().max().item()
    assert err < 0.02 * max(1.0, ref.abs().max().item()), err
