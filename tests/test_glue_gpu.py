"""The fused block-glue kernels (RMSNorm, GroupNorm + gate + skip, one-token conv) against the eager torch
formulas of the reference block (cdssm/models/modules.py:50-53, cdssm/models/block.py:213-224)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _tol(dtype):
    return 2.0 ** -7 if dtype == torch.bfloat16 else 2e-5


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,d", [(5, 128), (300, 768), (33, 2048), (2500, 256), (7, 4096)])   # both kernels
def test_rms_norm(ops, dtype, rows, d):
    g = torch.Generator(device="cuda").manual_seed(rows + d)
    x = (torch.randn(rows, d, generator=g, device="cuda") * 3).to(dtype)
    w = (1 + 0.2 * torch.randn(d, generator=g, device="cuda")).to(dtype)
    eps = 2.0 ** -14
    xf = x.float()
    want = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(dtype) * w
    got = ops.rms_norm(x, w, eps)
    assert got.dtype == dtype
    assert (got.float() - want.float()).abs().max() <= _tol(dtype) * want.float().abs().max()
    assert torch.equal(ops.rms_norm(x.view(rows, 1, d), w, eps).view(rows, d), got)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("per_token", [False, True])
@pytest.mark.parametrize("B,L,di", [(2, 37, 256), (1, 200, 1536), (3, 1, 4096),
                                    (2, 2101, 256), (3, 1400, 768),     # >= 4096 rows: the four-rows-per-block kernel
                                    (1, 20000, 256)])                   # more positions than 512 tiles of 32
def test_groupnorm_gate(ops, dtype, per_token, B, L, di):
    G = 32
    g = torch.Generator(device="cuda").manual_seed(L + di)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")
    y = (rn(B, L, di) * 2 + 0.3).to(dtype)
    proj = rn(B, L, 3 * di + 16).to(dtype)
    z = proj[..., :di]                                         # a strided column slice, as in the block
    xc = rn(B, L, di).to(dtype)
    gw, gb, D = (1 + 0.1 * rn(di)).to(dtype), (0.1 * rn(di)).to(dtype), rn(di).to(dtype)
    if per_token:
        n = F.group_norm(y.float().reshape(B * L, di, 1), G, gw.float(), gb.float(), 1e-5).to(dtype).reshape(B, L, di)
    else:
        n = F.group_norm(y.float().transpose(1, 2), G, gw.float(), gb.float(), 1e-5).to(dtype).transpose(1, 2)
    want = n * F.silu(z) + D * xc
    got = ops.groupnorm_gate(y, gw, gb, z, D, xc, G, 1e-5, per_token=per_token)
    assert got.shape == want.shape and got.dtype == dtype
    assert (got.float() - want.float()).abs().max() <= 2 * _tol(dtype) * want.float().abs().max()
    assert torch.equal(got, ops.groupnorm_gate(y, gw, gb, z, D, xc, G, 1e-5, per_token=per_token))   # deterministic


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("Dm", [256, 52])                      # 16-byte vectors / the element-wise kernel
def test_conv_step_equals_full_conv(ops, dtype, Dm):
    B, L = 3, 9
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(B, L, Dm, generator=g, device="cuda").to(dtype)
    w = (torch.randn(Dm, 1, 4, generator=g, device="cuda") / 2).to(dtype)
    b = (0.1 * torch.randn(Dm, generator=g, device="cuda")).to(dtype)
    full = ops.CUDAConv1dSiLUOp.apply(x, w, b)
    hist = torch.zeros(B, 3, Dm, device="cuda", dtype=dtype)
    wide = torch.cat([x, x], dim=-1)                           # rows strided, like x_gate inside the projection
    for t in range(L):
        out = ops.conv1d_silu_step(wide[:, t, :Dm], hist, w, b)
        assert (out.float() - full[:, t].float()).abs().max() <= _tol(dtype) * full.float().abs().max()
    assert torch.equal(hist, x[:, L - 3:])
