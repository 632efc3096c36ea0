"""Backward kernels of the fused dynamics and the K/Q normalisation (through autograd on the reference's operator
classes) against the float64 gradient oracle, which tests/test_grad_oracle.py checks by finite differences."""
import numpy as np
import pytest
import torch

from util import const_args, to_np

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("B,H,L,N", [(2, 4, 50, 2), (1, 3, 33, 4), (1, 24, 70, 16)])
def test_dynamics_backward(ops, orc, dtype, tol, B, H, L, N):
    from oracle import grad_oracle as go
    inp = orc.make_inputs(B, H, L, 8, N=N, seed=L + N, bf16=dtype == torch.bfloat16, context_length=256)
    rng = np.random.default_rng(L)
    ups = [rng.standard_normal(s).astype(np.float32) for s in ((B, L, H, N), (B, L, H, N // 2), (B, L, H), (B, L, H))]
    if dtype == torch.bfloat16:
        ups = [orc.bf16_round(u) for u in ups]
    gate = torch.from_numpy(inp["gate_raw"]).cuda().to(dtype).requires_grad_(True)
    lds = torch.from_numpy(inp["log_dt_scale"]).cuda().requires_grad_(True)
    rf = torch.from_numpy(inp["rope_freqs"]).cuda()
    outs = ops.DynamicsFusedFn.apply(gate, lds, rf, *const_args(inp["consts"]), H, N)
    loss = sum((o.float() * torch.from_numpy(u).cuda()).sum() for o, u in zip(outs, ups))
    loss.backward()
    wg, wl = go.dynamics_backward(*ups, inp["gate_raw"], inp["log_dt_scale"], inp["rope_freqs"], inp["consts"], H, N)
    assert gate.grad.dtype == dtype and lds.grad.dtype == torch.float32
    assert np.abs(to_np(gate.grad) - wg).max() <= tol * np.abs(wg).max()
    assert np.abs(to_np(lds.grad) - wl).max() <= tol * max(np.abs(wl).max(), 1e-6)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("rows,D", [(37, 64), (5, 128), (9, 40)])
def test_normalize_backward(ops, orc, dtype, tol, rows, D):
    from oracle import grad_oracle as go
    rng = np.random.default_rng(rows)
    r = lambda: rng.standard_normal((1, rows, 1, D)).astype(np.float32) * 2
    K, Q, gK, gQ = r(), r(), r(), r()
    if dtype == torch.bfloat16:
        K, Q, gK, gQ = (orc.bf16_round(x) for x in (K, Q, gK, gQ))
    k = torch.from_numpy(K).cuda().to(dtype).requires_grad_(True)
    q = torch.from_numpy(Q).cuda().to(dtype).requires_grad_(True)
    kn, qn = ops.NormalizeKQFn.apply(k, q)
    ((kn.float() * torch.from_numpy(gK).cuda()).sum() + (qn.float() * torch.from_numpy(gQ).cuda()).sum()).backward()
    for got, up, x in ((k.grad, gK, K), (q.grad, gQ, Q)):
        want = go.normalize_backward(up, x)
        assert np.abs(to_np(got) - want).max() <= tol * np.abs(want).max()


def test_scan_side_backward_is_not_implemented(ops):
    x = torch.randn(1, 8, 16, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = torch.randn(16, 1, 4, device="cuda", dtype=torch.bfloat16)
    out = ops.CUDAConv1dSiLUOp.apply(x, w, torch.zeros(16, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(NotImplementedError):
        out.sum().backward()
