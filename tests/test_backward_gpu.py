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


def _r(orc, rng, shape, dtype, scale=1.0, lo=None, hi=None):
    a = (rng.uniform(lo, hi, shape) if lo is not None else rng.standard_normal(shape) * scale).astype(np.float32)
    return orc.bf16_round(a) if dtype == torch.bfloat16 else a


def _t(a, dtype, grad=True):
    t = torch.from_numpy(a).cuda().to(dtype)
    return t.requires_grad_(True) if grad else t


def _check(got, want, tol, what):
    want = np.asarray(want)
    err = np.abs(to_np(got) - want).max() / max(np.abs(want).max(), 1e-30)
    assert err <= tol, (what, err)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("M,C,H,N,D", [(3, 16, 2, 2, 64), (2, 9, 3, 4, 40), (1, 64, 4, 2, 128)])
def test_intra_chunk_scan_backward(ops, orc, dtype, tol, M, C, H, N, D):
    """The kernel and the oracle both take the SAVED forward outputs as the previous states, so both see the same
    (for bf16: rounded) values; the oracle's forward supplies them."""
    from oracle import grad_oracle as go
    rng = np.random.default_rng(C + D)
    A = _r(orc, rng, (M, C, H, N), dtype, lo=-0.7, hi=0.7)
    K = _r(orc, rng, (M, C, H, D), dtype, scale=1.0 / np.sqrt(D))
    V = _r(orc, rng, (M, C, H, N), dtype)
    be = _r(orc, rng, (M, C, H), dtype, lo=0.1, hi=0.9)
    u1 = _r(orc, rng, (M, C, H, N, D), dtype)
    u2 = _r(orc, rng, (M, C, H, N), dtype)
    tA, tK, tV, tb = (_t(x, dtype) for x in (A, K, V, be))
    lh, cA = ops.IntraChunkScanFn.apply(tA, tK, tV, tb, N)
    torch.autograd.backward([lh, cA], [_t(u1, dtype, False), _t(u2, dtype, False)])
    want = go.intra_backward(u1, u2, A, K, V, be, to_np(lh), to_np(cA))
    for got, w, name in zip((tA.grad, tK.grad, tV.grad, tb.grad), want, ("A", "K", "V", "beta")):
        assert got.dtype == dtype
        _check(got, w, tol, name)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 3e-2)])
@pytest.mark.parametrize("B,NC,C,H,N,D", [(2, 3, 16, 2, 2, 64), (1, 4, 8, 3, 4, 40), (1, 2, 32, 4, 2, 128)])
def test_inter_chunk_and_correction_backward(ops, orc, dtype, tol, B, NC, C, H, N, D):
    from oracle import grad_oracle as go
    rng = np.random.default_rng(NC + D)
    tot = _r(orc, rng, (B, NC, H, N), dtype, lo=-0.7, hi=0.7)
    fin = _r(orc, rng, (B, NC, H, N, D), dtype)
    up = _r(orc, rng, (B, NC, H, N, D), dtype)
    ta, tf = _t(tot, dtype), _t(fin, dtype)
    cs = ops.InterChunkScanFn.apply(ta, tf, N)
    cs.backward(_t(up, dtype, False))
    wA, wH = go.inter_backward(up, tot, to_np(cs))
    _check(ta.grad, wA, tol, "total_A")
    _check(tf.grad, wH, tol, "final_local_h")
    A = _r(orc, rng, (B, NC, C, H, N), dtype, lo=-0.7, hi=0.7)
    K = _r(orc, rng, (B, NC, C, H, D), dtype, scale=1.0 / np.sqrt(D))
    be = _r(orc, rng, (B, NC, C, H), dtype, lo=0.1, hi=0.9)
    st = _r(orc, rng, (B, NC, H, N, D), dtype)
    upc = _r(orc, rng, (B, NC, C, H, N, D), dtype)
    tA, tK, tb, ts = (_t(x, dtype) for x in (A, K, be, st))
    for true_gradient in (True, False):        # the derivative of the forward / the reference kernel's order
        for t in (tA, tK, tb, ts):
            t.grad = None
        ops.EXACT_CORRECTION_TRUE_GRADIENT = true_gradient
        try:
            corr = ops.ExactCorrectionFn.apply(tA, tK, tb, ts, N)
            corr.backward(_t(upc, dtype, False))
        finally:
            ops.EXACT_CORRECTION_TRUE_GRADIENT = False
        want = go.correction_backward(upc, A, K, be, st, to_np(corr), reference_order=not true_gradient)
        for got, w, name in zip((tA.grad, tK.grad, tb.grad, ts.grad), want, ("A", "K", "beta", "chunk_states")):
            _check(got, w, tol, (name, true_gradient))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("B,L,Dm", [(2, 150, 256), (1, 5, 48), (3, 64, 130)])
def test_conv_backward(ops, orc, dtype, tol, B, L, Dm):
    from oracle import grad_oracle as go
    rng = np.random.default_rng(L + Dm)
    x = _r(orc, rng, (B, L, Dm), dtype)
    w = _r(orc, rng, (Dm, 1, 4), dtype, scale=0.5)
    b = _r(orc, rng, (Dm,), dtype, scale=0.2)
    up = _r(orc, rng, (B, L, Dm), dtype)
    tx, tw, tb = (_t(a, dtype) for a in (x, w, b))
    ops.CUDAConv1dSiLUOp.apply(tx, tw, tb).backward(_t(up, dtype, False))
    gx, gw, gb = go.conv_backward(up, x, w.reshape(Dm, 4), b)
    assert tw.grad.shape == (Dm, 1, 4)
    _check(tx.grad, gx, tol, "x")
    _check(tw.grad.reshape(Dm, 4), gw, tol, "weight")
    _check(tb.grad, gb, tol, "bias")
