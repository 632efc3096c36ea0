"""The six operator-level kernels against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from util import BF16_TOL, FP32_TOL, const_args, rel_err, to_dev, to_np

pytestmark = pytest.mark.gpu
DT = [(torch.float32, 0, FP32_TOL), (torch.bfloat16, 15, 2.0 ** -7)]


@pytest.mark.parametrize("dtype,mask,tol", DT)
@pytest.mark.parametrize("N", [2, 4, 16])
def test_dynamics(ops, orc, dtype, mask, tol, N):
    inp = orc.make_inputs(2, 6, 300, 32, N=N, seed=N, bf16=mask != 0)
    want = orc.dynamics(inp["gate_raw"], inp["log_dt_scale"], inp["rope_freqs"], inp["consts"], 6, N,
                        round_bf16=mask)
    got = ops.DynamicsFusedFn.apply(to_dev(inp["gate_raw"], dtype), to_dev(inp["log_dt_scale"], torch.float32),
                                    to_dev(inp["rope_freqs"], torch.float32), *const_args(inp["consts"]), 6, N)
    for g, w, name in zip(got, want, ("A_bar", "vp", "beta", "sel_C")):
        assert g.dtype == dtype and tuple(g.shape) == w.shape
        assert rel_err(to_np(g), w) <= tol, name


@pytest.mark.parametrize("dtype,mask,tol", DT)
@pytest.mark.parametrize("D", [64, 128, 48])
def test_normalize_kq(ops, orc, dtype, mask, tol, D):
    rng = np.random.default_rng(D)
    K = (rng.standard_normal((2, 33, 3, D)) * 3).astype(np.float32)
    Q = (rng.standard_normal((2, 33, 3, D)) * 0.2).astype(np.float32)
    if mask:
        K, Q = orc.bf16_round(K), orc.bf16_round(Q)
    wk, wq = orc.normalize_kq(K, Q, round_bf16=mask)
    gk, gq = ops.NormalizeKQFn.apply(to_dev(K, dtype), to_dev(Q, dtype))
    assert rel_err(to_np(gk), wk) <= tol and rel_err(to_np(gq), wq) <= tol


def _chunk_inputs(orc, BNC, C, H, D, N, seed, bf16):
    rng = np.random.default_rng(seed)
    mag = rng.uniform(0.3, 1.0, (BNC, C, H, N // 2))
    ang = rng.uniform(-3, 3, (BNC, C, H, N // 2))
    A = np.stack([mag * np.cos(ang), mag * np.sin(ang)], -1).reshape(BNC, C, H, N).astype(np.float32)
    K = rng.standard_normal((BNC, C, H, D)).astype(np.float32)
    K /= np.linalg.norm(K, axis=-1, keepdims=True)
    V = rng.standard_normal((BNC, C, H, N)).astype(np.float32)
    beta = rng.uniform(0, 1, (BNC, C, H)).astype(np.float32)
    if bf16:
        A, K, V, beta = (orc.bf16_round(x) for x in (A, K, V, beta))
    return A, K, V, beta


@pytest.mark.parametrize("dtype,mask,tol", [(torch.float32, 0, FP32_TOL), (torch.bfloat16, 15, BF16_TOL)])
@pytest.mark.parametrize("C,H,D,N", [(64, 3, 64, 2), (128, 2, 128, 2), (16, 2, 64, 16), (7, 1, 40, 4)])
def test_intra_inter_correction(ops, orc, dtype, mask, tol, C, H, D, N):
    B, NC = 2, 3
    A, K, V, beta = _chunk_inputs(orc, B * NC, C, H, D, N, seed=C + N, bf16=mask != 0)
    d = lambda x: to_dev(x, dtype)
    lh, cA = ops.IntraChunkScanFn.apply(d(A), d(K), d(V), d(beta), N)
    wlh, wcA = orc.intra_chunk(A, K, V, beta, N, round_bf16=mask)
    assert rel_err(to_np(lh), wlh) <= tol and rel_err(to_np(cA), wcA) <= tol
    tA = wcA.reshape(B, NC, C, H, N)[:, :, -1]
    fl = wlh.reshape(B, NC, C, H, N, D)[:, :, -1]
    cs = ops.InterChunkScanFn.apply(d(tA), d(fl), N)
    wcs = orc.inter_chunk(tA, fl, N, round_bf16=mask)
    assert rel_err(to_np(cs), wcs) <= tol
    r5 = lambda x: x.reshape(B, NC, *x.shape[1:])
    co = ops.ExactCorrectionFn.apply(d(r5(A)), d(r5(K)), d(r5(beta)), d(wcs), N)
    wco = orc.exact_correction(r5(A), r5(K), r5(beta), wcs, N, round_bf16=mask)
    assert tuple(co.shape) == (B, NC, C, H, N, D)
    assert rel_err(to_np(co), wco) <= tol


@pytest.mark.parametrize("dtype,mask,tol", DT)
@pytest.mark.parametrize("B,L,Dm", [(2, 100, 192), (1, 3, 40), (3, 1, 128)])
def test_conv1d_silu(ops, orc, dtype, mask, tol, B, L, Dm):
    rng = np.random.default_rng(L)
    x = rng.standard_normal((B, L, Dm)).astype(np.float32)
    w = (rng.standard_normal((Dm, 1, 4)) * 0.5).astype(np.float32)
    b = (rng.standard_normal(Dm) * 0.1).astype(np.float32)
    if mask:
        x, w, b = (orc.bf16_round(t) for t in (x, w, b))
    want = orc.conv1d_silu(x, w, b, round_bf16=mask)
    got = ops.CUDAConv1dSiLUOp.apply(to_dev(x, dtype), to_dev(w, dtype), to_dev(b, dtype))
    assert rel_err(to_np(got), want) <= tol


def test_errors_mirror_reference_checks(ops):
    x = torch.zeros(1, 4, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):                       # conv1d_silu.cu:241
        ops.CUDAConv1dSiLUOp.apply(x, torch.zeros(64, 1, 3, device="cuda"), torch.zeros(64, device="cuda"))
    K = torch.zeros(1, 4, 1, 256, device="cuda", dtype=torch.bfloat16)
    A = torch.zeros(1, 4, 1, 2, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):                       # intra_chunk_scan.cu:584
        ops.IntraChunkScanFn.apply(A, K, A, A[..., 0], 2)
