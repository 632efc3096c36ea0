"""The gradient oracle (oracle/grad_oracle.py) against central finite differences of its own float64 forward, and
its forward against the C oracle of the reference's dynamics kernel (CPU only)."""
import numpy as np
import pytest

from oracle import grad_oracle as go
from util import rel_err


def _case(orc, B, H, L, N, seed):
    inp = orc.make_inputs(B, H, L, 8, N=N, seed=seed, context_length=64)
    rng = np.random.default_rng(seed)
    lds = inp["log_dt_scale"].astype(np.float64)
    return inp["gate_raw"].astype(np.float64), lds, inp["rope_freqs"].astype(np.float64), inp["consts"], rng


@pytest.mark.parametrize("N", [2, 4])
def test_forward_matches_the_c_oracle(orc, N):
    B, H, L = 2, 3, 17
    gate, lds, rf, c, _ = _case(orc, B, H, L, N, 3)
    A, vp, beta, selc = go.dynamics_forward(gate, lds, rf, c, H, N)
    wA, wvp, wbeta, wselc = orc.dynamics(gate.astype(np.float32), lds.astype(np.float32), rf.astype(np.float32), c, H, N)
    for got, want in ((A, wA), (vp, wvp), (beta, wbeta), (selc, wselc)):
        assert np.abs(got - want).max() <= 2e-5 * max(np.abs(want).max(), 1.0)


@pytest.mark.parametrize("N", [2, 4])
def test_dynamics_backward_is_the_derivative_of_the_forward(orc, N):
    B, H, L = 1, 3, 9
    gate, lds, rf, c, rng = _case(orc, B, H, L, N, 5)
    NH = N // 2
    up = [rng.standard_normal(s) for s in ((B, L, H, N), (B, L, H, NH), (B, L, H), (B, L, H))]

    def loss(gate_, lds_):
        outs = go.dynamics_forward(gate_, lds_, rf, c, H, N)
        return sum(float((o * u).sum()) for o, u in zip(outs, up))

    gg, gl = go.dynamics_backward(*up, gate, lds, rf, c, H, N)
    h = 1e-6
    fd = np.zeros_like(gate)
    it = np.nditer(gate, flags=["multi_index"])
    for _ in it:
        i = it.multi_index
        p, m = gate.copy(), gate.copy()
        p[i] += h
        m[i] -= h
        fd[i] = (loss(p, lds) - loss(m, lds)) / (2 * h)
    # the hard min / abs / clamp kinks have measure zero on random inputs; everything else is smooth
    assert np.abs(gg - fd).max() <= 2e-5 * max(np.abs(fd).max(), 1.0)
    fdl = np.zeros_like(lds)
    for i in range(H):
        p, m = lds.copy(), lds.copy()
        p[i] += h
        m[i] -= h
        fdl[i] = (loss(gate, p) - loss(gate, m)) / (2 * h)
    assert np.abs(gl - fdl).max() <= 2e-5 * max(np.abs(fdl).max(), 1.0)


def test_normalize_backward_is_the_derivative_of_the_forward():
    rng = np.random.default_rng(0)
    x = rng.standard_normal((5, 16)) * 2
    up = rng.standard_normal((5, 16))
    g = go.normalize_backward(up, x)
    h = 1e-6
    fd = np.zeros_like(x)
    for i in np.ndindex(*x.shape):
        p, m = x.copy(), x.copy()
        p[i] += h
        m[i] -= h
        fd[i] = ((go.normalize_forward(p) - go.normalize_forward(m)) * up).sum() / (2 * h)
    assert np.abs(g - fd).max() <= 1e-6 * max(np.abs(fd).max(), 1.0)


def _fd(loss, x, h=1e-6):
    fd = np.zeros_like(x)
    for i in np.ndindex(*x.shape):
        p, m = x.copy(), x.copy()
        p[i] += h
        m[i] -= h
        fd[i] = (loss(p) - loss(m)) / (2 * h)
    return fd


def _close(a, b, tol=2e-6):
    assert np.abs(a - b).max() <= tol * max(np.abs(b).max(), 1.0)


def test_intra_forward_matches_the_c_oracle_and_backward_is_its_derivative(orc):
    rng = np.random.default_rng(1)
    M, C, H, N, D = 2, 5, 2, 4, 3
    A = rng.uniform(-0.9, 0.9, (M, C, H, N))
    K = rng.standard_normal((M, C, H, D)) * 0.6
    V = rng.standard_normal((M, C, H, N))
    beta = rng.uniform(0.1, 0.9, (M, C, H))
    lh, cA = go.intra_forward(A, K, V, beta)
    wlh, wcA = orc.intra_chunk(A.astype(np.float32), K.astype(np.float32), V.astype(np.float32), beta.astype(np.float32), N)
    _close(lh, wlh, 1e-5)
    _close(cA, wcA, 1e-5)
    u1, u2 = rng.standard_normal(lh.shape), rng.standard_normal(cA.shape)
    loss = lambda A_, K_, V_, b_: float((go.intra_forward(A_, K_, V_, b_)[0] * u1).sum() + (go.intra_forward(A_, K_, V_, b_)[1] * u2).sum())
    gA, gK, gV, gB = go.intra_backward(u1, u2, A, K, V, beta, lh, cA)
    _close(gA, _fd(lambda t: loss(t, K, V, beta), A))
    _close(gK, _fd(lambda t: loss(A, t, V, beta), K))
    _close(gV, _fd(lambda t: loss(A, K, t, beta), V))
    _close(gB, _fd(lambda t: loss(A, K, V, t), beta))


def test_inter_and_correction_backward_are_the_derivatives(orc):
    rng = np.random.default_rng(2)
    B, NC, C, H, N, D = 1, 4, 3, 2, 2, 3
    tA = rng.uniform(-0.9, 0.9, (B, NC, H, N))
    fh = rng.standard_normal((B, NC, H, N, D))
    cs = go.inter_forward(tA, fh)
    _close(cs, orc.inter_chunk(tA.astype(np.float32), fh.astype(np.float32), N), 1e-5)
    up = rng.standard_normal(cs.shape)
    gA, gH = go.inter_backward(up, tA, cs)
    _close(gA, _fd(lambda t: float((go.inter_forward(t, fh) * up).sum()), tA))
    _close(gH, _fd(lambda t: float((go.inter_forward(tA, t) * up).sum()), fh))
    A = rng.uniform(-0.9, 0.9, (B, NC, C, H, N))
    K = rng.standard_normal((B, NC, C, H, D)) * 0.6
    beta = rng.uniform(0.1, 0.9, (B, NC, C, H))
    corr = go.correction_forward(A, K, beta, cs)
    _close(corr, orc.exact_correction(A.astype(np.float32), K.astype(np.float32), beta.astype(np.float32),
                                      cs.astype(np.float32), N), 1e-5)
    up = rng.standard_normal(corr.shape)
    gA, gK, gB, gS = go.correction_backward(up, A, K, beta, cs, corr)
    _close(gA, _fd(lambda t: float((go.correction_forward(t, K, beta, cs) * up).sum()), A))
    _close(gK, _fd(lambda t: float((go.correction_forward(A, t, beta, cs) * up).sum()), K))
    _close(gB, _fd(lambda t: float((go.correction_forward(A, K, t, cs) * up).sum()), beta))
    _close(gS, _fd(lambda t: float((go.correction_forward(A, K, beta, t) * up).sum()), cs))


def test_conv_backward_is_the_derivative(orc):
    rng = np.random.default_rng(3)
    B, L, Dm = 2, 7, 3
    x, w, b = rng.standard_normal((B, L, Dm)), rng.standard_normal((Dm, 4)), rng.standard_normal(Dm)
    out = go.conv_forward(x, w, b)
    _close(out, orc.conv1d_silu(x.astype(np.float32), w.astype(np.float32), b.astype(np.float32)), 1e-5)
    up = rng.standard_normal(out.shape)
    gx, gw, gb = go.conv_backward(up, x, w, b)
    _close(gx, _fd(lambda t: float((go.conv_forward(t, w, b) * up).sum()), x))
    _close(gw, _fd(lambda t: float((go.conv_forward(x, t, b) * up).sum()), w))
    _close(gb, _fd(lambda t: float((go.conv_forward(x, w, t) * up).sum()), b))


def test_gradient_oracle_matches_the_reference_backward_kernels():
    """The pin of the gradient oracle: tests/golden/bwd_ref.npz holds what the reference's own backward kernels
    (compiled unmodified for sm_100, run on a B200 by tests/golden/make_golden_ref.py) returned for seeded inputs,
    their own forward outputs as saved tensors and seeded upstream gradients.  The float64 oracle reproduces them
    within the bfloat16 storage of the reference's outputs - the correction backward only in ``reference_order``
    (the reference adds the upstream gradient before the step it belongs behind, and its grad_beta is head_dim
    times the derivative)."""
    import os
    from golden.golden_cases import unbits
    from oracle import grad_oracle as go
    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "bwd_ref.npz"))
    f = lambda n: unbits(g[n]).astype(np.float64) if g[n].dtype == np.uint16 else g[n].astype(np.float64)
    B, NC, C, H, N, D = (int(x) for x in g["sizes"])
    close = lambda got, want, tol, what: rel_err(got, want) <= tol or pytest.fail(f"{what}: {rel_err(got, want):.3g} > {tol}")
    # dynamics
    c = dict(zip(("gating_c", "omega_thresh", "adt_delta", "adt_smoothness", "adt_eps"), g["dyn_consts"]))
    gg, gl = go.dynamics_backward(f("dyn_uA"), f("dyn_uvp"), f("dyn_ubeta"), f("dyn_uselc"), f("dyn_gate"), f("dyn_lds"),
                                  f("dyn_rope"), c, H, N)
    close(gg, f("dyn_ggate"), 2e-2, "dynamics grad_gate_raw")
    close(gl, f("dyn_glds"), 2e-2, "dynamics grad_log_dt_scale")
    # normalisation
    close(go.normalize_backward(f("nrm_uK"), f("nrm_K")), f("nrm_gK"), 1e-2, "normalize grad_K")
    close(go.normalize_backward(f("nrm_uQ"), f("nrm_Q")), f("nrm_gQ"), 1e-2, "normalize grad_Q")
    # intra-chunk scan
    got = go.intra_backward(f("intra_ulh"), f("intra_ucA"), f("A"), f("K"), f("V"), f("beta"), f("local_h"), f("cum_A"))
    for x, n in zip(got, ("intra_gA", "intra_gK", "intra_gV", "intra_gbeta")):
        close(x, f(n), 2e-2, n)
    # inter-chunk carry
    gA, gH = go.inter_backward(f("inter_u"), f("inter_tot"), f("inter_states"))
    close(gA, f("inter_gA"), 2e-2, "inter grad_total_A")
    close(gH, f("inter_gH"), 2e-2, "inter grad_final_h")
    # correction: the reference's order (and not the derivative of its forward)
    A5, K5, b5 = f("A").reshape(B, NC, C, H, N), f("K").reshape(B, NC, C, H, D), f("beta").reshape(B, NC, C, H)
    got = go.correction_backward(f("corr_u"), A5, K5, b5, f("corr_states"), f("corr_out"), reference_order=True)
    for x, n in zip(got, ("corr_gA", "corr_gK", "corr_gbeta", "corr_gstates")):
        close(x, f(n), 2e-2, n)
    true = go.correction_backward(f("corr_u"), A5, K5, b5, f("corr_states"), f("corr_out"), reference_order=False)
    assert rel_err(true[2] * D, f("corr_gbeta")) > 5e-2          # the true derivative is a different vector
    # conv
    gx, gw, gb = go.conv_backward(f("conv_u"), f("conv_x"), f("conv_w").reshape(-1, 4), f("conv_b"))
    close(gx, f("conv_gx"), 2e-2, "conv grad_x")
    close(np.asarray(gw).reshape(-1), f("conv_gw").reshape(-1), 2e-2, "conv grad_weight")
    close(gb, f("conv_gb"), 2e-2, "conv grad_bias")
