"""The gradient oracle (oracle/grad_oracle.py) against central finite differences of its own float64 forward, and
its forward against the C oracle of the reference's dynamics kernel (CPU only)."""
import numpy as np
import pytest

from oracle import grad_oracle as go


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
