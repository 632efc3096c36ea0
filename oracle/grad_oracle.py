"""Gradient oracle for the six operators (float64 numpy).

TEST INFRASTRUCTURE ONLY.  Forward and backward restatements, without any rounding, of dynamics_fused.cu:64-139 /
:187-386, normalize_kq.cu:118-160, intra_chunk_scan.cu:100-195 / :268-540, inter_chunk_scan.cu:52-84 / :115-190,
exact_correction.cu:83-150 / :230-375 (``reference_order=True``: what that kernel computes; False: the derivative of
its forward) and conv1d_silu.cu.
Pinned twice: tests/test_grad_oracle.py checks every backward function against central finite differences of its
forward function, and against tests/golden/bwd_ref.npz - the outputs of the reference's own backward kernels
(compiled unmodified for sm_100, run on a B200 by tests/golden/make_golden_ref.py).
"""
import numpy as np

EPS = 1e-6   # common.cuh:142


def _sig(x):
    return 1.0 / (1.0 + np.exp(-np.clip(x, -700.0, 700.0)))


def _sp(x):
    return np.where(x > 20.0, x, np.log1p(np.exp(np.minimum(x, 20.0))))


def _split(gate_raw, H, N):
    g = np.asarray(gate_raw, np.float64)
    B, L, _ = g.shape
    return g.reshape(B, L, N + 5, H)          # segment-major, head-minor (dynamics_fused.cu:60-81)


def _shared(g, lds, rf, c, N, pos0):
    """Per (b,l,h) quantities shared by the pairs.  Returns a dict of arrays (B,L,H)."""
    B, L, _, H = g.shape
    NH = N // 2
    pos = (np.arange(L, dtype=np.float64) + pos0)[None, :, None]
    rot = pos * np.asarray(rf, np.float64)[None, None, :]
    selB, selC, seldt, beta_raw, r_raw = (g[:, :, N + i] for i in range(5))
    a0_raw, w0 = g[:, :, 0], g[:, :, NH] + rot
    alpha0, w0a = _sp(a0_raw), np.abs(w0)
    s = _sp(np.asarray(lds, np.float64))[None, None, :]
    cf = alpha0 + w0a + c["adt_eps"]
    dt_raw = s / cf
    am = alpha0 + c["adt_eps"]
    dt_max = (2.0 - c["adt_delta"]) / am
    blend = _sig((c["omega_thresh"] - w0a) / c["adt_smoothness"])
    dt = blend * np.minimum(dt_raw, dt_max) + (1.0 - blend) * dt_raw + _sp(seldt)
    return dict(rot=rot, selB=selB, selC=selC, seldt=seldt, beta_raw=beta_raw, r_raw=r_raw, a0_raw=a0_raw, w0=w0,
                alpha0=alpha0, w0a=w0a, s=s, cf=cf, dt_raw=dt_raw, am=am, dt_max=dt_max, blend=blend, dt=dt,
                r=_sig(r_raw))


def dynamics_forward(gate_raw, log_dt_scale, rope_freqs, consts, H, N, pos0=0):
    """-> A_bar (B,L,H,N), vp_scale (B,L,H,N/2), beta (B,L,H), sel_C (B,L,H), float64."""
    g = _split(gate_raw, H, N)
    B, L = g.shape[:2]
    NH = N // 2
    sh = _shared(g, log_dt_scale, rope_freqs, consts, N, pos0)
    cr = consts["gating_c"] * sh["r"]
    A = np.empty((B, L, H, N))
    vp = np.empty((B, L, H, NH))
    for j in range(NH):
        alpha = np.maximum(_sp(g[:, :, j]), 0.0)
        omega = g[:, :, NH + j] + sh["rot"]
        tau = 0.5 * sh["dt"]
        ta, tw = tau * alpha, tau * omega
        den = (1 + ta) ** 2 + tw ** 2 + EPS
        mu_re = ((1 - ta) * (1 + ta) - tw ** 2) / den
        mu_im = (tw * (1 + ta) + (1 - ta) * tw) / den
        e = np.maximum(((1 - ta) ** 2 + tw ** 2) / den, 1e-8)
        scale = e ** ((cr - 1.0) / 2.0)
        A[..., 2 * j], A[..., 2 * j + 1] = mu_re * scale, -mu_im * scale
        vp[..., j] = np.minimum(np.sqrt(np.maximum(1.0 - e ** cr, EPS)), 1.0)
    return A, vp, _sig(sh["beta_raw"]) * _sig(sh["selB"]), _sig(sh["selC"])


def dynamics_backward(gA, gvp, gbeta, gselc, gate_raw, log_dt_scale, rope_freqs, consts, H, N, pos0=0):
    """-> grad_gate_raw (B,L,(N+5)H), grad_log_dt_scale (H), float64."""
    g = _split(gate_raw, H, N)
    B, L = g.shape[:2]
    NH = N // 2
    c = consts
    sh = _shared(g, log_dt_scale, rope_freqs, c, N, pos0)
    gA, gvp = np.asarray(gA, np.float64), np.asarray(gvp, np.float64)
    gbeta, gselc = np.asarray(gbeta, np.float64), np.asarray(gselc, np.float64)
    out = np.zeros_like(g)
    r, dt = sh["r"], sh["dt"]
    cr = c["gating_c"] * r
    expo = (cr - 1.0) / 2.0
    g_dt = np.zeros((B, L, H))
    g_r = np.zeros((B, L, H))
    for j in range(NH):
        a_raw = g[:, :, j]
        alpha = np.maximum(_sp(a_raw), 0.0)
        omega = g[:, :, NH + j] + sh["rot"]
        tau = 0.5 * dt
        ta, tw = tau * alpha, tau * omega
        opa, oma = 1 + ta, 1 - ta
        det = opa ** 2 + tw ** 2 + EPS
        num_re = oma * opa - tw ** 2
        mu_re, mu_im = num_re / det, 2 * tw / det
        e_raw = (oma ** 2 + tw ** 2) / det
        e = np.maximum(e_raw, 1e-8)
        free = e_raw > 1e-8
        scale, eff = e ** expo, e ** cr
        vp2 = 1.0 - eff
        # variance-preserving scale (dynamics_fused.cu:258-262)
        d_eff = np.where((vp2 > EPS) & (vp2 < 1.0), gvp[..., j] * (-0.5 / np.sqrt(np.maximum(vp2, EPS))), 0.0)
        # recurrence gate exponent (:264-282)
        d_scale = gA[..., 2 * j] * mu_re + gA[..., 2 * j + 1] * (-mu_im)
        d_e = np.where(free, d_eff * cr * e ** (cr - 1.0) + d_scale * expo * e ** (expo - 1.0), 0.0)
        g_r += d_eff * c["gating_c"] * np.log(e) * eff + d_scale * (c["gating_c"] / 2.0) * np.log(e) * scale
        # Cayley map (:288-340): e = num / det, mu = (num_re, 2 tw) / det, stored conjugated
        gm_re, gm_im = gA[..., 2 * j] * scale, -gA[..., 2 * j + 1] * scale
        d_ta = d_e * (-2 * oma) / det - d_e * e_raw * 2 * opa / det
        d_tw = d_e * 2 * tw / det - d_e * e_raw * 2 * tw / det
        d_ta += gm_re * (-2 * ta * det - num_re * 2 * opa) / det ** 2 + gm_im * (-2 * tw * 2 * opa) / det ** 2
        d_tw += gm_re * (-2 * tw * det - num_re * 2 * tw) / det ** 2 + gm_im * (2 * det - 4 * tw * tw) / det ** 2
        out[:, :, j] += d_ta * tau * _sig(a_raw)
        out[:, :, NH + j] += d_tw * tau
        g_dt += 0.5 * (d_ta * alpha + d_tw * omega)
    # adaptive time step (:348-372)
    capped = sh["dt_raw"] > sh["dt_max"]
    blend = sh["blend"]
    g_raw = g_dt * np.where(capped, 1.0 - blend, 1.0)
    g_max = g_dt * np.where(capped, blend, 0.0)
    g_blend = g_dt * (np.minimum(sh["dt_raw"], sh["dt_max"]) - sh["dt_raw"])
    g_s = g_raw / sh["cf"]
    g_cf = -g_raw * sh["s"] / sh["cf"] ** 2
    g_w0a = g_cf - g_blend * blend * (1 - blend) / c["adt_smoothness"]
    g_alpha0 = g_cf - g_max * (2.0 - c["adt_delta"]) / sh["am"] ** 2
    out[:, :, 0] += g_alpha0 * _sig(sh["a0_raw"])
    out[:, :, NH] += g_w0a * np.where(sh["w0"] >= 0, 1.0, -1.0)
    # gates (:208-217, :374-383)
    sb, sbe, sc = _sig(sh["selB"]), _sig(sh["beta_raw"]), _sig(sh["selC"])
    out[:, :, N] = gbeta * sbe * sb * (1 - sb)
    out[:, :, N + 1] = gselc * sc * (1 - sc)
    out[:, :, N + 2] = g_dt * _sig(sh["seldt"])
    out[:, :, N + 3] = gbeta * sb * sbe * (1 - sbe)
    out[:, :, N + 4] = g_r * r * (1 - r)
    glds = (g_s * _sig(np.asarray(log_dt_scale, np.float64))[None, None, :]).sum((0, 1))
    return out.reshape(B, L, (N + 5) * H), glds


def normalize_forward(x):
    x = np.asarray(x, np.float64)
    return x / np.sqrt((x ** 2).sum(-1, keepdims=True) + EPS)


def normalize_backward(g_out, x):
    """normalize_kq.cu:118-160: grad_in = (g - x_hat (g . x_hat)) * inv_norm."""
    x, g_out = np.asarray(x, np.float64), np.asarray(g_out, np.float64)
    inv = 1.0 / np.sqrt((x ** 2).sum(-1, keepdims=True) + EPS)
    xh = x * inv
    return (g_out - xh * (g_out * xh).sum(-1, keepdims=True)) * inv


# ---------------------------------------------------------------------------------------------
# The scan-side operators and the conv.  State rows come in complex pairs (rows 2j, 2j+1 = re, im); the stored
# A_bar pair multiplies the state pair as a complex number (intra_chunk_scan.cu:140-152).
def _cplx(x, axis):
    """Pairs (2j, 2j+1) along `axis` -> complex, that axis halved."""
    x = np.moveaxis(np.asarray(x, np.float64), axis, -1)
    return np.moveaxis(x[..., 0::2] + 1j * x[..., 1::2], -1, axis)


def _pairs(z, axis):
    z = np.moveaxis(z, axis, -1)
    out = np.empty(z.shape[:-1] + (2 * z.shape[-1],))
    out[..., 0::2], out[..., 1::2] = z.real, z.imag
    return np.moveaxis(out, -1, axis)


def intra_forward(A, K, V, beta):
    """intra_chunk_scan.cu:100-195.  A (M,C,H,N), K (M,C,H,D), V (M,C,H,N), beta (M,C,H) ->
    local_h (M,C,H,N,D), cum_A (M,C,H,N)."""
    a, v = _cplx(A, -1), _cplx(V, -1)                        # (M,C,H,P)
    K, beta = np.asarray(K, np.float64), np.asarray(beta, np.float64)
    M, C, H, P = a.shape
    D = K.shape[-1]
    z = np.zeros((M, H, P, D), complex)
    ca = np.ones((M, H, P), complex)
    lh = np.empty((M, C, H, P, D), complex)
    cA = np.empty((M, C, H, P), complex)
    for t in range(C):
        k, b = K[:, t][:, :, None, :], beta[:, t][:, :, None, None]
        u = (z * k).sum(-1, keepdims=True)
        z = a[:, t][..., None] * (z - b * u * k) + b * v[:, t][..., None] * k
        ca = a[:, t] * ca
        lh[:, t], cA[:, t] = z, ca
    return _pairs(lh, 3), _pairs(cA, 3)


def intra_backward(g_lh, g_cA, A, K, V, beta, local_h, cum_A):
    """Reverse walk with the SAVED forward outputs as the previous state / previous decay product
    (intra_chunk_scan.cu:268-540).  -> grad_A, grad_K, grad_V, grad_beta."""
    a, v = _cplx(A, -1), _cplx(V, -1)
    K, beta = np.asarray(K, np.float64), np.asarray(beta, np.float64)
    lh, cA = _cplx(local_h, 3), _cplx(cum_A, 3)
    glh, gcA = _cplx(g_lh, 3), _cplx(g_cA, 3)
    M, C, H, P = a.shape
    Gz = np.zeros_like(lh[:, 0])
    Gc = np.zeros_like(cA[:, 0])
    gA = np.empty_like(a)
    gV = np.empty_like(v)
    gK = np.zeros_like(K)
    gB = np.zeros_like(beta)
    for t in range(C - 1, -1, -1):
        Gz = Gz + glh[:, t]
        Gc = Gc + gcA[:, t]
        zp = lh[:, t - 1] if t > 0 else np.zeros_like(Gz)
        cp = cA[:, t - 1] if t > 0 else np.ones_like(Gc)
        k, b = K[:, t][:, :, None, :], beta[:, t][:, :, None, None]
        at, vt = a[:, t][..., None], v[:, t][..., None]
        u = (zp * k).sum(-1, keepdims=True)
        e = zp - b * u * k
        gA[:, t] = (Gz * np.conj(e)).sum(-1) + Gc * np.conj(cp)
        Ge = np.conj(at) * Gz
        s = (Gz * k).sum(-1, keepdims=True)
        gV[:, t] = (b * s)[..., 0]
        w = (Ge * k).sum(-1, keepdims=True)
        gB[:, t] = ((s * np.conj(vt)).real - (w * np.conj(u)).real).sum((2, 3))
        Gu = -b * w
        gK[:, t] = (b * (Gz * np.conj(vt)).real - b * (Ge * np.conj(u)).real + (Gu * np.conj(zp)).real).sum(2)
        Gz = Ge + Gu * k
        Gc = np.conj(a[:, t]) * Gc
    return _pairs(gA, -1), gK, _pairs(gV, -1), gB


def inter_forward(total_A, final_h):
    """inter_chunk_scan.cu:52-84.  total_A (B,NC,H,N), final_h (B,NC,H,N,D) -> chunk_states (B,NC,H,N,D)."""
    a, h = _cplx(total_A, -1), _cplx(final_h, 3)
    s = np.zeros_like(h[:, 0])
    out = np.empty_like(h)
    for c in range(a.shape[1]):
        out[:, c] = s
        s = a[:, c][..., None] * s + h[:, c]
    return _pairs(out, 3)


def inter_backward(g_states, total_A, chunk_states):
    """inter_chunk_scan.cu:115-190 (the saved chunk_states are the forward's s_c).  -> grad_total_A, grad_final_h."""
    a, s, g = _cplx(total_A, -1), _cplx(chunk_states, 3), _cplx(g_states, 3)
    G = np.zeros_like(s[:, 0])
    gA, gH = np.empty_like(a), np.empty_like(s)
    for c in range(a.shape[1] - 1, -1, -1):
        gH[:, c] = G
        gA[:, c] = (G * np.conj(s[:, c])).sum(-1)
        G = np.conj(a[:, c])[..., None] * G + g[:, c]
    return _pairs(gA, -1), _pairs(gH, 3)


def correction_forward(A, K, beta, states):
    """exact_correction.cu:83-150.  A (B,NC,C,H,N), K (B,NC,C,H,D), beta (B,NC,C,H), states (B,NC,H,N,D) ->
    corrections (B,NC,C,H,N,D): the state BEFORE each step."""
    a = _cplx(A, -1)
    K, beta = np.asarray(K, np.float64), np.asarray(beta, np.float64)
    r = _cplx(states, 3)
    C = a.shape[2]
    out = np.empty(a.shape[:2] + (C,) + r.shape[2:], complex)
    for t in range(C):
        out[:, :, t] = r
        k, b = K[:, :, t][:, :, :, None, :], beta[:, :, t][:, :, :, None, None]
        u = (r * k).sum(-1, keepdims=True)
        r = a[:, :, t][..., None] * (r - b * u * k)
    return _pairs(out, 4)


def correction_backward(g_corr, A, K, beta, states, corrections, reference_order=False):
    """exact_correction.cu:230-375, with the saved corrections as the state before each step.
    -> grad_A, grad_K, grad_beta, grad_states.  reference_order=True adds the upstream gradient of corrections[t]
    BEFORE step t is walked back, as the reference kernel does (exact_correction.cu:219-223): that is not the
    derivative of the forward (which stores corrections[t] before the step), but it is what the reference computes."""
    a = _cplx(A, -1)
    K, beta = np.asarray(K, np.float64), np.asarray(beta, np.float64)
    rs, g = _cplx(corrections, 4), _cplx(g_corr, 4)
    C = a.shape[2]
    Gr = np.zeros_like(rs[:, :, 0])
    gA = np.empty_like(a)
    gK = np.zeros_like(K)
    gB = np.zeros_like(beta)
    for t in range(C - 1, -1, -1):
        r = rs[:, :, t]
        if reference_order:
            Gr = Gr + g[:, :, t]
        k, b = K[:, :, t][:, :, :, None, :], beta[:, :, t][:, :, :, None, None]
        at = a[:, :, t][..., None]
        u = (r * k).sum(-1, keepdims=True)
        e = r - b * u * k
        gA[:, :, t] = (Gr * np.conj(e)).sum(-1)
        Ge = np.conj(at) * Gr
        w = (Ge * k).sum(-1, keepdims=True)
        gB[:, :, t] = -(w * np.conj(u)).real.sum((3, 4))
        if reference_order:      # the reference reduces an already reduced value over its D threads again (:347-359)
            gB[:, :, t] *= K.shape[-1]
        Gu = -b * w
        gK[:, :, t] = (-b * (Ge * np.conj(u)).real + (Gu * np.conj(r)).real).sum(3)
        Gr = Ge + Gu * k
        if not reference_order:
            Gr = Gr + g[:, :, t]
    return _pairs(gA, -1), gK, gB, _pairs(Gr, 3)


def _silu(p):
    return p * _sig(p)


def conv_forward(x, w, bias):
    """conv1d_silu.cu:25-90.  x (B,L,Dm), w (Dm,4), bias (Dm): causal 4-tap depthwise conv + SiLU."""
    x, w, bias = (np.asarray(t, np.float64) for t in (x, w, bias))
    B, L, Dm = x.shape
    xp = np.concatenate([np.zeros((B, 3, Dm)), x], 1)
    pre = bias + sum(w[:, j] * xp[:, j:j + L] for j in range(4))
    return _silu(pre)


def conv_backward(g_out, x, w, bias):
    """conv1d_silu.cu:94-219.  -> grad_x, grad_w (Dm,4), grad_bias."""
    x, w, bias, g_out = (np.asarray(t, np.float64) for t in (x, w, bias, g_out))
    B, L, Dm = x.shape
    xp = np.concatenate([np.zeros((B, 3, Dm)), x], 1)
    pre = bias + sum(w[:, j] * xp[:, j:j + L] for j in range(4))
    sg = _sig(pre)
    gp = g_out * sg * (1 + pre * (1 - sg))
    gpp = np.concatenate([gp, np.zeros((B, 3, Dm))], 1)
    gx = sum(w[:, j] * gpp[:, 3 - j:3 - j + L] for j in range(4))
    gw = np.stack([(gp * xp[:, j:j + L]).sum((0, 1)) for j in range(4)], -1)
    return gx, gw, gp.sum((0, 1))
