"""ctypes front end of the C oracle (oracle/cdssm_oracle.c).

TEST INFRASTRUCTURE ONLY.  All arrays are float32 numpy arrays in the reference's
layouts (cdssm/ops.py docstrings): q,k (B,L,H,D); v, A_bar (B,L,H,N); gate_raw
(B,L,(N+5)H); per-token scalars (B,L,H); states (B,H,N,D).
"""
import ctypes
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None

__all__ = ["build", "lib", "bf16_round", "derive_constants", "dynamics", "normalize_kq",
           "intra_chunk", "inter_chunk", "exact_correction", "conv1d_silu", "scan_reference",
           "scan_recurrent", "make_inputs", "set_threads", "rope_freqs_default", "ROUND_NONE", "ROUND_INPUTS", "ROUND_STATE",
           "ROUND_CARRY", "ROUND_OUTPUTS", "ROUND_REFERENCE", "ROUND_FP32_STATE", "ROUND_KEEP_DECAY"]


def build(force=False):
    so = os.path.join(_HERE, "liborc.so")
    src = os.path.join(_HERE, "cdssm_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE, "-B", "liborc.so"])
    return so


def lib():
    global _LIB
    if _LIB is None:
        _LIB = ctypes.CDLL(build())
        _LIB.orc_bf16_round.restype = ctypes.c_float
        _LIB.orc_bf16_round.argtypes = [ctypes.c_float]
    return _LIB


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(ctypes.c_void_p)


def _cf(x):
    return ctypes.c_float(float(x))


# Which of the reference's bfloat16 stores the oracle emulates (bit mask, see cdssm_oracle.c).
ROUND_NONE, ROUND_INPUTS, ROUND_STATE, ROUND_CARRY, ROUND_OUTPUTS = 0, 1, 2, 4, 8
ROUND_REFERENCE = 15          # the reference as it runs
ROUND_FP32_STATE = 13         # bfloat16 inputs/outputs/carry, fp32 per-token state
ROUND_KEEP_DECAY = 16         # modifier: A_bar stays float32 (not a reference behaviour; see cdssm_oracle.c)


def _mask(round_bf16):
    if round_bf16 is True:
        return ROUND_REFERENCE
    if round_bf16 is False or round_bf16 is None:
        return 0
    return int(round_bf16)


def set_threads(n):
    """Ask for an OpenMP team of n threads; returns the team size the library really runs with."""
    fn = lib().orc_set_threads
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_int]
    return int(fn(int(n)))


def bf16_round(a):
    """Round-to-nearest-even float32 -> bfloat16 -> float32, vectorised."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    u = a.view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    r = ((u + 0x7FFF + lsb) & 0xFFFF0000).astype(np.uint32)
    out = r.view(np.float32).copy()
    nan = np.isnan(a)
    out[nan] = a[nan]
    return out.reshape(a.shape)


def derive_constants(context_length):
    """Constants the reference derives from its config (cdssm/config/model.py:59-67,98-109)."""
    eps = 2.0 ** -7
    thr = math.sqrt(eps)
    return dict(gating_c=math.log(context_length), omega_thresh=thr, adt_delta=16.0 * eps,
                adt_smoothness=thr / 5.0, adt_eps=1.0)


def rope_freqs_default(H, base):
    """cdssm/models/block.py:59-62."""
    return (1.0 / (float(base) ** (np.arange(H, dtype=np.float32) / np.float32(H)))).astype(np.float32)


def dynamics(gate_raw, log_dt_scale, rope_freqs, consts, H, N, pos0=0, round_bf16=False):
    g, gp = _f(gate_raw)
    B, L = g.shape[0], g.shape[1]
    assert g.shape[2] == (N + 5) * H
    ld, ldp = _f(log_dt_scale)
    rf, rfp = _f(rope_freqs)
    A = np.empty((B, L, H, N), np.float32)
    vp = np.empty((B, L, H, N // 2), np.float32)
    be = np.empty((B, L, H), np.float32)
    sc = np.empty((B, L, H), np.float32)
    lib().orc_dynamics(gp, ldp, rfp, _cf(consts["gating_c"]), _cf(consts["omega_thresh"]),
                       _cf(consts["adt_delta"]), _cf(consts["adt_smoothness"]), _cf(consts["adt_eps"]),
                       B, L, H, N, int(pos0), _mask(round_bf16),
                       A.ctypes.data_as(ctypes.c_void_p), vp.ctypes.data_as(ctypes.c_void_p),
                       be.ctypes.data_as(ctypes.c_void_p), sc.ctypes.data_as(ctypes.c_void_p))
    return A, vp, be, sc


def normalize_kq(K, Q, round_bf16=False):
    k, kp = _f(K)
    q, qp = _f(Q)
    D = k.shape[-1]
    ko = np.empty_like(k)
    qo = np.empty_like(q)
    lib().orc_normalize_kq(kp, qp, ctypes.c_size_t(k.size // D), D, _mask(round_bf16),
                           ko.ctypes.data_as(ctypes.c_void_p), qo.ctypes.data_as(ctypes.c_void_p))
    return ko, qo


def intra_chunk(A, K, V, beta, N, round_bf16=False):
    a, ap = _f(A)
    k, kp = _f(K)
    v, vp = _f(V)
    b, bp = _f(beta)
    BNC, C, H, D = k.shape
    lh = np.empty((BNC, C, H, N, D), np.float32)
    cA = np.empty((BNC, C, H, N), np.float32)
    lib().orc_intra_chunk(ap, kp, vp, bp, BNC, C, H, D, N, _mask(round_bf16),
                          lh.ctypes.data_as(ctypes.c_void_p), cA.ctypes.data_as(ctypes.c_void_p))
    return lh, cA


def inter_chunk(total_A, final_local_h, N, s0=None, round_bf16=False, return_final=False):
    a, ap = _f(total_A)
    f, fp = _f(final_local_h)
    B, NC, H, _, D = f.shape
    cs = np.empty_like(f)
    fin = np.empty((B, H, N, D), np.float32)
    s0p = None
    if s0 is not None:
        s0, s0p = _f(s0)
    lib().orc_inter_chunk(ap, fp, s0p, B, NC, H, D, N, _mask(round_bf16),
                          cs.ctypes.data_as(ctypes.c_void_p), fin.ctypes.data_as(ctypes.c_void_p))
    return (cs, fin) if return_final else cs


def exact_correction(A, K, beta, chunk_states, N, round_bf16=False):
    a, ap = _f(A)
    k, kp = _f(K)
    b, bp = _f(beta)
    c, cp = _f(chunk_states)
    B, NC, C, H, D = k.shape
    out = np.empty((B, NC, C, H, N, D), np.float32)
    lib().orc_exact_correction(ap, kp, bp, cp, B, NC, C, H, D, N, _mask(round_bf16),
                               out.ctypes.data_as(ctypes.c_void_p))
    return out


def conv1d_silu(x, weight, bias, round_bf16=False):
    xx, xp = _f(x)
    w, wp = _f(np.asarray(weight).reshape(-1, 4))
    b, bp = _f(bias)
    B, L, Dm = xx.shape
    out = np.empty_like(xx)
    lib().orc_conv1d_silu(xp, wp, bp, B, L, Dm, _mask(round_bf16), out.ctypes.data_as(ctypes.c_void_p))
    return out


def _scan_common(fn, q, k, v, gate_raw, log_dt_scale, rope_freqs, consts, N, extra):
    qq, qp = _f(q)
    kk, kp = _f(k)
    vv, vp = _f(v)
    gg, gp = _f(gate_raw)
    ld, ldp = _f(log_dt_scale)
    rf, rfp = _f(rope_freqs)
    return (qp, kp, vp, gp, ldp, rfp, _cf(consts["gating_c"]), _cf(consts["omega_thresh"]),
            _cf(consts["adt_delta"]), _cf(consts["adt_smoothness"]), _cf(consts["adt_eps"])), \
        (qq, kk, vv, gg, ld, rf)


def scan_reference(q, k, v, gate_raw, log_dt_scale, rope_freqs, consts, N, C, h0=None,
                   shortcut_scale=0.0, pos0=0, round_bf16=False):
    """The path as the reference block runs it (all intermediates materialised).
    Returns (y (B,L,H,N), final carry (B,H,N,D))."""
    args, keep = _scan_common(None, q, k, v, gate_raw, log_dt_scale, rope_freqs, consts, N, None)
    B, L, H, D = keep[0].shape
    y = np.empty((B, L, H, N), np.float32)
    fin = np.empty((B, H, N, D), np.float32)
    h0p = None
    if h0 is not None:
        h0, h0p = _f(h0)
    rc = lib().orc_scan_reference(*args, _cf(shortcut_scale), h0p, B, L, H, D, N, int(C), int(pos0),
                                  _mask(round_bf16), y.ctypes.data_as(ctypes.c_void_p),
                                  fin.ctypes.data_as(ctypes.c_void_p))
    if rc != 0:
        raise RuntimeError("orc_scan_reference failed")
    return y, fin


def scan_recurrent(q, k, v, gate_raw, log_dt_scale, rope_freqs, consts, N, state=None,
                   shortcut_scale=0.0, pos0=0, round_bf16=False):
    """Token-by-token recurrence (defines the decode step).  Returns (y, state_after)."""
    args, keep = _scan_common(None, q, k, v, gate_raw, log_dt_scale, rope_freqs, consts, N, None)
    B, L, H, D = keep[0].shape
    y = np.empty((B, L, H, N), np.float32)
    st = np.zeros((B, H, N, D), np.float32) if state is None else np.array(state, np.float32, copy=True)
    st = np.ascontiguousarray(st)
    rc = lib().orc_scan_recurrent(*args, _cf(shortcut_scale), st.ctypes.data_as(ctypes.c_void_p),
                                  B, L, H, D, N, int(pos0), _mask(round_bf16),
                                  y.ctypes.data_as(ctypes.c_void_p))
    if rc != 0:
        raise RuntimeError("orc_scan_recurrent failed")
    return y, st


def make_inputs(B, H, L, D, N=2, seed=0, bf16=False, rope=True, context_length=None):
    """Seeded synthetic inputs with the distributions the benchmark configs name: q,k ~ N(0,1)
    drawn as (B,H,L,D) and L2-normalised over D; v ~ N(0,1) (B,H,L,N); beta_raw, sel_B, sel_C,
    sel_dt, r_gate ~ N(0,1) (B,H,L); per head alpha_raw ~ N(-1,0.5), omega ~ U(-pi,pi),
    log_dt_scale ~ N(0,0.5).  Everything is permuted to the (B,L,H,.) operator layout and the
    per-head alpha/omega are broadcast into the per-token gate slots.  Returns a dict of float32
    arrays (rounded to bfloat16 values when bf16=True)."""
    rng = np.random.default_rng(seed)
    NH = N // 2
    q = rng.standard_normal((B, H, L, D), dtype=np.float32)
    k = rng.standard_normal((B, H, L, D), dtype=np.float32)
    q /= np.linalg.norm(q, axis=-1, keepdims=True)
    k /= np.linalg.norm(k, axis=-1, keepdims=True)
    v = rng.standard_normal((B, H, L, N), dtype=np.float32)
    beta_raw, sel_B, sel_C, sel_dt, r_gate = [rng.standard_normal((B, H, L), dtype=np.float32) for _ in range(5)]
    alpha_raw = (-1.0 + 0.5 * rng.standard_normal((NH, H))).astype(np.float32)
    omega = rng.uniform(-math.pi, math.pi, (NH, H)).astype(np.float32)
    log_dt_scale = (0.5 * rng.standard_normal(H)).astype(np.float32)
    tr = lambda x: np.ascontiguousarray(np.moveaxis(x, 1, 2))  # (B,H,L,...) -> (B,L,H,...)
    segs = [np.broadcast_to(alpha_raw[j][None, None, :], (B, L, H)) for j in range(NH)]
    segs += [np.broadcast_to(omega[j][None, None, :], (B, L, H)) for j in range(NH)]
    segs += [tr(sel_B), tr(sel_C), tr(sel_dt), tr(beta_raw), tr(r_gate)]
    gate_raw = np.ascontiguousarray(np.concatenate(segs, axis=-1), dtype=np.float32)
    ctx = context_length or L
    out = dict(q=tr(q), k=tr(k), v=tr(v), gate_raw=gate_raw, log_dt_scale=log_dt_scale,
               rope_freqs=rope_freqs_default(H, ctx) if rope else np.zeros(H, np.float32),
               consts=derive_constants(ctx))
    if bf16:
        for name in ("q", "k", "v", "gate_raw"):
            out[name] = bf16_round(out[name])
    return out
