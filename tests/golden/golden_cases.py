"""Golden vectors from the reference's own CUDA kernels.

The reference has no tests or fixtures of its own and no CPU path, so the pin is made here:
``make_golden_ref.py`` runs the reference kernels (compiled unmodified for sm_100 by
oracle/build_ref.py) on a B200 over the cases below and stores what every stage produced;
``check_oracle_against_golden`` replays the CPU oracle stage by stage on the recorded stage
inputs and end to end on the raw inputs.

bfloat16 tensors are stored as their uint16 bit patterns.
"""
import numpy as np

# name -> sizes.  D = 64 cases use the reference's normalize_kq kernel; it is only correct for
# D = 64 (normalize_kq.cu:55-72 sizes its reduction for two warps), so the D = 128 case
# normalises with torch and records that.
CASES = {
    "d64_pad": dict(B=1, H=2, L=160, D=64, N=2, C=64, seed=11, shortcut=0.0),
    "d64_n4_shortcut": dict(B=2, H=2, L=128, D=64, N=4, C=64, seed=12, shortcut=0.5),
    "d128": dict(B=1, H=2, L=256, D=128, N=2, C=128, seed=13, shortcut=0.0),
}


def bits(t):
    """torch bf16 tensor -> uint16 numpy."""
    import torch
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def unbits(a):
    """uint16 bf16 bit patterns -> float32 numpy."""
    return (a.astype(np.uint32) << 16).view(np.float32)


def run_reference(ref, case, orc):
    """Run the reference pipeline (cdssm/models/block.py:181-211 over cdssm/models/ssd.py:56-111)
    by calling the reference extension's forward functions directly.  Returns a dict of numpy
    arrays (inputs and every stage output)."""
    import torch
    import torch.nn.functional as F
    B, H, L, D, N, C = (case[k] for k in "BHLDNC")
    inp = orc.make_inputs(B, H, L, D, N=N, seed=case["seed"], bf16=True)
    dev = "cuda"
    bf = lambda a: torch.from_numpy(a).to(dev).bfloat16()
    q, k, v, g = bf(inp["q"]), bf(inp["k"]), bf(inp["v"]), bf(inp["gate_raw"])
    # un-normalise q/k rows so that the normalisation is exercised
    scale = torch.linspace(0.5, 3.0, L, device=dev).view(1, L, 1, 1).bfloat16()
    q, k = (q * scale).contiguous(), (k * scale.flip(1)).contiguous()
    lds = torch.from_numpy(inp["log_dt_scale"]).to(dev)
    rf = torch.from_numpy(inp["rope_freqs"]).to(dev)
    c = inp["consts"]
    A, vp, beta, selc = ref.dynamics_fused_fwd_cuda(g, lds, rf, c["gating_c"], c["omega_thresh"],
                                                    c["adt_delta"], c["adt_smoothness"], c["adt_eps"], H, N)
    if D == 64:
        kn, qn = ref.normalize_kq_fwd_cuda(k, q)
    else:
        nrm = lambda x: (x.float() * torch.rsqrt((x.float() ** 2).sum(-1, keepdim=True) + 1e-6)).bfloat16()
        kn, qn = nrm(k), nrm(q)
    vg = v * vp.repeat_interleave(2, dim=-1)
    NC = -(-L // C)
    pad = NC * C - L
    Ap, Kp, Vp, bp = A, kn, vg, beta
    if pad:
        Ap = F.pad(A, (0, 0, 0, 0, 0, pad))
        Kp = F.pad(kn, (0, 0, 0, 0, 0, pad))
        Vp = F.pad(vg, (0, 0, 0, 0, 0, pad))
        bp = F.pad(beta, (0, 0, 0, pad))
    local_h, cum_A = ref.intra_chunk_scan_fwd_cuda(Ap.reshape(B * NC, C, H, N).contiguous(),
                                                   Kp.reshape(B * NC, C, H, D).contiguous(),
                                                   Vp.reshape(B * NC, C, H, N).contiguous(),
                                                   bp.reshape(B * NC, C, H).contiguous(), N)
    local_h = local_h.view(B, NC, C, H, N, D)
    cum_A = cum_A.view(B, NC, C, H, N)
    chunk_states = ref.inter_chunk_scan_fwd_cuda(cum_A[:, :, -1], local_h[:, :, -1], N)
    corr = ref.exact_correction_fwd_cuda(Ap.view(B, NC, C, H, N), Kp.view(B, NC, C, H, D),
                                         bp.view(B, NC, C, H), chunk_states, N)
    Y = (local_h + corr).reshape(B, -1, H, N, D)[:, :L]
    qk = torch.einsum("blhd,blhd->blh", qn, kn)
    shortcut = qk[..., None, None] * vg.unsqueeze(-1) * kn.unsqueeze(-2)
    Y = Y + torch.tensor([case["shortcut"]], device=dev).bfloat16() * shortcut
    y = torch.einsum("blhsd,blhd->blhs", Y, qn) * selc.unsqueeze(-1)
    torch.cuda.synchronize()
    out = dict(q=bits(q), k=bits(k), v=bits(v), gate_raw=bits(g), log_dt_scale=inp["log_dt_scale"],
               rope_freqs=inp["rope_freqs"], consts=np.array([c["gating_c"], c["omega_thresh"], c["adt_delta"],
                                                              c["adt_smoothness"], c["adt_eps"]], np.float64),
               sizes=np.array([B, H, L, D, N, C], np.int64), shortcut=np.array(case["shortcut"]),
               A_bar=bits(A), vp=bits(vp), beta=bits(beta), sel_C=bits(selc), k_norm=bits(kn), q_norm=bits(qn),
               cum_A=bits(cum_A), chunk_states=bits(chunk_states), y=bits(y),
               local_h_last=bits(local_h[:, :, -1]), corr_last=bits(corr[:, :, -1]))
    if B * NC * C * H * N * D <= 120000:
        out["local_h"] = bits(local_h)
        out["corrections"] = bits(corr)
    return out


def run_reference_backward(ref, orc):
    """One small case through the reference's BACKWARD kernels (called directly, each fed with the reference's own
    forward outputs as the saved tensors and a seeded random upstream gradient).  Returns a dict of numpy arrays:
    inputs, saved forward outputs, upstream gradients, and the reference's gradients, per operator."""
    import torch
    B, NC, C, H, N, D = 1, 2, 64, 2, 2, 64
    g = torch.Generator(device="cuda").manual_seed(31)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")
    out = {"sizes": np.array([B, NC, C, H, N, D], np.int64)}
    put = lambda name, t: out.__setitem__(name, bits(t) if t.dtype == torch.bfloat16 else t.detach().float().cpu().numpy())
    # dynamics
    L = 40
    inp = orc.make_inputs(B, H, L, D, N=N, seed=32, bf16=True, context_length=256)
    gate = torch.from_numpy(inp["gate_raw"]).cuda().bfloat16()
    lds, rf = torch.from_numpy(inp["log_dt_scale"]).cuda(), torch.from_numpy(inp["rope_freqs"]).cuda()
    c = inp["consts"]
    cs_ = (c["gating_c"], c["omega_thresh"], c["adt_delta"], c["adt_smoothness"], c["adt_eps"])
    ups = [rn(B, L, H, N).bfloat16(), rn(B, L, H, N // 2).bfloat16(), rn(B, L, H).bfloat16(), rn(B, L, H).bfloat16()]
    gg, gl = ref.dynamics_fused_bwd_cuda(*ups, gate, lds, rf, *cs_, H, N)
    out["dyn_consts"] = np.array(cs_, np.float64)
    for n, t in zip(("dyn_gate", "dyn_lds", "dyn_rope", "dyn_uA", "dyn_uvp", "dyn_ubeta", "dyn_uselc", "dyn_ggate", "dyn_glds"),
                    (gate, lds, rf, *ups, gg, gl)):
        put(n, t)
    # normalisation (head_dim 64: the only size the reference kernel is right for)
    Kq, Qq, gK, gQ = (rn(3, 7, H, D).bfloat16() for _ in range(4))
    wK, wQ = ref.normalize_kq_bwd_cuda(gK, gQ, Kq, Qq)
    for n, t in zip(("nrm_K", "nrm_Q", "nrm_uK", "nrm_uQ", "nrm_gK", "nrm_gQ"), (Kq, Qq, gK, gQ, wK, wQ)):
        put(n, t)
    # intra-chunk scan
    A = (rn(B * NC, C, H, N) * 0.4).bfloat16()
    K = (rn(B * NC, C, H, D) / 8).bfloat16()
    V, be = rn(B * NC, C, H, N).bfloat16(), torch.rand(B * NC, C, H, generator=g, device="cuda").bfloat16()
    lh, cA = ref.intra_chunk_scan_fwd_cuda(A, K, V, be, N)
    u1, u2 = rn(*lh.shape).bfloat16(), rn(*cA.shape).bfloat16()
    gi = ref.intra_chunk_scan_bwd_cuda(u1, u2, A, K, V, be, lh, cA, N)
    for n, t in zip(("A", "K", "V", "beta", "local_h", "cum_A", "intra_ulh", "intra_ucA", "intra_gA", "intra_gK",
                     "intra_gV", "intra_gbeta"), (A, K, V, be, lh, cA, u1, u2, *gi)):
        put(n, t)
    # inter-chunk carry
    tot, fin = (rn(B, NC + 2, H, N) * 0.4).bfloat16(), rn(B, NC + 2, H, N, D).bfloat16()
    cs = ref.inter_chunk_scan_fwd_cuda(tot, fin, N)
    up = rn(*cs.shape).bfloat16()
    wA, wH = ref.inter_chunk_scan_bwd_cuda(up, tot, cs, N)
    for n, t in zip(("inter_tot", "inter_fin", "inter_states", "inter_u", "inter_gA", "inter_gH"), (tot, fin, cs, up, wA, wH)):
        put(n, t)
    # correction
    A5, K5, b5 = A.view(B, NC, C, H, N), K.view(B, NC, C, H, D), be.view(B, NC, C, H)
    st = rn(B, NC, H, N, D).bfloat16()
    corr = ref.exact_correction_fwd_cuda(A5, K5, b5, st, N)
    upc = rn(*corr.shape).bfloat16()
    gc = ref.exact_correction_bwd_cuda(upc, A5, K5, b5, st, corr, N)
    for n, t in zip(("corr_states", "corr_out", "corr_u", "corr_gA", "corr_gK", "corr_gbeta", "corr_gstates"),
                    (st, corr, upc, *gc)):
        put(n, t)
    # conv
    x, w4 = rn(2, 37, 64).bfloat16(), (rn(64, 1, 4) / 2).bfloat16()
    bias, upx = (rn(64) / 5).bfloat16(), rn(2, 37, 64).bfloat16()
    gx = ref.conv1d_silu_bwd_cuda(x, w4, bias, upx)
    for n, t in zip(("conv_x", "conv_w", "conv_b", "conv_u", "conv_gx", "conv_gw", "conv_gb"), (x, w4, bias, upx, *gx)):
        put(n, t)
    torch.cuda.synchronize()
    return out


def _consts(g):
    c = g["consts"]
    return dict(gating_c=float(c[0]), omega_thresh=float(c[1]), adt_delta=float(c[2]),
                adt_smoothness=float(c[3]), adt_eps=float(c[4]))


def _ulp_close(x, ref, frac_exact, what):
    """bf16 results computed with different exp/log implementations: almost all bit-identical,
    the rest one bf16 ulp apart."""
    x, ref = np.asarray(x, np.float32), np.asarray(ref, np.float32)
    exact = np.mean(x == ref)
    err = np.abs(x - ref) / np.maximum(np.abs(ref), 1e-30)
    assert exact >= frac_exact, f"{what}: only {exact:.4f} bit-identical"
    assert err.max() <= 2.0 ** -7 + 1e-6, f"{what}: {err.max()} exceeds one bf16 ulp"


def check_oracle_against_golden(orc, g):
    B, H, L, D, N, C = (int(x) for x in g["sizes"])
    c = _consts(g)
    q, k, v, gate = (unbits(g[n]) for n in ("q", "k", "v", "gate_raw"))
    lds, rf = g["log_dt_scale"], g["rope_freqs"]
    R = orc.ROUND_REFERENCE
    # stage 1: dynamics
    A, vp, beta, selc = orc.dynamics(gate, lds, rf, c, H, N, round_bf16=R)
    _ulp_close(A, unbits(g["A_bar"]), 0.97, "A_bar")
    _ulp_close(vp, unbits(g["vp"]), 0.97, "vp_scale")
    _ulp_close(beta, unbits(g["beta"]), 0.97, "beta")
    _ulp_close(selc, unbits(g["sel_C"]), 0.97, "sel_C")
    # stage 2: normalisation
    kn, qn = orc.normalize_kq(k, q, round_bf16=R)
    _ulp_close(kn, unbits(g["k_norm"]), 0.99, "k_norm")
    _ulp_close(qn, unbits(g["q_norm"]), 0.99, "q_norm")
    # stage 3..5 on the recorded stage inputs
    gA, gvp, gbeta = unbits(g["A_bar"]), unbits(g["vp"]), unbits(g["beta"])
    gkn = unbits(g["k_norm"])
    vg = orc.bf16_round(v * np.repeat(gvp, 2, -1))
    NC = -(-L // C)
    pad = NC * C - L
    padl = lambda x: np.pad(x, [(0, 0), (0, pad)] + [(0, 0)] * (x.ndim - 2))
    Ap, Kp, Vp, bp = padl(gA), padl(gkn), padl(vg), padl(gbeta)
    lh, cA = orc.intra_chunk(Ap.reshape(B * NC, C, H, N), Kp.reshape(B * NC, C, H, D),
                             Vp.reshape(B * NC, C, H, N), bp.reshape(B * NC, C, H), N, round_bf16=R)
    lh = lh.reshape(B, NC, C, H, N, D)
    cA = cA.reshape(B, NC, C, H, N)
    tol = 2.0 ** -7
    from util import rel_err
    assert rel_err(cA, unbits(g["cum_A"])) <= tol
    assert rel_err(lh[:, :, -1], unbits(g["local_h_last"])) <= tol
    if "local_h" in g:
        assert rel_err(lh, unbits(g["local_h"])) <= tol
    cs = orc.inter_chunk(unbits(g["cum_A"])[:, :, -1], unbits(g["local_h_last"]), N, round_bf16=R)
    assert rel_err(cs, unbits(g["chunk_states"])) <= tol
    co = orc.exact_correction(Ap.reshape(B, NC, C, H, N), Kp.reshape(B, NC, C, H, D),
                              bp.reshape(B, NC, C, H), unbits(g["chunk_states"]), N, round_bf16=R)
    assert rel_err(co[:, :, -1], unbits(g["corr_last"])) <= tol
    if "corrections" in g:
        assert rel_err(co, unbits(g["corrections"])) <= tol
    # end to end from the raw inputs
    y, _ = orc.scan_reference(q, k, v, gate, lds, rf, c, N, C, shortcut_scale=float(g["shortcut"]), round_bf16=R)
    assert rel_err(y, unbits(g["y"])) <= 2e-2
