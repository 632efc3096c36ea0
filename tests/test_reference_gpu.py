"""Our kernels against the reference's OWN kernels (compiled unmodified for sm_100 into
oracle/_ref/ by oracle/build_ref.py), on the same bf16 inputs, on the GPU."""
import os
import sys

import numpy as np
import pytest
import torch

from util import BF16_TOL, const_args, rel_err, to_np

pytestmark = pytest.mark.gpu
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def ref():
    from oracle.build_ref import load_ref
    mod = load_ref()
    if mod is None:
        pytest.skip("reference extension not built (oracle/build_ref.py)")
    return mod


def _t(a):
    from golden.golden_cases import unbits
    return torch.from_numpy(unbits(a)).cuda().bfloat16()


@pytest.mark.parametrize("case", ["d64_pad", "d64_n4_shortcut", "d128"])
def test_against_reference_kernels(ops, orc, ref, case):
    from golden.golden_cases import CASES, run_reference, unbits
    c = CASES[case]
    g = run_reference(ref, c, orc)
    B, H, L, D, N, C = (int(x) for x in g["sizes"])
    consts = tuple(float(x) for x in g["consts"])
    lds, rf = torch.from_numpy(g["log_dt_scale"]).cuda(), torch.from_numpy(g["rope_freqs"]).cuda()
    q, k, v, gate = _t(g["q"]), _t(g["k"]), _t(g["v"]), _t(g["gate_raw"])
    # operator level: same inputs, same rounding points -> bf16-ulp agreement
    A, vp, beta, selc = ops.DynamicsFusedFn.apply(gate, lds, rf, *consts, H, N)
    for got, name in ((A, "A_bar"), (vp, "vp"), (beta, "beta"), (selc, "sel_C")):
        want = unbits(g[name])
        assert np.mean(to_np(got) == want) > 0.99, name
        assert rel_err(to_np(got), want) <= 2.0 ** -7, name
    kn, qn = ops.NormalizeKQFn.apply(k, q)
    assert rel_err(to_np(kn), unbits(g["k_norm"])) <= 2.0 ** -7
    assert rel_err(to_np(qn), unbits(g["q_norm"])) <= 2.0 ** -7
    cs = ops.InterChunkScanFn.apply(_t(g["cum_A"])[:, :, -1], _t(g["local_h_last"]), N)
    assert rel_err(to_np(cs), unbits(g["chunk_states"])) <= 2.0 ** -7
    # the fused path against the reference pipeline's final output
    y, _ = ops.scan_fused(q, k, v, gate, lds, rf, *consts, H, N, C, shortcut_scale=float(g["shortcut"]))
    assert rel_err(to_np(y), unbits(g["y"])) <= BF16_TOL


@pytest.mark.parametrize("B,H,L,D", [(2, 4, 512, 64), (1, 8, 300, 64), (1, 32, 1024, 128), (2, 4, 700, 128)])
def test_tensor_core_passes_against_reference_kernels(ops, orc, ref, B, H, L, D):
    """Shapes that take the tcgen05 passes (H a multiple of 4, head_dim 64 and 128), against the live
    reference pipeline on the same un-normalised bf16 inputs."""
    from oracle.ref_pipeline import reference_forward
    N, C = 2, D
    inp = orc.make_inputs(B, H, L, D, N=N, seed=100 + L + D, bf16=True)
    bf = lambda a: torch.from_numpy(a).cuda().bfloat16()
    q, k, v, gate = bf(inp["q"]), bf(inp["k"]), bf(inp["v"]), bf(inp["gate_raw"])
    scale = torch.linspace(0.5, 3.0, L, device="cuda").view(1, L, 1, 1).bfloat16()
    q, k = (q * scale).contiguous(), (k * scale.flip(1)).contiguous()
    lds, rf = torch.from_numpy(inp["log_dt_scale"]).cuda(), torch.from_numpy(inp["rope_freqs"]).cuda()
    consts = const_args(inp["consts"])
    want = reference_forward(ref, q, k, v, gate, lds, rf, consts, H, N, C, shortcut=0.5)
    y, _ = ops.scan_fused(q, k, v, gate, lds, rf, *consts, H, N, C, shortcut_scale=0.5, flags=ops.TENSOR_CORE_WA)
    assert ops.scan_fused_status() == 0
    assert rel_err(to_np(y), to_np(want)) <= BF16_TOL


def test_backward_kernels_against_reference_backward_kernels(ops, orc, ref):
    """dynamics and normalisation backward against the reference's own backward kernels on the same bf16 data."""
    B, H, L, N, D = 2, 4, 96, 2, 64
    inp = orc.make_inputs(B, H, L, D, N=N, seed=7, bf16=True, context_length=256)
    bf = lambda a: torch.from_numpy(a).cuda().bfloat16()
    g = torch.Generator(device="cuda").manual_seed(1)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda").bfloat16()
    gate, lds = bf(inp["gate_raw"]), torch.from_numpy(inp["log_dt_scale"]).cuda()
    rf = torch.from_numpy(inp["rope_freqs"]).cuda()
    consts = const_args(inp["consts"])
    ups = [rn(B, L, H, N), rn(B, L, H, N // 2), rn(B, L, H), rn(B, L, H)]
    want_g, want_l = ref.dynamics_fused_bwd_cuda(*ups, gate, lds, rf, *consts, H, N)
    gt = gate.clone().requires_grad_(True)
    lt = lds.clone().requires_grad_(True)
    outs = ops.DynamicsFusedFn.apply(gt, lt, rf, *consts, H, N)
    torch.autograd.backward(outs, ups)
    assert rel_err(to_np(gt.grad), to_np(want_g)) <= BF16_TOL
    assert rel_err(to_np(lt.grad), to_np(want_l)) <= BF16_TOL
    K, Q, gK, gQ = (rn(B, L, H, D) for _ in range(4))
    wK, wQ = ref.normalize_kq_bwd_cuda(gK, gQ, K, Q)
    kt, qt = K.clone().requires_grad_(True), Q.clone().requires_grad_(True)
    torch.autograd.backward(ops.NormalizeKQFn.apply(kt, qt), [gK, gQ])
    assert rel_err(to_np(kt.grad), to_np(wK)) <= BF16_TOL / 2
    assert rel_err(to_np(qt.grad), to_np(wQ)) <= BF16_TOL / 2


def test_scan_side_backward_kernels_against_reference_backward_kernels(ops, orc, ref):
    """intra / inter / correction / conv backward against the reference's own backward kernels, each fed with the
    reference's own forward outputs as the saved tensors."""
    B, NC, C, H, N, D = 2, 3, 64, 4, 2, 64
    g = torch.Generator(device="cuda").manual_seed(3)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda")
    A = (rn(B * NC, C, H, N) * 0.4).bfloat16()
    K = (rn(B * NC, C, H, D) / 8).bfloat16()
    V, be = rn(B * NC, C, H, N).bfloat16(), torch.rand(B * NC, C, H, generator=g, device="cuda").bfloat16()
    lh, cA = ref.intra_chunk_scan_fwd_cuda(A, K, V, be, N)
    u1, u2 = rn(*lh.shape).bfloat16(), rn(*cA.shape).bfloat16()
    want = ref.intra_chunk_scan_bwd_cuda(u1, u2, A, K, V, be, lh, cA, N)
    ts = [t.clone().requires_grad_(True) for t in (A, K, V, be)]
    torch.autograd.backward(ops.IntraChunkScanFn.apply(*ts, N), [u1, u2])
    for t, w, name in zip(ts, want, ("A", "K", "V", "beta")):
        assert rel_err(to_np(t.grad), to_np(w)) <= BF16_TOL, name
    # inter-chunk
    tot, fin = (rn(B, NC, H, N) * 0.4).bfloat16(), rn(B, NC, H, N, D).bfloat16()
    cs = ref.inter_chunk_scan_fwd_cuda(tot, fin, N)
    up = rn(*cs.shape).bfloat16()
    wA, wH = ref.inter_chunk_scan_bwd_cuda(up, tot, cs, N)
    ta, tf = tot.clone().requires_grad_(True), fin.clone().requires_grad_(True)
    ops.InterChunkScanFn.apply(ta, tf, N).backward(up)
    assert rel_err(to_np(ta.grad), to_np(wA)) <= BF16_TOL and rel_err(to_np(tf.grad), to_np(wH)) <= BF16_TOL
    # correction
    A5, K5, b5 = A.view(B, NC, C, H, N), K.view(B, NC, C, H, D), be.view(B, NC, C, H)
    corr = ref.exact_correction_fwd_cuda(A5, K5, b5, cs, N)
    upc = rn(*corr.shape).bfloat16()
    want = ref.exact_correction_bwd_cuda(upc, A5, K5, b5, cs, corr, N)
    ts = [t.clone().requires_grad_(True) for t in (A5, K5, b5, cs)]
    ops.ExactCorrectionFn.apply(*ts, N).backward(upc)
    for t, w, name in zip(ts, want, ("A", "K", "beta", "chunk_states")):
        assert rel_err(to_np(t.grad), to_np(w)) <= BF16_TOL, name
    # conv
    x, w4 = rn(2, 100, 256).bfloat16(), (rn(256, 1, 4) / 2).bfloat16()
    bias, upx = (rn(256) / 5).bfloat16(), rn(2, 100, 256).bfloat16()
    want = ref.conv1d_silu_bwd_cuda(x, w4, bias, upx)
    ts = [t.clone().requires_grad_(True) for t in (x, w4, bias)]
    ops.CUDAConv1dSiLUOp.apply(*ts).backward(upx)
    for t, w, name in zip(ts, want, ("x", "weight", "bias")):
        assert rel_err(to_np(t.grad), to_np(w).reshape(t.shape)) <= BF16_TOL, name
