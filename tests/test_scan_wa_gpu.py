"""The warp-autonomous tcgen05/TMA scan passes (bf16, N = 2, D = C in {64, 128}, H % 4 == 0) against the CPU
oracle and against the CUDA-core kernels, through the C ABI.  Flag bits 256 / 512 keep the CUDA-core local /
output pass, so each tensor-core pass is also checked on its own."""
import numpy as np
import pytest
import torch

from test_scan_gpu import oracle_scan, run_fused, unnormalise
from util import BF16_TOL, rel_err, to_np

pytestmark = pytest.mark.gpu
N = 2
KEEP_SIMT_LOCAL, KEEP_SIMT_OUTPUT = 256, 512


def _tol13(D):
    """Against the oracle with the kernel's fp32 state but the reference's bf16-rounded unit rows: the kernels
    keep the normalised q, k rows in fp32, which costs up to a bf16 ulp per element of a 64-term dot product
    (the CUDA-core kernels show the same difference); head_dim 128 averages it down further."""
    return BF16_TOL / 2 if D == 128 else 0.75 * BF16_TOL


def _inputs(orc, B, H, L, D, seed, scale=True):
    inp = orc.make_inputs(B, H, L, D, N=N, seed=seed, bf16=True, context_length=max(L, 2))
    if scale:
        inp = unnormalise(inp, np.random.default_rng(seed))
        inp["q"], inp["k"] = orc.bf16_round(inp["q"]), orc.bf16_round(inp["k"])
    return inp


@pytest.mark.parametrize("extra", [KEEP_SIMT_LOCAL, KEEP_SIMT_OUTPUT, 0])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,H,L", [(1, 4, 128), (1, 4, 256), (2, 8, 300), (1, 4, 1), (1, 4, 129), (2, 12, 1024),
                                   (3, 32, 512)])
def test_wa_matches_oracle_and_simt(ops, orc, B, H, L, D, extra):
    inp = _inputs(orc, B, H, L, D, seed=L + H)
    y, fin = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.TENSOR_CORE_WA | extra)
    assert ops.scan_fused_status() == 0
    ys, fs = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.FORCE_SIMT)
    wy, _ = oracle_scan(orc, inp, N, D, orc.ROUND_REFERENCE)
    wy13, wf13 = oracle_scan(orc, inp, N, D, orc.ROUND_FP32_STATE)
    assert rel_err(to_np(y), wy) <= BF16_TOL
    assert rel_err(to_np(y), wy13) <= _tol13(D)
    assert rel_err(to_np(y), to_np(ys)) <= BF16_TOL / 2
    scale = max(np.abs(wf13).max(), 1e-3)
    assert np.abs(to_np(fin) - wf13).max() <= 2e-2 * scale
    assert np.abs(to_np(fin) - to_np(fs)).max() <= 2e-2 * scale


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,H,L", [(2, 4, 32), (1, 8, 33), (1, 4, 127), (3, 4, 128 * 5 + 17), (1, 64, 384), (5, 4, 97)])
def test_wa_ragged_lengths_default_path(ops, orc, B, H, L, D):
    """Lengths around the sub-block and chunk sizes, more head groups than one block walks at a time; no
    flags: these shapes take the tensor-core passes by themselves."""
    inp = _inputs(orc, B, H, L, D, seed=7 * L + H)
    y, fin = run_fused(ops, inp, torch.bfloat16, N, D)
    assert ops.scan_fused_status() == 0
    ys, fs = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.FORCE_SIMT)
    wy13, wf13 = oracle_scan(orc, inp, N, D, orc.ROUND_FP32_STATE)
    assert rel_err(to_np(y), wy13) <= _tol13(D)
    assert rel_err(to_np(y), to_np(ys)) <= BF16_TOL / 2
    scale = max(np.abs(wf13).max(), 1e-3)
    assert np.abs(to_np(fin) - wf13).max() <= 2e-2 * scale


@pytest.mark.parametrize("D", [128, 64])
def test_wa_h0_shortcut_composition(ops, orc, D):
    B, H, L = 2, 4, 512
    inp = _inputs(orc, B, H, L, D, seed=77, scale=False)
    h0 = np.random.default_rng(1).standard_normal((B, H, N, D)).astype(np.float32)
    wy, wfin = oracle_scan(orc, inp, N, D, orc.ROUND_FP32_STATE, h0=h0, shortcut_scale=0.6)
    y, fin = run_fused(ops, inp, torch.bfloat16, N, D, h0=h0, shortcut_scale=0.6, flags=ops.TENSOR_CORE_WA)
    assert ops.scan_fused_status() == 0
    assert rel_err(to_np(y), wy) <= BF16_TOL / 2
    assert rel_err(to_np(fin), wfin) <= 2e-2
    cut = lambda s: {k: (v[:, s] if getattr(v, "ndim", 0) >= 3 else v) for k, v in inp.items()}
    y1, f1 = run_fused(ops, cut(slice(0, 256)), torch.bfloat16, N, D, h0=h0, shortcut_scale=0.6, flags=ops.TENSOR_CORE_WA)
    y2, f2 = run_fused(ops, cut(slice(256, None)), torch.bfloat16, N, D, h0=to_np(f1), shortcut_scale=0.6, pos0=256,
                       flags=ops.TENSOR_CORE_WA)
    assert torch.equal(torch.cat([y1, y2], 1), y) and torch.equal(f2, fin)


@pytest.mark.parametrize("D", [128, 64])
def test_wa_many_items_per_block(ops, orc, D):
    """More (chunk, head group) items than resident thread blocks: the persistent loop and its barrier
    phases across items."""
    B, H, L = 2, 8, D * 96 * (128 // D)
    inp = _inputs(orc, B, H, L, D, seed=9)
    y, fin = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.TENSOR_CORE_WA)
    assert ops.scan_fused_status() == 0
    ys, fs = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.FORCE_SIMT)
    assert rel_err(to_np(y), to_np(ys)) <= BF16_TOL / 2
    assert rel_err(to_np(fin), to_np(fs)) <= 2e-2


def test_wa_deterministic_and_in_bounds(ops, orc):
    B, H, L, D = 1, 4, 384, 128
    inp = _inputs(orc, B, H, L, D, seed=5)
    n = B * L * H * N
    big = torch.full((n + 512,), 7.0, device="cuda", dtype=torch.bfloat16)
    out = big[256:256 + n].view(B, L, H, N)
    y1, f1 = run_fused(ops, inp, torch.bfloat16, N, D, out=out, flags=ops.TENSOR_CORE_WA)
    y1 = y1.clone()
    y2, f2 = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.TENSOR_CORE_WA)
    assert torch.equal(y1, y2) and torch.equal(f1, f2)
    assert bool((big[:256] == 7).all()) and bool((big[256 + n:] == 7).all())


def test_wa_flag_rejects_unsupported_sizes(ops, orc):
    inp = orc.make_inputs(1, 4, 64, 32, N=2, seed=1, bf16=True)       # head_dim 32
    with pytest.raises(RuntimeError):
        run_fused(ops, inp, torch.bfloat16, 2, 32, flags=ops.TENSOR_CORE_WA)
    inp = orc.make_inputs(1, 3, 128, 128, N=2, seed=1, bf16=True)     # H not a multiple of 4
    with pytest.raises(RuntimeError):
        run_fused(ops, inp, torch.bfloat16, 2, 128, flags=ops.TENSOR_CORE_WA)
    inp = orc.make_inputs(1, 4, 128, 128, N=2, seed=1, bf16=True)     # chunk != head_dim
    with pytest.raises(RuntimeError):
        run_fused(ops, inp, torch.bfloat16, 2, 64, flags=ops.TENSOR_CORE_WA)


def test_wa_segmented_scan_equals_unsegmented(ops, orc):
    """Sequence segments as extra batch rows: the tensor-core output pass on the summary pass's local results."""
    from util import const_args, to_dev
    B, H, L, S, D = 1, 4, 1024, 4, 128
    inp = orc.make_inputs(B, H, L, D, N=N, seed=3, bf16=True)
    h0 = np.random.default_rng(3).standard_normal((B, H, N, D)).astype(np.float32) * 0.3
    d = lambda x: to_dev(x, torch.bfloat16)
    f = lambda x: to_dev(x, torch.float32)
    args = (d(inp["q"]), d(inp["k"]), d(inp["v"]), d(inp["gate_raw"]), f(inp["log_dt_scale"]), f(inp["rope_freqs"]),
            *const_args(inp["consts"]), H, N, D, f(h0))
    y, fin = ops.scan_fused(*args, shortcut_scale=0.4, pos0=7)
    ys, fs = ops.scan_fused_long(*args, segments=S, shortcut_scale=0.4, pos0=7)
    assert ops.scan_fused_status() == 0
    assert rel_err(to_np(ys), to_np(y)) <= 2.0 ** -7
    assert rel_err(to_np(fs), to_np(fin)) <= 2.0 ** -9


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("alpha_gate", [None, 2.0])
def test_wa_strong_decay(ops, orc, alpha_gate, D):
    """Gates pushed towards strong decay over 200 tokens.  alpha_gate None: half-sub-block decay products down
    to about 1e-27, still inside the range of the scaled walk (scalings up to 1e27); alpha_gate 2.0: down to
    about 1e-48, where the kernel falls back to the explicit walk.  Both must agree with the CUDA-core
    kernels and the oracle."""
    B, H, L = 1, 4, 512
    inp = _inputs(orc, B, H, L, D, seed=11)
    g = inp["gate_raw"].copy()
    g[:, 100:300, 6 * H:7 * H] += 8.0            # r gate: exponent of the decay magnitude at its maximum
    if alpha_gate is None:
        g[:, 100:300, 0:H] += 4.0                # decay-rate pre-activation
    else:
        g[:, 100:300, 0:H] = alpha_gate
        g[:, 100:300, H:2 * H] = 0.0             # no rotation: the Cayley map gets closest to zero
    inp["gate_raw"] = orc.bf16_round(g)
    y, fin = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.TENSOR_CORE_WA)
    assert ops.scan_fused_status() == 0
    ys, fs = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.FORCE_SIMT)
    wy13, _ = oracle_scan(orc, inp, N, D, orc.ROUND_FP32_STATE)
    assert np.isfinite(to_np(y)).all()
    assert rel_err(to_np(y), wy13) <= _tol13(D)
    assert rel_err(to_np(y), to_np(ys)) <= BF16_TOL / 2
    assert np.abs(to_np(fin) - to_np(fs)).max() <= 2e-2 * max(np.abs(to_np(fs)).max(), 1e-3)


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("path", ["tensor-core", "cuda-core", "segments"])
def test_float32_transition_option(ops, orc, D, path):
    """FP32_DECAY keeps A_bar in float32 between the dynamics and the scan (the oracle's ROUND_KEEP_DECAY bit);
    everything else rounds as before, so the results differ from the reference's only by A_bar's bf16 rounding."""
    from util import const_args, to_dev
    B, H, L = 2, 4, 640
    inp = _inputs(orc, B, H, L, D, seed=21)
    wy, wf = oracle_scan(orc, inp, N, D, orc.ROUND_FP32_STATE | orc.ROUND_KEEP_DECAY)
    wy_ref, _ = oracle_scan(orc, inp, N, D, orc.ROUND_FP32_STATE)
    if path == "segments":
        d = lambda x: to_dev(x, torch.bfloat16)
        f = lambda x: to_dev(x, torch.float32)
        y, fin = ops.scan_fused_long(d(inp["q"]), d(inp["k"]), d(inp["v"]), d(inp["gate_raw"]), f(inp["log_dt_scale"]),
                                     f(inp["rope_freqs"]), *const_args(inp["consts"]), H, N, D, segments=5, flags=ops.FP32_DECAY)
    else:
        extra = ops.TENSOR_CORE_WA if path == "tensor-core" else ops.FORCE_SIMT
        y, fin = run_fused(ops, inp, torch.bfloat16, N, D, flags=ops.FP32_DECAY | extra)
    assert ops.scan_fused_status() == 0
    assert rel_err(to_np(y), wy) <= _tol13(D)
    assert np.abs(to_np(fin) - wf).max() <= 2e-2 * max(np.abs(wf).max(), 1e-3)
    # and it is a different arithmetic from the default: the option is not silently ignored
    y0, _ = run_fused(ops, inp, torch.bfloat16, N, D)
    assert not torch.equal(y0, y)
    assert rel_err(to_np(y), wy) < rel_err(to_np(y), wy_ref) or rel_err(wy, wy_ref) < 1e-3
