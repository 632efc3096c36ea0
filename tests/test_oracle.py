"""CPU tests of the oracle itself: identities the algorithm must satisfy, and (when present)
the golden vectors produced by the reference's own kernels on a B200."""
import glob
import os

import numpy as np
import pytest
import torch

from util import rel_err

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def _args(inp, N=2):
    return (inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"], inp["rope_freqs"],
            inp["consts"], N)


def test_bf16_rounding_matches_torch(orc):
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 10.0 ** rng.integers(-20, 20, 4096),
                        np.array([0.0, -0.0, 1.00390625, 1.0078125, 3.0e38, 1e-40], np.float32)])
    want = torch.from_numpy(x).bfloat16().float().numpy()
    assert np.array_equal(orc.bf16_round(x), want)
    assert orc.lib().orc_bf16_round(1.00390625) == 1.0


def test_first_chunk_equals_recurrence(orc):
    inp = orc.make_inputs(2, 4, 192, 64, seed=0)
    y, _ = orc.scan_reference(*_args(inp), 64)
    yr, _ = orc.scan_recurrent(*_args(inp))
    assert np.abs(y[:, :64] - yr[:, :64]).max() == 0.0
    # beyond the first chunk the reference's chunk semantics differ from the recurrence
    assert rel_err(y, yr) > 1e-3


def test_single_chunk_whole_sequence_is_recurrence(orc):
    inp = orc.make_inputs(1, 2, 100, 32, seed=3)
    y, _ = orc.scan_reference(*_args(inp), 128)
    yr, _ = orc.scan_recurrent(*_args(inp))
    assert np.abs(y - yr).max() == 0.0


def test_dynamics_properties(orc):
    inp = orc.make_inputs(2, 4, 256, 64, N=4, seed=1)
    A, vp, beta, selc = orc.dynamics(inp["gate_raw"], inp["log_dt_scale"], inp["rope_freqs"],
                                     inp["consts"], 4, 4)
    mag2 = A[..., 0::2] ** 2 + A[..., 1::2] ** 2
    assert mag2.max() <= 1.0 + 1e-5                       # A-stability of the Cayley map
    # vp^2 + |mu|^(2 c r) = 1 and |A|^2 = |mu|^(2 c r)  (dynamics_fused.cu:112-131)
    free = (vp > 1.1e-3) & (vp < 1.0)
    assert np.abs((vp ** 2 + mag2)[free] - 1.0).max() < 2e-4
    assert beta.min() > 0 and beta.max() < 1 and selc.min() > 0 and selc.max() < 1


def test_normalised_rows_have_unit_norm(orc):
    rng = np.random.default_rng(2)
    K = rng.standard_normal((3, 5, 2, 64)).astype(np.float32) * 7
    Q = rng.standard_normal((3, 5, 2, 64)).astype(np.float32) * 0.01
    kn, qn = orc.normalize_kq(K, Q)
    assert np.abs(np.linalg.norm(kn, axis=-1) - 1).max() < 1e-5
    assert np.abs(np.linalg.norm(qn, axis=-1) - 1).max() < 6e-3   # the 1e-6 under the root shows at |q|~0.08


def test_zero_beta_is_pure_rotation(orc):
    BNC, C, H, D, N = 2, 16, 2, 32, 2
    rng = np.random.default_rng(4)
    ang = rng.uniform(-3, 3, (BNC, C, H))
    A = np.stack([np.cos(ang), np.sin(ang)], -1).astype(np.float32)
    K = rng.standard_normal((BNC, C, H, D)).astype(np.float32)
    cs = rng.standard_normal((1, BNC, H, N, D)).astype(np.float32)
    corr = orc.exact_correction(A[None], K[None], np.zeros((1, BNC, C, H), np.float32), cs, N)
    n0 = np.linalg.norm(cs, axis=(-2, -1))
    n = np.linalg.norm(corr, axis=(-2, -1))               # (1,BNC,C,H)
    assert np.abs(n - n0[:, :, None, :]).max() < 1e-4
    lh, cumA = orc.intra_chunk(A, K, np.ones((BNC, C, H, N), np.float32), np.zeros((BNC, C, H), np.float32), N)
    assert np.abs(lh).max() == 0.0
    assert np.abs(np.hypot(cumA[..., 0], cumA[..., 1]) - 1).max() < 1e-5


def test_zero_padding_wipes_carry(orc):
    inp = orc.make_inputs(1, 2, 70, 32, seed=5)
    _, fin = orc.scan_reference(*_args(inp), 64)           # second chunk is padded with zeros
    assert np.abs(fin).max() == 0.0


@pytest.mark.parametrize("mask", [0, 13, 15])
def test_segments_compose(orc, mask):
    inp = orc.make_inputs(2, 2, 256, 64, seed=6, bf16=mask != 0)
    a = _args(inp)
    y, fin = orc.scan_reference(*a, 64, round_bf16=mask)
    cut = lambda x, s: x[:, s] if getattr(x, "ndim", 0) >= 3 else x
    a1 = [cut(x, slice(0, 128)) for x in a]
    a2 = [cut(x, slice(128, None)) for x in a]
    y1, f1 = orc.scan_reference(*a1, 64, round_bf16=mask)
    y2, f2 = orc.scan_reference(*a2, 64, h0=f1, pos0=128, round_bf16=mask)
    assert np.array_equal(np.concatenate([y1, y2], 1), y)
    assert np.array_equal(f2, fin)


def test_fp32_state_mode_is_close_to_reference_rounding(orc):
    """The 'bf16 storage, fp32 state' statement stays within the bf16 parity budget of the
    reference's all-bf16 pipeline when the scan inputs are rounded at the same points."""
    inp = orc.make_inputs(2, 4, 512, 64, seed=0, bf16=True)
    y15, _ = orc.scan_reference(*_args(inp), 64, round_bf16=orc.ROUND_REFERENCE)
    y13, _ = orc.scan_reference(*_args(inp), 64, round_bf16=orc.ROUND_FP32_STATE)
    assert rel_err(y13, y15) < 1e-2


def test_composed_ops_equal_scan_reference(orc):
    """scan_reference is the composition of the per-kernel restatements."""
    B, H, L, D, N, C = 1, 2, 128, 32, 2, 64
    inp = orc.make_inputs(B, H, L, D, seed=7)
    A, vp, beta, selc = orc.dynamics(inp["gate_raw"], inp["log_dt_scale"], inp["rope_freqs"], inp["consts"], H, N)
    kn, qn = orc.normalize_kq(inp["k"], inp["q"])
    vg = inp["v"] * np.repeat(vp, 2, -1)
    NC = L // C
    rs = lambda x: x.reshape(B * NC, C, *x.shape[2:])
    lh, cA = orc.intra_chunk(rs(A), rs(kn), rs(vg), rs(beta), N)
    lh6 = lh.reshape(B, NC, C, H, N, D)
    cs = orc.inter_chunk(cA.reshape(B, NC, C, H, N)[:, :, -1], lh6[:, :, -1], N)
    co = orc.exact_correction(A.reshape(B, NC, C, H, N), kn.reshape(B, NC, C, H, D),
                              beta.reshape(B, NC, C, H), cs, N)
    Y = (lh6 + co).reshape(B, L, H, N, D)
    y = np.einsum("blhsd,blhd->blhs", Y, qn) * selc[..., None]
    yref, _ = orc.scan_reference(*_args(inp), C)
    assert rel_err(y, yref) < 1e-6


def test_conv1d_silu_matches_torch(orc):
    rng = np.random.default_rng(8)
    x = rng.standard_normal((2, 37, 24)).astype(np.float32)
    w = rng.standard_normal((24, 1, 4)).astype(np.float32)
    b = rng.standard_normal(24).astype(np.float32)
    want = torch.nn.functional.silu(torch.nn.functional.conv1d(
        torch.from_numpy(x).transpose(1, 2), torch.from_numpy(w), torch.from_numpy(b),
        padding=3, groups=24)[..., :37]).transpose(1, 2).numpy()
    assert np.abs(orc.conv1d_silu(x, w, b) - want).max() < 1e-5


# ---- golden vectors: outputs of the reference's own kernels, recorded on a B200 ------------
GOLDEN_FILES = sorted(glob.glob(os.path.join(GOLDEN, "ref_*.npz")))


@pytest.mark.skipif(not GOLDEN_FILES, reason="no golden vectors recorded yet")
@pytest.mark.parametrize("path", GOLDEN_FILES, ids=[os.path.basename(p) for p in GOLDEN_FILES])
def test_oracle_matches_reference_kernels(orc, path):
    from golden.golden_cases import check_oracle_against_golden
    check_oracle_against_golden(orc, np.load(path))
