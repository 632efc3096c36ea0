"""The fused scan and the decode step against the CPU oracle, through the C ABI."""
import numpy as np
import pytest
import torch

from util import BF16_TOL, FP32_TOL, const_args, rel_err, to_dev, to_np

pytestmark = pytest.mark.gpu


def run_fused(ops, inp, dtype, N, C, h0=None, **kw):
    H = inp["q"].shape[2]
    d = lambda x: to_dev(x, dtype)
    f = lambda x: to_dev(x, torch.float32)
    return ops.scan_fused(d(inp["q"]), d(inp["k"]), d(inp["v"]), d(inp["gate_raw"]), f(inp["log_dt_scale"]),
                          f(inp["rope_freqs"]), *const_args(inp["consts"]), H, N, C,
                          None if h0 is None else f(h0), **kw)


def oracle_scan(orc, inp, N, C, mask, **kw):
    return orc.scan_reference(inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"],
                              inp["rope_freqs"], inp["consts"], N, C, round_bf16=mask, **kw)


def unnormalise(inp, rng):
    """The benchmark inputs are unit rows; scale them so the in-kernel normalisation matters."""
    s = rng.uniform(0.25, 4.0, inp["q"].shape[:3] + (1,)).astype(np.float32)
    inp["q"] = inp["q"] * s
    inp["k"] = inp["k"] * s[::-1].copy()
    return inp


SHAPES = [  # B, H, L, D, N, C
    (2, 4, 512, 64, 2, 64),      # the reference-runnable configuration
    (1, 3, 1, 64, 2, 64),        # a single token
    (2, 2, 63, 64, 2, 64),       # C - 1
    (2, 2, 64, 64, 2, 64),       # exactly one chunk
    (2, 2, 65, 64, 2, 64),       # C + 1
    (1, 2, 197, 64, 2, 64),      # 3C + 5
    (1, 2, 384, 128, 2, 128),    # head_dim 128
    (1, 5, 150, 64, 4, 64),      # two complex pairs, odd head count
    (1, 2, 96, 32, 16, 32),      # the reference's default state_dim
    (1, 2, 100, 40, 2, 24),      # ragged head_dim, chunk != head_dim
    (1, 20, 130, 64, 2, 64),     # more (head,pair) units than one block holds
]


@pytest.mark.parametrize("B,H,L,D,N,C", SHAPES)
def test_fused_fp32(ops, orc, B, H, L, D, N, C):
    inp = unnormalise(orc.make_inputs(B, H, L, D, N=N, seed=L + D, context_length=max(L, 2)), np.random.default_rng(L))
    y, fin = run_fused(ops, inp, torch.float32, N, C)
    wy, wfin = oracle_scan(orc, inp, N, C, 0)
    assert rel_err(to_np(y), wy) <= FP32_TOL
    assert np.abs(to_np(fin) - wfin).max() <= FP32_TOL * max(np.abs(wfin).max(), 1e-3)


@pytest.mark.parametrize("B,H,L,D,N,C", SHAPES)
def test_fused_bf16_vs_reference_rounding(ops, orc, B, H, L, D, N, C):
    inp = orc.make_inputs(B, H, L, D, N=N, seed=L + D + 1, bf16=True, context_length=max(L, 2))
    inp = unnormalise(inp, np.random.default_rng(L))
    inp["q"], inp["k"] = orc.bf16_round(inp["q"]), orc.bf16_round(inp["k"])
    y, fin = run_fused(ops, inp, torch.bfloat16, N, C)
    assert y.dtype == torch.bfloat16 and fin.dtype == torch.float32
    wy, _ = oracle_scan(orc, inp, N, C, orc.ROUND_REFERENCE)        # the reference as it runs
    assert rel_err(to_np(y), wy) <= BF16_TOL
    wy13, wfin13 = oracle_scan(orc, inp, N, C, orc.ROUND_FP32_STATE)  # same rounding points as the kernel
    assert rel_err(to_np(y), wy13) <= BF16_TOL / 2
    assert np.abs(to_np(fin) - wfin13).max() <= 1e-2 * max(np.abs(wfin13).max(), 1e-3)


@pytest.mark.parametrize("dtype,mask,tol", [(torch.float32, 0, FP32_TOL), (torch.bfloat16, 13, 2.0 ** -7)])
def test_h0_shortcut_pos0_and_composition(ops, orc, dtype, mask, tol):
    B, H, L, D, N, C = 2, 3, 256, 64, 2, 64
    inp = orc.make_inputs(B, H, L, D, N=N, seed=21, bf16=mask != 0)
    rng = np.random.default_rng(5)
    h0 = rng.standard_normal((B, H, N, D)).astype(np.float32)
    wy, wfin = oracle_scan(orc, inp, N, C, mask, h0=h0, shortcut_scale=0.7)
    y, fin = run_fused(ops, inp, dtype, N, C, h0=h0, shortcut_scale=0.7)
    assert rel_err(to_np(y), wy) <= tol and rel_err(to_np(fin), wfin) <= max(tol, 1e-3)
    # two chunk-aligned segments chained through (final_state, pos0) equal the whole
    cut = lambda s: {k: (v[:, s] if getattr(v, "ndim", 0) >= 3 else v) for k, v in inp.items()}
    y1, f1 = run_fused(ops, cut(slice(0, 128)), dtype, N, C, h0=h0, shortcut_scale=0.7)
    y2, f2 = run_fused(ops, cut(slice(128, None)), dtype, N, C, h0=to_np(f1), shortcut_scale=0.7, pos0=128)
    assert torch.equal(torch.cat([y1, y2], 1), y)
    assert torch.equal(f2, fin)


def test_run_to_run_bit_identical(ops, orc):
    inp = orc.make_inputs(2, 4, 300, 64, seed=3, bf16=True)
    y1, f1 = run_fused(ops, inp, torch.bfloat16, 2, 64)
    y2, f2 = run_fused(ops, inp, torch.bfloat16, 2, 64)
    assert torch.equal(y1, y2) and torch.equal(f1, f2)      # no atomics on this path


def test_outputs_stay_inside_their_buffers(ops, orc):
    """compute-sanitizer is not available here: write into the middle of a poisoned buffer."""
    B, H, L, D, N, C = 1, 3, 70, 64, 2, 64
    inp = orc.make_inputs(B, H, L, D, seed=4, bf16=True)
    n = B * L * H * N
    big = torch.full((n + 512,), 7.0, device="cuda", dtype=torch.bfloat16)
    out = big[256:256 + n].view(B, L, H, N)
    run_fused(ops, inp, torch.bfloat16, N, C, out=out)
    torch.cuda.synchronize()
    assert bool((big[:256] == 7).all()) and bool((big[256 + n:] == 7).all())
    assert bool((out != 7).any())


def test_empty_inputs(ops, orc):
    z = lambda *s: torch.zeros(*s, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(2, device="cuda")
    c = orc.derive_constants(64)
    y, fin = ops.scan_fused(z(1, 0, 2, 64), z(1, 0, 2, 64), z(1, 0, 2, 2), z(1, 0, 14), f, f,
                            *const_args(c), 2, 2, 64)
    assert tuple(y.shape) == (1, 0, 2, 2) and float(fin.abs().max()) == 0.0


def test_unsupported_sizes_raise(ops, orc):
    z = lambda *s: torch.zeros(*s, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(1, device="cuda")
    c = const_args(orc.derive_constants(64))
    with pytest.raises(RuntimeError):
        ops.scan_fused(z(1, 8, 1, 256), z(1, 8, 1, 256), z(1, 8, 1, 2), z(1, 8, 7), f, f, *c, 1, 2, 64)
    with pytest.raises(RuntimeError):
        ops.scan_fused(z(1, 8, 1, 64).float(), z(1, 8, 1, 64), z(1, 8, 1, 2), z(1, 8, 7), f, f, *c, 1, 2, 64)


# ---------------------------------------------------------------- decode
@pytest.mark.parametrize("dtype,mask,tol", [(torch.float32, 0, FP32_TOL), (torch.bfloat16, 9, 2.0 ** -7)])
@pytest.mark.parametrize("B,H,D,N,T", [(3, 4, 64, 2, 40), (2, 3, 128, 2, 20), (2, 2, 64, 16, 12), (1, 5, 40, 4, 9)])
def test_decode_steps_equal_recurrence(ops, orc, dtype, mask, tol, B, H, D, N, T):
    inp = orc.make_inputs(B, H, T, D, N=N, seed=T, bf16=mask != 0, context_length=64)
    rng = np.random.default_rng(T)
    s0 = rng.standard_normal((B, H, N, D)).astype(np.float32)
    wy, wst = orc.scan_recurrent(inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"],
                                 inp["rope_freqs"], inp["consts"], N, state=s0, shortcut_scale=0.3,
                                 pos0=5, round_bf16=mask)
    d = lambda x: to_dev(x, dtype)
    state = to_dev(s0, torch.float32)
    lds, rf = to_dev(inp["log_dt_scale"], torch.float32), to_dev(inp["rope_freqs"], torch.float32)
    q, k, v, g = d(inp["q"]), d(inp["k"]), d(inp["v"]), d(inp["gate_raw"])
    ys = []
    for t in range(T):
        ys.append(ops.decode_step(state, q[:, t], k[:, t], v[:, t], g[:, t], lds, rf,
                                  *const_args(inp["consts"]), H, N, 5 + t, shortcut_scale=0.3))
    y = torch.stack(ys, 1)
    assert rel_err(to_np(y), wy) <= tol
    assert rel_err(to_np(state), wst) <= max(tol / 8, 1e-5)


def test_prefill_tail_state_feeds_decode(ops, orc):
    """Prefill T0 <= C tokens with the fused scan, continue with decode steps: inside one chunk
    the reference equals the recurrence, so the whole thing equals one scan of T0 + T1 tokens."""
    B, H, D, N, C, T0, T1 = 2, 3, 64, 2, 64, 40, 24
    inp = orc.make_inputs(B, H, T0 + T1, D, N=N, seed=9, context_length=64)
    full = {k: v for k, v in inp.items()}
    wy, _ = oracle_scan(orc, full, N, C, 0)
    head = {k: (v[:, :T0] if getattr(v, "ndim", 0) >= 3 else v) for k, v in inp.items()}
    y0, _, tail = run_fused(ops, head, torch.float32, N, C, return_tail_state=True)
    f = lambda x: to_dev(x, torch.float32)
    q, k, v, g = f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["gate_raw"])
    ys = [ops.decode_step(tail, q[:, t], k[:, t], v[:, t], g[:, t], f(inp["log_dt_scale"]),
                          f(inp["rope_freqs"]), *const_args(inp["consts"]), H, N, t) for t in range(T0, T0 + T1)]
    y = torch.cat([y0, torch.stack(ys, 1)], 1)
    assert rel_err(to_np(y), wy) <= FP32_TOL


# ---------------------------------------------------------------- sequence segments
@pytest.mark.parametrize("dtype,mask,tol", [(torch.float32, 0, 2e-5), (torch.bfloat16, 13, 2.0 ** -7)])
@pytest.mark.parametrize("B,H,L,D,N,C,S", [(2, 3, 512, 64, 2, 64, 4), (1, 2, 1024, 128, 2, 128, 8), (1, 2, 256, 32, 4, 32, 2)])
def test_segmented_scan_equals_unsegmented(ops, orc, dtype, mask, tol, B, H, L, D, N, C, S):
    inp = orc.make_inputs(B, H, L, D, N=N, seed=S, bf16=mask != 0)
    h0 = np.random.default_rng(S).standard_normal((B, H, N, D)).astype(np.float32) * 0.3
    d = lambda x: to_dev(x, dtype)
    f = lambda x: to_dev(x, torch.float32)
    args = (d(inp["q"]), d(inp["k"]), d(inp["v"]), d(inp["gate_raw"]), f(inp["log_dt_scale"]), f(inp["rope_freqs"]),
            *const_args(inp["consts"]), H, N, C, f(h0))
    y, fin = ops.scan_fused(*args, shortcut_scale=0.4, pos0=7)
    ys, fs = ops.scan_fused_long(*args, segments=S, shortcut_scale=0.4, pos0=7)
    assert rel_err(to_np(ys), to_np(y)) <= tol
    assert rel_err(to_np(fs), to_np(fin)) <= max(tol / 8, 1e-5)
    # the summary of the whole sequence is its carry-out and the product of the chunk decays
    carry, decay = ops.scan_summary(*args[1:4], *args[4:6], *const_args(inp["consts"]), H, N, C, f(h0), pos0=7)
    assert rel_err(to_np(carry), to_np(fin)) <= 1e-6
    A, _, _, _ = orc.dynamics(inp["gate_raw"], inp["log_dt_scale"], inp["rope_freqs"], inp["consts"], H, N,
                              pos0=7, round_bf16=mask)
    Ac = (A[..., 0::2] + 1j * A[..., 1::2]).reshape(B, L // C, C, H, N // 2).astype(np.complex128)
    gam = np.ones((B, H, N // 2), np.complex128)
    for c in range(L // C):
        g = np.prod(Ac[:, c], axis=1)
        if mask:
            g = orc.bf16_round(g.real.astype(np.float32)) + 1j * orc.bf16_round(g.imag.astype(np.float32))
        gam = gam * g
    got = to_np(decay)
    assert np.abs(got[..., 0::2] - gam.real).max() <= 2e-2 * max(np.abs(gam).max(), 1e-6)
    assert np.abs(got[..., 1::2] - gam.imag).max() <= 2e-2 * max(np.abs(gam).max(), 1e-6)


# ---------------------------------------------------------------- exact (sequential) semantics
@pytest.mark.parametrize("dtype,mask,tol", [(torch.float32, 0, FP32_TOL), (torch.bfloat16, 9, BF16_TOL / 2)])
@pytest.mark.parametrize("B,H,L,D,N", [(2, 3, 300, 64, 2), (1, 2, 200, 128, 2), (1, 2, 70, 40, 4)])
def test_exact_semantics_is_the_sequential_recurrence(ops, orc, dtype, mask, tol, B, H, L, D, N):
    inp = orc.make_inputs(B, H, L, D, N=N, seed=L, bf16=mask != 0, context_length=512)
    s0 = np.random.default_rng(L).standard_normal((B, H, N, D)).astype(np.float32) * 0.5
    wy, wst = orc.scan_recurrent(inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"],
                                 inp["rope_freqs"], inp["consts"], N, state=s0, shortcut_scale=0.2, pos0=3,
                                 round_bf16=mask)
    y, fin, tail = run_fused(ops, inp, dtype, N, 64, h0=s0, shortcut_scale=0.2, pos0=3, semantics="exact",
                             return_tail_state=True)
    assert rel_err(to_np(y), wy) <= tol
    assert rel_err(to_np(fin), wst) <= max(tol / 4, 1e-5) and torch.equal(fin, tail)
    # the reference's chunk semantics equal the recurrence inside the first chunk when the carry-in is
    # zero (a non-zero carry is read one step early, exact_correction.cu:90-94) and differ beyond it
    wy0, _ = orc.scan_recurrent(inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"],
                                inp["rope_freqs"], inp["consts"], N, shortcut_scale=0.2, pos0=3, round_bf16=mask)
    yr, _ = run_fused(ops, inp, dtype, N, 64, shortcut_scale=0.2, pos0=3)
    if L > 64:
        assert rel_err(to_np(yr), wy0) > 10 * tol
    assert rel_err(to_np(yr[:, :64]), wy0[:, :64]) <= tol


def test_exact_prefill_feeds_decode_beyond_one_chunk(ops, orc):
    B, H, D, N, T0, T1 = 2, 2, 64, 2, 150, 10
    inp = orc.make_inputs(B, H, T0 + T1, D, N=N, seed=12, context_length=256)
    wy, _ = orc.scan_recurrent(inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"],
                               inp["rope_freqs"], inp["consts"], N)
    head = {k: (v[:, :T0] if getattr(v, "ndim", 0) >= 3 else v) for k, v in inp.items()}
    y0, state = run_fused(ops, head, torch.float32, N, 64, semantics="exact")
    f = lambda x: to_dev(x, torch.float32)
    q, k, v, g = f(inp["q"]), f(inp["k"]), f(inp["v"]), f(inp["gate_raw"])
    ys = [ops.decode_step(state, q[:, t], k[:, t], v[:, t], g[:, t], f(inp["log_dt_scale"]), f(inp["rope_freqs"]),
                          *const_args(inp["consts"]), H, N, t) for t in range(T0, T0 + T1)]
    y = torch.cat([y0, torch.stack(ys, 1)], 1)
    assert rel_err(to_np(y), wy) <= FP32_TOL


@pytest.mark.parametrize("dtype,mask,tol", [(torch.float32, 0, FP32_TOL), (torch.bfloat16, 13, BF16_TOL / 2)])
@pytest.mark.parametrize("B,H,D,N,C,T", [(2, 3, 64, 2, 64, 3 * 64 + 7), (1, 2, 64, 4, 64, 130), (1, 4, 128, 2, 128, 300),
                                         (1, 2, 40, 2, 24, 60)])
def test_reference_decode_steps_equal_the_chunked_scan(ops, orc, dtype, mask, tol, B, H, D, N, C, T):
    """T reference-compatible decode steps from the start of a sequence reproduce the reference's chunked scan
    over T tokens - beyond the first chunk too, where the plain recurrence (decode_step) does not."""
    inp = orc.make_inputs(B, H, T, D, N=N, seed=T + D, bf16=mask != 0, context_length=512)
    wy, _ = oracle_scan(orc, inp, N, C, mask, shortcut_scale=0.3)
    d = lambda x: to_dev(x, dtype)
    lds, rf = to_dev(inp["log_dt_scale"], torch.float32), to_dev(inp["rope_freqs"], torch.float32)
    q, k, v, g = d(inp["q"]), d(inp["k"]), d(inp["v"]), d(inp["gate_raw"])
    st = ops.reference_decode_state(torch.zeros(B, H, N, D, device="cuda"), dtype)
    ys = [ops.decode_step_reference(st, q[:, t], k[:, t], v[:, t], g[:, t], lds, rf, *const_args(inp["consts"]), H, N, C,
                                    t, shortcut_scale=0.3) for t in range(T)]
    y = torch.stack(ys, 1)
    assert rel_err(to_np(y), wy) <= tol
    yf, _ = run_fused(ops, inp, dtype, N, C, shortcut_scale=0.3)
    assert rel_err(to_np(y), to_np(yf)) <= tol
    if T > C:   # the plain recurrence really is something else there
        wrec, _ = orc.scan_recurrent(inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"],
                                     inp["rope_freqs"], inp["consts"], N, shortcut_scale=0.3, round_bf16=mask)
        assert rel_err(wrec, wy) > 10 * tol


def test_reference_decode_continues_a_chunk_aligned_prefill(ops, orc):
    B, H, D, N, C, L0, T = 2, 4, 64, 2, 64, 128, 64 + 9
    inp = orc.make_inputs(B, H, L0 + T, D, N=N, seed=5, bf16=True, context_length=512)
    full, _ = run_fused(ops, inp, torch.bfloat16, N, C)
    head = {k: (v[:, :L0] if getattr(v, "ndim", 0) >= 3 else v) for k, v in inp.items()}
    _, carry = run_fused(ops, head, torch.bfloat16, N, C)
    st = ops.reference_decode_state(carry, torch.bfloat16)
    d = lambda x: to_dev(x, torch.bfloat16)
    lds, rf = to_dev(inp["log_dt_scale"], torch.float32), to_dev(inp["rope_freqs"], torch.float32)
    q, k, v, g = d(inp["q"]), d(inp["k"]), d(inp["v"]), d(inp["gate_raw"])
    pos = torch.tensor([L0], dtype=torch.int32, device="cuda")      # the graph-replayable form of the position
    ys = []
    for t in range(L0, L0 + T):
        ys.append(ops.decode_step_reference(st, q[:, t], k[:, t], v[:, t], g[:, t], lds, rf,
                                            *const_args(inp["consts"]), H, N, C, pos))
        pos += 1
    y = torch.stack(ys, 1)
    assert rel_err(to_np(y), to_np(full[:, L0:])) <= BF16_TOL / 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_decode_step_with_projection_slices_and_value_residual(ops, orc, dtype):
    """k and v as column slices of a wider projection and the value residual folded into the kernel: the same
    bits as contiguous copies and an eager torch.lerp in front of the plain step."""
    B, H, D, N = 5, 4, 64, 2
    g = torch.Generator(device="cuda").manual_seed(8)
    rn = lambda *s: torch.randn(*s, generator=g, device="cuda").to(dtype)
    proj = rn(B, H * D + H * N + 24)                       # [k | v | something else], row width a multiple of 8
    k, v = proj[:, :H * D].view(B, H, D), proj[:, H * D:H * D + H * N].view(B, H, N)
    assert not k.is_contiguous()
    q, gate, v_first = rn(B, H, D), rn(B, (N + 5) * H), rn(B, H, N)
    mix = torch.sigmoid(torch.randn(H, generator=g, device="cuda") * 2).to(dtype)     # both lerp branches
    lds, rf = torch.zeros(H, device="cuda"), torch.linspace(0.1, 1.0, H, device="cuda")
    consts = (3.0, 2 ** -3.5, 0.125, 2 ** -3.5 / 5, 1.0)
    s0 = torch.randn(B, H, N, D, generator=g, device="cuda") * 0.3
    s1, s2 = s0.clone(), s0.clone()
    y1 = ops.decode_step(s1, q, k, v, gate, lds, rf, *consts, H, N, 7, shortcut_scale=0.4, v_first=v_first, mix=mix)
    vm = torch.lerp(v_first, v.contiguous(), mix[None, :, None])
    y2 = ops.decode_step(s2, q, k.contiguous(), vm, gate, lds, rf, *consts, H, N, 7, shortcut_scale=0.4)
    assert torch.equal(y1, y2) and torch.equal(s1, s2)
