"""The allocation-free entry point (cdssm_b200_scan_fused_fwd_noalloc) against the ordinary one.

Collected last on purpose (file name): a failure here cannot hide the results of the other tests
in a run that stops at the first failure.  The test calls the C ABI directly with buffers the
caller owns, twice in a row (the built-in scratch keeps the first call's contents), and expects
exactly the ordinary entry point's results: both run the same kernels."""
import ctypes

import numpy as np
import pytest
import torch

from util import const_args

pytestmark = pytest.mark.gpu


def _call(lib, name, t, consts, dims, extra_ws=None):
    q, k, v, g, lds, rf, h0, y, fin, tail = t
    args = [0 if x is None else x.data_ptr() for x in (q, k, v, g, lds, rf, h0, y, fin, tail)]
    if extra_ws is not None:
        args += [extra_ws.data_ptr() + (-extra_ws.data_ptr()) % 256, extra_ws.numel() - 256]
    args += [ctypes.c_float(c) for c in consts] + [ctypes.c_float(0.25)] + list(dims)
    args += [0, 0, 0, torch.cuda.current_stream().cuda_stream]          # pos0, dtype=bf16, flags
    return getattr(lib, name)(*args)


@pytest.mark.parametrize("B,H,L,D,N,C", [(2, 4, 300, 64, 2, 64), (1, 3, 200, 128, 4, 128)])
def test_noalloc_entry_matches_allocating_entry(ops, orc, B, H, L, D, N, C):
    import cdssm_b200
    lib = cdssm_b200._lib.lib()
    inp = orc.make_inputs(B, H, L, D, N=N, seed=31, bf16=True)
    dev = torch.device("cuda", 0)
    bf = lambda a: torch.from_numpy(a).to(dev).bfloat16().contiguous()
    f32 = lambda a: torch.from_numpy(a).to(dev).float().contiguous()
    h0 = f32(np.random.default_rng(2).standard_normal((B, H, N, D)).astype(np.float32))
    base = [bf(inp["q"]), bf(inp["k"]), bf(inp["v"]), bf(inp["gate_raw"]), f32(inp["log_dt_scale"]),
            f32(inp["rope_freqs"]), h0]
    outs = lambda: [torch.full((B, L, H, N), 3.0, device=dev, dtype=torch.bfloat16),
                    torch.full((B, H, N, D), 3.0, device=dev), torch.full((B, H, N, D), 3.0, device=dev)]
    consts, dims = const_args(inp["consts"]), (B, L, H, D, N, C)
    ws = torch.empty(ops.scan_fused_workspace_bytes(B, L, H, D, N, C) + 512, dtype=torch.uint8, device=dev)
    ref = outs()
    assert _call(lib, "cdssm_b200_scan_fused_fwd", base + ref, consts, dims, extra_ws=ws) == 0
    torch.cuda.synchronize()
    for attempt in range(2):                      # second call finds the first call's scratch contents
        got = outs()
        assert _call(lib, "cdssm_b200_scan_fused_fwd_noalloc", base + got, consts, dims) == 0
        torch.cuda.synchronize()
        for a, b, name in zip(got, ref, ("y", "final_state", "tail_state")):
            err = float((a.float() - b.float()).abs().max() / b.float().abs().max().clamp_min(1e-30))
            assert err <= 2.0 ** -7, (attempt, name, err)      # same kernels: in practice exactly equal
            assert torch.equal(a, b), (attempt, name)


def test_noalloc_entry_on_the_tensor_core_passes_reports_its_status(ops, orc):
    """A shape that takes the tcgen05 passes (no tail_state): their records and carries live in the built-in
    scratch, and the status word is read through the entry point made for callers without a workspace."""
    import cdssm_b200
    lib = cdssm_b200._lib.lib()
    B, H, L, D, N, C = 1, 4, 512, 128, 2, 128
    inp = orc.make_inputs(B, H, L, D, N=N, seed=32, bf16=True)
    dev = torch.device("cuda", 0)
    bf = lambda a: torch.from_numpy(a).to(dev).bfloat16().contiguous()
    f32 = lambda a: torch.from_numpy(a).to(dev).float().contiguous()
    base = [bf(inp["q"]), bf(inp["k"]), bf(inp["v"]), bf(inp["gate_raw"]), f32(inp["log_dt_scale"]),
            f32(inp["rope_freqs"]), None]
    outs = lambda: [torch.full((B, L, H, N), 3.0, device=dev, dtype=torch.bfloat16),
                    torch.full((B, H, N, D), 3.0, device=dev), None]
    consts, dims = const_args(inp["consts"]), (B, L, H, D, N, C)
    ws = torch.empty(ops.scan_fused_workspace_bytes(B, L, H, D, N, C) + 512, dtype=torch.uint8, device=dev)
    ref = outs()
    assert _call(lib, "cdssm_b200_scan_fused_fwd", base + ref, consts, dims, extra_ws=ws) == 0
    torch.cuda.synchronize()
    for attempt in range(2):
        got = outs()
        assert _call(lib, "cdssm_b200_scan_fused_fwd_noalloc", base + got, consts, dims) == 0
        status = ctypes.c_int(-1)
        assert lib.cdssm_b200_scan_fused_noalloc_status(ctypes.addressof(status),
                                                        torch.cuda.current_stream().cuda_stream) == 0
        assert status.value == 0
        assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1]), attempt


def test_noalloc_entry_refuses_sizes_beyond_its_scratch(ops):
    import cdssm_b200
    lib = cdssm_b200._lib.lib()
    limit = lib.cdssm_b200_scan_fused_noalloc_max_bytes()
    assert limit == 16 << 20
    B, H, L, D, N, C = 4, 32, 16384, 128, 2, 128
    assert ops.scan_fused_workspace_bytes(B, L, H, D, N, C) > limit
    one = torch.zeros(8, device="cuda")          # never touched: the call is refused before any launch
    t = [one] * 10
    consts = (1.0, 0.1, 0.1, 0.02, 1.0)
    assert _call(lib, "cdssm_b200_scan_fused_fwd_noalloc", t, consts, (B, L, H, D, N, C)) == -3
