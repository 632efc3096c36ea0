"""Host-side partitioning logic, on CPU: two gloo ranks hand the (Gamma, b) segment summaries to each
other and the carry composition reproduces the unsharded oracle.  (The GPU path runs the same
sharding code with the CUDA kernels in place of the oracle.)"""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
B, H, L, D, N, C = 2, 3, 320, 32, 2, 64


def _segment_summary(orc, inp, lo, hi, mask):
    """(Gamma, b) of tokens [lo, hi): product of the per-chunk decay products and the carry-out from
    a zero carry-in, computed with the oracle."""
    sl = {k: (v[:, lo:hi] if getattr(v, "ndim", 0) >= 3 else v) for k, v in inp.items()}
    _, b_seg = orc.scan_reference(sl["q"], sl["k"], sl["v"], sl["gate_raw"], sl["log_dt_scale"], sl["rope_freqs"],
                                  sl["consts"], N, C, pos0=lo, round_bf16=mask)
    A, _, _, _ = orc.dynamics(sl["gate_raw"], sl["log_dt_scale"], sl["rope_freqs"], sl["consts"], H, N,
                              pos0=lo, round_bf16=mask)
    n = hi - lo
    assert n % C == 0
    Ac = (A[..., 0::2] + 1j * A[..., 1::2]).reshape(B, n // C, C, H, N // 2)
    gam = np.ones((B, H, N // 2), np.complex64)
    for c in range(n // C):
        g = np.ones((B, H, N // 2), np.complex64)
        for t in range(C):
            g = (Ac[:, c, t] * g).astype(np.complex64)
        if mask & 4:
            g = orc.bf16_round(g.real.copy()) + 1j * orc.bf16_round(g.imag.copy())
        gam = (g * gam).astype(np.complex64)
    dec = np.empty((B, H, N), np.float32)
    dec[..., 0::2], dec[..., 1::2] = gam.real, gam.imag
    return dec, b_seg, sl


def _worker(rank, world, port, mask, out_q):
    sys.path.insert(0, ROOT)
    import oracle as orc
    import cdssm_b200.sharding as sh
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    inp = orc.make_inputs(B, H, L, D, N=N, seed=3, bf16=mask != 0)
    lo, hi = sh.segment_bounds(L, C, world)[rank]
    dec, b_seg, sl = _segment_summary(orc, inp, lo, hi, mask)
    # sequence parallelism is opt-in: an initialised default group alone means "this rank's own sequences"
    assert sh.sequence_ranks() == (0, 1)
    assert sh.sequence_ranks(sequence_parallel=True) == (rank, world)
    assert sh.sequence_ranks(group=dist.group.WORLD) == (rank, world)
    decs, outs = sh.exchange_summaries(torch.from_numpy(dec), torch.from_numpy(b_seg))
    carry_in, final = sh.compose_carries(decs, outs)
    y, fin = orc.scan_reference(sl["q"], sl["k"], sl["v"], sl["gate_raw"], sl["log_dt_scale"], sl["rope_freqs"],
                                sl["consts"], N, C, h0=carry_in[rank].numpy(), pos0=lo, round_bf16=mask)
    out_q.put((rank, y, final.numpy()))
    dist.barrier()
    dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("mask", [0, 13])
def test_two_rank_segment_handoff_matches_unsharded(orc, mask):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mask, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    inp = orc.make_inputs(B, H, L, D, N=N, seed=3, bf16=mask != 0)
    wy, wfin = orc.scan_reference(inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"],
                                  inp["rope_freqs"], inp["consts"], N, C, round_bf16=mask)
    y = np.concatenate([r[1] for r in res], 1)
    tol = 1e-5 if mask == 0 else 2.0 ** -7
    assert np.abs(y - wy).max() <= tol * np.abs(wy).max()
    assert np.abs(res[0][2] - wfin).max() <= 1e-5 * max(np.abs(wfin).max(), 1e-3)


def test_partitions():
    import cdssm_b200.sharding as sh
    assert list(sh.batch_shard(16, 4, 3)) == [12, 13, 14, 15]
    with pytest.raises(ValueError):
        sh.batch_shard(6, 4, 0)
    assert sh.segment_bounds(1000, 128, 4) == [(0, 256), (256, 512), (512, 768), (768, 1000)]
    assert sh.segment_bounds(100, 128, 3) == [(0, 100), (100, 100), (100, 100)]
    b = sh.segment_bounds(1 << 20, 128, 8)
    assert b[0] == (0, 1 << 17) and b[-1][1] == 1 << 20 and all(x[1] == y[0] for x, y in zip(b, b[1:]))


def test_compose_carries_is_the_serial_recurrence():
    import cdssm_b200.sharding as sh
    g = torch.Generator().manual_seed(0)
    S, Bq, Hq, Nq, Dq = 5, 2, 3, 4, 8
    dec = torch.randn(S, Bq, Hq, Nq, generator=g) * 0.5
    out = torch.randn(S, Bq, Hq, Nq, Dq, generator=g)
    h0 = torch.randn(Bq, Hq, Nq, Dq, generator=g)
    cin, fin = sh.compose_carries(dec, out, h0)
    s = torch.complex(h0[..., 0::2, :], h0[..., 1::2, :])
    for k in range(S):
        assert torch.allclose(torch.complex(cin[k][..., 0::2, :], cin[k][..., 1::2, :]), s, atol=1e-6)
        a = torch.complex(dec[k][..., 0::2], dec[k][..., 1::2])[..., None]
        s = a * s + torch.complex(out[k][..., 0::2, :], out[k][..., 1::2, :])
    assert torch.allclose(torch.complex(fin[..., 0::2, :], fin[..., 1::2, :]), s, atol=1e-6)


def test_sequence_ranks_without_a_process_group():
    import cdssm_b200.sharding as sh
    assert sh.sequence_ranks() == (0, 1)
    with pytest.raises(RuntimeError):
        sh.sequence_ranks(sequence_parallel=True)
