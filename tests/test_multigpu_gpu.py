"""Two ranks, one GPU each (NCCL over NVLink, NVLS off): batch sharding is bit-identical to one GPU,
sequence-segment sharding agrees within fp32 re-association.  Skipped with fewer than two GPUs."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
B, H, L, D, N, C = 4, 4, 1024, 128, 2, 128


def _worker(rank, world, port, q_out):
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch.distributed as dist
    import oracle as orc
    from cdssm_b200 import ops, sharding
    from util import const_args
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world, device_id=dev)
    inp = orc.make_inputs(B, H, L, D, N=N, seed=5, bf16=True)
    t = lambda a, dt: torch.from_numpy(a).to(dev).to(dt)
    full = [t(inp[n], torch.bfloat16) for n in ("q", "k", "v", "gate_raw")]
    lds, rf = t(inp["log_dt_scale"], torch.float32), t(inp["rope_freqs"], torch.float32)
    consts = const_args(inp["consts"])
    # (a) batch shard
    mine = sharding.batch_shard(B, world, rank)
    sl = [x[mine.start:mine.stop].contiguous() for x in full]
    y_b, f_b = ops.scan_fused(*sl, lds, rf, *consts, H, N, C)
    # (b) sequence shard: rank r holds tokens [r*L/world, (r+1)*L/world)
    lo, hi = rank * L // world, (rank + 1) * L // world
    seg = [x[:, lo:hi].contiguous() for x in full]
    tm = {}
    y_s, f_s = ops.scan_fused_long(*seg, lds, rf, *consts, H, N, C, segments=2, sequence_parallel=True, timings=tm)
    torch.cuda.synchronize()
    q_out.put((rank, y_b.float().cpu().numpy(), f_b.cpu().numpy(), y_s.float().cpu().numpy(), f_s.cpu().numpy(), tm))
    dist.barrier()
    dist.destroy_process_group()


def test_two_gpu_batch_and_sequence_sharding(ops, orc):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=300) for _ in procs], key=lambda r: r[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    from util import const_args, to_dev, to_np
    inp = orc.make_inputs(B, H, L, D, N=N, seed=5, bf16=True)
    d = lambda x: to_dev(x, torch.bfloat16)
    f = lambda x: to_dev(x, torch.float32)
    y1, f1 = ops.scan_fused(d(inp["q"]), d(inp["k"]), d(inp["v"]), d(inp["gate_raw"]), f(inp["log_dt_scale"]),
                            f(inp["rope_freqs"]), *const_args(inp["consts"]), H, N, C)
    y1, f1 = to_np(y1), to_np(f1)
    yb = np.concatenate([r[1] for r in res], 0)
    fb = np.concatenate([r[2] for r in res], 0)
    assert np.array_equal(yb, y1) and np.array_equal(fb, f1)           # independent units: bit-identical
    ys = np.concatenate([r[3] for r in res], 1)
    assert np.abs(ys - y1).max() <= 2.0 ** -7 * np.abs(y1).max()
    assert np.abs(res[1][4] - f1).max() <= 1e-5 * max(np.abs(f1).max(), 1e-3)
    assert all(r[5]["handoff_ms"] >= 0 for r in res)
