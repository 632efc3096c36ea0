"""Benchmark of the fused CD-SSM scan (the scan-kernel sweep configuration).

    python bench.py --gpus N --steps K --warmup W            # this implementation
    python bench.py --impl reference ...                     # the CPU restatement, timed

One step = one pass of the fused scan path over the whole synthetic batch.  At N > 1 the batch
is split over the ranks (strong scaling, no data-path collective).  Prints ONE JSON line.
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {  # the scan-kernel sweep: bf16 q/k/v, fp32 state, seed 2
    "cfg2_L4096": dict(B=16, H=32, D=128, N=2, C=128, L=4096, seed=2),
    "cfg2_L16384": dict(B=16, H=32, D=128, N=2, C=128, L=16384, seed=2),
    "cfg2_L65536": dict(B=16, H=32, D=128, N=2, C=128, L=65536, seed=2),
    "cfg0": dict(B=2, H=4, D=64, N=2, C=64, L=512, seed=0),
    # long-context: one sequence per head, split into contiguous segments (over GPUs and within one)
    # whole-model workloads (random-initialised LM; library GEMMs around the scan path)
    "cfg1_prefill": dict(lm=dict(d_model=768, n_layers=12, vocab_size=32000, state_dim=2, context_length=2048),
                         B=8, L=2048, seed=1, H=24, D=64, N=2, C=64),
    "cfg3_decode": dict(lm=dict(d_model=2048, n_layers=24, vocab_size=32000, state_dim=2, context_length=4608),
                        B=256, L=4096, decode_steps=512, seed=3, H=64, D=64, N=2, C=64),
    # the one-token decode kernel alone: cfg3's per-layer shapes, graph replay over 24 layers' states
    "decode_kernel": dict(decode_kernel=True, B=256, H=64, D=64, N=2, layers=24, L=4608, seed=3),
    "cfg4_L1M": dict(B=1, H=32, D=128, N=2, C=128, L=1 << 20, seed=4, seq_parallel=True, segments=16),
}
DEFAULT_WORKLOAD = "cfg2_L65536"


def algorithmic_bytes(w, elem=2):
    """q, k read; v read; the N+5 per-token gate values read; y written (per token-head)."""
    per_th = (2 * w["D"] + w["N"] + (w["N"] + 5) + w["N"]) * elem
    return per_th * w["B"] * w["L"] * w["H"]


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# ------------------------------------------------------------------ synthetic inputs
def head_params(w):
    import torch
    g = torch.Generator().manual_seed(w["seed"])
    H, NH = w["H"], w["N"] // 2
    alpha_raw = -1.0 + 0.5 * torch.randn(NH, H, generator=g)
    omega = (torch.rand(NH, H, generator=g) * 2 - 1) * math.pi
    log_dt_scale = 0.5 * torch.randn(H, generator=g)
    return alpha_raw, omega, log_dt_scale


def make_batch_slice(w, b, device, dtype):
    """Inputs of batch element b, drawn in the configuration's (H,L,.) shapes from a generator
    seeded by (seed, b), so a shard does not depend on how many GPUs share the batch; then
    permuted to the operator layout (L,H,.)."""
    import torch
    H, L, D, N = w["H"], w["L"], w["D"], w["N"]
    g = torch.Generator(device=device).manual_seed(w["seed"] * 1000003 + b)
    rn = lambda *s: torch.randn(*s, generator=g, device=device, dtype=torch.float32)
    q = torch.nn.functional.normalize(rn(H, L, D), dim=-1).transpose(0, 1).to(dtype).contiguous()
    k = torch.nn.functional.normalize(rn(H, L, D), dim=-1).transpose(0, 1).to(dtype).contiguous()
    v = rn(H, L, N).transpose(0, 1).to(dtype).contiguous()
    beta_raw, sel_B, sel_C, sel_dt, r_gate = [rn(H, L).t() for _ in range(5)]
    alpha_raw, omega, _ = head_params(w)
    segs = [alpha_raw[j].to(device).expand(L, H) for j in range(N // 2)]
    segs += [omega[j].to(device).expand(L, H) for j in range(N // 2)]
    segs += [sel_B, sel_C, sel_dt, beta_raw, r_gate]
    gate = torch.cat(segs, dim=-1).to(dtype).contiguous()
    return q, k, v, gate


def consts_for(w):
    eps = 2.0 ** -7
    thr = math.sqrt(eps)
    return (math.log(w["L"]), thr, 16.0 * eps, thr / 5.0, 1.0)


def parity_spot_check(w, q, k, v, gate, lds, rope, consts, y, heads=4, tokens=4096):
    """Untimed: batch row 0, the first `heads` heads and the first `tokens` positions of the benchmarked output
    against the CPU oracle with the reference's rounding (the scan is causal and heads are independent, so the
    slice is a complete problem of its own).  Returns max|dy| / max|y_ref|."""
    import numpy as np
    import oracle
    oracle.build()
    oracle.set_threads(cpu_threads())
    H, N = w["H"], w["N"]
    T, hs = min(tokens, q.shape[1]), min(heads, H)
    f = lambda t: t.float().cpu().numpy()
    segs = gate.shape[-1] // H
    g = gate[0:1, :T].reshape(1, T, segs, H)[..., :hs].reshape(1, T, segs * hs)
    cd = dict(zip(("gating_c", "omega_thresh", "adt_delta", "adt_smoothness", "adt_eps"), consts))
    ref, _ = oracle.scan_reference(f(q[0:1, :T, :hs]), f(k[0:1, :T, :hs]), f(v[0:1, :T, :hs]), f(g), f(lds[:hs]),
                                   f(rope[:hs]), cd, N, w["C"], round_bf16=oracle.ROUND_REFERENCE)
    got = f(y[0:1, :T, :hs])
    return float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))


def reference_gpu_leg(w, q, k, v, gate, lds, rope, consts, ops, tokens=4096, reps=3):
    """Context figure, outside the product path: the reference's OWN kernels (compiled unmodified for sm_100
    into oracle/_ref by oracle/build_ref.py) and its glue, on the first `tokens` positions of the benchmark
    inputs, CUDA-event timed, beside this library's fused call on the same slice.  None if the extension
    was not built."""
    import torch
    from oracle.build_ref import load_ref
    from oracle.ref_pipeline import reference_forward
    ref = load_ref()
    if ref is None:
        return None
    H, N, C = w["H"], w["N"], w["C"]
    T = min(tokens, q.shape[1])
    sl = [t[:, :T].contiguous() for t in (q, k, v, gate)]

    def timed(fn):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    ref_ms = timed(lambda: reference_forward(ref, *sl, lds, rope, consts, H, N, C))
    our_ms = timed(lambda: ops.scan_fused(*sl, lds, rope, *consts, H, N, C))
    return {"ms": ref_ms, "this_library_ms": our_ms,
            "workload": f"B={q.shape[0]} H={H} L={T} head_dim={w['D']} (first {T} tokens of the benchmark inputs)",
            "what": "dynamics_fused + normalize (torch for head_dim 128) + intra_chunk_scan + inter_chunk_scan + "
                    "exact_correction kernels of the reference recompiled for sm_100, with the reference's torch glue"}


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc, self.index = [], None, index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")] + [time.time()])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.th.join(timeout=2)

    def summary(self, t0=None, t1=None):
        rows = [r for r in self.rows if len(r) >= 7 and r[0].isdigit()]
        if t0 is not None:   # prefer the samples taken while the timed regions ran
            inside = [r for r in rows if t0 <= r[-1] <= t1 + 0.2]
            rows = inside or rows
        self.rows = rows
        sm = sorted(int(r[0]) for r in rows)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        mx = max(int(r[1]) for r in self.rows if len(r) >= 6 and r[1].isdigit())
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": mx, "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------ CPU baseline (oracle port)
def cpu_sample_workload(w):
    """A bounded slice of the workload with the same per-token work: one
    batch element, all heads, at most 16384 positions (about 0.5 M token-heads per step)."""
    s = dict(w)
    s["B"] = 1
    s["L"] = min(w["L"], 16384)
    return s


def run_cpu_oracle(w, steps, warmup):
    """Time the CPU restatement of the reference path (oracle/cdssm_oracle.c, all-bf16 rounding
    like the reference) on a bounded sample.  Returns (tokens/s, seconds per step, sample dict)."""
    import numpy as np
    import oracle
    oracle.build()
    # a launcher may have exported OMP_NUM_THREADS=1: ask for the host threads this process may use and
    # report the team size the library really got
    team = oracle.set_threads(cpu_threads())
    s = cpu_sample_workload(w)
    inp = oracle.make_inputs(s["B"], s["H"], s["L"], s["D"], N=s["N"], seed=s["seed"], bf16=True,
                             context_length=w["L"])
    args = (inp["q"], inp["k"], inp["v"], inp["gate_raw"], inp["log_dt_scale"], inp["rope_freqs"],
            inp["consts"], s["N"], s["C"])
    for _ in range(warmup):
        oracle.scan_reference(*args, round_bf16=oracle.ROUND_REFERENCE)
    t0 = time.perf_counter()
    for _ in range(steps):
        y, _ = oracle.scan_reference(*args, round_bf16=oracle.ROUND_REFERENCE)
    dt = (time.perf_counter() - t0) / steps
    # tokens/s of the FULL workload's definition (a token = one position across all H heads):
    # the sample has H_s of H heads, so scale token-heads to tokens of the full head count
    tok_heads_per_s = s["B"] * s["L"] * s["H"] / dt
    return tok_heads_per_s / w["H"], dt, s, team


def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def reference_arm(args, w, rank):
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    tps, dt, s, cores = run_cpu_oracle(w, steps, warmup)
    sample = (f"B={s['B']} H={s['H']} L={s['L']} of the workload's B={w['B']} H={w['H']} L={w['L']} "
              f"(same D, N, C); tokens/s = token-heads/s / {w['H']} heads")
    line = {"impl": "reference", "metric": "scan_tokens_per_s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": dt * 1e3,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": workload_config(args.workload, w),
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0,
            "note": "the reference has no CPU implementation (cdssm/ops.py imports its CUDA extension only); "
                    "this times the C restatement of its kernels with OpenMP over all host threads"}
    print(json.dumps(line))


def workload_config(name, w):
    return {"workload": f"{name}: fused CD-SSM scan, B={w['B']} H={w['H']} head_dim={w['D']} state_dim={w['N']} "
                        f"chunk={w['C']} L={w['L']}, bf16 q/k/v/gates, fp32 state, seed {w['seed']}",
            "l2": "inputs (>= 1 GB per GPU) are larger than the 126 MB L2",
            "layout": "operator layout (B,L,H,.), rope_freqs = L^(-h/H), constants from context_length = L"}


# ------------------------------------------------------------------ whole-model workloads
def lm_arm(args, w, rank, world, local_rank):
    """cfg1: prefill tokens/s of the 12-layer LM; cfg3: greedy decode tokens/s after a 4096-token
    prefill.  Batch-sharded over ranks (replicas, no communication)."""
    import torch
    from cdssm_b200.model import CdssmConfig, CdssmLM
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    cfg = CdssmConfig(**w["lm"])
    lm = CdssmLM(cfg, device=dev, dtype=torch.bfloat16, seed=w["seed"])
    Bl = w["B"] // world
    g = torch.Generator().manual_seed(w["seed"] * 7919 + rank)
    ids = torch.randint(0, cfg.vocab_size, (Bl, w["L"]), generator=g)
    decode = "decode_steps" in w

    def sync():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        sync()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    with ClockSampler(local_rank) as clocks:
        t_begin = time.time()
        if not decode:
            hids = ids.pin_memory()
            last = torch.empty(Bl, cfg.vocab_size, dtype=torch.bfloat16).pin_memory()

            rows = min(Bl, 8)
            if args.no_graph:
                def step():      # end to end: ids from pinned host memory, last-position logits back
                    d = hids.to(dev, non_blocking=True)
                    for b0 in range(0, Bl, rows):
                        last[b0:b0 + rows].copy_(lm.forward(d[b0:b0 + rows])[:, -1], non_blocking=True)
            else:
                # the forward pass of a (rows, L) slice captured once as a CUDA graph and replayed per slice
                fgraph, gids, glogits = lm.make_forward_graph(rows, w["L"])

                def step():
                    for b0 in range(0, Bl, rows):
                        gids.copy_(hids[b0:b0 + rows], non_blocking=True)
                        fgraph.replay()
                        last[b0:b0 + rows].copy_(glogits[:, -1], non_blocking=True)

            for _ in range(args.warmup):
                step()
            ms_step = timed(step, args.steps) / args.steps
            tokens, launches = w["B"] * w["L"], None
            h2d, d2h = ids.numel() * 8 * world, last.numel() * 2 * world
            # share of the fused scan path in the step: the same scan_fused calls (4 rows x L tokens, one per
            # layer and slice) on random tensors of the model's shapes, timed alone
            from cdssm_b200 import ops
            Hh, Nn, Dd = cfg.n_heads, cfg.state_dim, cfg.head_dim
            rb = rows
            sq, sk = (torch.randn(rb, w["L"], Hh, Dd, device=dev).bfloat16() for _ in range(2))
            sv = torch.randn(rb, w["L"], Hh, Nn, device=dev).bfloat16()
            sg = torch.randn(rb, w["L"], (Nn + 5) * Hh, device=dev).bfloat16()
            p0 = lm.blocks[0]

            def scans():
                for _ in range(cfg.n_layers * ((Bl + rb - 1) // rb)):
                    ops.scan_fused(sq, sk, sv, sg, p0.log_dt_scale, p0.rope_freqs, *cfg.dyn_consts, Hh, Nn, cfg.chunk_size)

            scans()
            scan_ms = timed(scans, args.steps) / args.steps
            scan_share = {"scan_ms_per_step": scan_ms, "share": scan_ms / ms_step,
                          "what": f"{cfg.n_layers * ((Bl + rb - 1) // rb)} scan_fused calls of ({rb},{w['L']},{Hh},{Dd}) per step, "
                                  "timed alone on random inputs (tensor-core passes: head_dim 64, H a multiple of 4)"}
        else:
            dids = ids.to(dev)
            caches = []
            lm.prefill(dids[:min(Bl, 16), :256])    # warm-up of the library handles before the prefill is timed
            torch.cuda.synchronize()
            p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            p0.record()
            for b0 in range(0, Bl, 16):             # prefill in slices: activations of 16 x 4096 tokens
                logits, c = lm.prefill(dids[b0:b0 + 16])
                caches.append((logits[:, -1].argmax(-1), c))
            p1.record()
            torch.cuda.synchronize()
            prefill_ms = p0.elapsed_time(p1)
            tok = torch.cat([c[0] for c in caches])
            cache = {"pos": w["L"], "layers": [
                {k: torch.cat([c[1]["layers"][i][k] for c in caches]) for k in ("state", "conv")}
                for i in range(cfg.n_layers)]}
            del caches
            htok = torch.empty(Bl, dtype=torch.int64).pin_memory()
            graph, buf = lm.make_decode_graph(cache, Bl)     # one captured decode step, replayed
            buf.copy_(tok)

            def step():      # one greedy token for every sequence; the token ids go back to the host
                graph.replay()
                htok.copy_(buf, non_blocking=True)

            for _ in range(args.warmup):
                step()
            n = max(args.steps, 8)
            ms_step = timed(step, n) / n
            args.steps = n
            tokens = w["B"]
            h2d, d2h = 0, Bl * 8 * world
        t_end = time.time()
    if rank == 0:
        val = tokens / (ms_step / 1e3)
        H, N, D = cfg.n_heads, cfg.state_dim, cfg.head_dim
        line = {"metric": "decode_tokens_per_s" if decode else "prefill_tokens_per_s", "value": val,
                "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
                "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"{args.workload}: CD-SSM LM d_model={cfg.d_model} layers={cfg.n_layers} "
                                       f"heads={H} (reference-derived, d_inner/64) state_dim={N} vocab={cfg.vocab_size} "
                                       f"B={w['B']} L={w['L']}" + (f", {w['decode_steps']}-step greedy decode measured per step"
                                                                  if decode else ", random token ids, forward pass of up to 8 rows at a time "
                                                                  + ("issued eagerly" if args.no_graph else "replayed from one CUDA graph")),
                           "l2": "weights + activations per step exceed the 126 MB L2"},
                "clocks": clocks.summary(t_begin, t_end),
                "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "note": "the timed step already starts from host token ids / ends with host results"},
                "gpu_launches": args.steps * cfg.n_layers * (2 if decode else 4),
                "roofline": None}
        if not decode:
            line["scan_share"] = scan_share
        if decode:
            line["prefill"] = {"ms": prefill_ms, "tokens_per_s": Bl * w["L"] / (prefill_ms / 1e3) * world,
                               "what": f"the {w['L']}-token prefill that fills the decode cache, {Bl} sequences in slices "
                                       "of 16, issued eagerly, once (rank 0's time)"}
            per_bh = 2 * N * D * 4 + 2 * D * 2 + (3 * N + 5) * 2
            line["decode_state_bytes_per_step"] = cfg.n_layers * w["B"] * H * per_bh / world
        print(json.dumps(line))
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def decode_kernel_arm(args, w, local_rank):
    """cdssm_b200_decode_step alone at cfg3's per-layer shapes: one CUDA graph holds one launch per layer over 24
    separate (B,H,N,D) fp32 states (201 MB, more than the L2), replayed; reports microseconds per launch and
    the fraction of the HBM roofline against the 1302 algorithmic bytes per (batch, head).  `floor` is the same
    harness around a plain in-place torch kernel over the same states (two thirds of the bytes): what a launch
    of this size costs with no arithmetic at all."""
    import torch
    from cdssm_b200 import ops
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    B, H, D, N, layers = w["B"], w["H"], w["D"], w["N"], w["layers"]
    g = torch.Generator(device=dev).manual_seed(w["seed"])
    rn = lambda *s: torch.randn(*s, generator=g, device=dev)
    q, k = rn(B, H, D).bfloat16(), rn(B, H, D).bfloat16()
    v, gate = rn(B, H, N).bfloat16(), rn(B, (N + 5) * H).bfloat16()
    lds = torch.zeros(H, device=dev)
    rope = (1.0 / (float(w["L"]) ** (torch.arange(H, dtype=torch.float32) / H))).to(dev)
    consts = consts_for(w)
    y = torch.empty(B, H, N, device=dev, dtype=torch.bfloat16)
    states = [rn(B, H, N, D) * 0.1 for _ in range(layers)]

    def replayed(fn, reps):
        for s in states:
            fn(s)
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            for s in states:
                fn(s)
        for _ in range(max(3, args.warmup)):
            gr.replay()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            gr.replay()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps / layers * 1e3      # microseconds per launch

    reps = max(20, args.steps)
    with ClockSampler(local_rank) as clocks:
        t0 = time.time()
        us = replayed(lambda s: ops.decode_step(s, q, k, v, gate, lds, rope, *consts, H, N, 4096, out=y), reps)
        floor_us = replayed(lambda s: s.mul_(1.0), reps)
        # the step that reproduces the reference's chunked scan: local state and correction per (batch, head) are
        # read and written every token (the carry and the chunk decay only change at chunk boundaries)
        rstates = {id(s): ops.reference_decode_state(s) for s in states}
        ref_us = replayed(lambda s: ops.decode_step_reference(rstates[id(s)], q, k, v, gate, lds, rope, *consts, H, N,
                                                              D, 4096 + 17, out=y), reps)
        t1 = time.time()
    per_bh = 2 * N * D * 4 + 2 * D * 2 + (3 * N + 5) * 2
    abytes = B * H * per_bh
    peak, peak_kind = peaks()
    achieved = abytes / (us * 1e-6) / 1e9
    line = {"metric": "decode_kernel_us_per_layer", "value": us, "unit": "us", "n_gpus": 1, "steps": reps,
            "warmup": max(3, args.warmup), "ms_per_step": us * layers / 1e3, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32 state, bf16 activations", "data": "synthetic",
            "config": {"workload": f"decode_kernel: one-token decode step, B={B} H={H} head_dim={D} state_dim={N}, "
                                   f"{layers} layers' states ({layers * B * H * N * D * 4 / 1e6:.0f} MB) per graph replay",
                       "l2": "the states of one replay exceed the 126 MB L2"},
            "clocks": clocks.summary(t0, t1), "e2e": None, "gpu_launches": reps * layers,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": None, "peak_kind": peak_kind, "kernel": "decode_step_kernel<bf16, 8>",
                         "algorithmic_bytes_per_launch": abytes},
            "floor": {"us": floor_us, "bytes": 2 * B * H * N * D * 4,
                      "what": "in-place torch elementwise kernel over the same states in the same replay harness"},
            "reference_compatible_step": {
                "us": ref_us, "bytes": B * H * (per_bh + 2 * N * D * 4),
                "frac": B * H * (per_bh + 2 * N * D * 4) / (ref_us * 1e-6) / 1e9 / peak,
                "what": "decode_step_reference inside a chunk: local state + correction read and written per token"}}
    print(json.dumps(line))


# ------------------------------------------------------------------ the GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--segments", type=int, default=0, help="cfg4: segments per sequence over all GPUs (default: the workload's)")
    ap.add_argument("--no-graph", action="store_true", help="cfg1_prefill: issue the forward pass eagerly instead of replaying a CUDA graph")
    ap.add_argument("--flags", type=int, default=0, help="scan_fused flags (1 = the CUDA-core kernels instead of the tensor-core passes, 4096 = float32 transition)")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        reference_arm(args, w, rank)
        return
    if args.warmup < 3:
        args.warmup = 3
    if "lm" in w:
        return lm_arm(args, w, rank, world, local_rank)
    if w.get("decode_kernel"):
        if rank == 0:
            decode_kernel_arm(args, w, local_rank)
        return

    import torch
    import cdssm_b200
    from cdssm_b200 import ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the scan path has no CPU fallback")
    cdssm_b200._lib.lib()
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    dt = torch.bfloat16
    H, N, C, L, D = w["H"], w["N"], w["C"], w["L"], w["D"]
    seq_par = bool(w.get("seq_parallel"))
    nseg = max(1, (args.segments or w.get("segments", 1)) // world)   # segments per rank
    if seq_par:
        # rank r holds tokens [r*L/world, (r+1)*L/world) of every sequence; the data are drawn in 8
        # fixed pieces so that they do not depend on the number of GPUs
        pieces = 8
        if pieces % world:
            raise SystemExit(f"{pieces} sequence pieces do not split over {world} ranks")
        wp = dict(w, L=L // pieces)
        parts = [make_batch_slice(wp, 1000 + i, dev, dt) for i in range(rank * pieces // world, (rank + 1) * pieces // world)]
        q, k, v, gate = (torch.cat([p[i] for p in parts], 0).unsqueeze(0).contiguous() for i in range(4))
        Bl, Ll = 1, L // world
    else:
        if w["B"] % world:
            raise SystemExit(f"batch {w['B']} does not split over {world} ranks")
        Bl, Ll = w["B"] // world, L
        mine = range(rank * Bl, (rank + 1) * Bl)      # contiguous batch shard, no data-path collective
        parts = [make_batch_slice(w, b, dev, dt) for b in mine]
        q, k, v, gate = (torch.stack([p[i] for p in parts]) for i in range(4))
    del parts
    _, _, lds = head_params(w)
    lds = lds.to(dev)
    rope = (1.0 / (float(L) ** (torch.arange(H, dtype=torch.float32) / H))).to(dev)
    consts = consts_for(w)
    y = torch.empty(Bl, Ll, H, N, dtype=dt, device=dev)
    # the library takes its tcgen05/TMA passes by itself for these shapes unless another path is asked for
    tc_shapes = N == 2 and D == C and D in (64, 128) and H % 4 == 0
    uses_wa = bool(args.flags & 128) or (not (args.flags & (1 | 32)) and tc_shapes)

    def step():
        if seq_par:
            return ops.scan_fused_long(q, k, v, gate, lds, rope, *consts, H, N, C, segments=nseg, sequence_parallel=world > 1, flags=args.flags)
        return ops.scan_fused(q, k, v, gate, lds, rope, *consts, H, N, C, flags=args.flags, out=y)

    def sync_all():
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()

    def timed(fn, n):
        sync_all()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        sync_all()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if dist is not None:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    with ClockSampler(local_rank) as clocks:
        for _ in range(args.warmup):
            step()
        t_begin = time.time()
        ms_total = timed(step, args.steps)
        # end to end: pinned host inputs -> device -> scan -> result back on the host, every step
        e2e = None
        if not args.no_e2e:
            def pinned_copy(t):
                h = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
                h.copy_(t)
                return h

            hq, hk, hv, hg = (pinned_copy(t) for t in (q, k, v, gate))
            hy = torch.empty(y.shape, dtype=dt, pin_memory=True)
            dq, dk, dv, dg = (torch.empty_like(t) for t in (q, k, v, gate))

            def e2e_step():
                dq.copy_(hq, non_blocking=True)
                dk.copy_(hk, non_blocking=True)
                dv.copy_(hv, non_blocking=True)
                dg.copy_(hg, non_blocking=True)
                if seq_par:
                    out, _ = ops.scan_fused_long(dq, dk, dv, dg, lds, rope, *consts, H, N, C,
                                                 segments=nseg, sequence_parallel=world > 1, flags=args.flags)
                else:
                    out, _ = ops.scan_fused(dq, dk, dv, dg, lds, rope, *consts, H, N, C, flags=args.flags, out=y)
                hy.copy_(out, non_blocking=True)

            e2e_steps = max(2, min(args.steps, 5))
            e2e_step()
            e2e_ms = timed(e2e_step, e2e_steps)
            h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hg)) * world
            d2h = hy.numel() * hy.element_size() * world
            e2e = {"value": w["B"] * L / (e2e_ms / e2e_steps / 1e3), "unit": "tokens/s",
                   "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                   "ms_per_step": e2e_ms / e2e_steps}
        extra = {}
        if seq_par:
            tm = {}
            ops.scan_fused_long(q, k, v, gate, lds, rope, *consts, H, N, C,
                                segments=nseg, sequence_parallel=world > 1, flags=args.flags, timings=tm)
            t3 = torch.tensor([tm["summary_ms"], tm["handoff_ms"], tm["scan_ms"]], device=dev)
            if dist is not None:
                dist.all_reduce(t3, op=dist.ReduceOp.MAX)
            extra["segment_passes_ms"] = {"summary": float(t3[0]), "exposed_handoff": float(t3[1]), "scan": float(t3[2])}
        elif uses_wa:
            # the dominant kernel: the output pass, timed as a call that reuses the local results already in the
            # workspace (records pre-pass + carry pass + output pass; the first two are a few percent of it)
            def output_step():
                return ops.scan_fused(q, k, v, gate, lds, rope, *consts, H, N, C, flags=args.flags | ops.REUSE_LOCAL, out=y)
            output_step()
            extra["output_call_ms"] = timed(output_step, args.steps) / args.steps
        else:
            # the dominant kernel alone: the output pass = whole step minus (local pass + carry pass)
            def summary_step():
                return ops.scan_summary(k, v, gate, lds, rope, *consts, H, N, C)
            summary_step()
            extra["summary_ms"] = timed(summary_step, args.steps) / args.steps
        t_end = time.time()
        # untimed: how much of the output is finite.  At 2^20 tokens the reference's own arithmetic (bfloat16 A_bar,
        # carry without erasure) overflows on some heads; ops.FP32_DECAY (--flags 4096) is the bounded variant.
        out_now = step()[0]
        torch.cuda.synchronize()
        fin_cnt = torch.stack([torch.isfinite(out_now.float()).sum(), torch.tensor(out_now.numel(), device=dev)]).double()
        if dist is not None:
            dist.all_reduce(fin_cnt)
        finite_fraction = float(fin_cnt[0] / fin_cnt[1])
        del out_now
        parity_err = None
        if rank == 0 and not seq_par:
            step()
            torch.cuda.synchronize()
            parity_err = parity_spot_check(w, q, k, v, gate, lds, rope, consts, y)
    ms_step = ms_total / args.steps
    tokens = w["B"] * L
    scaling = "strong"
    if rank == 0:
        peak, peak_kind = peaks()
        abytes = algorithmic_bytes(w) / world                       # per GPU per step
        achieved = abytes / (ms_step / 1e3) / 1e9
        line = {"metric": "scan_tokens_per_s", "value": tokens / (ms_step / 1e3), "unit": "tokens/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": workload_config(args.workload, w),
                "clocks": clocks.summary(t_begin, t_end), "e2e": e2e,
                "gpu_launches": (4 if uses_wa else 3) * args.steps,
                "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                             "frac": achieved / peak, "traffic": None, "peak_kind": peak_kind,
                             "kernel": ("the whole step (wa_dynamics + scan_wa local pass + scan_carry + scan_wa output "
                                        "pass)" if uses_wa else
                                        "the whole step (scan_walk local pass + scan_carry + scan_walk output pass)"),
                             "algorithmic_bytes_per_launch": abytes}}
        if "output_call_ms" in extra:
            out_ms = extra["output_call_ms"]
            line["roofline"]["dominant_kernel"] = {
                "name": "wa::scan_wa_kernel<D, true> (output pass)",
                "ms": out_ms,
                "achieved": abytes / (out_ms / 1e3) / 1e9, "frac": abytes / (out_ms / 1e3) / 1e9 / peak,
                "how": "a call that reuses the local pass in the workspace (records pre-pass + carry pass + output "
                       "pass), CUDA-event timed; algorithmic bytes of the whole step"}
            # Streams of the four launches per token-head (bf16): pre-pass reads gates + v and writes a 16-byte
            # record; local pass reads k + record; output pass reads q, k + record and writes y.  The records are
            # re-read from HBM once they no longer fit the 126 MB L2 (they do at cfg2 L=4096: 33 MB).
            th = w["B"] * L * H / world
            rec_bytes = 16 * th
            rec_reads = 2 * rec_bytes if rec_bytes > 100e6 else 0.0
            streams = ((N + 5) + N) * 2 * th + rec_bytes + D * 2 * th + 2 * D * 2 * th + N * 2 * th + rec_reads
            line["roofline"]["traffic"] = streams
            line["roofline"]["traffic_how"] = ("sum of the kernels' HBM streams (gates, v, 16-byte records written once and "
                                               "read twice unless they fit L2, k twice, q once, y); agrees with the ncu "
                                               "dram byte counts of the same kernels at cfg2 L=4096 and L=16384 to a few "
                                               "percent")
        if "summary_ms" in extra:
            out_ms = ms_step - extra["summary_ms"]
            line["roofline"]["dominant_kernel"] = {
                "name": "scan_walk_kernel<bf16,16,true> (output pass)", "ms": out_ms,
                "achieved": abytes / (out_ms / 1e3) / 1e9, "frac": abytes / (out_ms / 1e3) / 1e9 / peak,
                "how": "step time minus the time of local pass + carry pass (scan_summary), both CUDA-event timed"}
            line["roofline"]["traffic"] = 1.55 * abytes
            line["roofline"]["traffic_how"] = ("dram bytes read+written per step from an ncu capture of the CUDA-core "
                                               "kernels at cfg2 L=4096, scaled by tokens")
        if "segment_passes_ms" in extra:
            line["segment_passes_ms"] = extra["segment_passes_ms"]
        line["output_finite_fraction"] = finite_fraction
        if not args.no_cpu_baseline and world == 1 and not seq_par:
            try:
                rg = reference_gpu_leg(w, q, k, v, gate, lds, rope, consts, ops)
            except Exception as e:   # context only: never fail the benchmark line over it
                rg = {"unavailable": f"{type(e).__name__}: {e}"[:200]}
            if rg is not None:
                line["reference_gpu"] = rg
        if parity_err is not None:
            line["parity_err"] = parity_err
            line["parity_how"] = ("batch row 0, heads 0-3, first 4096 tokens of the benchmarked y against the CPU oracle "
                                  "with the reference's bf16 rounding; max|dy| / max|y|, bound 2e-2")
        if not args.no_cpu_baseline and world == 1:
            tps, dt_s, s, team = run_cpu_oracle(w, 5, 1)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": team, "kind": "port",
                                    "sample": f"B={s['B']} H={s['H']} L={s['L']} slice, {dt_s * 1e3:.0f} ms per pass; "
                                              "C restatement of the reference kernels (the reference has no CPU path)"}
        print(json.dumps(line))
        if parity_err is not None and not parity_err <= 2e-2:
            raise SystemExit(f"parity spot check failed: {parity_err:.4g} > 2e-2")
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
