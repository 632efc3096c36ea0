"""CD-SSM language model glue around the fused scan path: prefill and cached one-token decode.

This is the caller side of the hot path (the reference's cdssm/models/{model,block}.py), written
from the behaviour of the reference so that benchmark configurations 1 (prefill) and 3 (batched
recurrent decode) can run on random-initialised weights.  Projections, norms and the LM head are
ordinary torch library calls (plumbing); the scan path itself is ``ops.scan_fused`` /
``ops.decode_step`` and the depthwise conv is ``ops.CUDAConv1dSiLUOp``.

Layer structure restated from cdssm/models/block.py:140-229, constants from
cdssm/config/model.py:38-109, initialisation from cdssm/models/init.py:13-126 and
cdssm/models/block.py:90-138.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import ops


@dataclass
class CdssmConfig:
    """The five user values of the reference config plus everything it derives from them."""
    d_model: int = 768
    n_layers: int = 12
    context_length: int = 8192
    vocab_size: int = 50257
    state_dim: int = 16

    def __post_init__(self):
        assert self.state_dim % 2 == 0
        self.d_inner = 2 * self.d_model
        self.head_dim = 64
        self.n_heads = self.d_inner // self.head_dim
        self.chunk_size = self.head_dim
        self.ssm_norm_groups = 32
        self.conv_kernel_size = 4
        self.rope_base = float(self.context_length)
        self.gating_c = math.log(self.context_length)
        self.band_fraction = 2.0 / (self.n_layers + 1)
        io_eps = 2.0 ** -7                                    # bfloat16 machine epsilon
        self.eps_norm = io_eps ** 2
        self.eps_log = io_eps ** 2
        self.adt_eps = 1.0
        self.omega_thresh = math.sqrt(io_eps)
        self.adt_delta = 16.0 * io_eps
        self.adt_smoothness = self.omega_thresh / 5.0

    @property
    def dyn_consts(self):
        return (self.gating_c, self.omega_thresh, self.adt_delta, self.adt_smoothness, self.adt_eps)


def _rms_norm(x, weight, eps):
    if x.shape[-1] % 8 == 0:
        return ops.rms_norm(x, weight, eps)           # one kernel
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * weight


class CdssmBlockParams:
    """Weights of one block, initialised like the reference (T-Fixup scaling, spectral gate biases,
    identity Q projection, shortcut and skip switched off)."""

    def __init__(self, cfg: CdssmConfig, layer_idx: int, gen: torch.Generator, device, dtype):
        N, H, di, dm = cfg.state_dim, cfg.n_heads, cfg.d_inner, cfg.d_model
        G = N + 5
        layer_scale = 1.0 / math.sqrt(2 * cfg.n_layers)
        std_in = math.sqrt(2.0 / (dm + di)) * layer_scale
        std_dyn = math.sqrt(2.0 / (di + di)) * layer_scale / math.sqrt(cfg.n_layers)
        rn = lambda *s: torch.randn(*s, generator=gen, dtype=torch.float32)
        w_in = rn(3 * di + H * N, dm) * std_in
        w_in[3 * di:] = rn(H * N, dm) * (std_in / math.sqrt(cfg.head_dim))      # V rows: small init
        w_gate = torch.cat([rn(N * H, di) * std_dyn, rn(5 * H, di) / math.sqrt(di)])
        b_gate = torch.zeros(G * H)
        ln2 = math.log(2.0)
        b_gate[N * H:(N + 1) * H] = ln2              # sel_B
        b_gate[(N + 1) * H:(N + 2) * H] = ln2        # sel_C
        b_gate[(N + 4) * H:(N + 5) * H] = ln2        # r_gate
        # spectral init: per layer a sliding log-timescale band; alpha = 1/tau, omega log-spaced
        log_range = math.log(float(cfg.context_length))
        frac = layer_idx / max(cfg.n_layers - 1, 1)
        width = cfg.band_fraction * log_range
        start = frac * (log_range - width)
        NH = N // 2
        sub = width / max(NH, 1)
        for j in range(NH):
            j0 = start + j * sub / NH
            j1 = j0 + width
            tau = torch.exp(torch.linspace(j0, j1, H))
            b_gate[j * H:(j + 1) * H] = torch.log(torch.exp(1.0 / tau) - 1 + cfg.eps_log)
            fmin, fmax = 1.0 / math.exp(j1), min(0.5, 1.0 / math.exp(j0))
            b_gate[(NH + j) * H:(NH + j + 1) * H] = torch.exp(
                torch.linspace(math.log(max(fmin, cfg.eps_log)), math.log(fmax), H))
        to = lambda t: t.to(device=device, dtype=dtype).contiguous()
        self.norm_w = to(torch.ones(dm))
        self.w_in, self.b_in = to(w_in), to(torch.zeros(3 * di + H * N))
        self.conv_w = to(rn(di, 1, 4) / 2.0)          # std 1/sqrt(kernel)
        self.conv_b = to(torch.zeros(di))
        self.w_gate, self.b_gate = to(w_gate), to(b_gate)
        self.log_dt_scale = torch.zeros(H, device=device, dtype=torch.float32)
        self.rope_freqs = (1.0 / (cfg.rope_base ** (torch.arange(H, dtype=torch.float32) / H))).to(device)
        self.w_q = to(torch.eye(di))
        self.w_readout = to(rn(di, H * N) / math.sqrt(H * N))
        self.w_out = to(rn(dm, di) * std_in)
        self.gn_w, self.gn_b = to(torch.ones(di)), to(torch.zeros(di))
        self.D = to(torch.zeros(di))
        self.v_residual_gate = torch.zeros(H, device=device, dtype=torch.float32)
        self.shortcut_scale = 0.0
        self.merge_q_and_gate_projections()


    def merge_q_and_gate_projections(self):
        """Q_proj and gate_proj read the same conv output: keep their weights as the two row blocks of ONE matrix,
        so that a decode step runs one product for both (the separate weights stay available as views)."""
        di = self.w_q.shape[0]
        self.w_qg = torch.cat([self.w_q, self.w_gate]).contiguous()
        self.b_qg = torch.cat([torch.zeros(di, device=self.b_gate.device, dtype=self.b_gate.dtype), self.b_gate])
        self.w_q, self.w_gate = self.w_qg[:di], self.w_qg[di:]

    def residual_mix(self, dtype):
        """sigmoid(v_residual_gate) in the activation dtype (block.py:167-171), computed once per value of the
        parameter instead of two small kernels per layer and token."""
        g = self.v_residual_gate
        key = (g.data_ptr(), g._version, dtype)
        if getattr(self, "_mix_key", None) != key:
            self._mix = torch.sigmoid(g).to(dtype)[None, None, :, None]
            self._mix_key = key
        return self._mix

    def load_reference(self, sd, prefix, device, dtype):
        """Take this block's weights from a reference state dict (parameter names of
        cdssm/models/block.py:35-88 under `prefix`, e.g. "blocks.3.")."""
        to = lambda name: sd[prefix + name].to(device=device, dtype=dtype).contiguous()
        f32 = lambda name: sd[prefix + name].to(device=device, dtype=torch.float32).contiguous()
        self.norm_w = to("norm.weight")
        self.w_in, self.b_in = to("in_proj.weight"), to("in_proj.bias")
        self.conv_w, self.conv_b = to("conv.weight"), to("conv.bias")
        self.w_gate, self.b_gate = to("gate_proj.weight"), to("gate_proj.bias")
        self.log_dt_scale = f32("log_dt_scale")
        self.w_q, self.w_readout, self.w_out = to("Q_proj.weight"), to("readout_proj.weight"), to("out_proj.weight")
        self.gn_w, self.gn_b = to("ssm_norm.weight"), to("ssm_norm.bias")
        self.D = to("D")
        self.v_residual_gate = f32("v_residual_gate")
        self.shortcut_scale = float(sd[prefix + "shortcut_scale"].float().item())
        self.merge_q_and_gate_projections()


class CdssmLM:
    """Embedding -> n_layers blocks -> RMSNorm -> tied LM head, inference only."""

    @classmethod
    def from_reference_checkpoint(cls, ckpt, device="cuda", dtype=torch.bfloat16):
        """Build the model from a checkpoint of the reference trainer: a dict (or the path of a torch.save'd
        dict) with "config" (the dataclass fields of cdssm/config/model.py; the derived ones are recomputed)
        and "model_state_dict" (cdssm/training/trainer.py:205-214, read like cdssm/inference/predict.py:10-30,
        including the "_orig_mod." prefix a compiled model leaves on its keys)."""
        if isinstance(ckpt, (str, bytes)) or hasattr(ckpt, "__fspath__"):
            ckpt = torch.load(ckpt, map_location="cpu", weights_only=False)
        c = ckpt["config"]
        cfg = CdssmConfig(**{k: c[k] for k in ("d_model", "n_layers", "context_length", "vocab_size", "state_dim")})
        sd = {k.replace("_orig_mod.", ""): v for k, v in ckpt["model_state_dict"].items()}
        lm = cls(cfg, device=device, dtype=dtype, seed=0)
        lm.load_reference_state_dict(sd)
        return lm

    def load_reference_state_dict(self, sd):
        self.embedding = sd["embedding.weight"].to(device=self.device, dtype=self.dtype).contiguous()
        self.final_norm_w = sd["final_norm.weight"].to(device=self.device, dtype=self.dtype).contiguous()
        for i, p in enumerate(self.blocks):
            p.load_reference(sd, f"blocks.{i}.", self.device, self.dtype)

    def __init__(self, cfg: CdssmConfig, device="cuda", dtype=torch.bfloat16, seed=0):
        self.cfg, self.device, self.dtype = cfg, torch.device(device), dtype
        gen = torch.Generator().manual_seed(seed)
        self.embedding = (torch.randn(cfg.vocab_size, cfg.d_model, generator=gen) *
                          math.sqrt(1.0 / cfg.d_model)).to(device=device, dtype=dtype)
        self.blocks = [CdssmBlockParams(cfg, i, gen, device, dtype) for i in range(cfg.n_layers)]
        self.final_norm_w = torch.ones(cfg.d_model, device=device, dtype=dtype)
        self.per_token_group_norm = False   # False = the reference's sequence-wide GroupNorm statistics

    # ------------------------------------------------------------------ one block
    def _block(self, p: CdssmBlockParams, x, v_first, pos0, cache, scan_flags):
        cfg = self.cfg
        B, L, _ = x.shape
        H, N, di = cfg.n_heads, cfg.state_dim, cfg.d_inner
        xn = _rms_norm(x, p.norm_w, cfg.eps_norm)
        if L > 1:
            # One product per consumer (row blocks of the in_proj weight are contiguous views): each output is
            # dense, so neither the conv nor the scan has to copy a column slice of a wide projection first.
            z, x_gate, K, V = (F.linear(xn, p.w_in[a:b], p.b_in[a:b]) for a, b in
                               ((0, di), (di, 2 * di), (2 * di, 3 * di), (3 * di, 3 * di + H * N)))
        else:
            z, x_gate, K, V = F.linear(xn, p.w_in, p.b_in).split([di, di, di, H * N], dim=-1)
        K = K.reshape(B, L, H, cfg.head_dim)
        V = V.reshape(B, L, H, N)
        decoding = cache is not None and "state" in cache     # a populated cache: one-token step
        mix = None
        if v_first is None:
            v_first = V.contiguous() if decoding else V     # one small copy per step; the kernels read it densely
        elif decoding:                          # the decode kernel applies the value residual itself
            mix = p.residual_mix(V.dtype)
        else:                                   # value residual across layers (block.py:167-171)
            V = torch.lerp(v_first, V, p.residual_mix(V.dtype))
        if not decoding:
            x_conv = ops.CUDAConv1dSiLUOp.apply(x_gate, p.conv_w, p.conv_b)
            if cache is not None:               # last three inputs of the causal 4-tap conv
                hist = torch.zeros(B, 3, di, device=x.device, dtype=x.dtype)
                n = min(3, L)
                hist[:, 3 - n:] = x_gate[:, L - n:]
                cache["conv"] = hist
        else:                                   # decode: one output from the cached history, shifted in place
            x_conv = ops.conv1d_silu_step(x_gate[:, 0], cache["conv"], p.conv_w, p.conv_b).unsqueeze(1)
        if decoding:                            # one product for Q and the gates; the step kernel reads the slices
            qg = F.linear(x_conv, p.w_qg, p.b_qg)
            Q, gates = qg[..., :di].unflatten(-1, (H, cfg.head_dim)), qg[..., di:]
        else:
            gates = F.linear(x_conv, p.w_gate, p.b_gate)
            Q = F.linear(x_conv, p.w_q).reshape(B, L, H, cfg.head_dim)
        if decoding:
            y = ops.decode_step(cache["state"], Q[:, 0], K[:, 0], V[:, 0], gates[:, 0], p.log_dt_scale,
                                p.rope_freqs, *cfg.dyn_consts, H, N, pos0, shortcut_scale=p.shortcut_scale,
                                v_first=None if mix is None else v_first[:, 0], mix=mix).unsqueeze(1)
        elif cache is not None:
            y, _, tail = ops.scan_fused(Q, K, V, gates, p.log_dt_scale, p.rope_freqs, *cfg.dyn_consts, H, N,
                                        cfg.chunk_size, shortcut_scale=p.shortcut_scale, pos0=pos0,
                                        return_tail_state=True)
            cache["state"] = tail
        else:
            y, _ = ops.scan_fused(Q, K, V, gates, p.log_dt_scale, p.rope_freqs, *cfg.dyn_consts, H, N,
                                  cfg.chunk_size, shortcut_scale=p.shortcut_scale, pos0=pos0, flags=scan_flags)
        y = F.linear(y.reshape(B, L, H * N), p.w_readout)
        # The reference normalises over (channels of the group) x (ALL positions of the sequence)
        # (block.py:216-222: group_norm on (B, d_inner, L)), which makes its forward non-causal.  A
        # cached decode cannot reproduce that, so the prefill/decode path - and forward() when
        # per_token_group_norm is set - takes the statistics per token instead.
        per_token = cache is not None or self.per_token_group_norm
        if (di // cfg.ssm_norm_groups) % 8 == 0 and di <= 8192:
            y = ops.groupnorm_gate(y, p.gn_w, p.gn_b, z, p.D, x_conv, cfg.ssm_norm_groups, 1e-5, per_token=per_token)
        else:
            if per_token:
                y = F.group_norm(y.float().reshape(B * L, di, 1), cfg.ssm_norm_groups, p.gn_w.float(),
                                 p.gn_b.float(), 1e-5).to(x.dtype).reshape(B, L, di)
            else:
                y = F.group_norm(y.float().transpose(1, 2), cfg.ssm_norm_groups, p.gn_w.float(), p.gn_b.float(),
                                 1e-5).to(x.dtype).transpose(1, 2)
            y = y * F.silu(z) + p.D * x_conv
        # the residual add rides in the product's epilogue
        return torch.addmm(x.reshape(B * L, -1), y.reshape(B * L, di), p.w_out.t()).reshape(B, L, -1), v_first

    # ------------------------------------------------------------------ public API
    @torch.no_grad()
    def forward(self, input_ids, scan_flags=0):
        """Prefill: (B,L) token ids -> (B,L,vocab) logits (cdssm/models/model.py:37-51)."""
        x = self.embedding[input_ids]
        v_first = None
        for p in self.blocks:
            x, v_first = self._block(p, x, v_first, 0, None, scan_flags)
        return F.linear(_rms_norm(x, self.final_norm_w, 2.0 ** -14), self.embedding)

    @torch.no_grad()
    def prefill(self, input_ids, last_only=True):
        """Prefill that also returns the decode cache: per layer the recurrent state after the last
        token (B,H,N,D) fp32 and the last three conv inputs; plus the position counter."""
        x = self.embedding[input_ids]
        caches, v_first = [], None
        for p in self.blocks:
            c = {}
            x, v_first = self._block(p, x, v_first, 0, c, 0)
            caches.append(c)
        if last_only:
            x = x[:, -1:]
        logits = F.linear(_rms_norm(x, self.final_norm_w, 2.0 ** -14), self.embedding)
        return logits, {"layers": caches, "pos": input_ids.shape[1]}

    @torch.no_grad()
    def decode(self, token_ids, cache):
        """One token per sequence: (B,) ids -> (B,vocab) logits; the cache is updated in place.
        The reference instead re-runs the whole window per token (cdssm/inference/predict.py:53-67)."""
        x = self.embedding[token_ids].unsqueeze(1)
        v_first = None
        # one position counter: the host integer, or - once a decode graph exists - the device int32 that
        # makes the step graph-replayable (see position())
        pos = cache["pos_dev"] if "pos_dev" in cache else cache["pos"]
        for p, c in zip(self.blocks, cache["layers"]):
            x, v_first = self._block(p, x, v_first, pos, c, 0)
        if "pos_dev" in cache:
            cache["pos_dev"] += 1
        else:
            cache["pos"] += 1
        return F.linear(_rms_norm(x[:, 0], self.final_norm_w, 2.0 ** -14), self.embedding)

    @staticmethod
    def position(cache):
        """Number of tokens the cache has seen (reads the device counter if a decode graph owns it)."""
        return int(cache["pos_dev"].item()) if "pos_dev" in cache else int(cache["pos"])

    def make_forward_graph(self, batch, length, scan_flags=0):
        """Capture forward() for a fixed (batch, length) as one CUDA graph: a prefill of a few thousand tokens is
        some 200 short launches per pass and otherwise bound by the host that issues them.  Returns
        (graph, ids, logits): write token ids into ``ids`` (batch, length), ``graph.replay()``, read ``logits``
        (batch, length, vocab).  The scan workspace belongs to the capture stream and stays alive with the graph."""
        dev = self.device
        ids = torch.zeros(batch, length, dtype=torch.int64, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):               # warm-up outside capture: workspaces, lazy library handles
            for _ in range(2):
                self.forward(ids, scan_flags)
        torch.cuda.current_stream(dev).wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            logits = self.forward(ids, scan_flags)
        return graph, ids, logits

    def make_decode_graph(self, cache, batch):
        """Capture one greedy decode step as a CUDA graph: static token buffer in, next tokens out,
        position in device memory.  Returns (graph, token_buffer); replay advances the cache."""
        dev = self.device
        cache["pos_dev"] = torch.tensor([cache.pop("pos")], dtype=torch.int32, device=dev)
        tok = torch.zeros(batch, dtype=torch.int64, device=dev)
        side = torch.cuda.Stream(device=dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        snapshot = [{k: v.clone() for k, v in c.items()} for c in cache["layers"]]
        with torch.cuda.stream(side):               # warm-up outside capture, then restore the cache
            for _ in range(2):
                tok.copy_(self.decode(tok, cache).argmax(-1))
        torch.cuda.current_stream(dev).wait_stream(side)
        for c, s0 in zip(cache["layers"], snapshot):
            for k in c:
                c[k].copy_(s0[k])
        cache["pos_dev"] -= 2
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            tok.copy_(self.decode(tok, cache).argmax(-1))
        return graph, tok
