"""The reference's scan path run with the reference's OWN kernels (oracle/_ref, built by build_ref.py).

TEST AND BENCHMARK INFRASTRUCTURE ONLY: nothing in the product package imports this file.

``reference_forward`` restates the glue the reference wraps around its kernels - cdssm/models/block.py:181-211
(dynamics, normalisation, vp scale, shortcut, read-out, sel_C gate) over cdssm/models/ssd.py:56-111 (pad,
chunk views, three kernels, add) - and calls the extension's forward functions for everything else.
"""


def reference_forward(ref, q, k, v, gate_raw, log_dt_scale, rope_freqs, consts, H, N, C, shortcut=0.0,
                      stages=None):
    """q, k (B,L,H,D), v (B,L,H,N), gate_raw (B,L,(N+5)H): bf16 CUDA tensors.  Returns y (B,L,H,N) bf16.
    ``stages``: optional dict that receives the intermediate tensors."""
    import torch
    import torch.nn.functional as F
    B, L, _, D = q.shape
    A, vp, beta, selc = ref.dynamics_fused_fwd_cuda(gate_raw, log_dt_scale, rope_freqs, *consts, H, N)
    if D == 64:
        kn, qn = ref.normalize_kq_fwd_cuda(k, q)
    else:   # the reference kernel sizes its reduction for head_dim 64 only (normalize_kq.cu:55-72)
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
    if shortcut != 0.0:
        qk = torch.einsum("blhd,blhd->blh", qn, kn)
        sc = qk[..., None, None] * vg.unsqueeze(-1) * kn.unsqueeze(-2)
        Y = Y + torch.tensor([shortcut], device=q.device).bfloat16() * sc
    y = torch.einsum("blhsd,blhd->blhs", Y, qn) * selc.unsqueeze(-1)
    if stages is not None:
        stages.update(A_bar=A, vp=vp, beta=beta, sel_C=selc, k_norm=kn, q_norm=qn, cum_A=cum_A,
                      chunk_states=chunk_states, local_h=local_h, corrections=corr)
    return y
