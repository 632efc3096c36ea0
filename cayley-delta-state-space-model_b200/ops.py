"""Operator API of the CD-SSM scan path on B200.

Level 1 mirrors the reference's cdssm/ops.py: the same six ``torch.autograd.Function``
classes, positional signatures, tensor layouts and dtypes (cdssm/ops.py:13-195), so
cdssm/models/{block,ssd,modules}.py can import this module in its place.  Forward only:
``backward`` raises NotImplementedError.

Level 2 is the fused path: :func:`scan_fused` (dynamics + normalisation + vp scale + chunked
scan + read-out in one call) and :func:`decode_step`.

Every function launches hand-written sm_100a kernels through the C ABI of
libcdssm_b200.so on the current CUDA stream.  There is no CPU, eager-PyTorch or Triton
fallback: tensors must be CUDA tensors and the library must be built.
"""
import torch
from torch import Tensor
from torch.autograd import Function

from . import _lib
from ._lib import CdssmError, check

__all__ = ["CUDAConv1dSiLUOp", "DynamicsFusedFn", "NormalizeKQFn", "IntraChunkScanFn",
           "InterChunkScanFn", "ExactCorrectionFn", "scan_fused", "decode_step", "decode_step_reference", "reference_decode_state",
           "scan_fused_workspace_bytes", "scan_fused_status", "set_wait_limit_ns", "selftest_bounded_wait", "rms_norm", "groupnorm_gate", "conv1d_silu_step", "scan_summary", "scan_fused_long", "compose_carries",
           "CdssmError"]

_DT = {torch.bfloat16: _lib.BF16, torch.float32: _lib.F32}


def _dtype_code(t: Tensor) -> int:
    if t.dtype not in _DT:
        raise CdssmError(f"unsupported dtype {t.dtype}: use bfloat16 (the reference's type) or float32")
    return _DT[t.dtype]


def _prep(t: Tensor, dtype=None, name="tensor") -> Tensor:
    """The reference launchers call .contiguous() and never check dtypes (e.g.
    intra_chunk_scan.cu:573-603); here a wrong device or dtype is an error, not garbage."""
    if not t.is_cuda:
        raise CdssmError(f"{name} must be a CUDA tensor (no CPU fallback exists)")
    if dtype is not None and t.dtype != dtype:
        raise CdssmError(f"{name} has dtype {t.dtype}, expected {dtype}")
    return t.contiguous()


def _f32(t: Tensor, name) -> Tensor:
    """Per-head fp32 vectors; a bf16 buffer (a model cast with .bfloat16()) is converted."""
    if not t.is_cuda:
        raise CdssmError(f"{name} must be a CUDA tensor")
    return t.detach().to(torch.float32).contiguous()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return None if t is None else t.data_ptr()


class CUDAConv1dSiLUOp(Function):
    """Causal depthwise conv (kernel 4) + bias + SiLU; cdssm/ops.py:13-28."""

    @staticmethod
    def forward(ctx, x: Tensor, weight: Tensor, bias: Tensor) -> Tensor:
        x = _prep(x, name="x")
        if weight.shape[-1] != 4:
            raise CdssmError("Only kernel_size=4 is supported")   # conv1d_silu.cu:241
        B, L, Dm = x.shape
        w = _prep(weight.detach().to(x.dtype), name="weight").reshape(Dm, 4)
        b = _prep(bias.detach().to(x.dtype), name="bias")
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            check(_lib.lib().cdssm_b200_conv1d_silu_fwd(_p(x), _p(w), _p(b), _p(out), B, L, Dm,
                                                        _dtype_code(x), _stream()), "conv1d_silu_fwd")
        ctx.save_for_backward(x, w, b)
        ctx.param_meta = (weight.shape, weight.dtype, bias.dtype)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        """(grad_x, grad_weight, grad_bias), as cdssm/ops.py:22-28 (conv1d_silu.cu:94-219)."""
        x, w, b = ctx.saved_tensors
        B, L, Dm = x.shape
        go = _prep(grad_out.to(x.dtype), name="grad_out")
        gx = torch.empty_like(x)
        gw = torch.empty(Dm, 4, dtype=torch.float32, device=x.device)
        gb = torch.empty(Dm, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            check(_lib.lib().cdssm_b200_conv1d_silu_bwd(_p(go), _p(x), _p(w), _p(b), _p(gx), _p(gw), _p(gb), B, L, Dm,
                                                        _dtype_code(x), _stream()), "conv1d_silu_bwd")
        wshape, wdt, bdt = ctx.param_meta
        return gx, gw.reshape(wshape).to(wdt), gb.to(bdt)


class DynamicsFusedFn(Function):
    """gate_raw -> A_bar, vp_scale, beta, sel_C_gate; cdssm/ops.py:31-81."""

    @staticmethod
    def forward(ctx, gate_raw: Tensor, log_dt_scale: Tensor, rope_freqs: Tensor, gating_c: float,
                omega_thresh: float, adt_delta: float, adt_smoothness: float, adt_eps: float,
                n_heads: int, state_dim: int):
        g = _prep(gate_raw, name="gate_raw")
        B, L, GH = g.shape
        H, N = int(n_heads), int(state_dim)
        if GH != (N + 5) * H:
            raise CdssmError(f"gate_raw last dim {GH} != (state_dim+5)*n_heads = {(N + 5) * H}")
        lds, rf = _f32(log_dt_scale, "log_dt_scale"), _f32(rope_freqs, "rope_freqs")
        o = dict(dtype=g.dtype, device=g.device)
        A = torch.empty(B, L, H, N, **o)
        vp = torch.empty(B, L, H, N // 2, **o)
        beta = torch.empty(B, L, H, **o)
        selc = torch.empty(B, L, H, **o)
        with torch.cuda.device(g.device):
            check(_lib.lib().cdssm_b200_dynamics_fwd(
                _p(g), _p(lds), _p(rf), _p(A), _p(vp), _p(beta), _p(selc), gating_c, omega_thresh,
                adt_delta, adt_smoothness, adt_eps, B, L, H, N, 0, _dtype_code(g), _stream()),
                "dynamics_fwd")
        ctx.save_for_backward(g, lds, rf)
        ctx.consts = (gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps)
        ctx.dims = (B, L, H, N)
        ctx.lds_dtype = log_dt_scale.dtype
        return A, vp, beta, selc

    @staticmethod
    def backward(ctx, grad_A_bar, grad_vp_scale, grad_beta, grad_sel_C):
        """(grad_gate_raw, grad_log_dt_scale, None x 8), as cdssm/ops.py:68-81 (dynamics_fused.cu:145-387)."""
        g, lds, rf = ctx.saved_tensors
        B, L, H, N = ctx.dims
        z = lambda t, shape: (torch.zeros(shape, dtype=g.dtype, device=g.device) if t is None
                              else _prep(t.to(g.dtype), name="upstream gradient"))
        gA, gvp = z(grad_A_bar, (B, L, H, N)), z(grad_vp_scale, (B, L, H, N // 2))
        gb, gc = z(grad_beta, (B, L, H)), z(grad_sel_C, (B, L, H))
        gg = torch.empty_like(g)
        glds = torch.empty(H, dtype=torch.float32, device=g.device)
        with torch.cuda.device(g.device):
            check(_lib.lib().cdssm_b200_dynamics_bwd(
                _p(gA), _p(gvp), _p(gb), _p(gc), _p(g), _p(lds), _p(rf), _p(gg), _p(glds), *ctx.consts, B, L, H, N, 0,
                _dtype_code(g), _stream()), "dynamics_bwd")
        return (gg, glds.to(ctx.lds_dtype)) + (None,) * 8


class NormalizeKQFn(Function):
    """L2-normalise K and Q over the last dim; cdssm/ops.py:84-97."""

    @staticmethod
    def forward(ctx, K: Tensor, Q: Tensor):
        K = _prep(K, name="K")
        Q = _prep(Q, dtype=K.dtype, name="Q")
        if K.shape != Q.shape:
            raise CdssmError("K and Q must have the same shape")
        D = K.shape[-1]
        Ko, Qo = torch.empty_like(K), torch.empty_like(Q)
        with torch.cuda.device(K.device):
            check(_lib.lib().cdssm_b200_normalize_kq_fwd(_p(K), _p(Q), _p(Ko), _p(Qo),
                                                         K.numel() // D, D, _dtype_code(K), _stream()),
                  "normalize_kq_fwd")
        ctx.save_for_backward(K, Q)
        return Ko, Qo

    @staticmethod
    def backward(ctx, grad_K_out, grad_Q_out):
        """(grad_K, grad_Q), as cdssm/ops.py:93-97 (normalize_kq.cu:89-163)."""
        K, Q = ctx.saved_tensors
        D = K.shape[-1]
        z = lambda t: torch.zeros_like(K) if t is None else _prep(t.to(K.dtype), name="upstream gradient")
        gKo, gQo = z(grad_K_out), z(grad_Q_out)
        gK, gQ = torch.empty_like(K), torch.empty_like(Q)
        with torch.cuda.device(K.device):
            check(_lib.lib().cdssm_b200_normalize_kq_bwd(_p(gKo), _p(gQo), _p(K), _p(Q), _p(gK), _p(gQ),
                                                         K.numel() // D, D, _dtype_code(K), _stream()),
                  "normalize_kq_bwd")
        return gK, gQ


class IntraChunkScanFn(Function):
    """Chunk-local delta-rule scan from a zero state; cdssm/ops.py:100-135."""

    @staticmethod
    def forward(ctx, A_flat: Tensor, K_flat: Tensor, V_flat: Tensor, beta_flat: Tensor, state_dim: int):
        K = _prep(K_flat, name="K_flat")
        A = _prep(A_flat, dtype=K.dtype, name="A_flat")
        V = _prep(V_flat, dtype=K.dtype, name="V_flat")
        be = _prep(beta_flat, dtype=K.dtype, name="beta_flat")
        BNC, C, H, D = K.shape
        N = int(state_dim)
        local_h = torch.empty(BNC, C, H, N, D, dtype=K.dtype, device=K.device)
        cum_A = torch.empty(BNC, C, H, N, dtype=K.dtype, device=K.device)
        with torch.cuda.device(K.device):
            check(_lib.lib().cdssm_b200_intra_chunk_scan_fwd(
                _p(A), _p(K), _p(V), _p(be), _p(local_h), _p(cum_A), BNC, C, H, D, N,
                _dtype_code(K), _stream()), "intra_chunk_scan_fwd")
        ctx.save_for_backward(A, K, V, be, local_h, cum_A)
        ctx.state_dim = N
        return local_h, cum_A

    @staticmethod
    def backward(ctx, grad_local_h, grad_cum_A):
        """(grad_A, grad_K, grad_V, grad_beta, None), as cdssm/ops.py:123-135 (intra_chunk_scan.cu:215-553)."""
        A, K, V, be, local_h, cum_A = ctx.saved_tensors
        BNC, C, H, D = K.shape
        N = ctx.state_dim
        glh = torch.zeros_like(local_h) if grad_local_h is None else _prep(grad_local_h.to(K.dtype), name="grad_local_h")
        gca = torch.zeros_like(cum_A) if grad_cum_A is None else _prep(grad_cum_A.to(K.dtype), name="grad_cum_A")
        gA, gV = torch.empty_like(A), torch.empty_like(V)
        gK = torch.empty(BNC, C, H, D, dtype=torch.float32, device=K.device)
        gB = torch.empty(BNC, C, H, dtype=torch.float32, device=K.device)
        with torch.cuda.device(K.device):
            check(_lib.lib().cdssm_b200_intra_chunk_scan_bwd(
                _p(glh), _p(gca), _p(A), _p(K), _p(V), _p(be), _p(local_h), _p(cum_A), _p(gA), _p(gK), _p(gV), _p(gB),
                BNC, C, H, D, N, _dtype_code(K), _stream()), "intra_chunk_scan_bwd")
        return gA, gK.to(K.dtype), gV, gB.to(be.dtype), None


class InterChunkScanFn(Function):
    """Carry recurrence across chunks; cdssm/ops.py:138-163."""

    @staticmethod
    def forward(ctx, total_A: Tensor, final_local_h: Tensor, state_dim: int) -> Tensor:
        f = _prep(final_local_h, name="final_local_h")
        a = _prep(total_A, dtype=f.dtype, name="total_A")
        B, NC, H, N, D = f.shape
        out = torch.empty_like(f)
        with torch.cuda.device(f.device):
            check(_lib.lib().cdssm_b200_inter_chunk_scan_fwd(_p(a), _p(f), _p(out), B, NC, H, D,
                                                             int(state_dim), _dtype_code(f), _stream()),
                  "inter_chunk_scan_fwd")
        ctx.save_for_backward(a, out)
        ctx.state_dim = int(state_dim)
        return out

    @staticmethod
    def backward(ctx, grad_chunk_states):
        """(grad_total_A, grad_final_local_h, None), as cdssm/ops.py:157-163 (inter_chunk_scan.cu:89-196)."""
        a, states = ctx.saved_tensors
        B, NC, H, N, D = states.shape
        g = _prep(grad_chunk_states.to(states.dtype), name="grad_chunk_states")
        gA, gH = torch.empty_like(a), torch.empty_like(states)
        with torch.cuda.device(states.device):
            check(_lib.lib().cdssm_b200_inter_chunk_scan_bwd(_p(g), _p(a), _p(states), _p(gA), _p(gH), B, NC, H, D,
                                                             ctx.state_dim, _dtype_code(states), _stream()),
                  "inter_chunk_scan_bwd")
        return gA, gH, None


# The reference's correction backward kernel adds the upstream gradient of corrections[t] BEFORE it walks step t
# back (exact_correction.cu:219-223), although the forward stores corrections[t] before the step (:90-94), and its
# grad_beta is head_dim times too large (:347-359): its gradient is not the derivative of its forward.  The drop-in default reproduces the reference (what its training
# runs with); set this to True for the true derivative.
EXACT_CORRECTION_TRUE_GRADIENT = False


class ExactCorrectionFn(Function):
    """Propagate chunk carries through erase+rotate; cdssm/ops.py:166-195."""

    @staticmethod
    def forward(ctx, A_chunk: Tensor, K_chunk: Tensor, beta_chunk: Tensor, chunk_states: Tensor,
                state_dim: int) -> Tensor:
        K = _prep(K_chunk, name="K_chunk")
        A = _prep(A_chunk, dtype=K.dtype, name="A_chunk")
        be = _prep(beta_chunk, dtype=K.dtype, name="beta_chunk")
        cs = _prep(chunk_states, dtype=K.dtype, name="chunk_states")
        B, NC, C, H, D = K.shape
        N = int(state_dim)
        out = torch.empty(B, NC, C, H, N, D, dtype=K.dtype, device=K.device)
        with torch.cuda.device(K.device):
            check(_lib.lib().cdssm_b200_exact_correction_fwd(
                _p(A), _p(K), _p(be), _p(cs), _p(out), B, NC, C, H, D, N, _dtype_code(K), _stream()),
                "exact_correction_fwd")
        ctx.save_for_backward(A, K, be, out)
        ctx.state_dim = N
        return out

    @staticmethod
    def backward(ctx, grad_corrections):
        """(grad_A, grad_K, grad_beta, grad_chunk_states, None), as cdssm/ops.py:188-195
        (exact_correction.cu:169-383)."""
        A, K, be, corr = ctx.saved_tensors
        B, NC, C, H, D = K.shape
        N = ctx.state_dim
        g = _prep(grad_corrections.to(K.dtype), name="grad_corrections")
        gA = torch.empty_like(A)
        gK = torch.empty(B, NC, C, H, D, dtype=torch.float32, device=K.device)
        gB = torch.empty(B, NC, C, H, dtype=torch.float32, device=K.device)
        gS = torch.empty(B, NC, H, N, D, dtype=K.dtype, device=K.device)
        with torch.cuda.device(K.device):
            check(_lib.lib().cdssm_b200_exact_correction_bwd(
                _p(g), _p(A), _p(K), _p(be), _p(corr), _p(gA), _p(gK), _p(gB), _p(gS), B, NC, C, H, D, N,
                0 if EXACT_CORRECTION_TRUE_GRADIENT else 1, _dtype_code(K), _stream()), "exact_correction_bwd")
        return gA, gK.to(K.dtype), gB.to(be.dtype), gS, None


# ------------------------------------------------------------------------------------------
# Level 2: the fused path
# ------------------------------------------------------------------------------------------
FORCE_SIMT = 1
REUSE_LOCAL = 8
EXACT = 32
TENSOR_CORE_WA = 128
KEEP_SIMT_LOCAL, KEEP_SIMT_OUTPUT = 256, 512   # tests: one tensor-core pass at a time
TEST_WITHHOLD = 2048   # self-test of the bounded waits: see include/cdssm_b200.h
FP32_DECAY = 4096      # keep the transition A_bar in float32 (NOT the reference's arithmetic): the reference's
#                        bfloat16 A_bar lets its carry grow without bound over some 1e5 tokens, see the header

_workspaces = {}


def scan_fused_workspace_bytes(B, L, H, D, N, C) -> int:
    return int(_lib.lib().cdssm_b200_scan_fused_workspace_bytes(B, L, H, D, N, C))


def _workspace(device, nbytes):
    """One grow-only scratch buffer per (device, stream); the library itself allocates nothing."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(nbytes + 256, dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    off = (-buf.data_ptr()) % 256
    return buf.data_ptr() + off, buf.numel() - off


def scan_fused(q: Tensor, k: Tensor, v: Tensor, gate_raw: Tensor, log_dt_scale: Tensor,
               rope_freqs: Tensor, gating_c: float, omega_thresh: float, adt_delta: float,
               adt_smoothness: float, adt_eps: float, n_heads: int, state_dim: int,
               chunk_size: int, h0: Tensor = None, *, shortcut_scale: float = 0.0, pos0: int = 0,
               return_tail_state: bool = False, flags: int = 0, out: Tensor = None, segs: int = 1,
               semantics: str = "reference", strict: bool = False):
    """The scan path of one CD-SSM block in a single call.

    Equals, in the reference (cdssm/models/block.py:181-211): DynamicsFusedFn -> NormalizeKQFn
    -> V * vp_scale -> SSDChunkwiseScan (cdssm/models/ssd.py:39-111) -> shortcut -> einsum
    read-out -> sel_C gate, with the reference's chunk semantics, but without ever storing a
    (B,L,H,N,D) tensor.

    q, k: (B,L,H,D) un-normalised; v: (B,L,H,N) before the vp scale; gate_raw: (B,L,(N+5)H);
    log_dt_scale, rope_freqs: (H).  h0: optional (B,H,N,D) float32 carry into the first chunk.
    segs > 1: the batch rows are ``segs`` consecutive segments of B/segs longer sequences (row b
    starts at position pos0 + (b % segs) * L); see :func:`scan_fused_long`.
    Returns (y (B,L,H,N), final_state (B,H,N,D) float32[, tail_state]); final_state is the carry
    after the last chunk (feed it as h0 of the next chunk-aligned segment together with pos0);
    tail_state is the recurrent state after the last token (what decode_step continues from).
    semantics="exact" runs the plain sequential recurrence instead of the reference's chunk semantics
    (identical inside the first chunk); h0/final_state are then the recurrent state.
    strict=True synchronises the stream after the call and raises if a bounded device-side wait of the
    tensor-core kernels ran out (the outputs are undefined then); without it the call stays asynchronous
    and :func:`scan_fused_status` reports the same word on demand.
    """
    if semantics not in ("reference", "exact"):
        raise CdssmError("semantics must be 'reference' (the reference's chunked scan, bug for bug) or "
                         "'exact' (the sequential recurrence)")
    if semantics == "exact":
        flags = int(flags) | EXACT
    q = _prep(q, name="q")
    k = _prep(k, dtype=q.dtype, name="k")
    v = _prep(v, dtype=q.dtype, name="v")
    g = _prep(gate_raw, dtype=q.dtype, name="gate_raw")
    B, L, H, D = q.shape
    N, C = int(state_dim), int(chunk_size)
    if H != int(n_heads) or k.shape != q.shape or tuple(v.shape) != (B, L, H, N) or \
            tuple(g.shape) != (B, L, (N + 5) * H):
        raise CdssmError("scan_fused: inconsistent shapes")
    lds, rf = _f32(log_dt_scale, "log_dt_scale"), _f32(rope_freqs, "rope_freqs")
    if h0 is not None:
        h0 = _prep(h0, dtype=torch.float32, name="h0")
        if tuple(h0.shape) != (B, H, N, D):
            raise CdssmError("h0 must be (B,H,N,D)")
    dev = q.device
    y = out if out is not None else torch.empty(B, L, H, N, dtype=q.dtype, device=dev)
    if out is not None and (tuple(out.shape) != (B, L, H, N) or out.dtype != q.dtype or not out.is_contiguous()):
        raise CdssmError("out must be a contiguous (B,L,H,N) tensor of the input dtype")
    final = torch.empty(B, H, N, D, dtype=torch.float32, device=dev)
    tail = torch.empty(B, H, N, D, dtype=torch.float32, device=dev) if return_tail_state else None
    if B * L == 0:   # nothing to scan: the carry passes through
        final.zero_() if h0 is None else final.copy_(h0)
        if tail is not None:
            tail.copy_(final)
        return (y, final, tail) if return_tail_state else (y, final)
    with torch.cuda.device(dev):
        ws_ptr, ws_bytes = _workspace(dev, scan_fused_workspace_bytes(B, L, H, D, N, C))
        if segs == 1:
            check(_lib.lib().cdssm_b200_scan_fused_fwd(
                _p(q), _p(k), _p(v), _p(g), _p(lds), _p(rf), _p(h0), _p(y), _p(final), _p(tail), ws_ptr,
                ws_bytes, gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps, shortcut_scale,
                B, L, H, D, N, C, int(pos0), _dtype_code(q), int(flags), _stream()), "scan_fused_fwd")
        else:
            if return_tail_state:
                raise CdssmError("tail_state is not available for segmented batches")
            check(_lib.lib().cdssm_b200_scan_fused_segmented_fwd(
                _p(q), _p(k), _p(v), _p(g), _p(lds), _p(rf), _p(h0), _p(y), _p(final), ws_ptr, ws_bytes,
                gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps, shortcut_scale, B, L, H, D, N,
                C, int(pos0), int(segs), _dtype_code(q), int(flags), _stream()), "scan_fused_segmented_fwd")
    if strict:
        code = scan_fused_status(dev)
        if code != 0:
            raise CdssmError(f"scan_fused: a device-side wait ran out (status {code}); the outputs are undefined")
    return (y, final, tail) if return_tail_state else (y, final)


def decode_step(state: Tensor, q: Tensor, k: Tensor, v: Tensor, gate_raw: Tensor,
                log_dt_scale: Tensor, rope_freqs: Tensor, gating_c: float, omega_thresh: float,
                adt_delta: float, adt_smoothness: float, adt_eps: float, n_heads: int,
                state_dim: int, pos: int, *, shortcut_scale: float = 0.0, out: Tensor = None,
                v_first: Tensor = None, mix: Tensor = None) -> Tensor:
    """One recurrent step for every sequence of a batch; ``state`` (B,H,N,D) float32 is updated
    in place.  q, k: (B,H,D); v: (B,H,N); gate_raw: (B,(N+5)H); returns y (B,H,N).
    k and v may be column slices of a wider per-token projection (only their batch stride is free).
    ``v_first`` (B,H,N) with ``mix`` (H): the value residual v <- lerp(v_first, v, mix[head]) of
    cdssm/models/block.py:167-171 is applied inside the kernel.

    The reference has no such step (cdssm/inference/predict.py:53-67 re-runs the full forward
    for every new token); the update is one iteration of intra_chunk_scan.cu:117-167 with the
    gates of dynamics_fused.cu:64-139 at position ``pos``.
    """
    if not q.is_cuda:
        raise CdssmError("q must be a CUDA tensor (no CPU fallback exists)")
    B, H, D = q.shape
    N = int(state_dim)
    dt = q.dtype

    def rows(t, shape, name):
        """Rows dense inside; only the batch stride may be larger (a column slice of a projection)."""
        ok = t.is_cuda and t.dtype == dt and tuple(t.shape) == tuple(shape)
        inner = 1
        for i in range(len(shape) - 1, 0, -1):
            ok = ok and t.stride(i) == inner
            inner *= shape[i]
        ok = ok and t.stride(0) >= inner and (t.stride(0) * t.element_size()) % 16 == 0 and t.data_ptr() % 16 == 0
        return t if ok else _prep(t, dtype=dt, name=name)       # anything else: a dense copy (as before)

    q = rows(q, (B, H, D), "q")
    k, v = rows(k, (B, H, D), "k"), rows(v, (B, H, N), "v")
    g = rows(gate_raw, (B, (N + 5) * H), "gate_raw")
    if not state.is_cuda or state.dtype != torch.float32 or not state.is_contiguous():
        raise CdssmError("state must be a contiguous float32 CUDA tensor (B,H,N,D)")
    if H != int(n_heads) or tuple(state.shape) != (B, H, N, D) or tuple(k.shape) != (B, H, D) or \
            tuple(v.shape) != (B, H, N) or tuple(g.shape) != (B, (N + 5) * H):
        raise CdssmError("decode_step: inconsistent shapes")
    if (v_first is None) != (mix is None):
        raise CdssmError("decode_step: v_first and mix go together")
    if v_first is not None:
        v_first = _prep(v_first, dtype=q.dtype, name="v_first")
        mix = _prep(mix.reshape(-1), dtype=q.dtype, name="mix")
        if tuple(v_first.shape) != (B, H, N) or mix.numel() != H:
            raise CdssmError("decode_step: v_first must be (B,H,N) and mix (H)")
    lds, rf = _f32(log_dt_scale, "log_dt_scale"), _f32(rope_freqs, "rope_freqs")
    y = out if out is not None else torch.empty(B, H, N, dtype=q.dtype, device=q.device)
    pos_dev, pos_i = (pos, 0) if isinstance(pos, Tensor) else (None, int(pos))
    if pos_dev is not None and (pos_dev.dtype != torch.int32 or not pos_dev.is_cuda):
        raise CdssmError("a tensor position must be an int32 CUDA tensor")   # device memory: graph-replayable
    with torch.cuda.device(q.device):
        check(_lib.lib().cdssm_b200_decode_step_strided(
            _p(state), _p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(v_first), _p(mix), _p(g),
            g.stride(0), _p(lds), _p(rf),
            _p(y), gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps, shortcut_scale, B, H, D, N, pos_i,
            _p(pos_dev), _dtype_code(q), _stream()), "decode_step")
    return y


def reference_decode_state(carry: Tensor, dtype=torch.bfloat16):
    """State of :func:`decode_step_reference` at a chunk boundary from the carry (B,H,N,D) float32 that
    scan_fused returned as final_state (or zeros at the start of a sequence): a dict of the local state, the
    correction (the carry rounded to the storage type), the carry and the chunk's cumulative decay."""
    carry = _prep(carry, dtype=torch.float32, name="carry").clone()
    B, H, N, D = carry.shape
    gamma = torch.zeros(B, H, N, dtype=torch.float32, device=carry.device)
    gamma[..., 0::2] = 1.0
    return {"local": torch.zeros_like(carry), "correction": carry.to(dtype).float().clone(), "carry": carry, "decay": gamma}


def decode_step_reference(state: dict, q: Tensor, k: Tensor, v: Tensor, gate_raw: Tensor, log_dt_scale: Tensor,
                          rope_freqs: Tensor, gating_c: float, omega_thresh: float, adt_delta: float,
                          adt_smoothness: float, adt_eps: float, n_heads: int, state_dim: int, chunk_size: int,
                          pos, *, shortcut_scale: float = 0.0, out: Tensor = None) -> Tensor:
    """One token of the reference's CHUNKED scan (see cdssm_b200_decode_step_reference): unlike
    :func:`decode_step`, T of these steps reproduce scan_fused / the reference forward over T tokens for any T.
    ``state`` comes from :func:`reference_decode_state` and is updated in place; ``pos`` is the token's position
    from the start of the sequence (int, or an int32 CUDA tensor for graph replay)."""
    q = _prep(q, name="q")
    k = _prep(k, dtype=q.dtype, name="k")
    v = _prep(v, dtype=q.dtype, name="v")
    g = _prep(gate_raw, dtype=q.dtype, name="gate_raw")
    B, H, D = q.shape
    N = int(state_dim)
    for name in ("local", "correction", "carry"):
        t = state[name]
        if not t.is_cuda or t.dtype != torch.float32 or not t.is_contiguous() or tuple(t.shape) != (B, H, N, D):
            raise CdssmError(f"decode_step_reference: state['{name}'] must be a contiguous float32 (B,H,N,D) CUDA tensor")
    if tuple(state["decay"].shape) != (B, H, N) or state["decay"].dtype != torch.float32:
        raise CdssmError("decode_step_reference: state['decay'] must be float32 (B,H,N)")
    if H != int(n_heads) or tuple(v.shape) != (B, H, N) or tuple(g.shape) != (B, (N + 5) * H):
        raise CdssmError("decode_step_reference: inconsistent shapes")
    lds, rf = _f32(log_dt_scale, "log_dt_scale"), _f32(rope_freqs, "rope_freqs")
    y = out if out is not None else torch.empty(B, H, N, dtype=q.dtype, device=q.device)
    pos_dev, pos_i = (pos, 0) if isinstance(pos, Tensor) else (None, int(pos))
    if pos_dev is not None and (pos_dev.dtype != torch.int32 or not pos_dev.is_cuda):
        raise CdssmError("a tensor position must be an int32 CUDA tensor")
    with torch.cuda.device(q.device):
        check(_lib.lib().cdssm_b200_decode_step_reference(
            _p(state["local"]), _p(state["correction"]), _p(state["carry"]), _p(state["decay"]), _p(q), _p(k), _p(v),
            _p(g), _p(lds), _p(rf), _p(y), gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps,
            shortcut_scale, B, H, D, N, int(chunk_size), pos_i, _p(pos_dev), _dtype_code(q), _stream()),
            "decode_step_reference")
    return y


def scan_fused_status(device=None) -> int:
    """Status word of the last scan_fused call on this device and stream (synchronises the stream).
    0 means every bounded device-side wait of the tensor-core kernel completed; anything else is
    the code of the wait that ran out, and that call's outputs are undefined."""
    import ctypes
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None:
        return 0
    out = ctypes.c_int(0)
    ptr = buf.data_ptr() + ((-buf.data_ptr()) % 256)
    with torch.cuda.device(device):
        rc = _lib.lib().cdssm_b200_scan_fused_status(ptr, ctypes.addressof(out), key[1])
    if rc not in (0, -5):
        check(rc, "scan_fused_status")
    return out.value


def rms_norm(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    """RMSNorm over the last dimension in one kernel (cdssm/models/modules.py:50-53)."""
    x = _prep(x, name="x")
    w = _prep(weight, dtype=x.dtype, name="weight")
    d = x.shape[-1]
    out = torch.empty_like(x)
    with torch.cuda.device(x.device):
        check(_lib.lib().cdssm_b200_rmsnorm_fwd(_p(x), _p(w), _p(out), x.numel() // d, d, float(eps),
                                                _dtype_code(x), _stream()), "rmsnorm_fwd")
    return out


def groupnorm_gate(y: Tensor, gn_weight: Tensor, gn_bias: Tensor, z: Tensor, skip: Tensor, x_conv: Tensor,
                   groups: int, eps: float = 1e-5, per_token: bool = False) -> Tensor:
    """GroupNorm(y) * silu(z) + skip * x_conv for (B,L,di) tensors (cdssm/models/block.py:213-224) in two kernels
    (statistics over channels x all positions, as the reference takes them) or, with per_token=True, in one
    (statistics per token: the causal form used with a decode cache).  z may be a column slice of a wider
    projection (rows strided)."""
    y = _prep(y, name="y")
    xc = _prep(x_conv, dtype=y.dtype, name="x_conv")
    B, L, di = y.shape
    if not z.is_cuda or z.dtype != y.dtype or tuple(z.shape) != (B, L, di) or z.stride(-1) != 1 or \
            (L > 1 and z.stride(0) != L * z.stride(1)):
        z = z.contiguous()
    zs = z.stride(1) if L > 1 else (z.stride(0) if B > 1 else di)
    if (zs * z.element_size()) % 16 or z.data_ptr() % 16:      # the kernel reads 16-byte pieces
        z, zs = z.contiguous(), di
    gw, gb, sk = (_prep(t, dtype=y.dtype, name="groupnorm parameter") for t in (gn_weight, gn_bias, skip))
    out = torch.empty_like(y)
    with torch.cuda.device(y.device):
        stats = None
        if not per_token:
            n_stats = int(_lib.lib().cdssm_b200_groupnorm_stats_floats(B, L, int(groups)))
            stats = torch.empty(n_stats, dtype=torch.float32, device=y.device)   # results first, then scratch
            check(_lib.lib().cdssm_b200_groupnorm_stats(_p(y), _p(stats), B, L, di, int(groups), float(eps),
                                                        _dtype_code(y), _stream()), "groupnorm_stats")
        check(_lib.lib().cdssm_b200_groupnorm_gate_fwd(_p(y), _p(stats), _p(gw), _p(gb), _p(z), zs, _p(sk), _p(xc),
                                                       _p(out), B, L, di, int(groups), float(eps), _dtype_code(y),
                                                       _stream()), "groupnorm_gate_fwd")
    return out


def conv1d_silu_step(x: Tensor, hist: Tensor, weight: Tensor, bias: Tensor) -> Tensor:
    """One position of the causal depthwise conv + SiLU: x (B,Dm) (rows may be strided), hist (B,3,Dm) the last
    three inputs, shifted in place.  Returns (B,Dm)."""
    if not x.is_cuda or x.stride(-1) != 1:
        x = x.contiguous()
    B, Dm = x.shape
    if hist.dtype != x.dtype or not hist.is_contiguous() or tuple(hist.shape) != (B, 3, Dm):
        raise CdssmError("conv1d_silu_step: hist must be a contiguous (B,3,Dm) tensor of the input dtype")
    w = _prep(weight, dtype=x.dtype, name="weight")
    b = _prep(bias, dtype=x.dtype, name="bias")
    out = torch.empty(B, Dm, dtype=x.dtype, device=x.device)
    with torch.cuda.device(x.device):
        check(_lib.lib().cdssm_b200_conv1d_silu_step(_p(x), x.stride(0) if B > 1 else Dm, _p(hist), _p(w), _p(b),
                                                     _p(out), B, Dm, _dtype_code(x), _stream()), "conv1d_silu_step")
    return out


def set_wait_limit_ns(limit_ns: int) -> int:
    """Limit of the bounded device-side waits of the tensor-core kernels (0 = the 400 ms default).
    Returns the previous limit."""
    return int(_lib.lib().cdssm_b200_set_wait_limit_ns(int(limit_ns)))


def selftest_bounded_wait(limit_ns: int = 1_000_000, device=None) -> int:
    """Runs the wait primitive of the tensor-core kernels on a barrier that nothing signals.
    Returns 1 if the wait gave up after ``limit_ns`` as it must, 2 if it claimed to be signalled."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    st = torch.zeros(1, dtype=torch.int32, device=device)
    with torch.cuda.device(device):
        check(_lib.lib().cdssm_b200_selftest_bounded_wait(_p(st), int(limit_ns), _stream()), "selftest_bounded_wait")
    return int(st.item())


def scan_summary(k: Tensor, v: Tensor, gate_raw: Tensor, log_dt_scale: Tensor, rope_freqs: Tensor,
                 gating_c: float, omega_thresh: float, adt_delta: float, adt_smoothness: float,
                 adt_eps: float, n_heads: int, state_dim: int, chunk_size: int, h0: Tensor = None, *,
                 pos0: int = 0, segs: int = 1, flags: int = 0):
    """Summary of chunk-aligned segments: (carry_out (B,H,N,D), total_decay (B,H,N)) float32, the
    carry after the last chunk for carry-in h0 and the product of the chunk decays.  Reads k, v and
    the gates only (about half of the scan's bytes).  Of ``flags`` only FP32_DECAY applies."""
    k = _prep(k, name="k")
    v = _prep(v, dtype=k.dtype, name="v")
    g = _prep(gate_raw, dtype=k.dtype, name="gate_raw")
    B, L, H, D = k.shape
    N, C = int(state_dim), int(chunk_size)
    lds, rf = _f32(log_dt_scale, "log_dt_scale"), _f32(rope_freqs, "rope_freqs")
    if h0 is not None:
        h0 = _prep(h0, dtype=torch.float32, name="h0")
    carry = torch.zeros(B, H, N, D, dtype=torch.float32, device=k.device)
    decay = torch.zeros(B, H, N, dtype=torch.float32, device=k.device)
    decay[..., 0::2] = 1.0
    if B * L == 0:
        return (carry if h0 is None else h0.clone()), decay
    with torch.cuda.device(k.device):
        ws_ptr, ws_bytes = _workspace(k.device, scan_fused_workspace_bytes(B, L, H, D, N, C))
        check(_lib.lib().cdssm_b200_scan_summary_fwd(
            _p(k), _p(v), _p(g), _p(lds), _p(rf), _p(h0), _p(carry), _p(decay), ws_ptr, ws_bytes, gating_c,
            omega_thresh, adt_delta, adt_smoothness, adt_eps, B, L, H, D, N, C, int(pos0), int(segs),
            _dtype_code(k), int(flags) & FP32_DECAY, _stream()), "scan_summary_fwd")
    return carry, decay


def scan_fused_long(q: Tensor, k: Tensor, v: Tensor, gate_raw: Tensor, log_dt_scale: Tensor,
                    rope_freqs: Tensor, gating_c: float, omega_thresh: float, adt_delta: float,
                    adt_smoothness: float, adt_eps: float, n_heads: int, state_dim: int, chunk_size: int,
                    h0: Tensor = None, *, segments: int = 1, sequence_parallel: bool = False, group=None,
                    shortcut_scale: float = 0.0, pos0: int = 0, flags: int = 0, timings: dict = None):
    """The fused scan of long sequences cut into chunk-aligned segments, on one GPU or - only with
    ``sequence_parallel=True`` (or an explicit ``group``) - one contiguous piece per rank of a
    torch.distributed group (rank r holds tokens [r*L, (r+1)*L) of every sequence; ``group=None`` is then
    the default group).  Without either, an initialised process group is ignored: in a data-parallel job
    every rank scans its own sequences.  ``h0`` is the carry into the FIRST token of the whole sequence;
    rank 0's value is broadcast to the group.

    Pass A summarises every segment (k, v, gates only); the ranks exchange their (decay, carry)
    summaries with one small all-gather; the carries into all segments follow from the serial
    composition; pass B scans all segments at once as a batch of B*segments rows.
    Returns (y (B,L,H,N), final_state (B,H,N,D)): final_state is the carry after this rank's last
    token (on the last rank: of the whole sequence)."""
    from . import sharding
    B, L, H, D = q.shape
    N, C, S = int(state_dim), int(chunk_size), int(segments)
    if L % (S * C):
        raise CdssmError(f"length {L} does not split into {S} chunk-aligned segments of chunk {C}")
    Ls = L // S
    seg = lambda t: t.contiguous().view(B * S, Ls, *t.shape[2:])
    consts = (gating_c, omega_thresh, adt_delta, adt_smoothness, adt_eps)
    rank, world = sharding.sequence_ranks(sequence_parallel, group)
    if world > 1 and h0 is not None:
        h0 = _prep(h0, dtype=torch.float32, name="h0").clone()
        torch.distributed.broadcast(h0, torch.distributed.get_global_rank(group, 0) if group is not None else 0,
                                    group=group)
    base = pos0 + rank * L
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if timings is not None else None
    if ev: ev[0].record()
    carry, decay = scan_summary(seg(k), seg(v), seg(gate_raw), log_dt_scale, rope_freqs, *consts, n_heads, N, C,
                                pos0=base, segs=S, flags=flags)
    if ev: ev[1].record()
    if world > 1:
        # this rank's piece as one summary, exchanged with the other ranks (one small all-gather)
        _, piece_out, piece_dec = compose_carries(decay, carry, None, B, S, layout="rows", want_carry_in=False)
        decs, outs = sharding.exchange_summaries(piece_dec, piece_out, group)
        ins, _, _ = compose_carries(decs, outs, h0, B, world, layout="gathered")
        h_in = ins[rank].contiguous()
    else:
        h_in = h0
    h_rows, final, _ = compose_carries(decay, carry, h_in, B, S, layout="rows")
    if ev: ev[2].record()
    y, _ = scan_fused(seg(q), seg(k), seg(v), seg(gate_raw), log_dt_scale, rope_freqs, *consts, n_heads, N, C,
                      h_rows, shortcut_scale=shortcut_scale, pos0=base, segs=S,
                      flags=flags | REUSE_LOCAL)   # pass A's local results
    if ev:
        ev[3].record()
        torch.cuda.synchronize()
        timings.update(summary_ms=ev[0].elapsed_time(ev[1]), handoff_ms=ev[1].elapsed_time(ev[2]),
                       scan_ms=ev[2].elapsed_time(ev[3]))
    return y.view(B, L, H, N), final


def compose_carries(decay: Tensor, carry_out: Tensor, h0, batch: int, segments: int, layout: str = "rows",
                    want_carry_in: bool = True):
    """Chain segment summaries on the GPU: carry_in[g] = s; s <- decay[g] * s + carry_out[g].

    layout "rows": decay (B*S,H,N), carry_out (B*S,H,N,D) are the rows of a segmented batch;
    layout "gathered": decay (S,B,H,N), carry_out (S,B,H,N,D) (one summary per rank).
    Returns (carry_in like carry_out or None, final (B,H,N,D), total_decay (B,H,N))."""
    decay = _prep(decay, dtype=torch.float32, name="decay")
    carry_out = _prep(carry_out, dtype=torch.float32, name="carry_out")
    H, N, D = carry_out.shape[-3:]
    B, S = int(batch), int(segments)
    bs, ss = (S, 1) if layout == "rows" else (1, B)
    if h0 is not None:
        h0 = _prep(h0, dtype=torch.float32, name="h0")
    dev = carry_out.device
    cin = torch.empty_like(carry_out) if want_carry_in else None
    final = torch.empty(B, H, N, D, dtype=torch.float32, device=dev)
    tot = torch.empty(B, H, N, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        check(_lib.lib().cdssm_b200_compose_carries(_p(decay), _p(carry_out), _p(h0), _p(cin), _p(final), _p(tot),
                                                    B, S, H, D, N, bs, ss, _stream()), "compose_carries")
    return cin, final, tot
