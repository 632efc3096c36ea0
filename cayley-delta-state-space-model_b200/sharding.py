"""Host-side partitioning of the scan over GPUs (one process per GPU, torch.distributed).

Two partitions exist, both derived from the structure of the reference kernels:

* (batch, head): every kernel of the path is independent across (b, h) (the reference grids are
  ``(B*NC, H)`` / ``(B, H)``, e.g. cdssm/csrc/kernels/inter_chunk_scan.cu:221), so a batch shard
  needs no communication at all and its result is bit-identical to the unsharded one.

* sequence segments: in the reference's semantics the carry between chunks is the diagonal-linear
  recurrence ``s <- gamma_c * s + l_c`` (inter_chunk_scan.cu:73-83) and neither gamma_c nor l_c
  depends on the carry.  A contiguous, chunk-aligned segment is therefore summarised by
  ``(Gamma, b)``: the product of its gamma_c and its carry-out from a zero carry-in.  Ranks
  exchange those summaries (H*(N*D + N) floats each), every rank composes the carry into its own
  segment locally and then runs its segment with that carry ("local correction").
"""
import torch


def batch_shard(batch: int, world: int, rank: int) -> range:
    """Contiguous slice of the batch owned by ``rank`` (batch must split evenly)."""
    if batch % world:
        raise ValueError(f"batch {batch} does not split over {world} ranks")
    per = batch // world
    return range(rank * per, (rank + 1) * per)


def segment_bounds(length: int, chunk: int, parts: int):
    """Chunk-aligned contiguous segments covering [0, length): list of (start, stop).
    Chunks are dealt as evenly as possible; trailing parts may be empty when there are fewer
    chunks than parts."""
    n_chunks = -(-length // chunk)
    out, c0 = [], 0
    for p in range(parts):
        n = n_chunks // parts + (1 if p < n_chunks % parts else 0)
        start, stop = min(c0 * chunk, length), min((c0 + n) * chunk, length)
        out.append((start, stop))
        c0 += n
    return out


def complex_mul_rows(decay: torch.Tensor, state: torch.Tensor) -> torch.Tensor:
    """decay (..., N) as re/im interleaved complex pairs times state (..., N, D) row pairs."""
    re, im = decay[..., 0::2, None], decay[..., 1::2, None]
    sr, si = state[..., 0::2, :], state[..., 1::2, :]
    out = torch.empty_like(state)
    out[..., 0::2, :] = re * sr - im * si
    out[..., 1::2, :] = re * si + im * sr
    return out


def complex_mul_pairs(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """Element-wise product of two (..., N) tensors of re/im interleaved complex pairs."""
    out = torch.empty_like(b)
    out[..., 0::2] = a[..., 0::2] * b[..., 0::2] - a[..., 1::2] * b[..., 1::2]
    out[..., 1::2] = a[..., 0::2] * b[..., 1::2] + a[..., 1::2] * b[..., 0::2]
    return out


def compose_carries(decay: torch.Tensor, carry_out: torch.Tensor, h0: torch.Tensor = None):
    """Carries into consecutive segments from their summaries.

    decay (S, B, H, N) and carry_out (S, B, H, N, D): summary of segment g.  Returns
    (carry_in (S, B, H, N, D), final (B, H, N, D)) with carry_in[0] = h0 (or 0) and
    carry_in[g+1] = decay[g] * carry_in[g] + carry_out[g]."""
    S = decay.shape[0]
    s = torch.zeros_like(carry_out[0]) if h0 is None else h0.to(carry_out.dtype).clone()
    ins = []
    for g in range(S):
        ins.append(s)
        s = complex_mul_rows(decay[g], s) + carry_out[g]
    return torch.stack(ins), s


def sequence_ranks(sequence_parallel: bool = False, group=None):
    """(rank, world) of the sequence-parallel scan.  Sequence parallelism is opt-in: it is taken only when
    asked for (``sequence_parallel=True``) or when a process group is passed explicitly.  A process group
    that merely happens to be initialised - the usual state of a data-parallel job, where every rank scans
    its own sequences - means a single piece: (0, 1)."""
    if not sequence_parallel and group is None:
        return 0, 1
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()):
        raise RuntimeError("sequence_parallel needs an initialised torch.distributed process group")
    return dist.get_rank(group), dist.get_world_size(group)


def exchange_summaries(decay: torch.Tensor, carry_out: torch.Tensor, group=None):
    """All-gather the (Gamma, b) summaries of every rank's segment.  decay (B,H,N), carry_out
    (B,H,N,D) of the local segment -> (world, B,H,N), (world, B,H,N,D).  One small collective;
    no kernel ever reads another GPU's memory."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    packed = torch.cat([decay.reshape(-1), carry_out.reshape(-1)]).contiguous()
    gathered = [torch.empty_like(packed) for _ in range(world)]
    dist.all_gather(gathered, packed, group=group)
    n = decay.numel()
    decs = torch.stack([g[:n].view_as(decay) for g in gathered])
    outs = torch.stack([g[n:].view_as(carry_out) for g in gathered])
    return decs, outs
