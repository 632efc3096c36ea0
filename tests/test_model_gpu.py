"""The LM glue (prefill and cached decode) on the fused scan path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _make(dtype):
    from cdssm_b200.model import CdssmConfig, CdssmLM
    cfg = CdssmConfig(d_model=128, n_layers=3, context_length=64, vocab_size=1000, state_dim=2)
    m = CdssmLM(cfg, device="cuda", dtype=dtype, seed=1)
    # switch on the paths that are off at initialisation so that the test exercises them
    for i, p in enumerate(m.blocks):
        p.shortcut_scale = 0.3
        p.D = torch.full_like(p.D, 0.1)
        p.v_residual_gate += 0.5 * i
    return m


@pytest.fixture(scope="module")
def lm(ops):
    return _make(torch.bfloat16)


@pytest.fixture(scope="module")
def lm32(ops):
    return _make(torch.float32)


def test_config_derivation():
    from cdssm_b200.model import CdssmConfig
    c = CdssmConfig(d_model=768, n_layers=12, context_length=2048, vocab_size=32000, state_dim=2)
    assert (c.d_inner, c.n_heads, c.head_dim, c.chunk_size) == (1536, 24, 64, 64)   # config/model.py:59-62
    assert abs(c.omega_thresh - 2 ** -3.5) < 1e-12 and c.adt_delta == 0.125 and c.adt_eps == 1.0


@pytest.mark.parametrize("which,tol", [("lm32", 2e-3), ("lm", 1e-1)])
def test_prefill_then_decode_equals_forward_inside_first_chunk(request, which, tol):
    """Within one chunk the reference's forward is the plain recurrence, so prefill + cached decode
    steps must reproduce the full forward (this also checks the conv cache and positions).  The fp32
    model pins the logic; the bf16 model only differs by GEMM rounding (batched vs one row)."""
    m = request.getfixturevalue(which)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 1000, (3, 60), generator=g).cuda()
    m.per_token_group_norm = True      # the reference's sequence-wide GroupNorm is not causal
    full = m.forward(ids).float()
    m.per_token_group_norm = False
    assert torch.isfinite(full).all()
    assert (m.forward(ids).float() - full).abs().max() > 0          # and the two do differ
    logits, cache = m.prefill(ids[:, :37])
    outs = [logits[:, -1].float()]
    for t in range(37, 59):
        outs.append(m.decode(ids[:, t], cache).float())
    got = torch.stack(outs, 1)                       # predictions for positions 36..58
    want = full[:, 36:59]
    err = (got - want).abs().max() / want.abs().max()
    assert err < tol, float(err)
    assert cache["pos"] == 59


def test_graph_replayed_decode_equals_eager_decode(lm32):
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 1000, (4, 20), generator=g).cuda()
    _, c1 = lm32.prefill(ids)
    _, c2 = lm32.prefill(ids)
    tok = torch.full((4,), 7, dtype=torch.int64, device="cuda")
    eager = []
    t = tok.clone()
    for _ in range(5):
        t = lm32.decode(t, c1).argmax(-1)
        eager.append(t.clone())
    graph, buf = lm32.make_decode_graph(c2, 4)
    buf.copy_(tok)
    replayed = []
    for _ in range(5):
        graph.replay()
        replayed.append(buf.clone())
    assert all(torch.equal(a, b) for a, b in zip(eager, replayed))
    assert torch.allclose(c1["layers"][-1]["state"], c2["layers"][-1]["state"], atol=1e-5)
    # one position counter: the replays advanced it, and an eager step after the graph continues from there
    assert lm32.position(c1) == 25 and lm32.position(c2) == 25
    a = lm32.decode(eager[-1], c1)
    b = lm32.decode(replayed[-1], c2)
    assert torch.allclose(a, b, atol=1e-4) and lm32.position(c2) == 26


def test_one_token_prompt(lm32):
    """A prompt of a single token is a prefill (empty cache), not a decode step."""
    ids = torch.tensor([[5], [9]], device="cuda")
    logits, cache = lm32.prefill(ids)
    assert logits.shape == (2, 1, 1000) and lm32.position(cache) == 1
    nxt = lm32.decode(logits[:, -1].argmax(-1), cache)
    lm32.per_token_group_norm = True
    full = lm32.forward(torch.cat([ids, logits[:, -1].argmax(-1)[:, None]], 1)).float()
    lm32.per_token_group_norm = False
    assert (nxt.float() - full[:, 1]).abs().max() <= 2e-3 * full.abs().max()


def test_forward_is_deterministic_and_batch_independent(lm):
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 1000, (4, 150), generator=g).cuda()
    a = lm.forward(ids)
    b = lm.forward(ids)
    assert torch.equal(a, b)
    c = lm.forward(ids[1:3])
    assert (c.float() - a[1:3].float()).abs().max() <= 2e-2 * a.float().abs().max()


def test_graph_replayed_forward_equals_eager_forward(lm):
    """forward() captured as one CUDA graph (static ids in, logits out) and replayed on new token ids: the same
    bits as the eager pass, twice in a row (nothing in the graph depends on state of an earlier replay)."""
    B, L = 2, 200                                  # head_dim 64, 4 heads: the tensor-core scan passes
    graph, ids_buf, logits = lm.make_forward_graph(B, L)
    g = torch.Generator().manual_seed(11)
    for _ in range(2):
        ids = torch.randint(0, lm.cfg.vocab_size, (B, L), generator=g).cuda()
        want = lm.forward(ids)
        ids_buf.copy_(ids)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(logits, want)
