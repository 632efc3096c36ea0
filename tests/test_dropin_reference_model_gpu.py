"""The drop-in claim, end to end: the reference's OWN model code (cdssm/models/{block,ssd,modules}.py, loaded
unmodified from $CDSSM_REFERENCE_ROOT) runs on this library's operator module installed as ``cdssm.ops``.

(a) its CDSSMBlock forward on our six operators equals the same block on the reference's own kernels
    (oracle/_ref, when built);
(b) model.py's restated block (the fused scan path) equals the reference block on copied weights.

Skipped when no reference checkout is readable: the reference sources are never part of this repository.
"""
import importlib
import os
import sys
import types

import pytest
import torch

from util import BF16_TOL, rel_err, to_np

pytestmark = pytest.mark.gpu


def _reference_root():
    root = os.environ.get("CDSSM_REFERENCE_ROOT", "")
    if not root or not os.path.isdir(os.path.join(root, "cdssm", "models")):
        pytest.skip("set CDSSM_REFERENCE_ROOT to a checkout of the reference to run the drop-in test")
    return root


def _purge():
    for k in [k for k in sys.modules if k == "cdssm" or k.startswith("cdssm.")]:
        del sys.modules[k]


def _load_reference_models(root, ops_module=None, ext=None):
    """Import the reference's model modules from `root` without running cdssm/__init__.py (global torch
    settings, allocator configuration).  ops_module: what ``cdssm.ops`` resolves to; if None the reference's own
    ops.py is used, on top of `ext` as ``cdssm._C``."""
    _purge()
    pkg = types.ModuleType("cdssm")
    pkg.__path__ = [os.path.join(root, "cdssm")]
    sys.modules["cdssm"] = pkg
    if ops_module is not None:
        sys.modules["cdssm.ops"] = ops_module
        pkg.ops = ops_module
    else:
        sys.modules["cdssm._C"] = ext
        pkg._C = ext
    block = importlib.import_module("cdssm.models.block")
    cfg = importlib.import_module("cdssm.config.model")
    return block, cfg


def _make_block(block_mod, cfg_mod, N, seed):
    torch.manual_seed(seed)
    cfg = cfg_mod.CDSSMConfig(d_model=128, n_layers=2, context_length=512, vocab_size=256, state_dim=N)
    blk = block_mod.CDSSMBlock(cfg, layer_idx=1)
    with torch.no_grad():   # switch on what the reference's init leaves at zero, so that it is tested
        blk.shortcut_scale.fill_(0.4)
        blk.D.normal_(std=0.5)
        blk.v_residual_gate.normal_()
        blk.log_dt_scale.normal_(std=0.3)
        blk.Q_proj.weight.add_(0.05 * torch.randn_like(blk.Q_proj.weight))
    blk = blk.cuda().bfloat16().eval()
    # the kernels read rope_freqs as float32 (dynamics_fused.cu:50-56); .bfloat16() above also cast this buffer
    blk.rope_freqs = blk.rope_freqs.float()
    return cfg, blk


@pytest.mark.parametrize("N", [2, 16])
def test_reference_block_runs_on_our_operators(ops, N):
    root = _reference_root()
    B, L = 2, 200                                       # not a multiple of the 64-token chunk: the pad path
    try:
        block_mod, cfg_mod = _load_reference_models(root, ops_module=ops)
        assert block_mod.DynamicsFusedFn is ops.DynamicsFusedFn
        cfg, blk = _make_block(block_mod, cfg_mod, N, seed=5)
        torch.manual_seed(9)
        x = torch.randn(B, L, cfg.d_model, device="cuda").bfloat16()
        v_first = torch.randn(B, L, cfg.n_heads, N, device="cuda").bfloat16()
        with torch.no_grad():
            y_ours, _ = blk(x, v_first)
            y_ours0, v0 = blk(x, None)
        state = {k: v.clone() for k, v in blk.state_dict().items()}
        assert torch.isfinite(y_ours.float()).all()

        # (b) the restated block of model.py (fused scan path) on the same weights
        from cdssm_b200.model import CdssmConfig, CdssmLM
        lm = CdssmLM(CdssmConfig(d_model=128, n_layers=2, context_length=512, vocab_size=256, state_dim=N),
                     device="cuda", dtype=torch.bfloat16, seed=0)
        p = lm.blocks[1]
        p.load_reference(state, "", "cuda", torch.bfloat16)
        p.rope_freqs = blk.rope_freqs.float()
        with torch.no_grad():
            y_model, _ = lm._block(p, x, v_first, 0, None, 0)
            y_model0, _ = lm._block(p, x, None, 0, None, 0)
        scale = float(y_ours.float().abs().max())
        assert rel_err(to_np(y_model), to_np(y_ours)) <= BF16_TOL, "model.py block differs from the reference block"
        assert rel_err(to_np(y_model0), to_np(y_ours0)) <= BF16_TOL
        assert scale > 0.1

        # (a) the same reference block on the reference's own kernels
        from oracle.build_ref import load_ref
        ext = load_ref()
        if ext is None:
            pytest.skip("reference extension not built (oracle/build_ref.py): only the self-consistency part ran")
        block_ref, cfg_ref = _load_reference_models(root, ops_module=None, ext=ext)
        _, blk_ref = _make_block(block_ref, cfg_ref, N, seed=5)
        blk_ref.load_state_dict(state)
        blk_ref.rope_freqs = blk.rope_freqs.float()
        with torch.no_grad():
            y_ref, _ = blk_ref(x, v_first)
            y_ref0, _ = blk_ref(x, None)
        assert rel_err(to_np(y_ours), to_np(y_ref)) <= BF16_TOL, "reference block on our operators differs"
        assert rel_err(to_np(y_ours0), to_np(y_ref0)) <= BF16_TOL
        assert rel_err(to_np(y_model), to_np(y_ref)) <= BF16_TOL
        # (c) a training step: backward through the reference block on our six operators against the same block on
        # the reference's own backward kernels
        probe = torch.randn_like(y_ref)
        grads = []
        for b_ in (blk, blk_ref):
            b_.zero_grad(set_to_none=True)
            xin = x.clone().requires_grad_(True)
            out, _ = b_(xin, v_first)
            (out.float() * probe.float()).sum().backward()
            grads.append({"x": xin.grad, **{k: p.grad for k, p in b_.named_parameters() if p.grad is not None}})
        assert set(grads[0]) == set(grads[1]) and "gate_proj.weight" in grads[0] and "log_dt_scale" in grads[0]
        for name in grads[0]:
            ref_g = grads[1][name].float()
            if float(ref_g.abs().max()) == 0.0:
                assert float(grads[0][name].float().abs().max()) == 0.0, name
                continue
            assert rel_err(to_np(grads[0][name]), to_np(ref_g)) <= 5e-2, name
    finally:
        _purge()


def test_reference_checkpoint_loads_and_matches_the_reference_lm(ops, tmp_path):
    """A checkpoint in the reference trainer's format (trainer.py:205-214), written by the reference's own LM
    class, loaded by CdssmLM.from_reference_checkpoint: same logits as the reference model on our operators."""
    import dataclasses
    root = _reference_root()
    try:
        _load_reference_models(root, ops_module=ops)
        model_mod = importlib.import_module("cdssm.models.model")
        cfg_mod = importlib.import_module("cdssm.config.model")
        torch.manual_seed(3)
        cfg = cfg_mod.CDSSMConfig(d_model=128, n_layers=3, context_length=256, vocab_size=512, state_dim=2)
        ref_lm = model_mod.CDSSMLMHeadModel(cfg)
        with torch.no_grad():
            for blk in ref_lm.blocks:
                blk.shortcut_scale.fill_(0.3)
                blk.v_residual_gate.normal_()
        path = tmp_path / "ckpt.pt"
        torch.save({"model_state_dict": {"_orig_mod." + k: v for k, v in ref_lm.state_dict().items()},
                    "config": dataclasses.asdict(cfg), "step": 7}, path)
        ref_lm = ref_lm.cuda().bfloat16().eval()
        for blk in ref_lm.blocks:
            blk.rope_freqs = blk.rope_freqs.float()
        ids = torch.randint(0, 512, (2, 150), generator=torch.Generator().manual_seed(4)).cuda()
        with torch.no_grad():
            want = ref_lm(ids).float()
        from cdssm_b200.model import CdssmLM
        lm = CdssmLM.from_reference_checkpoint(str(path))
        assert (lm.cfg.n_layers, lm.cfg.n_heads, lm.cfg.state_dim) == (3, 4, 2)
        got = lm.forward(ids).float()
        assert rel_err(to_np(got), to_np(want)) <= 3e-2      # 3 layers of bf16 GEMMs and norms on top of the scan
    finally:
        _purge()
