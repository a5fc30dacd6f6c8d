"""Host-side behaviour of the module API that needs no GPU: class surface,
cache objects, parameter names, argument errors, the rgd_triton import shim."""
import inspect
import sys

import pytest
import torch

import rgd_triton_b200 as R
from rgd_triton_b200 import compat, functional as F_, ops


def test_module_surface_matches_reference_signatures():
    sig = lambda f: list(inspect.signature(f).parameters)
    assert sig(ops.FlashAttention.forward) == ["self", "q", "k", "v", "bias", "causal", "softmax_scale"]
    assert sig(ops.L2Normalize.forward) == ["self", "x", "eps"]
    assert sig(ops.FusedL2Normalize2.forward) == ["self", "x1", "x2", "eps"]
    assert sig(ops.FusedHeadLayerNorm.forward) == ["self", "query", "key", "heads_second", "eps"]
    assert sig(ops.FusedRMSNorm.__init__) == ["self", "normalized_shape", "eps", "elementwise_affine", "device", "dtype"]
    assert sig(ops.FusedRMSNorm.forward) == ["self", "x", "weight"]
    assert sig(ops.FusedRMSNorm2.forward) == ["self", "x1", "x2", "weight1", "weight2"]
    assert sig(ops.RoPE.forward) == ["self", "query", "key", "pos_emb", "seq_cutoff", "heads_second"]
    assert sig(ops.FusedLNRoPE.forward) == ["self", "query", "key", "pos_emb", "seq_cutoff", "heads_second", "eps"]
    d = lambda f, n: inspect.signature(f).parameters[n].default
    assert d(ops.FusedHeadLayerNorm.forward, "heads_second") is True and d(ops.FusedHeadLayerNorm.forward, "eps") == 1e-6
    assert d(ops.L2Normalize.forward, "eps") == 1e-6 and d(ops.FusedLNRoPE.forward, "eps") == 1e-6
    assert sig(F_.flash_attn_func) == ["q", "k", "v", "bias", "causal", "softmax_scale", "return_lse", "kernel_cache"]
    assert sig(F_.triton_rms_func_fn) == ["x", "w", "norm_eps", "kernel_cache"]
    assert sig(F_.triton_fused_ln_rope_fn)[:6] == ["query", "key", "pos_emb", "seq_cutoff", "heads_second", "norm_eps"]


def test_cache_slots_and_enable_cache():
    slots = {ops.FlashAttention: ("fwd", "bwd_odot", "bwd"), ops.L2Normalize: ("fwd", "bwd"),
             ops.FusedL2Normalize2: ("fwd", "bwd"), ops.FusedHeadLayerNorm: ("fwd", "bwd"),
             ops.RoPE: ("fwd", "bwd"), ops.FusedLNRoPE: ("fwd", "bwd")}
    for cls, names in slots.items():
        m = cls()
        assert all(getattr(m.cache, n) is None for n in names)
        m.enable_cache(False)
        assert m.cache is None
        m.enable_cache()
        assert m.cache is not None and all(getattr(m.cache, n) is None for n in names)
    m = ops.FusedRMSNorm(8)
    assert (m.cache.fwd, m.cache.bwd, m.cache.bwd_dw) == (None, None, None)
    old = m.cache
    m.enable_cache(True)
    assert m.cache is not old


def test_rmsnorm_parameters_and_state_dict():
    m = ops.FusedRMSNorm(16, eps=1e-5)
    assert list(m.state_dict()) == ["weight"] and torch.equal(m.weight, torch.ones(16))
    assert m.normalized_shape == (16,) and m.eps == 1e-5
    m2 = ops.FusedRMSNorm2((16, 24), dtype=torch.bfloat16)
    assert list(m2.state_dict()) == ["weight1", "weight2"]
    assert m2.weight2.shape == (24,) and m2.weight1.dtype == torch.bfloat16
    m3 = ops.FusedRMSNorm(16, elementwise_affine=False)
    assert m3.weight is None and list(m3.state_dict()) == []
    with pytest.raises(AssertionError):
        ops.FusedRMSNorm((16,))
    with pytest.raises(AssertionError):
        ops.FusedRMSNorm2(16)
    with pytest.raises(AssertionError):
        m3(torch.zeros(1, 2, 16))          # no weight passed
    m2.load_state_dict({"weight1": torch.full((16,), 2.0), "weight2": torch.full((24,), 3.0)})
    assert m2.weight1[0].item() == 2.0


def test_cpu_tensors_are_refused_not_computed():
    """There is no CPU fallback: every operator raises on CPU tensors."""
    x = torch.randn(2, 3, 16)
    q = torch.randn(1, 2, 4, 16)
    pos = torch.randn(2, 8, 8)
    calls = [
        lambda: ops.L2Normalize()(x),
        lambda: ops.FusedL2Normalize2()(x, x),
        lambda: ops.FusedRMSNorm(16)(x),
        lambda: ops.FusedRMSNorm2((16, 16))(x, x),
        lambda: ops.FusedHeadLayerNorm()(q, q),
        lambda: ops.RoPE()(q, q, pos),
        lambda: ops.FusedLNRoPE()(q, q, pos),
        lambda: ops.FlashAttention()(q.half(), q.half(), q.half()),
    ]
    for c in calls:
        with pytest.raises(AssertionError):
            c()


def test_shape_and_dtype_errors_match_the_reference_convention():
    with pytest.raises(AssertionError):
        F_._check_rows([torch.zeros(2, 3)], "x")                       # not 3-D
    with pytest.raises(AssertionError):
        F_._check_rows([torch.zeros(2, 3, 4, dtype=torch.float64)], "x")
    q = torch.zeros(1, 4, 2, 8, dtype=torch.float16)
    with pytest.raises(AssertionError):
        F_._check_attn(q.float(), q.float(), q.float())               # fp32 attention unsupported
    with pytest.raises(AssertionError):
        big = torch.zeros(1, 4, 2, 256, dtype=torch.float16)
        F_._check_attn(big, big, big)                                   # head_dim > 128
    with pytest.raises(AssertionError):
        F_._head_dims(torch.zeros(1, 2, 4, 8), torch.zeros(1, 3, 4, 8), True)
    assert F_._cutoffs(None, 5, 7) == (5, 7)
    assert F_._cutoffs(3, 5, 7) == (3, 3)
    assert F_._cutoffs((2, 6), 5, 7) == (2, 6)
    x = torch.zeros(2, 3, 8)
    w, sb, per = F_._prep_weight(torch.ones(8), x)
    assert (sb, per) == (0, False)
    w, sb, per = F_._prep_weight(torch.ones(1, 1, 8), x)
    assert (sb, per) == (0, False)
    w, sb, per = F_._prep_weight(torch.ones(2, 1, 8), x)
    assert (sb, per) == (8, True)
    with pytest.raises(AssertionError):
        F_._prep_weight(torch.ones(7), x)
    with pytest.raises(AssertionError):
        F_._prep_weight(torch.ones(3, 1, 8), x)


def test_compat_installs_reference_import_names():
    assert "rgd_triton" not in sys.modules or getattr(sys.modules["rgd_triton"], "__rgd_b200__", False)
    compat.install()
    try:
        from rgd_triton.ops import FusedRMSNorm, FlashAttention
        from rgd_triton.triton.flash_attn.flash_attn_triton_cached import flash_attn_func
        from rgd_triton.triton.normalization.rmsnorm_cached import triton_rms_func_fn
        from rgd_triton.triton.rope.fused_ln_rope_cached import triton_fused_ln_rope_fn
        assert FusedRMSNorm is ops.FusedRMSNorm and flash_attn_func is F_.flash_attn_func
        assert triton_rms_func_fn is F_.triton_rms_func_fn and triton_fused_ln_rope_fn is F_.triton_fused_ln_rope_fn
        FlashAttention()       # constructs (the reference's own constructor raises ModuleNotFoundError)
    finally:
        compat.uninstall()
    assert "rgd_triton" not in sys.modules


def test_package_exports():
    for n in ("FlashAttention", "L2Normalize", "FusedL2Normalize2", "FusedHeadLayerNorm", "FusedRMSNorm",
              "FusedRMSNorm2", "RoPE", "FusedLNRoPE", "CachableModule"):
        assert hasattr(R, n)
