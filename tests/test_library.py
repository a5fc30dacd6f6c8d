"""The custom-operator registration (torch.ops.rgd_b200.*) without a GPU: every operator exists
and its fake (shape-only) implementation returns what the kernels would."""
import torch
from torch._subclasses.fake_tensor import FakeTensorMode

from rgd_triton_b200 import library  # noqa: F401  (registers the operators)


def test_every_operator_is_registered():
    for name in ("l2norm", "l2norm_bwd", "rmsnorm", "rmsnorm_bwd", "headln", "headln_bwd", "rope", "lnrope",
                 "lnrope_bwd", "attn", "attn_bwd"):
        assert hasattr(torch.ops.rgd_b200, name), name


def test_fake_implementations_give_the_kernels_shapes():
    bf = torch.bfloat16
    with FakeTensorMode():
        x1 = torch.empty(2, 7, 64, device="cuda", dtype=bf)
        x2 = torch.empty(2, 9, 96, device="cuda", dtype=bf)
        y1, y2 = torch.ops.rgd_b200.l2norm([x1, x2], 1e-6)
        assert y1.shape == x1.shape and y2.shape == x2.shape and y2.dtype == bf
        w1 = torch.empty(64, device="cuda", dtype=torch.float32)
        w2 = torch.empty(96, device="cuda", dtype=torch.float32)
        g = torch.ops.rgd_b200.rmsnorm_bwd([x1, x2], [w1, w2], [x1, x2], 1e-6)
        assert [t.shape for t in g] == [x1.shape, x2.shape, w1.shape, w2.shape] and g[2].dtype == torch.float32
        q = torch.empty(2, 100, 4, 128, device="cuda", dtype=bf)
        k = torch.empty(2, 77, 4, 128, device="cuda", dtype=bf)
        pos = torch.empty(2, 128, 64, device="cuda", dtype=bf)
        qo, ko = torch.ops.rgd_b200.lnrope(q, k, pos, 100, 77, False, 1e-5)
        assert qo.shape == q.shape and ko.shape == k.shape
        qo, ko = torch.ops.rgd_b200.rope(q, k, pos, 50, 50, False, False)
        assert qo.shape == q.shape
        o, lse = torch.ops.rgd_b200.attn(q, k, k, None, False, 0.1)
        assert o.shape == q.shape and lse.shape == (2, 4, 128) and lse.dtype == torch.float32
        dq, dk, dv, dbias = torch.ops.rgd_b200.attn_bwd(q, k, k, None, o, lse, o, False, 0.1, False)
        assert dq.shape == q.shape and dk.shape == k.shape and dv.shape == k.shape
