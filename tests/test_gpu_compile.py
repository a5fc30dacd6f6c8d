"""torch.compile traces the modules without graph breaks (fullgraph=True) through the registered
custom operators, and the compiled results equal the eager ones bit for bit (same kernels)."""
import pytest
import torch

from rgd_triton_b200 import ops
from tests._util import attention_backward, gen, randn, rotary_table

pytestmark = pytest.mark.gpu


def _both(module_call, inputs, grads_of=()):
    """Run eager and compiled (aot_eager: no code generation, only the tracing) forward + backward."""
    outs = []
    for compiled in (False, True):
        ins = [t.detach().clone().requires_grad_(True) for t in inputs]
        fn = torch.compile(module_call, fullgraph=True, backend="aot_eager") if compiled else module_call
        o = fn(*ins)
        o = o if isinstance(o, tuple) else (o,)
        g = torch.autograd.grad(o, ins + list(grads_of), [torch.ones_like(t) for t in o])
        outs.append([t.detach() for t in o] + list(g))
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_norms_compile():
    g = gen(1)
    bf = torch.bfloat16
    x1, x2 = randn(g, 2, 50, 256, dtype=bf).cuda(), randn(g, 2, 70, 384, dtype=bf).cuda()
    l2, l22 = ops.L2Normalize(), ops.FusedL2Normalize2()
    _both(lambda a: l2(a), [x1])
    _both(lambda a, b: l22(a, b), [x1, x2])
    m = ops.FusedRMSNorm(256, dtype=bf).cuda()
    _both(lambda a: m(a), [x1], [m.weight])
    m2 = ops.FusedRMSNorm2((256, 384), dtype=bf).cuda()
    _both(lambda a, b: m2(a, b), [x1, x2], [m2.weight1, m2.weight2])


def test_head_operators_compile():
    g = gen(2)
    bf = torch.bfloat16
    q, k = randn(g, 2, 130, 4, 128, dtype=bf).cuda(), randn(g, 2, 90, 4, 128, dtype=bf).cuda()
    pos = rotary_table(140, 64, bf).cuda()
    hl, rp, lr = ops.FusedHeadLayerNorm(), ops.RoPE(), ops.FusedLNRoPE()
    _both(lambda a, b: hl(a, b, False, 1e-6), [q, k])
    _both(lambda a, b: rp(a, b, pos, (100, 90), False), [q, k])
    _both(lambda a, b: lr(a, b, pos, 100, False, 1e-5), [q, k])


def test_attention_compiles():
    g = gen(3)
    q, k, v = (randn(g, 2, 200, 3, 64, dtype=torch.float16).cuda() for _ in range(3))
    bias = randn(g, 2, 3, 200, 200, dtype=torch.float16).cuda()
    fa = ops.FlashAttention()
    with attention_backward("two_kernel"):      # bit-equality of dq needs the form without reductions at head_dim 64
        _both(lambda a, b, c: fa(a, b, c), [q, k, v])
        _both(lambda a, b, c: fa(a, b, c, bias, True), [q, k, v])
