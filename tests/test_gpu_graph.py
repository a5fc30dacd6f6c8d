"""CUDA-graph capture of the module set: forward + backward of every operator is captured once
into a torch.cuda.CUDAGraph (after warm-up calls, which do the one-time kernel attribute set-up
outside the capture) and replayed on new input values; the replayed results equal the eager ones
bit for bit.  rgd_rmsnorm_bwd_static is not part of this (its first call per device resolves a
symbol address and belongs before any capture)."""
import pytest
import torch

from rgd_triton_b200 import _lib, ops
from tests._util import attention_backward, gen, randn, rotary_table

pytestmark = pytest.mark.gpu


def _capture_and_replay(step, inputs, fresh):
    """step(*inputs) -> tensors (outputs and gradients).  Captures step on static input buffers,
    then replays it after the buffers were overwritten with `fresh` values and compares with an
    eager evaluation on those values."""
    static = [t.clone() for t in inputs]
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(3):
            step(*static)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step(*static)
    for s_, f in zip(static, fresh):
        s_.copy_(f)
    graph.replay()
    torch.cuda.synchronize()
    want = step(*[f.clone() for f in fresh])
    torch.cuda.synchronize()
    for a, b in zip(captured, want):
        assert torch.equal(a, b)
    assert _lib.load().rgd_device_status() == 0


def _fwd_bwd(call, params=()):
    def step(*ins):
        ins = [t.detach().requires_grad_(True) for t in ins]
        outs = call(*ins)
        outs = outs if isinstance(outs, tuple) else (outs,)
        grads = torch.autograd.grad(outs, ins + list(params), [torch.ones_like(o) for o in outs])
        return [o.detach() for o in outs] + list(grads)
    return step


def test_norm_modules_capture():
    g = gen(11)
    bf = torch.bfloat16
    mk = lambda: [randn(g, 2, 300, 3072, dtype=bf).cuda(), randn(g, 2, 77, 1024, dtype=bf).cuda()]
    a, b = mk(), mk()
    l2, l22 = ops.L2Normalize(), ops.FusedL2Normalize2()
    _capture_and_replay(_fwd_bwd(lambda x: l2(x)), a[:1], b[:1])
    _capture_and_replay(_fwd_bwd(lambda x, y: l22(x, y)), a, b)
    m = ops.FusedRMSNorm(3072, dtype=bf).cuda()
    _capture_and_replay(_fwd_bwd(lambda x: m(x), [m.weight]), a[:1], b[:1])
    m2 = ops.FusedRMSNorm2((3072, 1024), dtype=bf).cuda()
    _capture_and_replay(_fwd_bwd(lambda x, y: m2(x, y), [m2.weight1, m2.weight2]), a, b)


def test_head_modules_capture():
    g = gen(12)
    bf = torch.bfloat16
    mk = lambda: [randn(g, 2, 260, 4, 128, dtype=bf).cuda(), randn(g, 2, 190, 4, 128, dtype=bf).cuda()]
    a, b = mk(), mk()
    pos = rotary_table(300, 64, bf).cuda()
    hl, rp, lr = ops.FusedHeadLayerNorm(), ops.RoPE(), ops.FusedLNRoPE()
    _capture_and_replay(_fwd_bwd(lambda q, k: hl(q, k, False, 1e-6)), a, b)
    _capture_and_replay(_fwd_bwd(lambda q, k: rp(q, k, pos, (200, 190), False)), a, b)
    _capture_and_replay(_fwd_bwd(lambda q, k: lr(q, k, pos, 200, False, 1e-5)), a, b)


@pytest.mark.parametrize("d,bias_kind", [(128, None), (64, "matrix"), (128, "vector"), (32, "matrix")])
def test_attention_captures(d, bias_kind):
    g = gen(13 + d)
    dt = torch.bfloat16
    B, T_, H = 2, 384, 3
    mk = lambda: [randn(g, B, T_, H, d, dtype=dt).cuda() for _ in range(3)]
    a, b = mk(), mk()
    bias = None
    if bias_kind == "matrix":
        bias = randn(g, B, H, T_, T_, dtype=dt).cuda()
    elif bias_kind == "vector":
        bias = randn(g, B, 1, 1, T_, dtype=dt).cuda()
    fa = ops.FlashAttention()
    with attention_backward("two_kernel"):
        _capture_and_replay(_fwd_bwd(lambda q, k, v: fa(q, k, v, bias, d == 64)), a, b)


def test_single_pass_attention_backward_captures():
    """The single-pass backward (head_dim 64: accumulator zero-fill, one kernel, rounding kernel)
    inside a graph: o, dk, dv of the replay bit-equal to eager, dq to within one rounding step."""
    g = gen(99)
    dt = torch.float16
    mk = lambda: [randn(g, 2, 640, 3, 64, dtype=dt).cuda() for _ in range(3)]
    a, b = mk(), mk()
    bias = randn(g, 2, 3, 640, 640, dtype=dt).cuda()
    fa = ops.FlashAttention()
    step = _fwd_bwd(lambda q, k, v: fa(q, k, v, bias))
    static = [t.clone() for t in a]
    with attention_backward("single_pass"):
        for _ in range(3):
            step(*static)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            captured = step(*static)
        for s_, f in zip(static, b):
            s_.copy_(f)
        graph.replay()
        torch.cuda.synchronize()
        want = step(*[f.clone() for f in b])
    torch.cuda.synchronize()
    for i in (0, 2, 3):
        assert torch.equal(captured[i], want[i])
    assert (captured[1].float() - want[1].float()).abs().max().item() <= 2 ** -9 * want[1].float().abs().max().item()
    assert _lib.load().rgd_device_status() == 0
