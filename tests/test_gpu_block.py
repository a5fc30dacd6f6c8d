"""Fifth benchmark configuration at reduced size: an MMDiT-style joint attention
block built from the operator set — FusedRMSNorm2 on a text and an image stream,
a shared QKV projection (torch Linear, outside the operator set), FusedHeadLayerNorm
on q / k, RoPE on the image tokens only (image tokens first, seq_cutoff = number of
image tokens), FlashAttention over the concatenated tokens with a bias that masks
padded text keys — forward and backward against an fp32 eager evaluation of the
same block."""
import math

import pytest
import torch
import torch.nn.functional as F

from rgd_triton_b200 import ops
from tests._util import gen, randn, rotary_table

pytestmark = pytest.mark.gpu


def eager_block(text, image, w1, w2, wqkv, pos, text_len, H, D, R, eps=1e-6):
    """fp32 reference of the block (returns the attention output)."""
    B, Nt, C = text.shape
    Ni = image.shape[1]
    rms = lambda x, w: x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w
    x = torch.cat([rms(image, w2), rms(text, w1)], dim=1)             # image tokens first
    qkv = (x @ wqkv.t()).view(B, Ni + Nt, 3, H, D)
    q, k, v = qkv.unbind(2)
    ln = lambda t: F.layer_norm(t, (D,), eps=eps)
    q, k = ln(q), ln(k)

    def rope(t):
        xr = t[:, :Ni, :, :R]
        s, c = pos[0, :Ni, None, :], pos[1, :Ni, None, :]
        rot = torch.stack((-xr[..., 1::2], xr[..., 0::2]), -1).flatten(-2)
        out = torch.cat([xr * c + rot * s, t[:, :Ni, :, R:]], -1)
        return torch.cat([out, t[:, Ni:]], 1)

    q, k = rope(q), rope(k)
    key_ok = torch.arange(Ni + Nt)[None, :] < (Ni + text_len)[:, None]          # [B, T]
    bias = torch.where(key_ok, 0.0, -1e4)[:, None, None, :].expand(B, H, Ni + Nt, Ni + Nt)
    s = torch.einsum("bthd,bshd->bhts", q, k) / math.sqrt(D) + bias
    return torch.einsum("bhts,bshd->bthd", s.softmax(-1), v), bias


@pytest.mark.parametrize("dtype", [torch.bfloat16])
def test_mmdit_block_forward_backward(dtype):
    g = gen(5)
    B, Nt, Ni, C, H, D, R = 2, 128, 384, 512, 4, 128, 64
    text, image = randn(g, B, Nt, C), randn(g, B, Ni, C)
    w1, w2 = 1 + 0.02 * torch.randn(C, generator=g), 1 + 0.02 * torch.randn(C, generator=g)
    wqkv = torch.randn(3 * H * D, C, generator=g) / math.sqrt(C)
    pos = rotary_table(Ni + Nt + 1, R, torch.float32)
    text_len = torch.tensor([64, 100])
    dout = randn(g, B, Ni + Nt, H, D)

    # fp32 eager
    leaves = [t.clone().requires_grad_(True) for t in (text, image, w1, w2)]
    ref_out, bias = eager_block(*leaves, wqkv, pos, text_len, H, D, R)
    ref_grads = torch.autograd.grad(ref_out, leaves, dout)

    # operator set on the GPU, low precision
    dev = "cuda"
    t_, i_ = (t.to(dtype).to(dev).requires_grad_(True) for t in (text, image))
    norm = ops.FusedRMSNorm2((C, C), dtype=dtype).to(dev)
    with torch.no_grad():
        norm.weight1.copy_(w1)
        norm.weight2.copy_(w2)
    hln, rope, attn = ops.FusedHeadLayerNorm(), ops.RoPE(), ops.FlashAttention()
    nt, ni = norm(t_, i_)
    x = torch.cat([ni, nt], dim=1)
    qkv = (x @ wqkv.to(dtype).to(dev).t()).view(B, Ni + Nt, 3, H, D)
    q, k, v = qkv.unbind(2)                       # strided views: channel stride 1, row stride 3*H*D
    q, k = hln(q, k, heads_second=False, eps=1e-6)
    q, k = rope(q, k, pos.to(dtype).to(dev), seq_cutoff=Ni, heads_second=False)
    out = attn(q, k, v, bias.to(dtype).to(dev).contiguous())
    grads = torch.autograd.grad(out, [t_, i_, norm.weight1, norm.weight2], dout.to(dtype).to(dev))

    def rel(a, b):
        return ((a.detach().float().cpu() - b).norm() / b.norm()).item()

    assert rel(out, ref_out.detach()) < 2e-2
    for name, a, b in zip(("d_text", "d_image", "d_w1", "d_w2"), grads, ref_grads):
        assert rel(a, b) < 4e-2, f"{name}: relative error {rel(a, b):.3e}"
    # padded text keys get no gradient through attention: rows past text_len of d_text come
    # only from their own query positions, so they are finite and small but not required zero
    assert all(torch.isfinite(gr.float()).all() for gr in grads)
