"""tcgen05 flash attention over packed sequences against an fp32 PyTorch reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference(q, k, v, lens, causal, scale):
    """fp32 attention per sequence; returns (out [T, Hq, D], lse [Hq, T])."""
    hq, hkv = q.shape[1], k.shape[1]
    outs, lses = [], []
    s = 0
    for n in lens:
        qi = q[s:s + n].float().transpose(0, 1)  # [Hq, n, D]
        ki = k[s:s + n].float().transpose(0, 1).repeat_interleave(hq // hkv, 0)
        vi = v[s:s + n].float().transpose(0, 1).repeat_interleave(hq // hkv, 0)
        z = torch.einsum("hqd,hkd->hqk", qi, ki) * scale
        if causal:
            z = z.masked_fill(torch.ones(n, n, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
        lses.append(torch.logsumexp(z, -1))
        outs.append(torch.einsum("hqk,hkd->hqd", torch.softmax(z, -1), vi).transpose(0, 1))
        s += n
    return torch.cat(outs), torch.cat(lses, 1)


def _inputs(lens, hq, hkv, d, seed=0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    t = sum(lens)
    q = torch.randn(t, hq, d, generator=g, device="cuda").bfloat16()
    k = torch.randn(t, hkv, d, generator=g, device="cuda").bfloat16()
    v = torch.randn(t, hkv, d, generator=g, device="cuda").bfloat16()
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device="cuda")
    return q, k, v, cu


CASES = [([1], 4, 2, 64), ([17, 1, 257], 4, 2, 128), ([128, 256, 129], 8, 2, 64), ([300, 700], 8, 8, 128), ([4700], 4, 1, 128), ([1000, 33, 515], 6, 2, 128)]


@pytest.mark.parametrize("lens,hq,hkv,d", CASES)
@pytest.mark.parametrize("causal", [True, False])
def test_flash_attention_forward(lens, hq, hkv, d, causal):
    from unirl_b200.ops._ext import require_ext

    C = require_ext()
    q, k, v, cu = _inputs(lens, hq, hkv, d)
    scale = 1.0 / math.sqrt(d)
    out, lse = C.attn_varlen_fwd(q, k, v, cu, max(lens), causal, scale)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0, "a bounded wait expired inside the attention kernel"
    ref, ref_lse = _reference(q, k, v, lens, causal, scale)
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, f"max |out - ref| = {err}"
    torch.testing.assert_close(lse, ref_lse, atol=2e-3, rtol=1e-3)


def test_flash_attention_forward_on_strided_views_of_a_fused_qkv_buffer():
    from unirl_b200.ops._ext import require_ext

    C = require_ext()
    lens, hq, hkv, d = [200, 333], 8, 2, 128
    t = sum(lens)
    g = torch.Generator(device="cuda").manual_seed(3)
    qkv = torch.randn(t, (hq + 2 * hkv) * d, generator=g, device="cuda").bfloat16()
    q = qkv[:, : hq * d].view(t, hq, d)
    k = qkv[:, hq * d : (hq + hkv) * d].view(t, hkv, d)
    v = qkv[:, (hq + hkv) * d :].view(t, hkv, d)
    cu = torch.tensor([0, 200, 533], dtype=torch.int32, device="cuda")
    out, _ = C.attn_varlen_fwd(q, k, v, cu, 333, True, 1.0 / math.sqrt(d))
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0
    ref, _ = _reference(q, k, v, lens, True, 1.0 / math.sqrt(d))
    assert (out.float() - ref).abs().max().item() < 2e-2


BWD_CASES = [([1], 4, 2, 64), ([17, 1, 257], 4, 2, 128), ([128, 256, 129], 8, 2, 64), ([300, 700], 4, 4, 128), ([1000, 33, 515], 6, 2, 128), ([4700], 4, 1, 128)]


@pytest.mark.parametrize("lens,hq,hkv,d", BWD_CASES)
@pytest.mark.parametrize("causal", [True, False])
def test_flash_attention_backward(lens, hq, hkv, d, causal):
    """dQ, dK, dV of the tcgen05 backward against autograd through the fp32 reference."""
    from unirl_b200.ops._ext import require_ext

    C = require_ext()
    q, k, v, cu = _inputs(lens, hq, hkv, d, seed=5)
    scale = 1.0 / math.sqrt(d)
    g = torch.randn(q.shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(6)).bfloat16()
    out, lse = C.attn_varlen_fwd(q, k, v, cu, max(lens), causal, scale)
    dq, dk, dv = C.attn_varlen_bwd(g, q, k, v, out, lse, cu, max(lens), causal, scale)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0, "a bounded wait expired inside the attention kernels"
    qr, kr, vr = (x.detach().float().requires_grad_() for x in (q, k, v))
    ref, _ = _reference(qr, kr, vr, lens, causal, scale)
    (ref * g.float()).sum().backward()
    for name, got, want in (("dq", dq, qr.grad), ("dk", dk, kr.grad), ("dv", dv, vr.grad)):
        err = (got.float() - want).abs().max().item()
        tol = 2e-2 * max(1.0, want.abs().max().item())
        assert err < tol, f"{name}: max err {err} (tolerance {tol})"


def test_varlen_attention_op_is_native_and_differentiable():
    """The public op routes bf16 head_dim 64 / 128 problems to the native kernels (forward and backward)."""
    from unirl_b200.ops.attention import _varlen_impl, varlen_attention, varlen_attention_reference

    assert _varlen_impl() == "native"
    lens, hq, hkv, d = [150, 90], 8, 4, 128
    q, k, v, cu = _inputs(lens, hq, hkv, d, seed=9)
    q.requires_grad_(); k.requires_grad_(); v.requires_grad_()
    out = varlen_attention(q, k, v, cu, max(lens), True)
    out.float().pow(2).sum().backward()
    qr, kr, vr = (x.detach().float().requires_grad_() for x in (q, k, v))
    ref = varlen_attention_reference(qr, kr, vr, cu, True)
    ref.pow(2).sum().backward()
    assert (out.float() - ref).abs().max().item() < 2e-2
    for got, want in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert (got.float() - want).abs().max().item() < 3e-2 * max(1.0, want.abs().max().item())
