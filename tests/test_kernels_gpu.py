"""sm_100a kernels vs plain PyTorch fp32 references of the same op (run on the B200 box)."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _C():
    from unirl_b200.ops._ext import require_ext

    return require_ext()


def _close(a, b, atol, rtol, what=""):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"{what}: max err {err.max().item():.4e} (tol {tol.max().item():.3e}), mean err {err.mean().item():.3e}"


@pytest.mark.parametrize("rows,dim,dtype", [(7, 256, torch.bfloat16), (33, 2560, torch.bfloat16), (5, 100, torch.float32), (2051, 2560, torch.bfloat16),
                                            (1500, 1536, torch.bfloat16), (1100, 3584, torch.bfloat16)])
def test_rmsnorm_fwd_bwd(rows, dim, dtype):
    from unirl_b200.ops.norm import rmsnorm, rmsnorm_reference

    torch.manual_seed(0)
    x = torch.randn(rows, dim, device="cuda", dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(dim, device="cuda")).to(dtype).requires_grad_()
    y = rmsnorm(x, w, 1e-6)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = rmsnorm_reference(xr, wr, 1e-6)
    yr.backward(g.float())
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    _close(y, yr, tol, tol, "rmsnorm fwd")
    _close(x.grad, xr.grad, tol, tol, "rmsnorm dx")
    _close(w.grad, wr.grad, tol * 4, tol, "rmsnorm dw")


def test_add_rmsnorm_and_modulate():
    from unirl_b200.ops.norm import add_rmsnorm, layernorm_modulate, layernorm_modulate_reference, rmsnorm_reference

    torch.manual_seed(1)
    x = torch.randn(19, 512, device="cuda", dtype=torch.bfloat16)
    r = torch.randn_like(x)
    w = torch.randn(512, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        y, r2 = add_rmsnorm(x, r, w, 1e-6)
    rr = (x.float() + r.float()).to(torch.bfloat16)
    _close(r2, rr, 1e-2, 1e-2, "residual")
    _close(y, rmsnorm_reference(rr, w, 1e-6), 3e-2, 3e-2, "add_rmsnorm")
    xx = torch.randn(2, 9, 384, device="cuda", dtype=torch.bfloat16)
    sh, sc = torch.randn(2, 384, device="cuda", dtype=torch.bfloat16), torch.randn(2, 384, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        _close(layernorm_modulate(xx, sh, sc), layernorm_modulate_reference(xx.float(), sh.float(), sc.float(), 1e-6), 5e-2, 3e-2, "adaLN")


@pytest.mark.parametrize("hq,hkv,d", [(4, 2, 64), (32, 8, 128)])
def test_qk_norm_rope_fwd_bwd(hq, hkv, d):
    from unirl_b200.ops.rope import qk_norm_rope, qk_norm_rope_reference

    torch.manual_seed(2)
    t = 37
    qkv = torch.randn(t, (hq + 2 * hkv) * d, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    qw = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_()
    kw = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16).requires_grad_()
    pos = torch.randint(0, 5000, (t,), device="cuda")
    q, k, v = qk_norm_rope(qkv, qw, kw, pos, hq, hkv, d, 1e6, 1e-6)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    a, b, c = (x.detach().float().requires_grad_() for x in (qkv, qw, kw))
    qr, kr, vr = qk_norm_rope_reference(a, b, c, pos, hq, hkv, d, 1e6, 1e-6)
    torch.autograd.backward([qr, kr, vr], [gq.float(), gk.float(), gv.float()])
    _close(q, qr, 3e-2, 2e-2, "q")
    _close(k, kr, 3e-2, 2e-2, "k")
    _close(v, vr, 1e-6, 0, "v")
    _close(qkv.grad, a.grad, 4e-2, 3e-2, "dqkv")
    _close(qw.grad, b.grad, 0.5, 5e-2, "dqw")
    _close(kw.grad, c.grad, 0.5, 5e-2, "dkw")


def test_swiglu():
    from unirl_b200.ops.activation import swiglu, swiglu_reference

    torch.manual_seed(3)
    gu = torch.randn(45, 2 * 352, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = swiglu(gu)
    g = torch.randn_like(y)
    y.backward(g)
    r = gu.detach().float().requires_grad_()
    yr = swiglu_reference(r)
    yr.backward(g.float())
    _close(y, yr, 2e-2, 2e-2, "swiglu")
    _close(gu.grad, r.grad, 3e-2, 2e-2, "swiglu bwd")


@pytest.mark.parametrize("kind", ["clip", "drpo", "spo", "dppo"])
def test_policy_losses(kind):
    from unirl_b200.ops import policy_loss as PL

    torch.manual_seed(4)
    n = 5000
    new = (-2 + 0.3 * torch.randn(n, device="cuda")).requires_grad_()
    old = (new.detach() + 0.2 * torch.randn(n, device="cuda"))
    adv = torch.randn(n, device="cuda")
    newr = new.detach().clone().requires_grad_()
    if kind == "clip":
        (l, m), (lr, mr) = PL.ppo_clip(new, old, adv, 0.2, 0.28), PL.ppo_clip_reference(newr, old, adv, 0.2, 0.28)
    elif kind in ("drpo", "spo"):
        (l, m), (lr, mr) = PL.drpo(new, old, adv, 12.5, kind == "drpo"), PL.drpo_reference(newr, old, adv, 12.5, kind == "drpo")
    else:
        b, s = 50, 100
        nm, om = torch.randn(b, s, 4, 8, 8, device="cuda"), None
        om = nm + 0.01 * torch.randn_like(nm)
        sig = torch.full((1, s, 1, 1, 1), 0.05, device="cuda")
        new2, newr2 = new.view(b, s), newr.view(b, s)
        (l, m), (lr, mr) = PL.flow_dppo(new2, old.view(b, s), nm, om, adv.view(b, s), sig, 0.02), PL.flow_dppo_reference(
            newr2, old.view(b, s), nm, om, adv.view(b, s), sig, 0.02)
    l.mean().backward()
    lr.mean().backward()
    _close(l, lr, 1e-5, 1e-4, "loss")
    _close(new.grad, newr.grad, 1e-8, 1e-3, "dlogp")
    for k in mr:
        _close(m[k], mr[k], 1e-4, 2e-3, f"metric {k}")


def test_sampler_distribution_and_logp():
    from unirl_b200.ops.sampling import sample

    torch.manual_seed(5)
    v = 1000
    logits = torch.randn(1, v, device="cuda") * 2
    rows = logits.expand(4096, v).contiguous()
    tok, lp = sample(rows, 0.7, seed=11, step=3)
    ref = torch.log_softmax(logits[0] / 0.7, -1)
    _close(lp, ref[tok], 1e-4, 1e-4, "sampled logp")
    freq = torch.bincount(tok, minlength=v).float() / tok.numel()
    top = ref.exp().topk(5).indices
    assert (freq[top] - ref.exp()[top]).abs().max() < 0.03
    tok2, _ = sample(rows, 0.7, seed=11, step=3)
    assert torch.equal(tok, tok2), "sampler must be a pure function of (seed, step, row)"
    tok3, _ = sample(rows, 0.7, seed=11, step=4)
    assert not torch.equal(tok, tok3)
    g, glp = sample(logits.to(torch.bfloat16), 0.0)
    assert int(g) == int(logits.to(torch.bfloat16).float().argmax())


def test_adamw_and_sum_squares():
    from unirl_b200.ops.optim import adamw_reference, adamw_step, sum_squares

    torch.manual_seed(6)
    n = 100_003
    master = torch.randn(n, device="cuda")
    grad = torch.randn(n, device="cuda").to(torch.bfloat16)
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    low = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    ema = master.clone()
    rm, rmm, rv, rema = master.clone(), m.clone(), v.clone(), ema.clone()
    coef = torch.tensor([0.5], device="cuda")
    for step in (1, 2, 3):
        adamw_step(master, grad, m, v, lr=1e-3, weight_decay=0.01, step=step, low=low, ema=ema, ema_decay=0.99, grad_scale_tensor=coef)
        adamw_reference(rm, grad, rmm, rv, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=step, grad_scale=0.5, ema=rema, ema_decay=0.99)
    _close(master, rm, 1e-6, 1e-5, "adamw master")
    _close(low, rm.to(torch.bfloat16), 1e-2, 1e-2, "adamw low")
    _close(ema, rema, 1e-6, 1e-5, "ema")
    _close(sum_squares(grad), grad.float().pow(2).sum(), 1e-2, 1e-4, "sum_squares")


def _kept_mask(z, top_k, top_p):
    """The reference sampler's truncation on fp32 rows without ties: True where an entry survives."""
    filt = z.clone()
    if top_k and top_k < z.shape[-1]:
        kth = torch.topk(filt, top_k, -1).values[..., -1:]
        filt = filt.masked_fill(filt < kth, float("-inf"))
    if top_p < 1.0:
        sv, si = torch.sort(filt, -1, descending=True)
        pr = torch.softmax(sv, -1)
        drop = pr.cumsum(-1) - pr > top_p
        sv = sv.masked_fill(drop, float("-inf"))
        filt = torch.full_like(filt, float("-inf")).scatter(-1, si, sv)
    return torch.isfinite(filt)


@pytest.mark.parametrize("top_k,top_p", [(5, 1.0), (0, 0.8), (50, 0.9), (1, 1.0), (0, 0.05)])
def test_truncated_sampling_kernel(top_k, top_p):
    """Top-k / top-p sampling by radix selection: draws stay inside the reference's kept set, the recorded log-prob is the
    full-vocabulary one, and the draw frequencies follow the renormalised probabilities."""
    from unirl_b200.ops.sampling import sample

    torch.manual_seed(31)
    b, v, temp = 16, 1000, 0.7
    logits = torch.randn(b, v, device="cuda") * 2.0
    z = logits / temp
    keep = _kept_mask(z, top_k, top_p)
    full_lp = torch.log_softmax(z, -1)
    probs = torch.softmax(z.masked_fill(~keep, float("-inf")), -1)
    draws = 3000
    counts = torch.zeros(b, v, device="cuda")
    for step in range(draws):
        tok, lp = sample(logits, temp, top_k, top_p, seed=7, step=step)
        assert bool(keep.gather(1, tok[:, None]).all()), "a draw fell outside the kept set"
        if step < 3:
            torch.testing.assert_close(lp, full_lp.gather(1, tok[:, None]).squeeze(1), atol=1e-4, rtol=1e-4)
        counts.scatter_add_(1, tok[:, None], torch.ones(b, 1, device="cuda"))
    freq = counts / draws
    assert float((freq - probs).abs().max()) < 0.05, "draw frequencies do not follow the truncated distribution"


def test_truncated_sampling_large_vocab_bf16_is_deterministic():
    C = _C()
    torch.manual_seed(32)
    logits = (torch.randn(8, 151936, device="cuda") * 3.0).bfloat16()
    a = C.sample_truncated(logits, 1.0, 40, 0.95, 3, 11)
    b = C.sample_truncated(logits, 1.0, 40, 0.95, 3, 11)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), "same (seed, step) must give the same draw (tensor-parallel ranks rely on it)"
    z = logits.float()
    kth = torch.topk(z, 40, -1).values[:, -1:]
    assert bool((z.gather(1, a[0][:, None]) >= kth).all())
    torch.testing.assert_close(a[1], torch.log_softmax(z, -1).gather(1, a[0][:, None]).squeeze(1), atol=2e-3, rtol=1e-3)


@pytest.mark.parametrize("name", ["flow", "cps", "dance"])
def test_sde_step_matches_strategy(name):
    from unirl_b200.ops.sde_step import sde_step
    from unirl_b200.sde import get_sigma_schedule, make_strategy

    torch.manual_seed(7)
    st = make_strategy(name)
    sig = get_sigma_schedule(10, 3.0).cuda()
    x = torch.randn(3, 16, 32, 32, device="cuda", dtype=torch.bfloat16)
    v = torch.randn_like(x).requires_grad_()
    noise = torch.randn(x.shape, device="cuda")
    prev, lp, mean = sde_step(st, v, x, sig[2], sig[3], eta=0.7, noise=noise)
    rprev, rlp, rmean = st.denoise(v.detach(), x, sig[2], sig[3], eta=0.7, noise=noise)
    _close(prev, rprev, 2e-2, 1e-2, "prev (one bf16 ulp of storage rounding allowed)")
    _close(mean, rmean, 1e-5, 1e-5, "mean")
    _close(lp, rlp, 1e-3, 1e-3, "logp")
    stored = prev.to(torch.bfloat16)
    p2, lp2, m2 = sde_step(st, v, x, sig[2], sig[3], eta=0.7, prev_sample=stored)
    vr = v.detach().clone().requires_grad_()
    _, rlp2, rm2 = st.denoise(vr, x, sig[2], sig[3], eta=0.7, prev_sample=stored)
    _close(lp2, rlp2, 1e-3, 1e-3, "replay logp")
    (lp2.sum() + 0.01 * m2.sum()).backward()
    (rlp2.sum() + 0.01 * rm2.sum()).backward()
    _close(v.grad, vr.grad, 1e-4, 2e-2, "replay dv")


@pytest.mark.parametrize("dtype,shape", [(torch.float32, (2, 70, 96)), (torch.bfloat16, (3, 333, 1536))])
def test_layernorm_modulate_backward_kernel(dtype, shape):
    """adaLN with gradients: dx, dshift, dscale of the kernel pair against autograd through the fp32 PyTorch statement."""
    from unirl_b200.ops.norm import layernorm_modulate, layernorm_modulate_reference

    torch.manual_seed(13)
    b, l, d = shape
    x = torch.randn(b, l, d, device="cuda").to(dtype).requires_grad_()
    sh = (torch.randn(b, d, device="cuda") * 0.3).to(dtype).requires_grad_()
    sc = (torch.randn(b, d, device="cuda") * 0.3).to(dtype).requires_grad_()
    xr, shr, scr = (t.detach().float().requires_grad_() for t in (x, sh, sc))
    y = layernorm_modulate(x, sh, sc, 1e-6)
    yr = layernorm_modulate_reference(xr, shr, scr, 1e-6)
    g = torch.randn_like(yr)
    y.backward(g.to(dtype))
    yr.backward(g)
    tol = 3e-2 if dtype == torch.bfloat16 else 2e-4
    _close(y, yr, tol, tol, "adaLN forward")
    _close(x.grad, xr.grad, tol, tol, "dx")
    _close(sh.grad, shr.grad, tol * (l ** 0.5), tol, "dshift (a sum over the tokens)")
    _close(sc.grad, scr.grad, tol * (l ** 0.5), tol, "dscale")


@pytest.mark.parametrize("interleaved", [True, False])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_table_driven_rotary_kernel(interleaved, dtype):
    """Rotation by per-token tables shared over the batch: forward and gradient against the fp32 PyTorch statement, both pairings."""
    from unirl_b200.ops.rope import rope_table, rope_table_reference

    torch.manual_seed(12)
    b, l, h, d = 2, 37, 3, 64
    ang = torch.rand(l, d // 2, device="cuda") * 6.28
    cos, sin = ang.cos(), ang.sin()
    x = torch.randn(b, l, h, d, device="cuda").to(dtype).requires_grad_()
    xr = x.detach().float().requires_grad_()
    y, yr = rope_table(x, cos, sin, interleaved), rope_table_reference(xr, cos, sin, interleaved)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    _close(y, yr, tol, tol, "rotated")
    g = torch.randn_like(yr)
    y.backward(g.to(dtype))
    yr.backward(g)
    _close(x.grad, xr.grad, tol, tol, "gradient (the rotation by the opposite angle)")
    # three leading dimensions collapse the same way as two
    x3 = torch.randn(l, h, d, device="cuda").to(dtype)
    _close(rope_table(x3, cos, sin, interleaved), rope_table_reference(x3.float(), cos, sin, interleaved), tol, tol, "no batch dimension")


def test_sde_step_with_guidance_combined_in_the_kernel():
    """Two branches of a classifier-free-guidance pass go to the step kernel separately: same transition, log-prob and gradients as the
    combination formed first (fp32 reference), in sampling and in differentiable replay."""
    from unirl_b200.ops.sde_step import sde_step
    from unirl_b200.sde import get_sigma_schedule, make_strategy

    torch.manual_seed(11)
    st = make_strategy("flow")
    sig = get_sigma_schedule(10, 3.0).cuda()
    g = 4.5
    x = torch.randn(3, 16, 32, 32, device="cuda")
    vc, vu = torch.randn_like(x).requires_grad_(), torch.randn_like(x).requires_grad_()
    noise = torch.randn(x.shape, device="cuda")
    prev, lp, mean = sde_step(st, vc, x, sig[2], sig[3], eta=0.7, noise=noise, noise_pred_uncond=vu, guidance_scale=g)
    ref_v = (vu + g * (vc - vu)).detach()
    rprev, rlp, rmean = st.denoise(ref_v, x, sig[2], sig[3], eta=0.7, noise=noise)
    _close(prev, rprev, 1e-5, 1e-5, "prev")
    _close(mean, rmean, 1e-5, 1e-5, "mean")
    _close(lp, rlp, 1e-3, 1e-3, "logp")
    _, lp2, m2 = sde_step(st, vc, x, sig[2], sig[3], eta=0.7, prev_sample=prev, noise_pred_uncond=vu, guidance_scale=g)
    rc, ru = vc.detach().clone().requires_grad_(), vu.detach().clone().requires_grad_()
    _, rlp2, rm2 = st.denoise(ru + g * (rc - ru), x, sig[2], sig[3], eta=0.7, prev_sample=prev)
    _close(lp2, rlp2, 1e-3, 1e-3, "replay logp")
    (lp2.sum() + 0.01 * m2.sum()).backward()
    (rlp2.sum() + 0.01 * rm2.sum()).backward()
    _close(vc.grad, rc.grad, 1e-4, 2e-2, "replay dv_cond")
    _close(vu.grad, ru.grad, 1e-4, 2e-2, "replay dv_uncond")


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 512, 320), (1000, 6144, 2560), (257, 2560, 9728), (64, 384, 128)])
def test_gemm_tcgen05(m, n, k):
    C = _C()
    torch.manual_seed(8)
    a = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.5).to(torch.bfloat16)
    r = torch.randn(m, n, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    c = C.gemm_bf16_tn(a, b, None, 0)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0, "a bounded wait expired inside the GEMM"
    _close(c, ref, 0.15, 2e-2, "gemm")
    c2 = C.gemm_bf16_tn(a, b, r, 1)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0
    _close(c2, ref + r.float(), 0.15, 2e-2, "gemm+residual")


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (300, 520, 136), (1000, 2560, 6144), (2560, 9728, 1003), (72, 384, 128), (4096, 2560, 9728)])
@pytest.mark.parametrize("a_mn,b_mn", [(False, True), (True, True), (True, False), (False, False)])
def test_gemm_tcgen05_operand_layouts(m, n, k, a_mn, b_mn):
    """Every operand layout of the tcgen05 GEMM against an fp32 product: K-major / MN-major A and B (the layouts of the forward,
    input-gradient and weight-gradient GEMMs), bf16 output, fp32 overwrite and fp32 accumulation."""
    C = _C()
    if (not a_mn and k % 8) or (not b_mn and k % 8) or (a_mn and m % 8):
        pytest.skip("this layout needs 16-byte aligned rows")
    torch.manual_seed(18)
    a = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.5).to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    a_in = a.t().contiguous() if a_mn else a
    b_in = b.t().contiguous() if b_mn else b
    c = C.gemm_bf16(a_in, b_in, a_mn, b_mn)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0, "a bounded wait expired inside the GEMM"
    _close(c, ref, 0.2, 2e-2, "bf16 out")
    acc = torch.full((m, n), 3.0, device="cuda")
    C.gemm_bf16(a_in, b_in, a_mn, b_mn, acc, False)
    _close(acc, ref, 0.05, 1e-2, "fp32 overwrite")
    C.gemm_bf16(a_in, b_in, a_mn, b_mn, acc, True)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0
    _close(acc, 2 * ref, 0.1, 1e-2, "fp32 accumulate")


def test_gemm_tcgen05_strided_operands_and_output():
    """Row-strided views (a column block of a wider matrix) as operands and as the fp32 accumulator."""
    C = _C()
    torch.manual_seed(19)
    big_a = (torch.randn(700, 512, device="cuda") * 0.5).to(torch.bfloat16)
    big_b = (torch.randn(700, 640, device="cuda") * 0.5).to(torch.bfloat16)
    a, b = big_a[:, 128:384], big_b[:, 64:576]  # stored [K=700, M=256] and [K=700, N=512]
    out = torch.zeros(256, 1024, device="cuda")
    C.gemm_bf16(a, b, True, True, out[:, 256:768], True)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0
    _close(out[:, 256:768], a.float().t() @ b.float(), 0.05, 1e-2, "strided dW")
    assert float(out[:, :256].abs().max()) == 0 and float(out[:, 768:].abs().max()) == 0


@pytest.mark.parametrize("t,v,k,temp", [(100, 1000, 64, 1.0), (517, 4096, 256, 0.7)])
def test_linear_dlogits_epilogue(t, v, k, temp):
    C = _C()
    torch.manual_seed(20)
    h = (torch.randn(t, k, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(v, k, device="cuda") * 0.05).to(torch.bfloat16)
    tgt = torch.randint(0, v, (t,), device="cuda", dtype=torch.int32)
    g = torch.randn(t, device="cuda")
    z = (h.float() @ w.float().t()) / temp
    lse = torch.logsumexp(z, -1)
    ref = (g / temp)[:, None] * (torch.nn.functional.one_hot(tgt.long(), v).float() - torch.softmax(z, -1))
    dz = C.linear_dlogits(h, w, tgt, lse, g, temp, 0)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0
    _close(dz, ref, 2e-2, 2e-2, "dZ")
    half = v // 2 // 8 * 8  # a vocabulary chunk that starts at a non-zero column
    dz2 = C.linear_dlogits(h, w[half:], tgt, lse, g, temp, half)
    _close(dz2, ref[:, half:], 2e-2, 2e-2, "dZ chunk")


@pytest.mark.parametrize("m,n,k", [(128, 6144, 2560), (128, 2560, 4096), (128, 19456, 2560), (77, 2560, 9728), (256, 2560, 4096), (130, 1096, 128)])
def test_gemm_skinny_cluster_split_k(m, n, k):
    C = _C()
    torch.manual_seed(12)
    a = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16)
    b = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    r = torch.randn(m, n, device="cuda").to(torch.bfloat16)
    ref = a.float() @ b.float().t()
    c = C.gemm_bf16_tn_skinny(a, b)
    c_again = C.gemm_bf16_tn_skinny(a, b)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0, "a bounded wait expired inside the GEMM"
    _close(c, ref, 0.05, 2e-2, "skinny gemm")
    assert torch.equal(c, c_again), "partials are summed in rank order: the result must be reproducible"
    out = torch.empty(m, n, device="cuda", dtype=torch.bfloat16)
    c2 = C.gemm_bf16_tn_skinny(a, b, r, out)
    torch.cuda.synchronize()
    assert c2.data_ptr() == out.data_ptr()
    _close(c2, ref + r.float(), 0.05, 2e-2, "skinny gemm + residual")
    for splits in (1, 2, 3, 5, 8):  # every cluster size the launcher may pick
        C.set_gemm_skinny_splits(splits)
        cs = C.gemm_bf16_tn_skinny(a, b, r)
        torch.cuda.synchronize()
        C.set_gemm_skinny_splits(0)
        assert C.gemm_status(True) == 0
        _close(cs, ref + r.float(), 0.05, 2e-2, f"skinny gemm, cluster of {splits}")


@pytest.mark.parametrize("m,inter,k,splits", [(128, 9728, 2560, 0), (100, 640, 256, 0), (128, 1024, 512, 2), (256, 4864, 2560, 0)])
def test_gemm_skinny_swiglu(m, inter, k, splits):
    C = _C()
    torch.manual_seed(13)
    a = (torch.randn(m, k, device="cuda") * 0.3).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device="cuda") * 0.05).to(torch.bfloat16)
    C.set_gemm_skinny_splits(splits)
    out = C.gemm_bf16_tn_skinny(a, w, None, None, 2)
    torch.cuda.synchronize()
    C.set_gemm_skinny_splits(0)
    assert C.gemm_status(True) == 0
    z = a.float() @ w.float().t()
    ref = torch.nn.functional.silu(z[:, :inter]) * z[:, inter:]
    _close(out, ref, 0.05, 3e-2, "skinny gemm + swiglu")


def test_gemm_swiglu_epilogue():
    C = _C()
    torch.manual_seed(9)
    m, inter, k = 300, 640, 256
    a = (torch.randn(m, k, device="cuda") * 0.3).to(torch.bfloat16)
    w = (torch.randn(2 * inter, k, device="cuda") * 0.3).to(torch.bfloat16)
    out = C.gemm_bf16_tn(a, w, None, 2)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0
    z = a.float() @ w.float().t()
    ref = torch.nn.functional.silu(z[:, :inter]) * z[:, inter:]
    _close(out, ref, 0.1, 3e-2, "gemm+swiglu")


@pytest.mark.parametrize("t,v,k,temp", [(100, 1000, 64, 1.0), (700, 4096, 256, 0.7), (130, 151936, 2560, 1.0)])
def test_linear_logprob_fwd_bwd(t, v, k, temp):
    from unirl_b200.ops.logprob import linear_logprob, linear_logprob_reference

    torch.manual_seed(10)
    h = (torch.randn(t, k, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = (torch.randn(v, k, device="cuda") * 0.05).to(torch.bfloat16).requires_grad_()
    tgt = torch.randint(0, v, (t,), device="cuda")
    lp = linear_logprob(h, w, tgt, temp)
    ref = linear_logprob_reference(h.detach(), w.detach(), tgt, temp)
    torch.cuda.synchronize()
    assert _C().gemm_status(True) == 0
    _close(lp, ref, 2e-2, 1e-3, "logprob")
    if v <= 4096:
        g = torch.randn(t, device="cuda")
        lp.backward(g)
        hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
        z = (hr @ wr.t()) / temp
        (torch.log_softmax(z, -1).gather(-1, tgt[:, None]).squeeze(-1) * g).sum().backward()
        _close(h.grad, hr.grad, 2e-2, 5e-2, "dH")
        _close(w.grad, wr.grad, 2e-2, 5e-2, "dW")


def test_linear_sample_matches_unfused():
    C = _C()
    torch.manual_seed(11)
    b, v, k = 64, 5000, 256
    h = (torch.randn(b, k, device="cuda") * 0.5).to(torch.bfloat16)
    w = (torch.randn(v, k, device="cuda") * 0.1).to(torch.bfloat16)
    tok, lp = C.linear_sample(h, w, 0.8, 123, 7, None)
    torch.cuda.synchronize()
    assert C.gemm_status(True) == 0
    ref = torch.log_softmax((h.float() @ w.float().t()) / 0.8, -1)
    _close(lp, ref.gather(-1, tok[:, None]).squeeze(-1), 3e-2, 1e-3, "fused sample logp")
    assert int(tok.min()) >= 0 and int(tok.max()) < v
    # same (seed, step) => same draw; other step => other draw
    tok2, _ = C.linear_sample(h, w, 0.8, 123, 7, None)
    assert torch.equal(tok, tok2)


@pytest.mark.parametrize("hq,hkv,d,page", [(4, 2, 64, 16), (32, 8, 128, 64), (28, 4, 128, 32)])
def test_paged_decode_attention(hq, hkv, d, page):
    from unirl_b200.ops.attention import kv_cache_write, paged_decode_attention, paged_decode_attention_reference

    torch.manual_seed(12)
    lens = [1, 17, 64, 65, 300, 1000]
    b = len(lens)
    max_pages = (max(lens) + page - 1) // page
    n_pages = b * max_pages + 3
    kc = torch.zeros(n_pages, hkv, page, d, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    perm = torch.randperm(n_pages)[: b * max_pages].view(b, max_pages).to(torch.int32).cuda()
    for i, n in enumerate(lens):
        k = torch.randn(n, hkv, d, device="cuda", dtype=torch.bfloat16)
        v = torch.randn(n, hkv, d, device="cuda", dtype=torch.bfloat16)
        pos = torch.arange(n, device="cuda")
        slots = perm[i, (pos // page)].long() * page + pos % page
        kv_cache_write(k, v, kc, vc, slots)
    q = torch.randn(b, hq, d, device="cuda", dtype=torch.bfloat16)
    sl = torch.tensor(lens, dtype=torch.int32, device="cuda")
    out = paged_decode_attention(q, kc, vc, perm, sl, None, None, max(lens))
    ref = paged_decode_attention_reference(q, kc, vc, perm, sl)
    _close(out, ref, 2e-2, 2e-2, "paged decode attention")


def test_kv_cache_write_matches_reference():
    from unirl_b200.ops.attention import kv_cache_write

    torch.manual_seed(13)
    kc = torch.zeros(10, 2, 16, 64, device="cuda", dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    k, v = torch.randn(20, 2, 64, device="cuda", dtype=torch.bfloat16), torch.randn(20, 2, 64, device="cuda", dtype=torch.bfloat16)
    slots = torch.randperm(160, device="cuda")[:20]
    kv_cache_write(k, v, kc, vc, slots)
    kr, vr = torch.zeros_like(kc).cpu(), torch.zeros_like(vc).cpu()
    kv_cache_write(k.cpu(), v.cpu(), kr, vr, slots.cpu())
    assert torch.equal(kc.cpu(), kr) and torch.equal(vc.cpu(), vr)


def test_rollout_replay_parity_and_train_step_tiny():
    """Decode path (paged KV, graph) vs packed replay path: same log-probs; one GRPO step runs."""
    from unirl_b200.models.qwen3 import Qwen3ARConditions, Qwen3Pipeline, Qwen3PipelineConfig
    from unirl_b200.models.qwen3.chat_template import pad_right
    from unirl_b200.types import ARSamplingParams, RolloutReq

    torch.manual_seed(14)
    pipe = Qwen3Pipeline.from_config(Qwen3PipelineConfig(model_precision="bf16", device="cuda"))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(3, 4096, (int(n),), generator=g).tolist() for n in (5, 40, 77, 130)]
    req = RolloutReq(sample_ids=[f"s{i}" for i in range(4)], group_ids=["a", "a", "b", "b"], request_conditions={"prompt": pad_right(prompts, 0)},
                     sampling_params=ARSamplingParams(temperature=1.0, top_p=1.0, top_k=0, max_new_tokens=40))
    with torch.no_grad():
        resp = pipe.generate(req)
    tr = resp.tracks["ar"]
    new = pipe.ar.replay(Qwen3ARConditions.from_dict(tr.conditions), segment=tr.segment, temperature=1.0)
    diff = (new.detach().cpu() - tr.segment.log_probs).abs()
    # Measured on this model (three seeds): mean 0.0012-0.0015, max 0.0046-0.0070 -- the same size as either path's distance from an fp32
    # replay (mean 0.0018), i.e. bf16 rounding of two different kernel sequences.  Bounds at about three times that.
    assert diff.mean() < 0.004 and diff.max() < 0.02, f"rollout/replay gap too large: mean {diff.mean():.4f} max {diff.max():.4f}"
    new.sum().backward()
    assert pipe.bundle.transformer.layers[0].qkv_proj.grad is not None


@pytest.mark.parametrize("cascade", [False, True])
def test_decode_bookkeeping_kernels_match_the_tensor_op_path(cascade):
    """record + advance and prepare as one kernel each: every state tensor identical to the element-wise composition, over several steps,
    with stop tokens, the length limit and rows that are already finished."""
    from unirl_b200.rollout.engine.native_ar.generator import _DecodeState

    torch.manual_seed(21)
    b, max_new, ps, pages = 37, 6, 16, 12
    dev = torch.device("cuda")
    states = [_DecodeState(b, max_new, dev) for _ in range(2)]
    pos0 = torch.randint(0, 100, (b,), device=dev)
    off = torch.randint(0, 50, (b,), device=dev)
    bt = torch.randint(1, 500, (b, pages), device=dev, dtype=torch.int32)
    stop = torch.tensor([3, 7], device=dev)
    shared = torch.randint(0, 3, (b,), device=dev, dtype=torch.int32) * ps
    for st in states:
        st.positions.copy_(pos0)
        st.rope_offset.copy_(off)
        st.finished[::5] = True
        if cascade:
            st.prefix_len = shared.clone()
            st.suffix_lens = torch.zeros(b, dtype=torch.int32, device=dev)
    ref, fused = states
    ref._native = lambda: None  # the tensor-op composition
    for step in range(8):
        tok = torch.randint(0, 10, (b,), device=dev)
        lp = -torch.rand(b, device=dev)
        for st in states:
            st.prepare(bt, ps)
            st.record(tok, lp, stop, fuse_advance=True)
            st.advance()
        for name in ("out_tokens", "out_logp", "cur_tokens", "positions", "slots", "rope_pos", "seq_lens", "lengths", "finished", "step_counter") + (("suffix_lens",) if cascade else ()):
            assert torch.equal(getattr(ref, name), getattr(fused, name)), (name, step)
    assert bool(fused.finished.all()) and int(fused.step_counter) == 8


def test_rope_with_fused_cache_write_matches_two_step_path():
    from unirl_b200.ops.attention import kv_cache_write
    from unirl_b200.ops.rope import qk_norm_rope, qk_norm_rope_cached

    torch.manual_seed(0)
    T, hq, hkv, d, page, pages = 37, 8, 2, 128, 16, 9
    qkv = torch.randn(T, (hq + 2 * hkv) * d, device="cuda").bfloat16()
    qw, kw = (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16(), (1 + 0.1 * torch.randn(d, device="cuda")).bfloat16()
    pos = torch.randint(0, 4000, (T,), device="cuda")
    slots = torch.randperm(pages * page, device="cuda")[:T]
    with torch.no_grad():
        q0, k0, v0 = qk_norm_rope(qkv, qw, kw, pos, hq, hkv, d, 1e6, 1e-6)
        kc0, vc0 = torch.zeros(pages, hkv, page, d, device="cuda", dtype=torch.bfloat16), torch.zeros(pages, hkv, page, d, device="cuda", dtype=torch.bfloat16)
        kv_cache_write(k0, v0, kc0, vc0, slots)
        for dense in (True, False):
            kc, vc = torch.zeros_like(kc0), torch.zeros_like(vc0)
            q, k, v = qk_norm_rope_cached(qkv, qw, kw, pos, hq, hkv, d, 1e6, 1e-6, kc, vc, slots, dense)
            assert torch.equal(q, q0) and torch.equal(kc, kc0) and torch.equal(vc, vc0)
            assert (k is None and v is None) if not dense else (torch.equal(k, k0) and torch.equal(v, v0))


def test_decode_attention_single_split_writes_output_directly():
    from unirl_b200.ops.attention import paged_decode_attention, paged_decode_attention_reference

    torch.manual_seed(1)
    b, hq, hkv, d, page, ctx = 80, 16, 4, 128, 32, 300  # 320 CTAs: one split, no merge pass
    pages_per = (ctx + page - 1) // page
    kc = torch.randn(b * pages_per, hkv, page, d, device="cuda").bfloat16()
    vc = torch.randn_like(kc)
    bt = torch.randperm(b * pages_per, device="cuda").view(b, pages_per).to(torch.int32)
    sl = torch.randint(ctx // 2, ctx + 1, (b,), device="cuda", dtype=torch.int32)
    q = torch.randn(b, hq, d, device="cuda").bfloat16()
    out = paged_decode_attention(q, kc, vc, bt, sl, None, None, ctx)
    ref = paged_decode_attention_reference(q, kc, vc, bt, sl)
    _close(out, ref, 2e-2, 2e-2, "decode attention, single split")


def test_padded_dense_attention_matches_reference_on_ragged_batch():
    from unirl_b200.ops.attention import varlen_attention, varlen_attention_reference

    torch.manual_seed(0)
    lens = [300, 257, 288, 310]
    t, hq, hkv, d = sum(lens), 8, 2, 128
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), device="cuda", dtype=torch.int32)
    q = torch.randn(t, hq, d, device="cuda").bfloat16().requires_grad_()
    k = torch.randn(t, hkv, d, device="cuda").bfloat16().requires_grad_()
    v = torch.randn(t, hkv, d, device="cuda").bfloat16().requires_grad_()
    go = torch.randn(t, hq, d, device="cuda").bfloat16()
    out = varlen_attention(q, k, v, cu, max(lens), True, None, lens)
    out.backward(go)
    got = (out.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone())
    qr, kr, vr = (x.detach().float().requires_grad_() for x in (q, k, v))
    ref = varlen_attention_reference(qr, kr, vr, cu, True, d**-0.5)
    ref.backward(go.float())
    for a, b, name in zip(got, (ref.detach(), qr.grad, kr.grad, vr.grad), ("out", "dq", "dk", "dv")):
        _close(a, b, 3e-2, 3e-2, f"padded dense attention {name}")


def test_cascade_decode_attention_matches_per_sequence_attention():
    """Groups of 4 sequences share their first pages: the shared-prefix kernel must equal plain paged attention over the full tables."""
    from types import SimpleNamespace

    from unirl_b200.ops.attention import paged_decode_attention, paged_decode_attention_cascade

    torch.manual_seed(0)
    b, rows, hq, hkv, d, page = 16, 4, 32, 8, 128, 64
    pre_pages = [3, 0, 9, 5]  # shared whole pages per group (one group has none)
    suf_len = torch.randint(1, 700, (b,))
    suf_pages = [(int(n) + page - 1) // page for n in suf_len]
    n_pages = sum(pre_pages) + sum(suf_pages) + 2
    kc = torch.randn(n_pages, hkv, page, d, device="cuda").bfloat16()
    vc = torch.randn_like(kc)
    perm = torch.randperm(n_pages).tolist()
    pre_t = torch.zeros(b // rows, max(pre_pages), dtype=torch.int32)
    suf_t = torch.zeros(b, max(suf_pages), dtype=torch.int32)
    full_t = torch.zeros(b, max(pre_pages) + max(suf_pages), dtype=torch.int32)
    for g, n in enumerate(pre_pages):
        pre_t[g, :n] = torch.tensor([perm.pop() for _ in range(n)], dtype=torch.int32)
    for i in range(b):
        own = torch.tensor([perm.pop() for _ in range(suf_pages[i])], dtype=torch.int32)
        suf_t[i, : suf_pages[i]] = own
        n = pre_pages[i // rows]
        full_t[i, :n] = pre_t[i // rows, :n]
        full_t[i, n : n + suf_pages[i]] = own
    pre_len = torch.tensor([n * page for n in pre_pages], dtype=torch.int32)
    full_len = (pre_len.repeat_interleave(rows) + suf_len).to(torch.int32)
    q = torch.randn(b, hq, d, device="cuda").bfloat16()
    want = paged_decode_attention(q, kc, vc, full_t.cuda(), full_len.cuda(), None, None, int(full_len.max()))
    cas = SimpleNamespace(prefix_tables=pre_t.cuda(), prefix_lens=pre_len.cuda(), suffix_tables=suf_t.cuda(), suffix_lens=suf_len.to(torch.int32).cuda(), rows=rows)
    got = paged_decode_attention_cascade(q, kc, vc, cas, None, None, int(full_len.max()))
    _close(got, want, 2e-2, 2e-2, "cascade decode attention")


def test_generator_with_shared_prefix_matches_unshared_generation():
    """Same seeds, same prompts (4 samples each): sharing the prompt pages must not change a single sampled token."""
    from unirl_b200.models.qwen3.modeling import Qwen3Config, Qwen3Transformer
    from unirl_b200.rollout.engine.native_ar.generator import ARGenerator

    cfg = Qwen3Config.tiny(num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=4096)
    model = Qwen3Transformer(cfg, dtype=torch.bfloat16, device="cuda").init_weights(0).eval().requires_grad_(False)
    g = torch.Generator().manual_seed(0)
    base = [torch.randint(16, 4096, (int(n),), generator=g) for n in (150, 64, 201)]
    prompts = [p for p in base for _ in range(4)]
    outs = []
    for share in (False, True):
        gen = ARGenerator(model, page_size=64, use_cuda_graph=True, seed=5, share_prefix=share)
        o = gen.generate(prompts, max_new_tokens=24, temperature=1.0, stop_token_ids=[2], seed=11)
        outs.append(o)
        gen.release_cache()
    same = sum(int(torch.equal(a, b)) for a, b in zip(outs[0].tokens, outs[1].tokens))
    assert same >= len(prompts) - 1, f"only {same} of {len(prompts)} sequences identical"  # a bf16 tie may flip one sample
    for a, b in zip(outs[0].log_probs, outs[1].log_probs):
        n = min(a.numel(), b.numel(), 4)
        assert float((a[:n] - b[:n]).abs().max()) < 0.05


def test_linear_weight_grad_accumulates_into_fp32_buffer():
    """The trainer hands its fp32 accumulator to the linear layer; dW must land there (twice after two backward passes) and
    the parameter's own .grad is only a placeholder."""
    from unirl_b200.ops.linear import linear

    torch.manual_seed(21)
    m, n, k = 640, 256, 192
    x = (torch.randn(m, k, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = torch.nn.Parameter((torch.randn(n, k, device="cuda") * 0.1).to(torch.bfloat16))
    buf = torch.zeros(n, k, device="cuda", dtype=torch.float32)
    w._wgrad_accum = lambda: buf
    gy = (torch.randn(m, n, device="cuda") * 0.2).to(torch.bfloat16)
    ref_w = gy.float().t() @ x.detach().float()
    ref_x = gy.float() @ w.detach().float()
    for rep in (1, 2):
        x.grad = None
        linear(x, w).backward(gy)
        torch.cuda.synchronize()
        assert getattr(w, "_wgrad_fused", False), "the fused path did not run"
        _close(buf, ref_w * rep, 2e-2 * rep, 1e-2, f"accumulated dW after {rep} pass(es)")
        _close(x.grad, ref_x, 0.05, 2e-2, "dX")
        w._wgrad_fused = False
        w.grad = None


def test_linear_logprob_weight_grad_accumulates_into_fp32_buffer():
    from unirl_b200.ops.logprob import linear_logprob, linear_logprob_reference

    torch.manual_seed(22)
    t, v, k = 300, 4096, 256
    h = (torch.randn(t, k, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_()
    w = torch.nn.Parameter((torch.randn(v, k, device="cuda") * 0.05).to(torch.bfloat16))
    tgt = torch.randint(0, v, (t,), device="cuda")
    g = torch.randn(t, device="cuda")
    buf = torch.zeros(v, k, device="cuda", dtype=torch.float32)
    w._wgrad_accum = lambda: buf
    linear_logprob(h, w, tgt, 0.8).backward(g)
    torch.cuda.synchronize()
    assert getattr(w, "_wgrad_fused", False)
    hr = h.detach().float().requires_grad_()
    wr = w.detach().float().requires_grad_()
    linear_logprob_reference(hr, wr, tgt, 0.8).backward(g)
    _close(buf, wr.grad, 2.5e-2, 5e-2, "fused lm_head dW")
    _close(h.grad, hr.grad, 2e-2, 5e-2, "lm_head dH")
    shared = torch.nn.Parameter(w.detach().clone())
    shared._wgrad_accum, shared._wgrad_shared = (lambda: buf), True
    linear_logprob(h, shared, tgt, 0.8).backward(g)
    assert not getattr(shared, "_wgrad_fused", False) and shared.grad is not None  # a shared weight keeps the ordinary gradient


def test_sharded_trainer_gradients_with_and_without_gemm_accumulation():
    """One backward pass of a small decoder under the flat sharded trainer (one rank): the fp32 gradient buffer filled by the
    GEMMs directly must match the buffer filled by bf16 weight gradients + the hook's add, and the gradient norm with it."""
    import unirl_b200.ops.linear as L
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.models.qwen3.modeling import AttnMeta, Qwen3Config, Qwen3Transformer
    from unirl_b200.ops.logprob import linear_logprob
    from unirl_b200.parallel.flat_shard import FlatShardedModel

    def run(fused: bool):
        torch.manual_seed(5)
        cfg = Qwen3Config.tiny(vocab_size=2048, hidden_size=256, intermediate_size=512, num_hidden_layers=2, head_dim=64)
        model = Qwen3Transformer(cfg, dtype=torch.bfloat16, device="cuda").init_weights(0)
        sh = FlatShardedModel(model, Comm.world(), block_class_names=("Qwen3DecoderLayer",))
        old = L._WGRAD_FUSION
        L._WGRAD_FUSION = fused
        try:
            n = 768  # >= 512 rows: the projections run on the tcgen05 GEMM, whose backward owns the accumulation
            tokens = torch.randint(0, cfg.vocab_size, (n,), device="cuda")
            meta = AttnMeta(mode="train", positions=torch.arange(n, device="cuda") % 256, cu_seqlens=torch.tensor([0, 256, 512, 768], dtype=torch.int32, device="cuda"),
                            max_seqlen=256, seq_lens_host=[256, 256, 256])
            sh.zero_grad()
            sh.set_grad_sync(True)
            h = model(tokens, meta)
            (linear_logprob(h, model.output_weight, torch.roll(tokens, -1), 1.0).mean() * -1.0).backward()
            sh.finish_grad_sync()
            norm = float(sh.grad_norm())
            grads = torch.cat([g.main_grad.detach().float().reshape(-1).clone() for g in sh.groups if g.main_grad is not None])
            fused_flags = [getattr(p, "_wgrad_accum", None) is not None for p in model.parameters()]
        finally:
            L._WGRAD_FUSION = old
        return norm, grads, any(fused_flags)

    n1, g1, has_accum = run(True)
    n0, g0, _ = run(False)
    assert has_accum, "the trainer did not expose its accumulators"
    assert abs(n1 - n0) <= 2e-2 * max(n0, 1e-6), (n1, n0)
    denom = float(g0.abs().max())
    assert float((g1 - g0).abs().max()) <= 2e-2 * denom, (float((g1 - g0).abs().max()), denom)
