import math

import pytest
import torch

from unirl_b200.algorithms.base import aggregate_token_loss, expand_per_token, gather_sde_field, resolve_clip_range
from unirl_b200.algorithms.normalizers import normalize_global, normalize_grouped
from unirl_b200.ops import policy_loss as PL
from unirl_b200.sde import (CPSSDEStrategy, DanceSDEStrategy, DPM2Strategy, FlowMatchSchedulePolicy, FlowSDEStrategy, StepStrategy,
                            calculate_dynamic_mu, generate_shared_noise, get_sigma_schedule, regen_initial_noise)
from unirl_b200.sde.noise import derive_group_seed
from unirl_b200.utils.scheduler_utils import AllSDEScheduler, WindowConfig, WindowScheduler, create_indices_scheduler


def test_sigma_schedules():
    s = get_sigma_schedule(4, 3.0)
    t = torch.linspace(1, 0, 5)
    assert torch.allclose(s, 3 * t / (1 + 2 * t)) and s[0] == 1 and s[-1] == 0
    mu = calculate_dynamic_mu(4096)
    assert abs(mu - 1.15) < 1e-6 and abs(calculate_dynamic_mu(256) - 0.5) < 1e-6
    d = get_sigma_schedule(4, mu=0.8)
    base = torch.linspace(1, 0.25, 4, dtype=torch.float64)
    assert torch.allclose(d[:-1].double(), math.exp(0.8) / (math.exp(0.8) + (1 / base - 1)), atol=1e-6) and d[-1] == 0
    pol = FlowMatchSchedulePolicy(use_dynamic_shifting=True)
    assert pol.image_seq_len(1024, 1024) == 4096
    assert torch.allclose(pol.compute_sigma(num_inference_steps=4, height=1024, width=1024), get_sigma_schedule(4, mu=1.15))


@pytest.mark.parametrize("cls", [FlowSDEStrategy, DanceSDEStrategy, CPSSDEStrategy])
def test_strategies_against_scalar_fp64(cls):
    torch.manual_seed(0)
    st = cls()
    x, v, eps = torch.randn(2, 3, 4, 4, dtype=torch.float64), torch.randn(2, 3, 4, 4, dtype=torch.float64), torch.randn(2, 3, 4, 4)
    s, s2, eta = 0.8, 0.6, 0.7
    prev, lp, mean = st.denoise(v.float(), x.float(), torch.tensor(s), torch.tensor(s2), eta=eta, noise=eps)
    dt = s2 - s
    if cls is CPSSDEStrategy:
        std = s2 * math.sin(eta * math.pi / 2)
        m = (x - s * v) * (1 - s2) + (x + v * (1 - s)) * math.sqrt(s2**2 - std**2)
        p = m + std * eps.double()
        ref_lp = (-(p - m) ** 2).mean(dim=(1, 2, 3))
    else:
        sd = eta if cls is DanceSDEStrategy else math.sqrt(s / (1 - s)) * eta
        m = x * (1 + sd**2 / (2 * s) * dt) + v * (1 + sd**2 * (1 - s) / (2 * s)) * dt
        sv = sd * math.sqrt(-dt)
        p = m + sv * eps.double()
        ref_lp = (-(p - m) ** 2 / (2 * sv**2) - math.log(sv) - 0.5 * math.log(2 * math.pi)).mean(dim=(1, 2, 3))
    assert torch.allclose(mean.double(), m, atol=1e-5) and torch.allclose(prev.double(), p, atol=1e-5) and torch.allclose(lp.double(), ref_lp, atol=1e-4)
    _, lp2, _ = st.denoise(v.float(), x.float(), torch.tensor(s), torch.tensor(s2), eta=eta, prev_sample=prev)
    assert torch.allclose(lp, lp2)
    _, none_lp, _ = st.denoise(v.float(), x.float(), torch.tensor(s), torch.tensor(s2), eta=0.0, noise=eps)
    assert none_lp is None


def test_sigma_one_uses_sigma_max_and_ode_and_dpm2():
    x, v = torch.randn(1, 2, 2), torch.randn(1, 2, 2)
    _, lp, _ = FlowSDEStrategy().denoise(v, x, torch.tensor(1.0), torch.tensor(0.9), eta=0.5, noise=torch.zeros(1, 2, 2))
    assert torch.isfinite(lp).all()
    p, lp, m = StepStrategy().denoise(v, x, torch.tensor(0.5), torch.tensor(0.3))
    assert lp is None and torch.allclose(p, x - 0.2 * v)
    sig = get_sigma_schedule(6, 3.0)
    d = DPM2Strategy()
    d.init_schedule(sig)
    cur = x
    for i in range(6):
        cur, a, b = d.denoise(v, cur, sig[i], sig[i + 1], step_index=i)
        assert a is None and torch.isfinite(cur).all()
    with pytest.raises(RuntimeError):
        DPM2Strategy().denoise(v, x, sig[0], sig[1])


def test_noise_is_group_deterministic_and_shard_safe():
    a = regen_initial_noise(["g0", "g1", "g0"], 7, (2, 3), "cpu")
    assert torch.equal(a[0], a[2]) and not torch.equal(a[0], a[1])
    b = regen_initial_noise(["g1"], 7, (2, 3), "cpu")
    assert torch.equal(b[0], a[1])
    assert derive_group_seed(7, "g0") != derive_group_seed(8, "g0")
    with pytest.raises(ValueError):
        generate_shared_noise(2, (1,), "cpu", noise_group_ids=["a"])


def test_index_schedulers():
    assert AllSDEScheduler(10, 0.5).get_sde_indices(3) == {0, 1, 2, 3, 4}
    s = AllSDEScheduler(10, [0.2, 1.0], num_sde_steps=3)
    assert s.get_sde_indices(5) == s.get_sde_indices(5) and len(s.get_sde_indices(5)) == 3 and min(s.get_sde_indices(5)) >= 2
    assert AllSDEScheduler(10, 1.0, num_sde_steps=0).get_sde_indices(1) == set()
    w = WindowScheduler(10, WindowConfig(strategy="progressive", window_size=4, iters_per_window=2))
    assert w.get_sde_indices(0) == {0, 1, 2, 3} and w.get_sde_indices(2) == {4, 5, 6, 7} and w.get_sde_indices(100) == {4, 5, 6, 7}
    wr = WindowScheduler(10, WindowConfig(strategy="progressive", window_size=4, iters_per_window=2, roll_back=True))
    assert wr.get_sde_indices(4) == {0, 1, 2, 3}
    assert isinstance(create_indices_scheduler(scheduler_config={"timestep_strategy": "window"}, num_timesteps=8), WindowScheduler)


def test_clip_loss_closed_form_and_metrics():
    new, old, adv = torch.tensor([0.0, 0.5, -0.5, 0.1]), torch.zeros(4), torch.tensor([1.0, 1.0, -1.0, -2.0])
    loss, m = PL.ppo_clip_reference(new, old, adv, 0.2, 0.3)
    r = new.exp()
    exp = torch.stack([-r[0], -torch.tensor(1.3), torch.tensor(0.8), 2 * r[3]])
    assert torch.allclose(loss, exp, atol=1e-6)
    assert abs(float(m["clipfrac_gt_one"]) - 0.25) < 1e-6 and abs(float(m["clipfrac_lt_one"]) - 0.25) < 1e-6
    assert resolve_clip_range(0.2, "linear_decay", 1.0) == 0.1 and abs(resolve_clip_range(0.2, "cosine_decay", 1.0)) < 1e-9


def test_drpo_loss_closed_form():
    new, old, adv = torch.tensor([-1.0, -2.5]), torch.tensor([-1.2, -2.0]), torch.tensor([2.0, -1.0])
    loss, m = PL.drpo_reference(new, old, adv, 12.5, True)
    r, mu = (new - old).exp(), old.exp()
    assert torch.allclose(loss, -adv * r + adv.abs() * mu * (r - 1) ** 2 / 25.0, atol=1e-6)
    plain, _ = PL.drpo_reference(new, old, adv, 12.5, False)
    assert torch.allclose(plain, -adv * r + adv.abs() * (r - 1) ** 2 / 25.0, atol=1e-6)
    assert abs(float(m["approx_kl"]) - float(((r - 1) - (new - old)).mean())) < 1e-6


def test_flow_dppo_mask():
    new, old = torch.tensor([[0.2, -0.2, 0.2]]), torch.zeros(1, 3)
    adv = torch.tensor([[1.0, 1.0, -1.0]])
    nm = torch.zeros(1, 3, 2, 2, 2)
    om = torch.ones(1, 3, 2, 2, 2) * torch.tensor([1.0, 1.0, 0.0]).view(1, 3, 1, 1, 1)
    loss, m = PL.flow_dppo_reference(new, old, nm, om, adv, torch.ones(1, 3, 1, 1, 1), 0.1)
    r = new.exp()
    assert torch.allclose(loss, torch.tensor([[0.0, -float(r[0, 1]), float(r[0, 2])]]), atol=1e-6)
    assert abs(float(m["masked_fraction"]) - 1 / 3) < 1e-6


def test_token_aggregation_and_helpers():
    le = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0])
    lens = torch.tensor([1, 2, 3])
    assert float(aggregate_token_loss(le, lens, "token-mean", 8)) == 3.5
    assert abs(float(aggregate_token_loss(le, lens, "seq-mean-token-sum-norm", 10)) - (1 + 5 + 15) / 3 / 10) < 1e-6
    assert abs(float(aggregate_token_loss(le, lens, "seq-mean-token-mean", 10)) - (1 + 2.5 + 5) / 3) < 1e-6
    assert expand_per_token(torch.tensor([1.0, 2.0, 3.0]), lens, dtype=torch.float32, device="cpu").tolist() == [1, 2, 2, 3, 3, 3]
    t = torch.arange(12.0).view(2, 3, 2)
    g = gather_sde_field(t, torch.tensor([5, 1, 3]), [3, 5])
    assert torch.equal(g, t[:, [2, 0]])
    with pytest.raises(ValueError):
        gather_sde_field(t, torch.tensor([5, 1, 3]), [2])
    r = torch.tensor([1.0, 2.0, 3.0, 10.0, 20.0, 30.0])
    a = normalize_grouped(r, [[0, 1, 2], [3, 4, 5]])
    assert torch.allclose(a[:3], a[3:], atol=1e-5)
    assert torch.allclose(normalize_global(r), (r - r.mean()) / (r.std() + 1e-8))
    assert normalize_grouped(r, [[0, 1, 2], [3, 4, 5]], clip_max=0.5).abs().max() <= 0.5


class _FakeDiffStage:
    """predict v = w * x (one scalar parameter), replay via the Flow strategy."""

    def __init__(self):
        self.w = torch.nn.Parameter(torch.tensor(0.5))
        self.strategy = FlowSDEStrategy()

    def replay(self, conds, *, segment, params, step_indices=None):
        from unirl_b200.models.types import ReplayResult

        lps, means = [], []
        for s in step_indices:
            x, nxt = segment.latents_at(s), segment.latents_at(s + 1)
            _, lp, mean = self.strategy.denoise(self.w * x, x, segment.sigmas[s], segment.sigmas[s + 1], eta=params.eta, prev_sample=nxt)
            lps.append(lp)
            means.append(mean)
        return ReplayResult(torch.stack(lps, 1), torch.stack(means, 1))

    def predict_noise_at_step(self, conds, *, sample, sigma, params):
        return self.w * sample


def _latent_segment():
    from unirl_b200.types import make_image_segment

    torch.manual_seed(0)
    sig = get_sigma_schedule(4, 3.0)
    lat = torch.randn(4, 5, 2, 4, 4)
    return make_image_segment(latents=lat, sigmas=sig, indices=torch.arange(5), sde_indices=torch.tensor([1, 2]))


def test_flow_grpo_dppo_nft_run_and_are_on_policy():
    from types import SimpleNamespace

    from unirl_b200.algorithms import DiffusionNFT, FlowDPPO, FlowGRPO

    params = SimpleNamespace(eta=0.7)
    adv = torch.tensor([1.0, -1.0, 0.5, -0.5])
    for cls, kw in ((FlowGRPO, {"old_logp_source": "replay", "clip_range": 0.2}), (FlowDPPO, {})):
        st = _FakeDiffStage()
        algo = cls(params=params, stage=st, **kw)
        seg = _latent_segment()
        algo.prepare_segment(conditions={}, segment=seg)
        assert seg.sde_logp.shape == (4, 2)
        res = algo.compute_loss_and_backward(conditions={}, segment=seg, advantages=adv, training_progress=0.0, loss_scale=1.0)
        assert res.has_backward and abs(res.metrics["ratio_mean"] - 1.0) < 1e-6 and st.w.grad is not None
        if cls is FlowDPPO:
            assert res.metrics["kl_new_old_max"] == 0.0 and res.metrics["unmasked_fraction"] == 1.0
    with pytest.raises(RuntimeError):
        FlowGRPO(params=params, stage=_FakeDiffStage()).prepare_segment(conditions={}, segment=_latent_segment())

    class Pol:
        import contextlib

        @contextlib.contextmanager
        def use_shadow(self):
            yield

    st = _FakeDiffStage()
    nft = DiffusionNFT(params=params, stage=st, nft_lora_policy=Pol(), shuffle_train_timesteps=False)
    res = nft.compute_loss_and_backward(conditions={}, segment=_latent_segment(), advantages=adv, training_progress=0.0, loss_scale=1.0)
    assert res.has_backward and res.num_steps_or_tokens == 3 and abs(res.metrics["prediction_deviation"]) < 1e-12
    with pytest.raises(TypeError):
        DiffusionNFT(params=params, stage=st, nft_lora_policy=object())
