"""Sharded trainer: flat-shard runtime vs a plain single-process AdamW, checkpoint format round trip, LoRA, weight sync."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from _spawn import run_ranks  # noqa: E402

from unirl_b200.distributed.group.comm import Comm
from unirl_b200.models.qwen3.modeling import AttnMeta, Qwen3Config, Qwen3Transformer, shard_param
from unirl_b200.parallel.flat_shard import FlatShardedModel


def _tiny(seed=0, layers=2):
    cfg = Qwen3Config.tiny(num_hidden_layers=layers, vocab_size=512, hidden_size=64, intermediate_size=128, head_dim=16)
    return Qwen3Transformer(cfg, dtype=torch.float32, device="cpu").init_weights(seed)


def _loss(model, tokens):
    n = tokens.numel()
    meta = AttnMeta(mode="train", positions=torch.arange(n), cu_seqlens=torch.tensor([0, n], dtype=torch.int32), max_seqlen=n)
    return model.logits(model(tokens, meta)).float().pow(2).mean()


def _sharded_steps(rank, world, steps):
    import torch.distributed as dist

    torch.manual_seed(0)
    model = _tiny()
    sh = FlatShardedModel(model, Comm.world(), block_class_names=("Qwen3DecoderLayer",), low_dtype=torch.float32)
    g = torch.Generator().manual_seed(1)
    data = [torch.randint(0, 512, (world, 24), generator=g) for _ in range(steps)]
    for i in range(steps):
        sh.zero_grad()
        sh.set_grad_sync(True)
        _loss(model, data[i][rank]).backward()
        sh.finish_grad_sync()
        norm = sh.grad_norm()
        coef = torch.clamp(1.0 / (norm + 1e-6), max=1.0).reshape(1)
        sh.optimizer_step(lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, step=i + 1, clip_coef=coef)
    return {n: p.detach().clone() for n, p in model.named_parameters()}, float(norm)


def test_flat_shard_two_ranks_match_single_process_adamw():
    steps, world = 3, 2
    outs = run_ranks(_sharded_steps, world, steps)
    (p0, n0), (p1, n1) = outs
    assert abs(n0 - n1) < 1e-6
    for k in p0:
        assert torch.equal(p0[k], p1[k]), f"replicas diverged on {k}"
    # single-process oracle: mean of per-rank gradients, global-norm clip, torch AdamW
    torch.manual_seed(0)
    ref = _tiny()
    opt = torch.optim.AdamW(ref.parameters(), lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01)
    g = torch.Generator().manual_seed(1)
    data = [torch.randint(0, 512, (world, 24), generator=g) for _ in range(steps)]
    for i in range(steps):
        opt.zero_grad()
        (sum(_loss(ref, data[i][r]) for r in range(world)) / world).backward()
        norm = torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        opt.step()
    assert abs(float(norm) - n0) < 1e-4
    for k, v in ref.named_parameters():
        assert torch.allclose(p0[k], v, atol=2e-5, rtol=1e-4), f"{k}: {(p0[k] - v).abs().max()}"


def test_backend_checkpoint_roundtrip_and_format(tmp_path):
    from unirl_b200.models.qwen3 import Qwen3Bundle, Qwen3PipelineConfig
    from unirl_b200.train.backend.fsdp import FSDPBackend
    from unirl_b200.distributed.group.remote import RankInfo

    def make():
        b = Qwen3Bundle.from_config(Qwen3PipelineConfig(model_precision="fp32", device="cpu"))
        be = FSDPBackend(bundle=b, block_class_names=("Qwen3DecoderLayer",), fsdp_cfg={"mixed_precision": False}, optimizer_cfg={"learning_rate": 1e-3},
                         scheduler_cfg={"type": "cosine", "total_steps": 10})
        be.setup(None, "cpu", RankInfo())
        return b, be

    b, be = make()
    tokens = torch.randint(0, 4096, (20,))
    for _ in range(2):
        be.zero_grad()
        be.set_grad_sync(True)
        _loss(b.transformer, tokens).backward()
        gn = be.optimizer_step(max_grad_norm=1.0)
        assert gn > 0
    path = str(tmp_path / "checkpoint-2")
    FSDPBackend.save.__wrapped__(be, path, step=2, mode="full")
    ck = torch.load(os.path.join(path, "checkpoint.pt"), weights_only=False)
    assert set(ck) >= {"policy_state_dict", "optimizer_state_dict", "optimizer_step_count", "step", "save_mode", "lora_config", "scheduler_state_dict"}
    assert "model.layers.0.self_attn.q_proj.weight" in ck["policy_state_dict"] and "lm_head.weight" in ck["policy_state_dict"]
    assert ck["optimizer_step_count"] == 2 and ck["step"] == 2 and ck["save_mode"] == "full" and os.path.exists(os.path.join(path, "manifest.json"))
    b2, be2 = make()
    be2.model.init_weights(seed=99)
    assert FSDPBackend.load.__wrapped__(be2, path) == 2
    for (n, p), (_, q) in zip(b.transformer.named_parameters(), b2.transformer.named_parameters()):
        assert torch.equal(p, q), n
    assert be2._optimizer_step_count == 2 and abs(be2.current_lr - be.current_lr) < 1e-12
    for g1, g2 in zip(be.sharded.groups, be2.sharded.groups):
        assert torch.allclose(g1.exp_avg, g2.exp_avg) and torch.allclose(g1.exp_avg_sq, g2.exp_avg_sq)
    # the next step is identical after resume
    for x in (be, be2):
        x.zero_grad(); x.set_grad_sync(True)
    _loss(b.transformer, tokens).backward(); _loss(b2.transformer, tokens).backward()
    be.optimizer_step(max_grad_norm=1.0); be2.optimizer_step(max_grad_norm=1.0)
    assert torch.allclose(b.transformer.layers[0].qkv_proj, b2.transformer.layers[0].qkv_proj, atol=1e-7)
    with pytest.raises(FileNotFoundError):
        FSDPBackend.load.__wrapped__(be2, str(tmp_path / "nope"))


def test_nonfinite_grad_norm_skips_update():
    from unirl_b200.models.qwen3 import Qwen3Bundle, Qwen3PipelineConfig
    from unirl_b200.train.backend.fsdp import FSDPBackend
    from unirl_b200.distributed.group.remote import RankInfo

    b = Qwen3Bundle.from_config(Qwen3PipelineConfig(model_precision="fp32", device="cpu"))
    be = FSDPBackend(bundle=b, block_class_names=("Qwen3DecoderLayer",), fsdp_cfg={"mixed_precision": False})
    be.setup(None, "cpu", RankInfo())
    before = b.transformer.norm.detach().clone()
    be.zero_grad(); be.set_grad_sync(True)
    (b.transformer.norm.sum() * float("inf")).backward()
    gn = be.optimizer_step(max_grad_norm=1.0)
    assert gn != gn or gn == float("inf")
    assert torch.equal(b.transformer.norm, before) and be._optimizer_step_count == 0


def test_lora_injection_merge_and_peft_keys():
    from unirl_b200.train.inject import inject_lora, inject_nft, lora_named_tensors
    from unirl_b200.utils.peft_merge import extract_lora_tensors, merged_state_dict

    m = _tiny()
    x = torch.randint(0, 512, (10,))
    meta = AttnMeta(mode="train", positions=torch.arange(10), cu_seqlens=torch.tensor([0, 10], dtype=torch.int32), max_seqlen=10)
    base = m(x, meta)
    n = inject_lora(m, rank=4, alpha=8, target_modules=("q_proj", "v_proj", "down_proj"))
    assert n == 6 and not m.layers[0].qkv_proj.requires_grad
    assert torch.allclose(m(x, meta), base, atol=1e-6), "zero-initialised lora_B must not change the output"
    for mod in m.layers:
        for ad in mod.lora.values():
            torch.nn.init.normal_(ad.lora_B, std=0.05)
    with_lora = m(x, meta)
    assert (with_lora - base).abs().max() > 1e-4
    keys = lora_named_tensors(m)
    assert "base_model.model.model.layers.0.self_attn.q_proj.lora_A.default.weight" in keys
    assert "model.layers.1.mlp.down_proj.lora_B.weight" in extract_lora_tensors(m)
    merged = dict(merged_state_dict(m))
    plain = _tiny()
    with torch.no_grad():
        for name, p in plain.named_parameters():
            p.copy_(merged[name])
    assert torch.allclose(plain(x, meta), with_lora, atol=1e-5), "folding (B·A)·alpha/r into the base rows must reproduce the adapter forward"
    m2 = _tiny()
    shadow = inject_nft(m2, rank=2, alpha=4, target_modules=("o_proj",))
    for mod in m2.layers:
        torch.nn.init.normal_(mod.lora["o_proj__default"].lora_B, std=0.1)
    out_live = m2(x, meta)
    with shadow.use_shadow():
        out_old = m2(x, meta)
    assert (out_live - out_old).abs().max() > 1e-5
    shadow.configure(decay=0.0, decay_type="constant", timing="rollout_end")
    shadow.on_rollout_end(0)
    with shadow.use_shadow():
        assert torch.allclose(m2(x, meta), out_live, atol=1e-6), "decay 0 copies the live adapter into the shadow"


def test_reshard_plan_matches_reference_sharding():
    from unirl_b200.distributed.weight_sync.full.reshard import execute_copy, plan_param

    cfg = Qwen3Config.tiny()
    full = Qwen3Transformer(cfg, dtype=torch.float32).init_weights(3)
    for tp in (1, 2):
        for name, p in full.named_parameters():
            ops = plan_param(name, tuple(p.shape), cfg, tp)
            for r in range(tp):
                want = shard_param(p.detach(), name, cfg, r, tp).contiguous()
                got = torch.full_like(want, float("nan")).reshape(-1)
                for op in ops:
                    if op.dst_tp_rank == r:
                        execute_copy(op, p.detach().reshape(-1), got)
                assert torch.equal(got.view_as(want), want), (name, tp, r)


def test_name_remap_and_buckets():
    from unirl_b200.distributed.weight_sync.full.base import apply_name_remap, validate_name_remap

    rules = validate_name_remap({"vision.*": None, "*": "transformer.*"})
    assert apply_name_remap("vision.proj", rules) is None and apply_name_remap("layers.0.w", rules) == "transformer.layers.0.w"
    with pytest.raises(ValueError):
        validate_name_remap({"*": "a.*", "b.*": "c.*"})
    with pytest.raises(ValueError):
        validate_name_remap({"a": "b"})


def test_checksums():
    from unirl_b200.distributed.weight_sync.checksum import compare_checksums, fingerprint_tensor, lora_checksum_multiset

    a = torch.arange(6, dtype=torch.bfloat16).view(2, 3)
    assert fingerprint_tensor(a) == fingerprint_tensor(a.clone()) and fingerprint_tensor(a) != fingerprint_tensor(a.view(3, 2))
    assert len(fingerprint_tensor(a)) == 16
    ok, bad = compare_checksums({"x": "1", "y": "2"}, {"x": "1", "y": "3"})
    assert not ok and bad == ["y"]
    t = {"m.lora_A.weight": torch.ones(2, 4), "m.lora_B.weight": torch.ones(4, 2)}
    folded = {"m.lora_A.weight": torch.ones(2, 4), "m.lora_B.weight": torch.ones(4, 2) * 2}
    assert lora_checksum_multiset(t, alpha=4, rank=2) == lora_checksum_multiset(folded, alpha=2, rank=2)


def _variant_steps(rank, world, steps, variant):
    torch.manual_seed(0)
    model = _tiny()
    comm = Comm.world()
    kw = {}
    if variant == "zero3":
        kw = {"reshard_after_forward": True}
    elif variant == "hsdp":  # 2 replicas x shard groups of 2
        comm_all = comm
        shard = comm_all.split([[0, 1], [2, 3]])
        kw = {"replicate_comm": comm_all.split([[0, 2], [1, 3]])}
        comm = shard
    sh = FlatShardedModel(model, comm, block_class_names=("Qwen3DecoderLayer",), low_dtype=torch.float32, **kw)
    g = torch.Generator().manual_seed(1)
    data = [torch.randint(0, 512, (world, 24), generator=g) for _ in range(steps)]
    released = []
    for i in range(steps):
        sh.release_all()
        released.append(sum(1 for gr in sh.groups if not gr._gathered))
        sh.zero_grad()
        sh.set_grad_sync(True)
        _loss(model, data[i][rank]).backward()
        sh.finish_grad_sync()
        norm = sh.grad_norm()
        coef = torch.clamp(1.0 / (norm + 1e-6), max=1.0).reshape(1)
        sh.optimizer_step(lr=1e-2, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, step=i + 1, clip_coef=coef)
        sh.gather_all()
    return {n: p.detach().clone() for n, p in model.named_parameters()}, float(norm), released


def test_zero3_residency_gives_the_same_training_as_resident_replicas():
    base = run_ranks(_variant_steps, 2, 3, "zero2")
    z3 = run_ranks(_variant_steps, 2, 3, "zero3")
    assert z3[0][2] == [2, 2, 2] and base[0][2] == [0, 0, 0], "both decoder blocks give their replica back between uses"
    assert abs(base[0][1] - z3[0][1]) < 1e-6
    for k in base[0][0]:
        torch.testing.assert_close(z3[0][0][k], base[0][0][k], atol=1e-6, rtol=1e-6)
        assert torch.equal(z3[0][0][k], z3[1][0][k])


def test_hsdp_four_ranks_match_flat_four_way_sharding():
    flat = run_ranks(_variant_steps, 4, 2, "zero2")
    hs = run_ranks(_variant_steps, 4, 2, "hsdp")
    assert abs(flat[0][1] - hs[0][1]) < 1e-5
    for k in flat[0][0]:
        torch.testing.assert_close(hs[0][0][k], flat[0][0][k], atol=2e-5, rtol=1e-4)  # reduction order differs (2-level vs flat)
        assert torch.equal(hs[0][0][k], hs[3][0][k])


class _Routed(torch.nn.Module):
    """Two 'experts' per block; a forward touches only the experts its ``route`` names, so the others get no gradient."""

    def __init__(self, width=16, blocks=3):
        super().__init__()
        self.inp = torch.nn.Linear(width, width)
        self.blocks = torch.nn.ModuleList(_RoutedBlock(width) for _ in range(blocks))
        self.out = torch.nn.Linear(width, 1)

    def forward(self, x, route):
        x = self.inp(x)
        for b, r in zip(self.blocks, route):
            x = b(x, r)
        return self.out(x).pow(2).mean()


class _RoutedBlock(torch.nn.Module):
    def __init__(self, width):
        super().__init__()
        self.experts = torch.nn.ModuleList(torch.nn.Linear(width, width) for _ in range(2))

    def forward(self, x, r):
        return x + sum(torch.tanh(self.experts[e](x)) for e in r)


_ROUTES = {0: [(0,), (0, 1), (1,)], 1: [(1,), (), (0, 1)]}  # rank 1 gives the middle block no gradient at all


def _routed_grads(rank, world, variant):
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.parallel.flat_shard import FlatShardedModel

    torch.manual_seed(0)
    model = _Routed().float()
    g = torch.Generator().manual_seed(5)
    xs = [torch.randn(4, 16, generator=g) for _ in range(2)]
    sh = FlatShardedModel(model, Comm.world() if world > 1 else None, block_class_names=("_RoutedBlock",), low_dtype=torch.float32,
                          reshard_after_forward=variant == "zero3")
    sh.zero_grad()
    sh.set_grad_sync(True)
    if world == 1:
        (sum(model(xs[r], _ROUTES[r]) for r in range(2)) / 2).backward()
    elif not (variant == "skip" and rank == 1):
        model(xs[rank], _ROUTES[rank]).backward()
    sh.finish_grad_sync()
    out = {}
    for gr in sh.groups:
        out[gr.name] = (gr.rank, gr.grad_shard.detach().clone() if gr.grad_shard is not None else None)
    return out, float(sh.grad_norm())


def test_reduce_order_does_not_depend_on_which_parameters_got_gradients():
    """Ranks route tokens to different experts, so different parameters receive gradients on each rank (one block gets none
    on rank 1).  Every group must still be reduced against the SAME group of the peer: the sharded gradient equals the
    single-process gradient of the averaged loss."""
    ref, ref_norm = run_ranks(_routed_grads, 1, "zero2")[0]
    for variant in ("zero2", "zero3"):
        res = run_ranks(_routed_grads, 2, variant)
        assert abs(res[0][1] - ref_norm) < 1e-5 and abs(res[1][1] - ref_norm) < 1e-5
        for name, (_, full) in ref.items():
            parts = [res[r][0][name][1] for r in range(2)]
            torch.testing.assert_close(torch.cat(parts)[: full.numel()], full[: sum(p.numel() for p in parts)], atol=1e-6, rtol=1e-5)


def test_rank_without_backward_still_joins_the_reductions():
    res = run_ranks(_routed_grads, 2, "skip")
    assert res[0][1] == res[1][1] and res[0][1] > 0
