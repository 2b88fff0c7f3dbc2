"""Unified text + image model: MoE routing, incremental decoding, rollout/replay alignment on both tracks, joint training."""
import os

import pytest
import torch

from unirl_b200.config.loader import compose
from unirl_b200.models.dit.diffusion import DiTDiffusionParams
from unirl_b200.models.unified import MoEFFN, UnifiedConditions, UnifiedConfig, UnifiedPipeline, UnifiedPipelineConfig, UnifiedTransformer
from unirl_b200.trainer.unified_model import UnifiedModelTrainer
from unirl_b200.types.primitives import Texts
from unirl_b200.types.rollout_req import RolloutReq
from unirl_b200.types.sampling import ARSamplingParams, ComposedSamplingParams, DiffusionSamplingParams


def test_moe_matches_dense_evaluation_of_the_selected_experts():
    cfg = UnifiedConfig.tiny()
    moe = MoEFFN(cfg, torch.float32, "cpu")
    for p in moe.parameters():
        torch.nn.init.normal_(p, std=0.1)
    x = torch.randn(9, cfg.hidden_size)
    probs = torch.softmax(x @ moe.router.t(), -1)
    w, idx = probs.topk(cfg.experts_per_token, -1)
    w = w / w.sum(-1, keepdim=True)
    want = torch.stack([sum(w[t, j] * moe.experts[int(idx[t, j])](x[t : t + 1])[0] for j in range(cfg.experts_per_token)) for t in range(9)]) + moe.shared(x)
    torch.testing.assert_close(moe(x), want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("preset", ["tiny-unified", "tiny-mot"])
def test_incremental_decode_and_both_tracks_replay(preset):
    pipe = UnifiedPipeline.from_config(UnifiedPipelineConfig(pretrained_model_ckpt_path=f"random:{preset}", model_precision="fp32", device="cpu",
                                                              autocast_precision="fp32", recaption=True))
    m = pipe.bundle.transformer
    ids = torch.randint(3, 500, (1, 7))
    ones = torch.ones_like(ids)
    with torch.no_grad():
        full = m.forward_text(ids, ones)
        caches = [{} for _ in m.layers]
        a = m.forward_text(ids[:, :4], ones[:, :4], caches)
        b = m.forward_text(ids[:, 4:], ones[:, 4:], caches, positions=torch.arange(4, 7)[None], key_mask=ones)
    assert float((torch.cat([a, b], 1) - full).abs().max()) < 1e-5
    sp = ComposedSamplingParams(ar=ARSamplingParams(max_new_tokens=5, temperature=1.0, top_p=1.0, top_k=0),
                                diffusion=DiffusionSamplingParams(num_inference_steps=3, guidance_scale=2.0, height=32, width=32, seed=1, sde_indices=[0, 1]))
    resp = pipe.generate(RolloutReq(sample_ids=["a/0", "a/1"], group_ids=["a", "a"], primitives={"text": Texts.from_list(["cat", "cat"])}, sampling_params=sp,
                                    stage_config={"mode": "t2i"}))
    ar, im = resp.tracks["ar"], resp.tracks["image"]
    lp = pipe.ar.replay(UnifiedConditions.from_dict(ar.conditions), segment=ar.segment)
    out = pipe.diffusion.replay(UnifiedConditions.from_dict(im.conditions), segment=im.segment, params=DiTDiffusionParams(guidance_scale=2.0))
    assert float((lp.detach() - ar.segment.log_probs).abs().max()) < 1e-4 and float((out.log_probs.detach() - im.segment.sde_logp).abs().max()) < 1e-5
    text_only = pipe.generate(RolloutReq(sample_ids=["a/0"], group_ids=["a"], primitives={"text": Texts.from_list(["hi"])}, sampling_params=sp,
                                         stage_config={"mode": "t2t"}))
    assert list(text_only.tracks) == ["ar"]


@pytest.mark.timeout(600)
def test_unified_trainer_one_step_for_two_tracks(tmp_path):
    cfg = compose("unified_model/tiny_unified_t2i_cpu", overrides=[])
    tr = UnifiedModelTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend, rollout_cfg=cfg.rollout,
                             reward_cfg=cfg.reward, ar_algorithm_cfg=cfg.ar_algorithm, image_algorithm_cfg=cfg.image_algorithm, stack_cfg=cfg.stack,
                             data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, logging_cfg=None, rollout_dump_dir=str(tmp_path))
    try:
        before = tr.backend.compute_local_param_checksums()[0]
        tr.train(num_rollouts=1)
        assert tr.backend.compute_local_param_checksums()[0] != before
        rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(rows) == 1 and any(k.startswith("train/ar/") for k in rows[0]) and any(k.startswith("train/image/") for k in rows[0])
        assert (tmp_path / "rollout_000000.jsonl").exists()
    finally:
        tr.shutdown()


@pytest.mark.timeout(600)
def test_unified_trainer_with_an_engine_pair_and_the_memory_choreography(tmp_path):
    """Two engines with weights of their own: extract → offload → wake → push → rollout (P → P·N → P·N·M) → sleep → onload → train.
    The adapter the engines hold after a synced step equals the trainer's; rewrites earn the mean reward of their images."""
    import json

    from unirl_b200.train_unified_model import main

    calls = []
    cfg = compose("unified_model/tiny_unified_two_engines_cpu", overrides=[])
    tr = UnifiedModelTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                             ar_rollout_cfg=cfg.ar_rollout, dit_rollout_cfg=cfg.dit_rollout, sync_cfg=cfg.sync, enable_fsdp_offload=True,
                             reward_cfg=cfg.reward, ar_algorithm_cfg=cfg.ar_algorithm, image_algorithm_cfg=cfg.image_algorithm, stack_cfg=cfg.stack,
                             data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, logging_cfg=None, rollout_dump_dir=str(tmp_path))
    try:
        for name in ("offload", "onload"):  # record the order of the choreography
            inner = getattr(tr.backend, name)
            setattr(tr.backend, name, (lambda inner=inner, name=name: (calls.append(name), inner())[1]))
        for tag, eng in (("ar", tr.ar_rollouts[0]), ("dit", tr.dit_rollouts[0])):
            for name in ("wake_up", "sleep", "set_lora_from_tensors"):
                inner = getattr(eng, name)
                setattr(eng, name, (lambda *a, inner=inner, n=f"{tag}.{name}", **k: (calls.append(n), inner(*a, **k))[1]))
        tr.train(num_rollouts=2)
        first = calls[: calls.index("offload", 2) + 1] if calls.count("offload") > 1 else calls
        assert first[:2] == ["onload", "offload"], first  # extract with the trainer resident, then make room
        assert first.index("ar.wake_up") > first.index("offload") and first.index("ar.set_lora_from_tensors") > first.index("dit.wake_up")
        assert first.index("ar.sleep") > first.index("dit.set_lora_from_tensors") and first.index("onload", 1) > first.index("dit.sleep")
        rows = [json.loads(l) for l in open(tmp_path / "rollout_000001.jsonl")]
        ar = [r for r in rows if r.get("track") == "ar"]
        img = [r for r in rows if r.get("track") == "image"]
        assert len(ar) == 2 * 2 and len(img) == 2 * 2 * 2  # P·N rewrites, P·N·M images
        for a in ar:
            kids = [i["reward"] for i in img if i["parent_id"] == a["sample_id"]]
            assert len(kids) == 2 and abs(a["reward"] - sum(kids) / 2) < 1e-5
        # the engines' adapters follow the trainer's (second step synced after the first optimizer step)
        tr.backend.onload()
        mine = {k: v for k, v in tr.backend.compute_local_param_checksums()[0].items() if "lora_" in k}
        theirs = {k: v for k, v in tr.dit_rollouts[0].compute_local_param_checksums()[0].items() if "lora_" in k}
        assert mine and len(theirs) == len(mine)
        train_rows = [r for r in tr.wandb_logger.history if "train/step" in r]
        assert len(train_rows) == 2 and any(k.startswith("train/ar/") for k in train_rows[0]) and any(k.startswith("train/image/") for k in train_rows[0])
    finally:
        tr.shutdown()


def test_meta_construction_and_per_rank_materialisation(tmp_path):
    """``from_meta_config`` allocates nothing; ``materialize`` fills by global tensor name, so an expert-parallel rank that keeps half of
    the experts holds exactly the values of the unsharded model for them; a native sharded checkpoint round-trips, each rank reading
    only what it kept."""
    from unirl_b200.models.unified.modeling import MoEFFN
    from unirl_b200.models.unified.pipeline import UnifiedBundle, UnifiedPipelineConfig, save_native_checkpoint

    cfg = UnifiedPipelineConfig(pretrained_model_ckpt_path="random:tiny-unified", model_precision="fp32", device="cpu", init_seed=5)
    meta = UnifiedBundle.from_meta_config(cfg)
    assert all(p.is_meta for p in meta.transformer.parameters()) and all(p.is_meta for p in meta.vae.parameters())
    full = meta.materialize("cpu")
    assert not any(p.is_meta for p in full.transformer.parameters()) and not any(p.is_meta for p in full.vae.parameters())
    again = UnifiedBundle.from_meta_config(cfg).materialize("cpu", with_aux=False)
    assert all(p.is_meta for p in again.vae.parameters()), "with_aux=False leaves the codec unallocated"
    ref = dict(full.transformer.named_parameters())
    for n, p in again.transformer.named_parameters():
        assert torch.equal(p, ref[n]), n

    class _EP:  # what MoEFFN.shard_experts needs from an expert-parallel context
        def __init__(self, rank, size):
            self.rank, self.size = rank, size

        def local_experts(self, n):
            per = n // self.size
            return list(range(self.rank * per, (self.rank + 1) * per))

    n_experts = full.transformer.cfg.num_experts
    seen = 0
    for rank in (0, 1):
        part = UnifiedBundle.from_meta_config(cfg).materialize("cpu", with_aux=False, ep=_EP(rank, 2))
        moes = [m for m in part.transformer.modules() if isinstance(m, MoEFFN)]
        assert moes and all(len(m.experts) == n_experts // 2 and m.expert_ids == _EP(rank, 2).local_experts(n_experts) for m in moes)
        for n, p in part.transformer.named_parameters():
            if ".experts." in n:
                pre, rest = n.split(".experts.")
                slot, leaf = rest.split(".", 1)
                g = f"{pre}.experts.{rank * (n_experts // 2) + int(slot)}.{leaf}"
                seen += 1
            else:
                g = n
            assert torch.equal(p, ref[g]), (n, g)
    assert seen == sum(1 for n in ref if ".experts." in n), "the two ranks together hold every expert exactly once"

    with torch.no_grad():  # a trained-looking model: perturb, save, reload
        for p in full.transformer.parameters():
            p.add_(torch.randn_like(p) * 0.01)
    save_native_checkpoint(full.transformer, str(tmp_path), "tiny-unified", shard_bytes=200_000)
    assert len([f for f in os.listdir(tmp_path) if f.endswith(".safetensors")]) > 1, "several shards"
    ck = UnifiedPipelineConfig(pretrained_model_ckpt_path=str(tmp_path), model_precision="fp32", device="cpu")
    loaded = UnifiedBundle.from_config(ck)
    for n, p in loaded.transformer.named_parameters():
        assert torch.equal(p, ref[n]), n
    part = UnifiedBundle.from_meta_config(ck).materialize("cpu", with_aux=False, ep=_EP(1, 2))
    first = next(m for m in part.transformer.modules() if isinstance(m, MoEFFN))
    name = next(n for n, m in part.transformer.named_modules() if m is first)
    assert torch.equal(first.experts[0].down, ref[f"{name}.experts.{n_experts // 2}.down"])


def test_bagel_guidance_window_and_renormalisation():
    """Bagel's sampling knobs: the text guidance acts only inside ``cfg_interval`` of the schedule, and the guided velocity is scaled back
    towards the conditional one's norm (whole-sample or per-token norms, clamped between ``cfg_renorm_min`` and 1)."""
    import pytest

    from unirl_b200.models.bagel import BagelDiffusionParams, BagelPipeline, BagelPipelineConfig, BagelStageParams

    with pytest.raises(Exception):
        BagelDiffusionParams(cfg_renorm_type="rows")
    sp = BagelDiffusionParams(cfg_text_scale=4.0, cfg_interval=(0.4, 1.0), cfg_renorm_min=0.0, cfg_renorm_type="global", samples_per_prompt=2)
    assert sp.num_inference_steps == 14 and sp.samples_per_prompt == 2
    pipe = BagelPipeline.from_config(BagelPipelineConfig(pretrained_model_ckpt_path="random:tiny-mot", model_precision="fp32", autocast_precision="fp32", device="cpu"))
    stage = pipe.diffusion
    p = stage._stage_params(sp)
    assert isinstance(p, BagelStageParams) and p.guidance_scale == 4.0 and p.cfg_interval == (0.4, 1.0) and p.eta == 1.0
    torch.manual_seed(0)
    vc, vu = torch.randn(2, 4, 6, 6), torch.randn(2, 4, 6, 6)
    plain = vu + 4.0 * (vc - vu)
    g = stage._guided(vu, vc, p)
    ratio = (vc.flatten(1).norm(dim=1) / plain.flatten(1).norm(dim=1)).clamp(max=1.0)
    torch.testing.assert_close(g, plain * ratio.view(2, 1, 1, 1))
    assert torch.all(g.flatten(1).norm(dim=1) <= vc.flatten(1).norm(dim=1) * (1 + 1e-5))
    pc = stage._stage_params(BagelDiffusionParams(cfg_text_scale=4.0, cfg_renorm_type="channel", cfg_renorm_min=0.5))
    gc = stage._guided(vu, vc, pc)
    r = (vc.norm(dim=1, keepdim=True) / (plain.norm(dim=1, keepdim=True) + 1e-8)).clamp(min=0.5, max=1.0)
    torch.testing.assert_close(gc, plain * r)
    # inside the window both branches are evaluated, outside only the conditional one
    tok = pipe.bundle.tokenizer
    from unirl_b200.models.unified.stages import UnifiedConditions
    from unirl_b200.types.conditions import TextTokenCondition

    ids = torch.tensor([[5, 6, 7, 8], [9, 10, 11, 12]])
    cond = UnifiedConditions(prompt=TextTokenCondition(input_ids=ids, attention_mask=torch.ones_like(ids)),
                             negative_prompt=TextTokenCondition(input_ids=torch.tensor([[1], [1]]), attention_mask=torch.ones(2, 1, dtype=torch.long)))
    x = torch.randn(2, *pipe.latent_shape(sp))
    inside = stage._branches(x, torch.tensor([0.7]), cond, p)
    outside = stage._branches(x, torch.tensor([0.2]), cond, p)
    assert inside[1] is not None and outside[1] is None and inside[0].shape == x.shape
    del tok
