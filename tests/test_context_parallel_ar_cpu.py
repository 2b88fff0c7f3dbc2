"""Context parallelism of the autoregressive replay on 2 gloo ranks: log-probs and gradients of the cut sequences equal the single-rank
replay, and a GRPO trainer step with one context-parallel replica equals the step of two data-parallel replicas."""
import pytest
import torch

from _spawn import run_ranks


def _body(rank, world):
    from unirl_b200.distributed.group.comm import Comm
    from unirl_b200.models.qwen3 import Qwen3Pipeline, Qwen3PipelineConfig
    from unirl_b200.models.qwen3.ar import pack_text_segment
    from unirl_b200.models.qwen3.conditions import Qwen3ARConditions
    from unirl_b200.parallel.context_parallel import ContextParallel
    from unirl_b200.types.conditions import TextTokenCondition

    pipe = Qwen3Pipeline.from_config(Qwen3PipelineConfig(pretrained_model_ckpt_path="random:tiny", model_precision="fp32", device="cpu"))
    model = pipe.bundle.transformer
    torch.manual_seed(3)
    vocab = model.cfg.vocab_size
    prompts = [torch.randint(3, vocab, (n,)) for n in (5, 9, 4)]
    responses = [torch.randint(3, vocab, (n,)) for n in (7, 1, 12)]  # lengths that do not divide by the group size; one response of a single token
    width = max(p.numel() for p in prompts)
    ids = torch.zeros(3, width, dtype=torch.long)
    mask = torch.zeros(3, width, dtype=torch.long)
    for i, p in enumerate(prompts):  # left-padded prompts, as the data pipeline delivers them
        ids[i, width - p.numel():] = p
        mask[i, width - p.numel():] = 1
    cond = Qwen3ARConditions(prompt=TextTokenCondition(input_ids=ids, attention_mask=mask))
    seg = pack_text_segment(responses, [torch.zeros(r.numel()) for r in responses], torch.ones(3, dtype=torch.bool))
    weights = torch.linspace(0.5, 1.5, sum(r.numel() for r in responses))

    def run():
        for p in model.parameters():
            p.grad = None
        lp = pipe.ar.replay(cond, segment=seg, temperature=1.0)
        (lp * weights).sum().backward()
        return lp.detach().clone(), torch.cat([p.grad.flatten() for p in model.parameters() if p.grad is not None])

    model.cp = None
    lp_ref, g_ref = run()
    model.cp = ContextParallel(Comm.world())
    lp_cp, g_cp = run()
    return {"lp_diff": float((lp_ref - lp_cp).abs().max()), "g_ref": g_ref, "g_cp": g_cp, "n": int(lp_ref.numel())}


def test_context_parallel_replay_matches_single_rank():
    r0, r1 = run_ranks(_body, 2)
    assert r0["n"] == 20 and r0["lp_diff"] < 1e-5 and r1["lp_diff"] < 1e-5, (r0["lp_diff"], r1["lp_diff"])
    total = r0["g_cp"] + r1["g_cp"]  # each rank holds the gradient of its tokens (keys' and values' gradients already summed over readers)
    scale = float(r0["g_ref"].abs().max())
    assert float((total - r0["g_ref"]).abs().max()) < 1e-4 * max(1.0, scale), float((total - r0["g_ref"]).abs().max())


@pytest.mark.timeout(900)
def test_grpo_trainer_with_a_context_parallel_replica_matches_data_parallel_replicas():
    """Two workers: two rollout engines (data parallel) and ONE trainer replica whose replay cuts every sequence over both ranks."""
    from test_e2e_cpu import _COLOC, _trainer

    from unirl_b200.config.loader import compose

    def run(extra):
        ov = [o for o in _COLOC if not o.startswith(("num_devices", "+pool_backend"))]
        tr = _trainer(compose("ar/qwen3_4b_grpo_b200", overrides=ov + extra + ["rollout.config.model_precision=fp32"]))
        try:
            req = tr._build_req(tr.data_source.get_samples(tr.batch_size), 0)
            result, _reward = tr.train_step(req, rollout_id=0)
            row = [r for r in tr.wandb_logger.history if "train/step" in r][0]
            return {**row, "grad_norm": float(result.grad_norm)}
        finally:
            tr.shutdown()

    # same two rollout engines in both runs; the trainer is two data-parallel replicas of 8 samples each in the first and ONE replica
    # (two micro-batches of the same 8 samples each) cut over two context-parallel ranks in the second: the same averaged gradient
    dp2 = run(["num_devices=2", "+pool_backend=mp"])
    cp2 = run(["num_devices=2", "+pool_backend=mp", "+train_parallel={sp: 2}", "+backend.fsdp_cfg.cp_size=2"])
    assert abs(cp2["train/ratio_mean"] - 1.0) < 1e-4 and cp2["train/rollout_replay_logp_absdiff_max"] < 1e-3
    assert abs(dp2["grad_norm"] - cp2["grad_norm"]) < 1e-5 * abs(dp2["grad_norm"]), (dp2["grad_norm"], cp2["grad_norm"])
