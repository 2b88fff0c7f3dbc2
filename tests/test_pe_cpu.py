"""Prompt-enhancement flow (AR → diffusion, two tracks, two optimizers) and the σ echo check."""
import pytest
import torch

from unirl_b200.config.loader import compose
from unirl_b200.rollout.engine.composed.engine import extract_enhanced_prompt
from unirl_b200.rollout.engine.sigma_verify import SigmaMismatchError, verify_sigmas
from unirl_b200.trainer.pe import PETrainer


def test_extract_enhanced_prompt():
    assert extract_enhanced_prompt("<think>hm</think> sure <prompt>a golden cat</prompt> bye", "cat") == "a golden cat"
    assert extract_enhanced_prompt("<prompt>x</prompt> then <prompt> final one", "cat") == "final one"
    assert extract_enhanced_prompt("<think>only thoughts</think>   ", "cat") == "cat"
    assert extract_enhanced_prompt("plain rewrite", "cat") == "plain rewrite"


def test_sigma_verify_scales_and_rejects():
    want = torch.tensor([1.0, 0.75, 0.4, 0.0])
    verify_sigmas(want.clone(), want)
    verify_sigmas(want[:-1] * 1000, want)  # 0..1000 scale without the terminal zero
    with pytest.raises(SigmaMismatchError):
        verify_sigmas(torch.tensor([1.0, 0.70, 0.4, 0.0]), want)
    with pytest.raises(SigmaMismatchError):
        verify_sigmas(torch.tensor([1.0, 0.75]), want)


@pytest.mark.timeout(600)
def test_pe_trainer_two_tracks_two_updates():
    cfg = compose("pe/tiny_pe_cpu", overrides=[])
    tr = PETrainer(cfg=cfg, batch_size=cfg.batch_size, ar_cfg=cfg.ar, diffusion_cfg=cfg.diffusion, reward_cfg=cfg.reward, data_source_cfg=cfg.data_source,
                   sampling_cfg=cfg.sampling, logging_cfg=None)
    try:
        before = (tr.ar["backend"].compute_local_param_checksums()[0], tr.diffusion["backend"].compute_local_param_checksums()[0])
        req = tr._build_req(tr.data_source.get_samples(tr.batch_size), 0)
        resp = tr.rollout.generate(req)
        ar, diff = resp.tracks["ar"], resp.tracks["diffusion"]
        assert len(ar.sample_ids) == 4 and len(diff.sample_ids) == 8 and diff.parent_track == "ar"
        assert diff.parent_ids == [s for s in ar.sample_ids for _ in range(2)], "children sit next to each other under their AR parent"
        results, reward = tr.train_step(req, rollout_id=0)
        assert results["ar"].has_backward and results["diffusion"].has_backward and 0.0 <= reward <= 1.0
        after = (tr.ar["backend"].compute_local_param_checksums()[0], tr.diffusion["backend"].compute_local_param_checksums()[0])
        assert after[0] != before[0] and after[1] != before[1]
    finally:
        tr.shutdown()
