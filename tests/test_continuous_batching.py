"""Continuous batching in the AR generator: retire / admit / compact, against fixed waves."""
import pytest
import torch


def _model(device, dtype):
    from unirl_b200.models.qwen3.modeling import Qwen3Config, Qwen3Transformer

    cfg = Qwen3Config.tiny(num_hidden_layers=2, hidden_size=128, intermediate_size=256, num_attention_heads=4, num_key_value_heads=2, head_dim=32, vocab_size=512)
    if device == "cuda":
        cfg = Qwen3Config.tiny(num_hidden_layers=2, hidden_size=512, intermediate_size=1024, num_attention_heads=8, num_key_value_heads=2, head_dim=128, vocab_size=4096)
    return Qwen3Transformer(cfg, dtype=dtype, device=device).init_weights(0).eval().requires_grad_(False), cfg


def _stops(vocab, frac):
    """A stop set covering `frac` of the vocabulary: random-init models then end sequences after about 1 / frac tokens."""
    g = torch.Generator().manual_seed(9)
    return torch.randperm(vocab, generator=g)[: int(vocab * frac)].tolist()


def test_continuous_batching_matches_waves_greedy_cpu():
    """Greedy decoding is a function of the prompt alone, so retiring, admitting and compacting rows must reproduce the wave
    generator's output exactly -- while taking fewer decode steps, because rows freed by short sequences are refilled."""
    from unirl_b200.rollout.engine.native_ar.generator import ARGenerator

    model, cfg = _model("cpu", torch.float32)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(8, cfg.vocab_size, (int(n),), generator=g) for n in torch.randint(5, 40, (22,), generator=g)]
    stops = _stops(cfg.vocab_size, 0.06)
    outs = {}
    for mode in (False, True):
        gen = ARGenerator(model, page_size=16, max_running=8, use_cuda_graph=False, poll_interval=4, seed=3, continuous=mode)
        outs[mode] = gen.generate(prompts, max_new_tokens=40, temperature=0.0, stop_token_ids=stops, seed=5)
    lens = [int(t.numel()) for t in outs[False].tokens]
    assert len(set(lens)) > 3, "the stop set should give a spread of response lengths"
    for a, b in zip(outs[False].tokens, outs[True].tokens):
        assert torch.equal(a, b)
    for a, b in zip(outs[False].log_probs, outs[True].log_probs):
        torch.testing.assert_close(a, b, atol=1e-4, rtol=1e-4)
    assert torch.equal(outs[False].finished, outs[True].finished)
    assert outs[True].num_steps < outs[False].num_steps, (outs[True].num_steps, outs[False].num_steps)


def test_continuous_batching_steps_follow_total_length_cpu():
    from unirl_b200.rollout.engine.native_ar.generator import ARGenerator

    model, cfg = _model("cpu", torch.float32)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(8, cfg.vocab_size, (12,), generator=g) for _ in range(32)]
    gen = ARGenerator(model, page_size=16, max_running=8, use_cuda_graph=False, poll_interval=2, seed=3, continuous=True)
    out = gen.generate(prompts, max_new_tokens=64, temperature=1.0, stop_token_ids=_stops(cfg.vocab_size, 0.1), seed=5)
    total = sum(int(t.numel()) for t in out.tokens)
    longest = max(int(t.numel()) for t in out.tokens)
    # ideal: total / 8 rows; waves would need about (32 / 8) * longest.  Allow the polling granularity and the drain of the last rows.
    assert out.num_steps <= total / 8 + longest + 4 * 2, (out.num_steps, total, longest)
    assert gen.cache.allocator.num_free == gen.cache.num_pages - 1, "every page except the scratch page went back to the allocator"


@pytest.mark.gpu
def test_continuous_batching_on_gpu_with_shared_prefixes_and_graphs():
    """bf16 on CUDA with shared prompt pages (4 samples per prompt), CUDA graphs per bucket and early stops: same tokens as fixed waves
    for the same seeds (the random stream is keyed on (sequence, token index)), fewer decode steps."""
    from unirl_b200.rollout.engine.native_ar.generator import ARGenerator

    model, cfg = _model("cuda", torch.bfloat16)
    g = torch.Generator().manual_seed(4)
    base = [torch.randint(16, cfg.vocab_size, (int(n),), generator=g) for n in torch.randint(40, 200, (24,), generator=g)]
    prompts = [p for p in base for _ in range(4)]
    stops = _stops(cfg.vocab_size, 0.03)
    outs = {}
    for mode in (False, True):
        gen = ARGenerator(model, page_size=64, max_running=32, use_cuda_graph=True, poll_interval=8, seed=5, continuous=mode)
        outs[mode] = gen.generate(prompts, max_new_tokens=96, temperature=1.0, stop_token_ids=stops, seed=11)
        gen.release_cache()
    # The random stream is keyed on (sequence, token index), so both modes draw with the same numbers; the logits differ in the last bf16
    # bits (the batch shape picks the GEMM path and its summation order), a near-tie flips now and then, and a flipped token changes the
    # rest of its sequence.  So: almost every sequence starts identically, and most are identical to the end.
    pairs = list(zip(outs[False].tokens, outs[True].tokens))
    head = sum(int(torch.equal(a[:12], b[:12])) for a, b in pairs)
    same = sum(int(torch.equal(a, b)) for a, b in pairs)
    assert head >= int(0.9 * len(prompts)) and same >= int(0.5 * len(prompts)), f"{head} of {len(prompts)} sequences agree on 12 tokens, {same} on all"
    assert outs[True].num_steps < 0.95 * outs[False].num_steps, (outs[True].num_steps, outs[False].num_steps)
    # A group of 4 samples shares its prompt pages and leaves the batch when its longest member stops, so a slot is busy for the
    # group's maximum length, not for its own: with geometric lengths that is about twice the mean.  Bound: the group-maximum lengths
    # packed perfectly into the 8 group slots, plus one full-length tail.
    lens = torch.tensor([int(t.numel()) for t in outs[True].tokens]).view(-1, 4)
    assert outs[True].num_steps <= int(lens.max(1).values.sum()) / 8 + 96 + 16, (outs[True].num_steps, lens.max(1).values.sum())
