"""Reward scorers, the HTTP reward service and its client (served from a thread on 127.0.0.1)."""
import os
import sys
import threading
import time

import pytest
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "reward_service"))

from unirl_b200.distributed.utils import free_port  # noqa: E402
from unirl_b200.reward.local.scorers import GenEvalScorer, OCRScorer, build_scorer  # noqa: E402
from unirl_b200.reward.remote import RemoteRewardBackend, decode_image, encode_image  # noqa: E402
from unirl_b200.types.primitives import Images, Texts  # noqa: E402
from unirl_b200.types.reward import RewardRequest  # noqa: E402


def _req(n=3, **kw):
    return RewardRequest(primitives={"text": Texts.from_list([f'a sign that says "hello {i}"' for i in range(n)])},
                         generated={"image": Images(pixels=torch.rand(n, 3, 32, 32, generator=torch.Generator().manual_seed(0)))},
                         sample_ids=[str(i) for i in range(n)], **kw)


def test_png_round_trip_is_lossless_to_8_bits():
    px = torch.rand(3, 17, 23)
    assert float((decode_image(encode_image(px)) - px).abs().max()) <= 0.5 / 255 + 1e-6


@pytest.mark.parametrize("name,lo,hi", [("clip", -1.0, 1.0), ("pickscore", -100.0, 100.0), ("hpsv2", -100.0, 100.0), ("aesthetic", 1.0, 10.0), ("image_reward", -50, 50)])
def test_model_scorers_are_deterministic_and_in_range(name, lo, hi):
    s = build_scorer(name, device="cpu", seed=3)
    a, b = s.compute_rewards(_req()).rewards, s.compute_rewards(_req()).rewards
    assert a == b and all(lo <= r <= hi for r in a)


def test_rule_scorers():
    ocr = OCRScorer().compute_rewards(_req(metadata=[{"ocr_text": "hello 0"}, {"ocr_text": "hellp 1"}, {"ocr_text": ""}])).rewards
    assert ocr[0] == 1.0 and 0.5 < ocr[1] < 1.0 and ocr[2] == 0.0
    meta = [{"include": [{"class": "dog", "count": 2}, {"class": "ball", "color": "red"}], "detections": [{"class": "dog"}, {"class": "dog"}, {"class": "ball", "color": "blue"}]}]
    assert GenEvalScorer().compute_rewards(RewardRequest(metadata=meta, sample_ids=["0"])).rewards == [0.5]


@pytest.mark.timeout(120)
def test_http_service_and_client_agree_with_local_scoring():
    import uvicorn
    from unirl_b200_reward_service.app import create_app

    port = free_port()
    server = uvicorn.Server(uvicorn.Config(create_app({"clip": {"seed": 3}}), host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    client = RemoteRewardBackend(f"http://127.0.0.1:{port}", scorers=["clip", "geneval"], weights={"clip": 2.0, "geneval": 1.0}, batch_size=2, concurrency=2)
    try:
        for _ in range(100):
            if client.is_available():
                break
            time.sleep(0.1)
        assert client.is_available()
        meta = [{"include": [{"class": "dog"}], "detections": [{"class": "dog"}]}] * 3
        out = client.compute_rewards(_req(metadata=meta))
        local = build_scorer("clip", device="cpu", seed=3).compute_rewards(_req()).rewards
        assert len(out.rewards) == 3 and all(abs(o - (2.0 * l + 1.0)) < 2e-2 for o, l in zip(out.rewards, local))  # PNG quantisation only
        assert set(out.component_rewards) == {"clip", "geneval"}
    finally:
        server.should_exit = True
        th.join(10)


def _tiny_clip_checkpoint(path):
    """A CLIP checkpoint in the Hugging Face layout (random weights, a 54-entry vocabulary), written with the library's own save calls."""
    import json
    import os

    from transformers import CLIPConfig, CLIPModel, CLIPTextConfig, CLIPTokenizer, CLIPVisionConfig

    cfg = CLIPConfig(text_config=CLIPTextConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, max_position_embeddings=16,
                                                eos_token_id=1, bos_token_id=0, pad_token_id=1).to_dict(),
                     vision_config=CLIPVisionConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=2, image_size=32, patch_size=8).to_dict(),
                     projection_dim=16)
    torch.manual_seed(0)
    model = CLIPModel(cfg).eval()
    model.save_pretrained(path)
    vocab = {"<|startoftext|>": 0, "<|endoftext|>": 1}
    for ch in "abcdefghijklmnopqrstuvwxyz":
        vocab[ch] = len(vocab)
        vocab[ch + "</w>"] = len(vocab)
    with open(os.path.join(path, "vocab.json"), "w") as f:
        json.dump(vocab, f)
    with open(os.path.join(path, "merges.txt"), "w") as f:
        f.write("#version: 0.2\n")
    tok = CLIPTokenizer(os.path.join(path, "vocab.json"), os.path.join(path, "merges.txt"))
    tok.save_pretrained(path)
    with open(os.path.join(path, "preprocessor_config.json"), "w") as f:
        json.dump({"image_mean": [0.5, 0.4, 0.3], "image_std": [0.2, 0.25, 0.3], "size": {"shortest_edge": 32}, "crop_size": 32}, f)
    return model, tok


def test_scorers_load_a_published_layout_checkpoint_and_follow_the_published_formulas(tmp_path):
    from unirl_b200.reward.local.scorers import build_scorer
    from unirl_b200.types.primitives import Texts
    from unirl_b200.types.reward import RewardRequest

    model, tok = _tiny_clip_checkpoint(str(tmp_path))
    px = torch.rand(3, 3, 32, 32, generator=torch.Generator().manual_seed(1))  # already at the model's size: no resampling in the way of the comparison
    prompts = ["a cab", "zz top", "quiet fox"]
    with torch.no_grad():
        mean, std = torch.tensor([0.5, 0.4, 0.3]).view(1, 3, 1, 1), torch.tensor([0.2, 0.25, 0.3]).view(1, 3, 1, 1)
        enc = tok(prompts, padding="max_length", truncation=True, max_length=16, return_tensors="pt")
        out = model(pixel_values=(px - mean) / std, input_ids=enc["input_ids"], attention_mask=enc["attention_mask"])
        logits = out.logits_per_image.diagonal()
    req = RewardRequest(primitives={"text": Texts(texts=prompts)}, generated={"image": px}, sample_ids=["a", "b", "c"])
    clip = build_scorer("clip", model_id=str(tmp_path), device="cpu", batch_size=2).compute_rewards(req)
    torch.testing.assert_close(torch.tensor(clip.rewards), logits / 30, rtol=1e-4, atol=1e-5)
    pick = build_scorer("pickscore", model_id=str(tmp_path), device="cpu").compute_rewards(req)
    torch.testing.assert_close(torch.tensor(pick.rewards), logits / 26, rtol=1e-4, atol=1e-5)
    hps = build_scorer("hpsv2", model_id=str(tmp_path), device="cpu").compute_rewards(req)
    torch.testing.assert_close(torch.tensor(hps.rewards), logits / model.logit_scale.exp().item(), rtol=1e-4, atol=1e-5)
    big = build_scorer("clip", model_id=str(tmp_path), device="cpu").score(torch.rand(2, 3, 80, 56), ["a", "b"])  # resized and cropped on the way in
    assert big.shape == (2,) and torch.isfinite(big).all()
    with pytest.raises(FileNotFoundError, match="never downloaded"):
        build_scorer("clip", model_id="openai/clip-vit-large-patch14", device="cpu")


def test_service_config_validation_and_gpu_ledger():
    from unirl_b200_reward_service.config import RewardModelCfg, ServiceCfg, from_dict
    from unirl_b200_reward_service.workers import WorkerPool

    with pytest.raises(ValueError, match="num_replicas"):
        RewardModelCfg(name="clip", num_replicas=0)
    with pytest.raises(ValueError, match="num_gpus"):
        RewardModelCfg(name="clip", num_gpus=-1)
    with pytest.raises(ValueError, match="duplicate"):
        from_dict({"rewards": [{"name": "clip"}, {"name": "clip"}]})
    cfg = from_dict({"isolation": "thread", "gpu_ids": [4, 5, 6], "rewards": [{"name": "ocr", "num_replicas": 2, "num_gpus": 1}, {"name": "geneval"}]})
    assert cfg.gpus_needed() == 2
    pool = WorkerPool(cfg)
    try:
        assert pool.owned["ocr"] == [[4], [5]] and pool.owned["geneval"] == [[]], "whole GPUs, each owned by one replica"
        with pytest.raises(ValueError, match="GPUs"):
            pool.add(RewardModelCfg(name="geneval2", num_gpus=2))  # one GPU left
        with pytest.raises(KeyError):
            pool.get("no-such-reward")
    finally:
        pool.close()
    with pytest.raises(ValueError, match="need 4 GPUs"):
        WorkerPool(ServiceCfg(rewards=[RewardModelCfg(name="ocr", num_replicas=2, num_gpus=2)], gpu_ids=[0, 1]))


@pytest.mark.parametrize("isolation", ["thread", "process"])
def test_request_form_routes_each_request_to_its_rewards_and_isolates_failures(isolation):
    from unirl_b200_reward_service.app import RewardGateway
    from unirl_b200_reward_service.config import from_dict

    cfg = from_dict({"isolation": isolation, "gpu_ids": [],
                     "rewards": [{"name": "ocr", "num_replicas": 2}, {"name": "sharp", "scorer": "clip", "kwargs": {"seed": 3, "device": "cpu"}}]})
    gw = RewardGateway(config=cfg)
    try:
        png = encode_image(torch.rand(3, 32, 32, generator=torch.Generator().manual_seed(0)))
        reqs = [{"prompt": 'a sign that says "hello"', "image_png_b64": png, "rewards": ["ocr", "sharp"], "metadata": {"ocr_text": "hello"}},
                {"prompt": 'a sign that says "world"', "image_png_b64": png, "rewards": ["ocr"], "metadata": {"ocr_text": "word"}},
                {"prompt": "a cat", "image_png_b64": png, "rewards": ["sharp", "no-such-reward"]}]
        out = gw.score({"requests": reqs})["results"]
        assert out[0]["rewards"]["ocr"] == 1.0 and set(out[0]["rewards"]) == {"ocr", "sharp"} and not out[0]["errors"]
        assert 0.0 < out[1]["rewards"]["ocr"] < 1.0 and set(out[1]["rewards"]) == {"ocr"}
        assert "sharp" in out[2]["rewards"] and "no-such-reward" in out[2]["errors"] and "no-such-reward" not in out[2]["rewards"]
        again = gw.score({"requests": reqs[:1]})["results"][0]["rewards"]
        assert again["ocr"] == out[0]["rewards"]["ocr"] and abs(again["sharp"] - out[0]["rewards"]["sharp"]) < 1e-5, "replicas of a group agree"
        st = gw.stats()
        assert st["ocr"]["replicas"] == 2 and st["ocr"]["calls"] == 2 and st["sharp"]["errors"] == 0
    finally:
        gw.close()
