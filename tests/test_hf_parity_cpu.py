"""Logit parity against the Hugging Face implementations (tiny random-init configs, CPU fp32): checks the key grammar,
the rotary convention, per-head q/k norm, grouped-query attention and the fused QKV / gate-up packing in one go."""

import pytest
import torch

transformers = pytest.importorskip("transformers")


def _packed_meta(b, l):
    from unirl_b200.models.qwen3.modeling import AttnMeta

    return AttnMeta(mode="train", positions=torch.arange(l).repeat(b), cu_seqlens=torch.arange(0, (b + 1) * l, l, dtype=torch.int32), max_seqlen=l)


@pytest.mark.parametrize("tie,bias", [(False, False), (True, False)])
def test_qwen3_logits_match_transformers(tie, bias):
    if not hasattr(transformers, "Qwen3ForCausalLM"):
        pytest.skip("transformers build without Qwen3")
    from unirl_b200.models.qwen3.modeling import Qwen3Config, Qwen3Transformer

    torch.manual_seed(0)
    hc = transformers.Qwen3Config(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                                  num_key_value_heads=2, head_dim=32, max_position_embeddings=256, rope_theta=10000.0, rms_norm_eps=1e-6,
                                  tie_word_embeddings=tie, attention_bias=bias)
    hf = transformers.Qwen3ForCausalLM(hc).eval().float()
    cfg = Qwen3Config.from_hf_dict(hc.to_dict())
    assert cfg.rope_theta == 10000.0 and cfg.tie_word_embeddings == tie
    model = Qwen3Transformer(cfg).float()
    model.load_hf_state_dict(hf.state_dict())
    ids = torch.randint(0, 320, (2, 17))
    with torch.no_grad():
        ref = hf(ids).logits
        out = model.logits(model(ids.reshape(-1), _packed_meta(2, 17))).view(2, 17, -1)
    assert torch.allclose(out, ref, atol=2e-5, rtol=1e-4), (out - ref).abs().max().item()
    back = model.hf_state_dict()
    for k, v in hf.state_dict().items():
        if k in back:
            assert torch.equal(back[k], v), k


def test_qwen25_vl_matches_transformers():
    """Vision tower (windowed + full attention blocks, 2x2 merger), 3-axis rotary positions and the decoder, from one
    checkpoint-format state dict.  ``tokens_per_second=1`` keeps the temporal axis of still images at the text position in
    every library version."""
    if not hasattr(transformers, "Qwen2_5_VLForConditionalGeneration"):
        pytest.skip("transformers build without Qwen2.5-VL")
    from unirl_b200.models.qwen3.modeling import AttnMeta
    from unirl_b200.models.qwen_vl.modeling import QwenVLConfig, QwenVLTransformer

    torch.manual_seed(0)
    hc = transformers.Qwen2_5_VLConfig(
        text_config=dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=512, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, rope_theta=10000.0,
                         tie_word_embeddings=False),
        vision_config=dict(depth=3, hidden_size=32, num_heads=2, intermediate_size=48, patch_size=4, temporal_patch_size=2, spatial_merge_size=2,
                           in_channels=3, out_hidden_size=64, window_size=16, fullatt_block_indexes=[1], tokens_per_second=1),
        image_token_id=5, video_token_id=6, vision_start_token_id=4)
    hf = transformers.Qwen2_5_VLForConditionalGeneration(hc).eval().float()
    cfg = QwenVLConfig.from_hf_dict(hc.to_dict())
    assert cfg.mrope_section == (2, 3, 3) and cfg.vision.fullatt_block_indexes == (1,) and cfg.vision.window_size == 16
    model = QwenVLTransformer(cfg, dtype=torch.float32)
    model.load_hf_state_dict(hf.state_dict())
    grid = torch.tensor([[1, 6, 10], [1, 4, 4]])  # 6x10 patches: partial windows on both edges; 4x4: exactly one window
    pv = torch.randn(int((grid[:, 1] * grid[:, 2]).sum()), 3 * 2 * 4 * 4)
    ids = torch.tensor([7, 8, 4] + [5] * (6 * 10 // 4) + [9, 10, 11, 4] + [5] * (4 * 4 // 4) + [12, 13, 14, 15])
    with torch.no_grad():
        kw = dict(input_ids=ids[None], pixel_values=pv, image_grid_thw=grid, attention_mask=torch.ones(1, len(ids), dtype=torch.long))
        try:
            ref = hf(**kw, mm_token_type_ids=(ids == 5).int()[None]).logits[0]
        except TypeError:  # library versions that infer the modality from the token ids
            ref = hf(**kw).logits[0]
        meta = AttnMeta(mode="train", cu_seqlens=torch.tensor([0, len(ids)], dtype=torch.int32), max_seqlen=len(ids))
        model.prepare_multimodal([ids], [{"pixel_values": pv, "image_grid_thw": grid}], meta)
        out = model.logits(model(ids, meta))
    assert torch.allclose(out, ref, atol=2e-5, rtol=1e-4), (out - ref).abs().max().item()
    back = model.hf_state_dict()
    for k, v in hf.state_dict().items():
        assert k in back and torch.equal(back[k].reshape(v.shape), v), k


def test_bundles_load_checkpoint_directories(tmp_path):
    """``config.json`` + ``*.safetensors`` written by the Hugging Face classes load through the bundles' public constructors."""
    import json

    from safetensors.torch import save_file

    if not (hasattr(transformers, "Qwen3ForCausalLM") and hasattr(transformers, "Qwen2_5_VLForConditionalGeneration")):
        pytest.skip("transformers build without the Qwen model classes")
    from unirl_b200.models.qwen3.bundle import Qwen3Bundle
    from unirl_b200.models.qwen3.config import Qwen3PipelineConfig
    from unirl_b200.models.qwen_vl.bundle import QwenVLBundle
    from unirl_b200.models.qwen_vl.config import QwenVLPipelineConfig

    torch.manual_seed(1)
    hc = transformers.Qwen3Config(vocab_size=320, hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                                  head_dim=32, max_position_embeddings=256, rope_theta=10000.0, tie_word_embeddings=False)
    hf = transformers.Qwen3ForCausalLM(hc).float()
    d = tmp_path / "qwen3"
    d.mkdir()
    save_file({k: v.contiguous() for k, v in hf.state_dict().items()}, str(d / "model.safetensors"))
    (d / "config.json").write_text(json.dumps(hc.to_dict()))
    b = Qwen3Bundle.from_config(Qwen3PipelineConfig(pretrained_model_ckpt_path=str(d), model_precision="fp32", device="cpu"))
    assert b.model_config.rope_theta == 10000.0
    assert torch.equal(b.transformer.embed_tokens.detach(), hf.state_dict()["model.embed_tokens.weight"])

    vc = transformers.Qwen2_5_VLConfig(
        text_config=dict(vocab_size=320, hidden_size=64, intermediate_size=128, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                         max_position_embeddings=512, rope_scaling={"type": "mrope", "mrope_section": [2, 3, 3]}, rope_theta=10000.0, tie_word_embeddings=False),
        vision_config=dict(depth=2, hidden_size=32, num_heads=2, intermediate_size=48, patch_size=4, temporal_patch_size=2, spatial_merge_size=2, in_channels=3,
                           out_hidden_size=64, window_size=16, fullatt_block_indexes=[1], tokens_per_second=1),
        image_token_id=5, video_token_id=6, vision_start_token_id=4)
    vl = transformers.Qwen2_5_VLForConditionalGeneration(vc).float()
    d2 = tmp_path / "qwen_vl"
    d2.mkdir()
    save_file({k: v.contiguous() for k, v in vl.state_dict().items()}, str(d2 / "model.safetensors"))
    (d2 / "config.json").write_text(json.dumps(vc.to_dict()))
    vb = QwenVLBundle.from_config(QwenVLPipelineConfig(pretrained_model_ckpt_path=str(d2), model_precision="fp32", device="cpu"))
    assert vb.model_config.vision.depth == 2 and vb.model_config.mrope_section == (2, 3, 3)
    assert torch.equal(vb.transformer.visual.merge_fc2.detach(), vl.state_dict()["model.visual.merger.mlp.2.weight"])


@pytest.mark.parametrize("act,proj", [("quick_gelu", True), ("gelu", False)])
def test_clip_text_tower_matches_transformers(tmp_path, act, proj):
    """Published-layout CLIP text checkpoints (with and without the projection head) land in the native encoder: last and penultimate
    hidden states and the pooled vector agree with ``transformers``."""
    from transformers import CLIPTextConfig, CLIPTextModel, CLIPTextModelWithProjection

    from unirl_b200.models.dit.text_keys import load_hf_text_encoder

    torch.manual_seed(0)
    hc = CLIPTextConfig(vocab_size=99, hidden_size=32, intermediate_size=64, num_hidden_layers=3, num_attention_heads=4, max_position_embeddings=16, hidden_act=act,
                        projection_dim=24, eos_token_id=98, bos_token_id=97, pad_token_id=98)
    hf = (CLIPTextModelWithProjection if proj else CLIPTextModel)(hc).eval()
    hf.save_pretrained(tmp_path)
    enc, cfg = load_hf_text_encoder(str(tmp_path), dtype=torch.float32)
    assert cfg.act == act and cfg.projection_dim == (24 if proj else 0)
    ids = torch.randint(0, 97, (3, 16))
    ids[:, 0] = 97
    for b, n in enumerate((5, 16, 9)):
        ids[b, n - 1:] = 98  # EOS, then padding with the same id: the pooled vector is taken at the FIRST one
    with torch.no_grad():
        out = hf(input_ids=ids, output_hidden_states=True)
        seq, pooled = enc(ids)
    torch.testing.assert_close(seq, out.hidden_states[-2], rtol=1e-4, atol=1e-5)  # SD3 conditions on the penultimate layer
    want = out.text_embeds if proj else out.pooler_output
    torch.testing.assert_close(pooled, want, rtol=1e-4, atol=1e-5)
    enc.cfg.penultimate = False
    torch.testing.assert_close(enc(ids)[0], out.last_hidden_state, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("umt5,d_kv", [(False, 8), (True, 8), (False, 6)])
def test_t5_encoder_matches_transformers(tmp_path, umt5, d_kv):
    """T5 v1.1 (one shared relative-position table) and UMT5 (one per layer) encoders: hidden states agree with ``transformers``,
    padding masked; the third case has heads narrower than width / heads, as the byte-level ByT5 glyph encoder does."""
    from transformers import T5Config, T5EncoderModel, UMT5Config, UMT5EncoderModel

    from unirl_b200.models.dit.text_keys import load_hf_text_encoder

    torch.manual_seed(1)
    kw = dict(vocab_size=120, d_model=32, d_kv=d_kv, d_ff=48, num_layers=3, num_heads=4, relative_attention_num_buckets=8, relative_attention_max_distance=20,
              feed_forward_proj="gated-gelu", dropout_rate=0.0)
    hf = (UMT5EncoderModel(UMT5Config(**kw)) if umt5 else T5EncoderModel(T5Config(**kw))).eval()
    with torch.no_grad():  # the library initialises some tables identically across layers: make every tensor distinct
        for p in hf.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    hf.save_pretrained(tmp_path)
    enc, cfg = load_hf_text_encoder(str(tmp_path), dtype=torch.float32)
    assert cfg.rel_bias_per_layer == umt5 and cfg.kind == "t5" and cfg.head_dim == (0 if d_kv == 8 else d_kv) and cfg.eos_token_id == 1
    ids = torch.randint(1, 120, (2, 23))
    mask = torch.ones(2, 23, dtype=torch.long)
    mask[1, 15:] = 0
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        got, pooled = enc(ids, mask)
    assert pooled is None
    torch.testing.assert_close(got[0], want[0], rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(got[1, :15], want[1, :15], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("family", ["qwen2", "llama", "qwen3"])
def test_llm_text_tower_matches_transformers(tmp_path, family):
    """Decoder-only text towers (Qwen-Image: Qwen2.5-VL's language model; HunyuanVideo: LLaMA; Z-Image: Qwen3) loaded from a checkpoint
    directory: last hidden states of a right-padded batch agree with ``transformers`` at every real token and are zero at the padding."""
    from unirl_b200.models.dit.llm_tower import LLMTextTower
    from unirl_b200.models.dit.text_keys import load_hf_text_encoder

    torch.manual_seed(2)
    kw = dict(vocab_size=300, hidden_size=64, intermediate_size=96, num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=128,
              rms_norm_eps=1e-6, rope_theta=10000.0, eos_token_id=7)
    if family == "qwen2":
        hf = transformers.Qwen2Model(transformers.Qwen2Config(**kw))
    elif family == "llama":
        hf = transformers.LlamaModel(transformers.LlamaConfig(**kw, attention_bias=False))
    else:
        if not hasattr(transformers, "Qwen3Model"):
            pytest.skip("transformers build without Qwen3")
        hf = transformers.Qwen3Model(transformers.Qwen3Config(**kw, head_dim=16))
    hf = hf.eval().float()
    with torch.no_grad():
        for p in hf.parameters():
            p.add_(torch.randn_like(p) * 0.02)  # biases and norm scales away from their constant initial values
    hf.save_pretrained(tmp_path)
    tower, info = load_hf_text_encoder(str(tmp_path), dtype=torch.float32)
    assert isinstance(tower, LLMTextTower) and info.kind == "llm" and info.hidden_size == 64 and info.eos_token_id == 7
    assert (tower.decoder.layers[0].qkv_bias is not None) == (family == "qwen2") and (tower.decoder.layers[0].q_norm is not None) == (family == "qwen3")
    ids = torch.randint(8, 300, (3, 21))
    mask = torch.ones(3, 21, dtype=torch.long)
    mask[0, 9:], mask[2, 17:] = 0, 0
    with torch.no_grad():
        want = hf(input_ids=ids, attention_mask=mask).last_hidden_state
        got, pooled = tower(ids, mask)
    assert pooled is None and got.shape == want.shape
    keep = mask.bool()
    torch.testing.assert_close(got[keep], want[keep], rtol=1e-4, atol=2e-5)
    assert float(got[~keep].abs().max()) == 0.0


def test_llm_text_tower_reads_the_language_model_of_a_vision_language_checkpoint():
    """Key grammars of vision-language files: ``model.language_model.*`` and ``language_model.model.*`` map to the decoder, vision and
    head tensors are left out; the configuration's text part is used."""
    from unirl_b200.models.dit.llm_tower import decoder_config_from_hf, language_model_tensors

    sd = {"model.language_model.layers.0.input_layernorm.weight": torch.ones(4), "model.visual.blocks.0.norm1.weight": torch.ones(4),
          "language_model.model.norm.weight": torch.ones(4), "visual.merger.mlp.0.weight": torch.ones(2, 2), "lm_head.weight": torch.ones(3, 4),
          "model.embed_tokens.weight": torch.ones(3, 4)}
    got = language_model_tensors(sd)
    assert sorted(got) == ["model.embed_tokens.weight", "model.layers.0.input_layernorm.weight", "model.norm.weight"]
    cfg = decoder_config_from_hf({"model_type": "qwen2_5_vl", "vision_config": {"depth": 2, "hidden_size": 8},
                                  "text_config": {"model_type": "qwen2_5_vl_text", "vocab_size": 50, "hidden_size": 32, "intermediate_size": 48, "num_hidden_layers": 1,
                                                  "num_attention_heads": 4, "num_key_value_heads": 2, "rope_theta": 1000000.0, "rms_norm_eps": 1e-6}})
    assert cfg.attention_bias and not cfg.qk_norm and cfg.head_dim == 8 and cfg.rope_theta == 1000000.0 and cfg.num_hidden_layers == 1


def test_qwen_image_bundle_loads_its_language_model_tower_from_the_checkpoint(tmp_path):
    """A checkpoint directory with the transformer and a ``text_encoder`` folder written by ``transformers`` (a Qwen2 decoder): the bundle
    builds the package's own decoder as the text tower, and the Qwen-Image text stage returns that model's hidden states past the template prefix."""
    import json

    from safetensors.torch import save_file

    from unirl_b200.models.dit.llm_tower import LLMTextTower
    from unirl_b200.models.qwen_image import QwenImagePipeline, QwenImagePipelineConfig
    from unirl_b200.models.qwen_image.pipeline import PROMPT_PREFIX, PROMPT_SUFFIX

    torch.manual_seed(4)
    rnd = QwenImagePipeline.from_config(QwenImagePipelineConfig(pretrained_model_ckpt_path="random:tiny-qwen-image", model_precision="fp32", autocast_precision="fp32", device="cpu"))
    tdim = rnd.bundle.spec.transformer.text_dim
    save_file({k: v.contiguous() for k, v in rnd.bundle.transformer.state_dict().items()}, str(tmp_path / "transformer.safetensors"))
    (tmp_path / "config.json").write_text(json.dumps({"preset": "tiny-qwen-image"}))
    hf = transformers.Qwen2Model(transformers.Qwen2Config(vocab_size=512, hidden_size=tdim, intermediate_size=2 * tdim, num_hidden_layers=2, num_attention_heads=4,
                                                          num_key_value_heads=2, max_position_embeddings=512, rope_theta=10000.0, eos_token_id=3)).eval().float()
    hf.save_pretrained(tmp_path / "text_encoder")
    pipe = QwenImagePipeline.from_config(QwenImagePipelineConfig(pretrained_model_ckpt_path=str(tmp_path), model_precision="fp32", autocast_precision="fp32", device="cpu",
                                                                 max_sequence_length=64))
    tower = pipe.bundle.text_encoders[0]
    assert isinstance(tower, LLMTextTower) and tower.cfg.hidden_size == tdim
    assert torch.equal(tower.decoder.embed_tokens.detach(), hf.state_dict()["embed_tokens.weight"])
    tok = pipe.bundle.tokenizers[0]  # no tokenizer folder: the byte tokenizer stands in, the tower does not care
    emb = pipe.text_embed.embed(["a red cube"])
    ids = torch.tensor([[int(i) % 512 for i in tok.encode(PROMPT_PREFIX + "a red cube" + PROMPT_SUFFIX)]])
    with torch.no_grad():
        want = hf(input_ids=ids).last_hidden_state[:, len(tok.encode(PROMPT_PREFIX)):][:, :64]
    torch.testing.assert_close(emb.embeds, want, rtol=1e-4, atol=2e-5)
    assert emb.pooled is None and int(emb.attn_mask.sum()) == want.shape[1]


def test_clip_vision_tower_matches_transformers(tmp_path):
    """The image encoder of the WAN image-to-video checkpoints: penultimate hidden states agree with ``transformers``' ``CLIPVisionModel``."""
    from transformers import CLIPVisionConfig as HFConfig
    from transformers import CLIPVisionModel

    from unirl_b200.models.dit.clip_vision import CLIPVisionTower

    torch.manual_seed(5)
    hf = CLIPVisionModel(HFConfig(hidden_size=32, intermediate_size=48, num_hidden_layers=3, num_attention_heads=4, image_size=28, patch_size=14, hidden_act="gelu")).eval()
    with torch.no_grad():
        for p in hf.parameters():
            p.add_(torch.randn_like(p) * 0.05)
    hf.save_pretrained(tmp_path)
    tower = CLIPVisionTower.from_hf(str(tmp_path), dtype=torch.float32)
    assert tower.cfg.num_tokens == 5
    px = torch.randn(2, 3, 28, 28)
    with torch.no_grad():
        want = hf(pixel_values=px, output_hidden_states=True).hidden_states[-2]
    torch.testing.assert_close(tower(px), want, rtol=1e-4, atol=1e-5)
    pics = torch.rand(2, 3, 40, 60)
    assert tower.encode(pics).shape == (2, 5, 32) and abs(float(tower.preprocess(torch.full((1, 3, 28, 28), 0.48145466))[0, 0].mean())) < 1e-6
