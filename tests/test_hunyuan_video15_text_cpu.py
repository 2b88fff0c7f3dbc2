"""HunyuanVideo-1.5 text conditioning: chat-templated LLM stream with the template prefix cut off, plus the glyph stream of quoted snippets."""
import torch

from unirl_b200.models.hunyuan_video15.pipeline import HunyuanVideo15Pipeline, HunyuanVideo15PipelineConfig, glyph_text


def test_quoted_snippets_become_the_glyph_prompt():
    assert glyph_text('a sign that says "OPEN" next to a door') == 'Text "OPEN". '
    assert glyph_text('“早上好” on a banner, "SALE" below, "SALE" again') == 'Text "早上好". Text "SALE". '
    assert glyph_text("no quoted text here") is None and glyph_text("") is None


def test_two_streams_share_one_sequence_and_unquoted_prompts_mask_the_glyph_part():
    pipe = HunyuanVideo15Pipeline.from_config(HunyuanVideo15PipelineConfig(pretrained_model_ckpt_path="random:tiny-hunyuan-video15", model_precision="fp32",
                                                                        autocast_precision="fp32", device="cpu"))
    stage = pipe.text_embed
    assert len(stage.encoders) == 2 and stage.encoders[1].cfg.kind == "t5"
    prompts = ['a neon sign reading "HELLO WORLD" at night', "a cat on a sofa", 'a neon sign reading "HELLO WORLD" at night']
    cond = stage.embed(prompts)
    width = pipe.bundle.spec.transformer.text_dim
    assert cond.embeds.shape[0] == 3 and cond.embeds.shape[-1] == width and cond.attn_mask.shape == cond.embeds.shape[:2] and cond.pooled is None
    # the LLM part alone (one encoder) is the front of the sequence
    stage_llm = type(stage)(stage.encoders[:1], stage.tokenizers[:1], "single", width, stage.max_sequence_length)
    llm = stage_llm.embed(prompts)
    n = llm.embeds.shape[1]
    torch.testing.assert_close(cond.embeds[:, :n], llm.embeds)
    assert torch.equal(cond.attn_mask[:, :n], llm.attn_mask)
    # glyph part: real tokens for the quoted prompt, nothing for the other; equal prompts give equal rows
    g_mask, g_seq = cond.attn_mask[:, n:], cond.embeds[:, n:]
    assert int(g_mask[0].sum()) > 0 and int(g_mask[1].sum()) == 0 and float(g_seq[1].abs().max()) == 0.0
    assert torch.equal(g_seq[0], g_seq[2]) and float(g_seq[0].abs().max()) > 0
    glyph_width = stage.encoders[1].cfg.hidden_size
    assert float(g_seq[0][..., glyph_width:].abs().max()) == 0.0, "the glyph stream is zero-padded to the LLM width"
    want, _ = stage.encoders[1](*[t.unsqueeze(0) for t in _byte_ids(stage, 'Text "HELLO WORLD". ')])
    k = int(g_mask[0].sum())
    torch.testing.assert_close(g_seq[0, :k, :glyph_width], want[0, :k])
    # the system prefix is cut: the LLM stream is shorter than prefix + prompt
    tok = stage.tokenizers[0]
    assert n <= max(len(tok.encode(p)) for p in prompts) + len(tok.encode(stage.suffix)) + 1


def _byte_ids(stage, text):
    enc, tok = stage.encoders[1], stage.tokenizers[1]
    ids, mask = stage._tokenize(tok, [text], min(enc.cfg.max_length, stage.glyph_max_length), enc.cfg.eos_token_id, enc.cfg.vocab_size)
    return ids[0], mask[0]


def test_published_geometry_names_the_byte_level_glyph_encoder():
    from unirl_b200.models.dit.config import resolve_family

    spec = resolve_family("random:hunyuan-video15")
    g = spec.text_encoders[1] if hasattr(spec, "text_encoders") else None
    assert g is not None and (g.kind, g.vocab_size, g.hidden_size, g.num_layers, g.num_heads, g.head_dim, g.ffn_dim) == ("t5", 384, 1472, 12, 6, 64, 3584)
