"""Prompt → ``TextEmbedCondition`` for the DiT families.

``combine="single"``    one encoder, its hidden states are the conditioning sequence.
``combine="sd3"``       CLIP-L and CLIP-G penultimate hidden states concatenated channel-wise, zero-padded to the T5
                        width and prepended to the T5 sequence; pooled = [CLIP-L pooled, CLIP-G pooled].
``combine="llm+clip"``  LLM hidden states as the sequence, CLIP pooled vector as the pooled conditioning (HunyuanVideo).
``combine="llm+glyph"`` LLM hidden states ++ a byte-level glyph encoder's hidden states of the prompt's quoted snippets, zero-padded
                        to the LLM width, along the token axis (HunyuanVideo-1.5; its own stage adds the chat template).

Identical prompts in a batch are encoded once (a GRPO batch repeats each prompt ``samples_per_prompt`` times).
Parity: ``unirl/models/sd3/text_embed.py:51-140`` (triple encoder + dedupe), ``unirl/models/wan21/text_embed.py``.
"""

from __future__ import annotations

import re
from typing import Any, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from unirl_b200.types.conditions import TextEmbedCondition
from unirl_b200.types.primitives import Texts


_QUOTED = re.compile(r"\"(.*?)\"|\u201c(.*?)\u201d")


def glyph_text(prompt: str) -> Optional[str]:
    """Quoted snippets of ``prompt`` (straight or curly quotes) as ``Text "a". Text "b". `` — first occurrences, in order; ``None``
    without any (``unirl/models/hunyuan_video15/text_embed.py:56-72``)."""
    found = [a or b for a, b in _QUOTED.findall(prompt or "")]
    found = list(dict.fromkeys(found)) if len(found) > 1 else found
    return (". ".join(f'Text "{t}"' for t in found) + ". ") if found else None


class TextEmbedStage:
    def __init__(self, encoders: Sequence[Any], tokenizers: Sequence[Any], combine: str = "single", text_dim: Optional[int] = None,
                 max_sequence_length: int = 256, glyph_max_length: int = 256):
        self.encoders, self.tokenizers, self.combine = list(encoders), list(tokenizers), combine
        self.text_dim = text_dim
        self.max_sequence_length = int(max_sequence_length)
        self.glyph_max_length = int(glyph_max_length)

    def append_glyph_stream(self, strs: List[str], seq: torch.Tensor, mask: torch.Tensor, k: int = 1) -> Tuple[torch.Tensor, torch.Tensor]:
        """``seq [B, L, D]`` / ``mask [B, L]`` of the prompts ``strs`` ++ the glyph encoder's (``encoders[k]``) hidden states of each
        prompt's quoted snippets, zero-padded to ``D``, along the token axis; a prompt without quotes contributes masked zeros."""
        enc = self.encoders[k]
        if enc.cfg.hidden_size > seq.shape[-1]:
            raise ValueError(f"the glyph encoder is wider ({enc.cfg.hidden_size}) than the conditioning sequence ({seq.shape[-1]})")
        glyphs = [glyph_text(s) for s in strs]
        some = [g for g in dict.fromkeys(glyphs) if g is not None]
        g_len = 1
        if some:
            cap, self.max_sequence_length = self.max_sequence_length, self.glyph_max_length
            try:
                g_all, _, m_all = self._encode_one(k, some)
            finally:
                self.max_sequence_length = cap
            g_all = g_all * m_all.unsqueeze(-1).to(g_all.dtype)
            g_len = g_all.shape[1]
        g_seq, g_mask = seq.new_zeros(len(strs), g_len, seq.shape[-1]), mask.new_zeros(len(strs), g_len)
        for i, g in enumerate(glyphs):
            if g is not None:
                j = some.index(g)
                g_seq[i, :, : g_all.shape[-1]] = g_all[j].to(g_seq.dtype)
                g_mask[i] = m_all[j].to(g_mask.dtype)
        return torch.cat([seq, g_seq], 1), torch.cat([mask, g_mask], 1)

    def _tokenize(self, tok: Any, texts: List[str], max_len: int, eos: int, vocab: int) -> Tuple[torch.Tensor, torch.Tensor]:
        rows = []
        for t in texts:
            ids = [int(i) % vocab for i in tok.encode(t)]
            if ids and ids[-1] == eos:  # a tokenizer that closes the sequence itself: one end marker, not two
                ids = ids[:-1]
            ids = ids[: max_len - 1] + [eos]
            rows.append(ids)
        width = max(len(r) for r in rows)
        ids = torch.zeros(len(rows), width, dtype=torch.long)
        mask = torch.zeros(len(rows), width, dtype=torch.long)
        for i, r in enumerate(rows):
            ids[i, : len(r)] = torch.tensor(r)
            mask[i, : len(r)] = 1
        return ids, mask

    def _encode_one(self, k: int, texts: List[str]) -> Tuple[torch.Tensor, Optional[torch.Tensor], torch.Tensor]:
        enc, tok = self.encoders[k], self.tokenizers[k]
        c = enc.cfg
        dev = next(enc.parameters()).device
        ids, mask = self._tokenize(tok, texts, min(c.max_length, self.max_sequence_length if c.kind != "clip" else c.max_length), c.eos_token_id, c.vocab_size)
        if c.kind == "clip":  # fixed-length context, as the CLIP towers are used
            ids = F.pad(ids, (0, c.max_length - ids.shape[1]), value=c.eos_token_id)
            mask = F.pad(mask, (0, c.max_length - mask.shape[1]), value=0)
        seq, pooled = enc(ids.to(dev), mask.to(dev))
        return seq, pooled, mask.to(dev)

    @torch.no_grad()
    def embed(self, texts: Any) -> TextEmbedCondition:
        strs = [t.to_str() if hasattr(t, "to_str") else str(t) for t in (texts.to_list() if isinstance(texts, Texts) else texts)]
        uniq: Dict[str, int] = {}
        for s in strs:
            uniq.setdefault(s, len(uniq))
        ulist = list(uniq)
        if self.combine == "single":
            seq, pooled, mask = self._encode_one(0, ulist)
        elif self.combine == "sd3":
            l_seq, l_pool, _ = self._encode_one(0, ulist)
            g_seq, g_pool, _ = self._encode_one(1, ulist)
            t_seq, _, t_mask = self._encode_one(2, ulist)
            clip = torch.cat([l_seq, g_seq], -1)
            clip = F.pad(clip, (0, t_seq.shape[-1] - clip.shape[-1]))
            seq = torch.cat([clip, t_seq], 1)
            mask = torch.cat([torch.ones(clip.shape[:2], dtype=t_mask.dtype, device=t_mask.device), t_mask], 1)
            pooled = torch.cat([l_pool, g_pool], -1)
        elif self.combine == "llm+clip":
            seq, _, mask = self._encode_one(0, ulist)
            _, pooled, _ = self._encode_one(1, ulist)
        elif self.combine == "llm+glyph":
            seq, pooled, mask = self._encode_one(0, ulist)
            if self.text_dim and seq.shape[-1] < self.text_dim:
                seq = F.pad(seq, (0, self.text_dim - seq.shape[-1]))
            seq, mask = self.append_glyph_stream(ulist, seq * mask.unsqueeze(-1).to(seq.dtype), mask)
        else:
            raise ValueError(f"unknown text combine mode {self.combine!r}")
        if self.text_dim and seq.shape[-1] != self.text_dim:
            seq = F.pad(seq, (0, self.text_dim - seq.shape[-1])) if seq.shape[-1] < self.text_dim else seq[..., : self.text_dim]
        idx = torch.tensor([uniq[s] for s in strs], device=seq.device)
        return TextEmbedCondition(embeds=seq[idx], pooled=None if pooled is None else pooled[idx], attn_mask=mask[idx])


__all__ = ["TextEmbedStage"]
