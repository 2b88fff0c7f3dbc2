"""Triple text encoder stage of SD3 (``unirl/models/sd3/text_embed.py:51-140``): see ``models/dit/text_embed.py`` (``combine="sd3"``)."""
from unirl_b200.models.dit.text_embed import TextEmbedStage as SD3TextEmbedStage

__all__ = ["SD3TextEmbedStage"]
