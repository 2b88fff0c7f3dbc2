from unirl_b200.types.segments.base import Segment, SegmentStatus  # noqa: F401
from unirl_b200.types.segments.latent import (  # noqa: F401
    LatentSegment,
    make_audio_segment,
    make_image_segment,
    make_video_segment,
)
from unirl_b200.types.segments.text import TextSegment  # noqa: F401
