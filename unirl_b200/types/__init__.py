"""Typed contracts shared by every layer (requests, tracks, segments, conditions, sampling)."""
from unirl_b200.types.conditions import (  # noqa: F401
    Condition,
    FusedMultimodalCondition,
    ImageEmbedCondition,
    ImageLatentCondition,
    Modality,
    TextEmbedCondition,
    TextTokenCondition,
)
from unirl_b200.types.media import MediaRef  # noqa: F401
from unirl_b200.types.media_preview import MediaPreview, build_media_preview_for_track  # noqa: F401
from unirl_b200.types.noise_recipe import NoiseRecipe  # noqa: F401
from unirl_b200.types.primitives import Audio, Audios, Image, Images, Text, Texts, Video, Videos  # noqa: F401
from unirl_b200.types.prompts import RolloutInputs  # noqa: F401
from unirl_b200.types.reward import RewardRequest, RewardResponse, RewardType  # noqa: F401
from unirl_b200.types.rollout_req import RolloutReq  # noqa: F401
from unirl_b200.types.rollout_resp import RolloutResp, RolloutTrack  # noqa: F401
from unirl_b200.types.sampling import (  # noqa: F401
    ARSamplingParams,
    BaseSamplingParams,
    ComposedSamplingParams,
    DiffusionSamplingParams,
    SamplingRequirements,
    get_ar_params,
    get_diffusion_params,
)
from unirl_b200.types.segments import (  # noqa: F401
    LatentSegment,
    Segment,
    SegmentStatus,
    TextSegment,
    make_audio_segment,
    make_image_segment,
    make_video_segment,
)
from unirl_b200.types.trajectory_store import Trajectory, TrajectoryBuilder, compute_trajectory_positions  # noqa: F401
