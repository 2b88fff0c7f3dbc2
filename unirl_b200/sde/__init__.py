from unirl_b200.sde.kernels import (  # noqa: F401
    CPSSDEStrategy,
    DanceSDEStrategy,
    DPM2Strategy,
    FlowSDEStrategy,
    SDEStrategy,
    StepStrategy,
    make_strategy,
)
from unirl_b200.sde.noise import generate_latents, generate_shared_noise, regen_initial_noise  # noqa: F401
from unirl_b200.sde.runtime import FlowMatchSchedulePolicy, calculate_dynamic_mu, ensure_req_sigmas, get_sigma_schedule  # noqa: F401
