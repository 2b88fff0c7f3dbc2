"""Klein's empirical μ: the exponential time-shift parameter depends on BOTH the image token count and the number of
inference steps (two straight lines fitted at 10 and 200 steps, blended linearly in the step count; above 4300 tokens
the 200-step line alone is used).  Parity: ``unirl/models/flux2_klein/schedule.py``."""
from __future__ import annotations

from dataclasses import dataclass

from unirl_b200.sde.runtime import FlowMatchSchedulePolicy


def compute_empirical_mu(image_seq_len: int, num_steps: int) -> float:
    a1, b1 = 8.73809524e-05, 1.89833333
    a2, b2 = 0.00016927, 0.45666666
    if image_seq_len > 4300:
        return float(a2 * image_seq_len + b2)
    m_200 = a2 * image_seq_len + b2
    m_10 = a1 * image_seq_len + b1
    a = (m_200 - m_10) / 190.0
    b = m_200 - 200.0 * a
    return float(a * num_steps + b)


@dataclass
class KleinSchedulePolicy(FlowMatchSchedulePolicy):
    use_dynamic_shifting: bool = True

    def compute_mu(self, image_seq_len: int, num_inference_steps: int) -> float:
        return compute_empirical_mu(image_seq_len, num_inference_steps)


__all__ = ["KleinSchedulePolicy", "compute_empirical_mu"]
