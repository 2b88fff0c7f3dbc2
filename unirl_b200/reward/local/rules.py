"""Rule-based text rewards: multiple-choice exact match, GSM8K final-number match, ``\\boxed{}`` math match,
and a symbolic-equivalence grader.  Parity: ``unirl/reward/local/{mc_exact_match,gsm8k_exact_match,math_boxed,mathverify}.py``
(the last uses the external ``math-verify`` grader when importable and falls back to normalised comparison).
"""

from __future__ import annotations

import re
import time
from dataclasses import dataclass
from fractions import Fraction
from typing import Any, Callable, Dict, List, Optional

from unirl_b200.reward.base import RewardBackend
from unirl_b200.types.reward import RewardRequest, RewardResponse

_THINK = re.compile(r"<think>.*?</think>", re.S)
_NUM = re.compile(r"-?\d[\d,]*\.?\d*(?:/\d+)?")


def strip_thinking(text: str) -> str:
    text = _THINK.sub("", text)
    return text.split("</think>")[-1] if "</think>" in text else text


def last_boxed(text: str) -> Optional[str]:
    i = text.rfind("\\boxed")
    if i < 0:
        return None
    j = text.find("{", i)
    if j < 0:
        return None
    depth = 0
    for k in range(j, len(text)):
        depth += text[k] == "{"
        depth -= text[k] == "}"
        if depth == 0:
            return text[j + 1 : k]
    return None


def normalize_math(s: str) -> str:
    s = s.strip().strip("$").replace("\\!", "").replace("\\,", "").replace("\\ ", "").replace(" ", "")
    s = re.sub(r"\\text\{(.*?)\}", r"\1", s)
    s = s.replace("\\dfrac", "\\frac").replace("\\tfrac", "\\frac").replace("\\left", "").replace("\\right", "")
    s = re.sub(r"\\frac\{([^{}]+)\}\{([^{}]+)\}", r"(\1)/(\2)", s)
    s = s.rstrip(".").replace(",", "")
    return s.lower()


def _as_number(s: str) -> Optional[Fraction]:
    s = s.replace("(", "").replace(")", "").replace("%", "")
    try:
        return Fraction(s)
    except (ValueError, ZeroDivisionError):
        try:
            return Fraction(float(s)).limit_denominator(10**9)
        except ValueError:
            return None


def math_equal(pred: str, gold: str) -> bool:
    a, b = normalize_math(pred), normalize_math(gold)
    if a == b:
        return True
    na, nb = _as_number(a), _as_number(b)
    return na is not None and nb is not None and na == nb


class _TextRuleBackend(RewardBackend):
    preferred_input_kind = "text"

    def _gold(self, meta: Optional[Dict[str, Any]]) -> Optional[str]:
        if not meta:
            return None
        for k in ("answer", "ground_truth", "gold", "label", "target"):
            if meta.get(k) is not None:
                return str(meta[k])
        return None

    def score(self, response: str, gold: Optional[str], meta: Optional[Dict[str, Any]]) -> float:
        raise NotImplementedError

    def compute_rewards(self, request: RewardRequest) -> RewardResponse:
        t0 = time.perf_counter()
        texts = request.generated.get("text")
        texts = list(texts.texts) if hasattr(texts, "texts") else list(texts or [])
        metas = request.metadata or [None] * len(texts)
        rewards, ok, errs = [], [], []
        for t, m in zip(texts, metas):
            try:
                rewards.append(float(self.score(t, self._gold(m), m)))
                ok.append(True)
                errs.append(None)
            except Exception as e:  # noqa: BLE001 - reported per sample; the service fails fast on it
                rewards.append(0.0)
                ok.append(False)
                errs.append(repr(e))
        return RewardResponse(rewards=rewards, successes=ok, errors=errs, compute_time=time.perf_counter() - t0)


class MCExactMatchRewardScorer(_TextRuleBackend):
    """Multiple choice: last standalone option letter (A–J) of the response equals the gold letter."""

    def __init__(self, base_device: str = "cpu", config: Any = None):
        pass

    def score(self, response, gold, meta):
        if gold is None:
            raise ValueError("mc_exact_match needs metadata['answer']")
        letters = re.findall(r"\b([A-J])\b", strip_thinking(response).upper())
        return 1.0 if letters and letters[-1] == gold.strip().upper()[:1] else 0.0


class GSM8KExactMatchRewardScorer(_TextRuleBackend):
    """Final number after ``####`` (or the last number in the response) equals the gold number."""

    def __init__(self, base_device: str = "cpu", config: Any = None):
        pass

    def score(self, response, gold, meta):
        if gold is None:
            raise ValueError("gsm8k_exact_match needs metadata['answer']")
        body = strip_thinking(response)
        tail = body.split("####")[-1] if "####" in body else body
        nums = _NUM.findall(tail)
        gold_n = _NUM.findall(gold.split("####")[-1])
        return 1.0 if nums and gold_n and math_equal(nums[-1], gold_n[-1]) else 0.0


class MathBoxedRewardScorer(_TextRuleBackend):
    def __init__(self, base_device: str = "cpu", config: Any = None):
        pass

    def score(self, response, gold, meta):
        if gold is None:
            raise ValueError("math_boxed needs metadata['answer']")
        pred = last_boxed(strip_thinking(response))
        gold_b = last_boxed(gold) or gold
        return 1.0 if pred is not None and math_equal(pred, gold_b) else 0.0


@dataclass
class MCExactMatchSpec:
    """The rule needs no settings; the class exists because recipes name it under the backend's ``config``."""


@dataclass
class GSM8KExactMatchSpec:
    pass


@dataclass
class MathBoxedSpec:
    pass


@dataclass
class MathVerifySpec:
    timeout_s: float = 5.0
    boxed_only: bool = False


class MathVerifyRewardScorer(_TextRuleBackend):
    def __init__(self, base_device: str = "cpu", config: Optional[MathVerifySpec] = None):
        self.config = config or MathVerifySpec()
        try:
            import math_verify  # type: ignore

            self._mv = math_verify
        except Exception:  # noqa: BLE001 - optional dependency
            self._mv = None

    def score(self, response, gold, meta):
        if gold is None:
            raise ValueError("mathverify needs metadata['answer']")
        body = strip_thinking(response)
        if self._mv is not None:
            try:
                return 1.0 if self._mv.verify(self._mv.parse(f"${gold}$"), self._mv.parse(body)) else 0.0
            except Exception:  # noqa: BLE001
                pass
        pred = last_boxed(body)
        if pred is None and not self.config.boxed_only:
            nums = _NUM.findall(body)
            pred = nums[-1] if nums else None
        return 1.0 if pred is not None and math_equal(pred, last_boxed(gold) or gold) else 0.0


__all__ = ["MCExactMatchRewardScorer", "GSM8KExactMatchRewardScorer", "MathBoxedRewardScorer", "MathVerifyRewardScorer", "MathVerifySpec", "MCExactMatchSpec",
           "GSM8KExactMatchSpec", "MathBoxedSpec",
           "last_boxed", "normalize_math", "math_equal", "strip_thinking"]
