#!/usr/bin/env python
"""Headline benchmark: RL-step throughput of Qwen3-4B GRPO (tokens/s) and weight-sync latency (ms).

One step = weight sync -> rollout (native paged-KV engine) -> reward -> group advantages -> sharded
training update, driven through the public ``ARTrainer.train_step`` API on synthetic prompts
(uniform-random token ids, length 256-1024, 8 samples per prompt, up to 4096 response tokens, random-init
bf16 weights).  Per GPU the work is fixed (weak scaling): 16 prompts x 8 samples.

    python bench.py [--gpus N --steps K --warmup W]            (N > 1: launched by torchrun, one rank per GPU)
    python bench.py --impl reference ...                       (the reference arm)

``value`` is device-timed (CUDA events around the rollout / sync / train phases, max over ranks);
``e2e.value`` is wall-clock around the complete ``train_step`` calls, including the host->device copies of the
step's prompts and the device->host reads of its rollout and loss.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

_T_START = time.time()  # the wall budget counts from here (or from the launcher's start, see _job_start)

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--model", default="qwen3-4b")
    ap.add_argument("--prompts-per-gpu", type=int, default=16)
    ap.add_argument("--group-size", type=int, default=8)
    ap.add_argument("--max-new-tokens", type=int, default=4096)
    ap.add_argument("--prompt-min", type=int, default=256)
    ap.add_argument("--prompt-max", type=int, default=1024)
    ap.add_argument("--micro-batch", type=int, default=4)
    ap.add_argument("--rollout-tp", type=int, default=1, help="tensor-parallel degree of each rollout engine (1: one engine per GPU that aliases the trainer replica; 2: fused TP all-reduce + reshard weight sync)")
    ap.add_argument("--algorithm", default="grpo", choices=["grpo", "drpo"])
    ap.add_argument("--budget-s", type=float, default=float(os.environ.get("UNIRL_B200_BENCH_BUDGET_S", "780")),
                    help="wall-clock budget of the whole run in seconds (launcher start to exit); warm-up and timed steps are capped to fit, "
                         "the work inside a step never shrinks; 0 = no cap")
    ap.add_argument("--ckpt-layers", type=int, default=-1, help="recompute only the first N decoder blocks in backward (-1 = recipe default)")
    return ap.parse_args()


def reference_arm(args) -> None:
    """The reference (Tencent-Hunyuan/UniRL) through its own public API, installed under baseline/_ref."""
    ref = os.path.join(ROOT, "baseline", "_ref")
    why = None
    if not os.path.isdir(os.path.join(ref, "unirl")):
        why = "reference package is not installed under baseline/_ref"
    else:
        missing = []
        for mod in ("ray", "hydra", "omegaconf", "peft", "diffusers", "tensordict"):
            try:
                __import__(mod)
            except Exception:
                missing.append(mod)
        if missing:
            why = ("reference installed with --no-deps, but its entrypoints (python -m unirl.train_ar: Hydra + Ray single controller, "
                   "FSDP2 trainer) need packages absent from this offline image: " + ", ".join(missing))
    if why is None:
        why = "reference AR recipes require an SGLang/vLLM rollout server, which is not installable offline"
    print(json.dumps({"impl": "reference", "unavailable": why}))


def _job_start() -> float:
    """Start of the job on the wall clock: the launcher's creation time when this rank was spawned by ``torch.distributed.run``
    (its own start-up and rendezvous are part of what a caller's time limit sees), else the start of this script."""
    try:
        import psutil

        parent = psutil.Process(os.getppid())
        if any("torch.distributed.run" in a or a.endswith("torchrun") for a in parent.cmdline()):
            return min(_T_START, parent.create_time())
    except Exception:
        pass
    return _T_START


class StepBudget:
    """Caps the number of warm-up and timed steps so the run ends inside a wall budget.

    Every rank measures its own step times; the decisions are taken on the slowest rank's numbers (MAX all-reduce), so all
    ranks run the same number of steps.  At least ``min_warmup`` warm-up steps and one timed step always run."""

    def __init__(self, budget_s: float, t_start: float, world: int, min_warmup: int = 3, teardown_s: float = 25.0):
        self.budget_s, self.t_start, self.world, self.min_warmup, self.teardown_s = budget_s, t_start, world, min_warmup, teardown_s
        self.step_s = 0.0

    def observe(self, seconds: float) -> None:
        self.step_s = seconds  # the latest step: the first one carries graph capture and allocator growth

    def _agree(self, elapsed: float, step_s: float):
        if self.world == 1:
            return elapsed, step_s
        import torch
        import torch.distributed as dist

        t = torch.tensor([elapsed, step_s], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]), float(t[1])

    def steps_that_fit(self) -> int:
        if self.budget_s <= 0:
            return 1 << 30
        elapsed, step_s = self._agree(time.time() - self.t_start, self.step_s)
        left = self.budget_s - self.teardown_s - elapsed
        return int(left // (step_s * 1.05)) if step_s > 0 else 1 << 30

    def plan_warmup(self, done: int, requested: int, timed_requested: int) -> bool:
        """True when another warm-up step should run."""
        if done >= requested:
            return False
        if done < self.min_warmup:
            return True
        return self.steps_that_fit() - 1 >= min(timed_requested, 4)  # extra warm-up only while >= 4 timed steps still fit

    def plan_timed(self, requested: int) -> int:
        return max(1, min(requested, self.steps_that_fit()))


class ClockSampler:
    """Samples SM clocks / throttle reasons with nvidia-smi while the timed region runs."""

    Q = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int):
        self.index, self.rows, self._stop, self._t = index, [], threading.Event(), None

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([c.strip() for c in out.split(",")])
            except Exception:
                pass
            self._stop.wait(0.5)

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=6)
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 7 for n, v in zip(names, r[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(self.rows)}


def main() -> None:
    args = parse_args()
    if args.impl == "reference":
        reference_arm(args)
        return

    import torch
    import torch.distributed as dist

    from unirl_b200.config.loader import compose
    from unirl_b200.ops._ext import launch_count, require_ext
    from unirl_b200.trainer.ar import ARTrainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device")
    torch.cuda.set_device(local)
    require_ext()
    tp = max(1, args.rollout_tp)
    preset = {"qwen3-4b": "random:qwen3-4b", "tiny": "random:tiny"}[args.model]
    vocab = 151936 if args.model == "qwen3-4b" else 4096
    n_prompts = args.prompts_per_gpu * world
    overrides = [
        f"num_devices={world}", f"batch_size={n_prompts}", f"bundle.config.pretrained_model_ckpt_path={preset}",
        f"rollout.config.pretrained_model_ckpt_path={preset}", f"rollout.config.tp_size={tp}", f"rollout.config.max_new_tokens={args.max_new_tokens}",
        f"rollout.config.max_running_requests={args.prompts_per_gpu * args.group_size * tp}",
        f"sampling.samples_per_prompt={args.group_size}", f"sampling.max_new_tokens={args.max_new_tokens}",
        f"data_source.vocab_size={vocab}", f"data_source.min_len={args.prompt_min}", f"data_source.max_len={args.prompt_max}",
        f"data_source.reserved_low_ids={1000 if vocab > 4096 else 16}", f"stack.micro_batch_size={args.micro_batch}",
        f"algorithm.horizon={args.max_new_tokens}", f"rollout_parallel={{tp: {tp}}}",
    ]
    if args.ckpt_layers >= 0:
        overrides.append(f"+backend.fsdp_cfg.checkpoint_layers={args.ckpt_layers}")
    if args.algorithm == "drpo":
        overrides += ["algorithm._target_=unirl_b200.algorithms.drpo.DRPO", "~algorithm.clip_range", "~algorithm.clip_range_high",
                      "+algorithm.drpo_epsilon=12.5"]
    cfg = compose("ar/qwen3_4b_grpo_b200", overrides=overrides)
    trainer = ARTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend,
                        rollout_cfg=cfg.rollout, reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack,
                        data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling, sync_cfg=cfg.get("sync"), logging_cfg=None)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_step(i: int):
        inputs = trainer.data_source.get_samples(trainer.batch_size)
        # stage this step's prompts in pinned host memory: the engine's H2D copy starts from there
        pt = inputs.primitives["prompt_tokens"]
        pt.input_ids, pt.attention_mask = pt.input_ids.pin_memory(), pt.attention_mask.pin_memory()
        h2d = pt.input_ids.numel() * pt.input_ids.element_size() * args.group_size
        req = trainer._build_req(inputs, i)
        result, reward = trainer.train_step(req, training_progress=0.0, sync_weights=True, rollout_id=i)
        row = trainer.wandb_logger.history[-2] if len(trainer.wandb_logger.history) >= 2 else {}
        rollout_row = next((r for r in reversed(trainer.wandb_logger.history) if "rollout/step" in r), {})
        n_tok = int(round(rollout_row.get("rollout/response_length_mean", 0.0) * n_prompts * args.group_size))
        dev_ms = dict(trainer.phase_timer.device_ms)
        sync_ms = float(trainer.last_sync_stats.get("sync_ms", 0.0))
        m = dict(getattr(result, "metrics", {}) or {})
        return {"tokens": n_tok, "device_ms": dev_ms, "sync_ms": sync_ms, "loss": float(result.loss), "reward": reward, "h2d": h2d,
                "d2h": n_tok * (8 + 4) + 8, "logp_gap": (m.get("rollout_replay_logp_absdiff_mean"), m.get("rollout_replay_logp_absdiff_max"))}

    budget = StepBudget(args.budget_s, _job_start(), world)
    n_warm = 0
    while budget.plan_warmup(n_warm, args.warmup, args.steps):
        t_w = time.time()
        one_step(n_warm)
        torch.cuda.synchronize()
        budget.observe(time.time() - t_w)
        n_warm += 1
    n_steps = budget.plan_timed(args.steps)
    barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ev0.record()
    t0 = time.perf_counter()
    rows = [one_step(n_warm + i) for i in range(n_steps)]
    ev1.record()
    barrier()
    wall = time.perf_counter() - t0
    launches = launch_count() - l0
    clocks = sampler.stop() if rank == 0 else {}
    span_ms = ev0.elapsed_time(ev1)
    dev_ms = sum(sum(v for k, v in r["device_ms"].items() if k in ("rollout", "train", "sync", "wake", "sleep", "reward")) for r in rows)
    t = torch.tensor([dev_ms, span_ms, wall * 1e3, max(r["sync_ms"] for r in rows)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dev_ms, span_ms, wall_ms, sync_ms = t.tolist()
    tokens = sum(r["tokens"] for r in rows)
    if rank == 0:
        out = {"metric": "rl_step_tokens_per_s", "value": tokens / (dev_ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": n_steps,
               "warmup": n_warm, "steps_requested": args.steps, "warmup_requested": args.warmup, "budget_s": args.budget_s,
               "ms_per_step": dev_ms / n_steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
               "dtype": "bf16", "data": "synthetic (uniform-random prompt token ids, random-init weights, token-hash reward)",
               "weight_sync_ms": sync_ms, "impl": "native",
               "config": {"model": "Qwen3-4B" if args.model == "qwen3-4b" else args.model, "algorithm": args.algorithm.upper(),
                          "global_batch": n_prompts * args.group_size, "prompts": n_prompts, "group_size": args.group_size,
                          "seq_len": f"prompt {args.prompt_min}-{args.prompt_max} + response <= {args.max_new_tokens}",
                          "tokens_counted": "generated response tokens", "tokens_per_step": tokens // max(1, n_steps),
                          "micro_batch": args.micro_batch, "parallelism": f"dp{world} trainer (sharded optimizer), rollout tp{tp}",
                          "l2_policy": "inputs_exceed_l2 (8 GB of bf16 weights + KV cache streamed every decode step)"},
               "clocks": clocks,
               "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": rows[-1]["h2d"], "d2h_bytes_per_step": rows[-1]["d2h"],
                       "ms_per_step": wall_ms / n_steps},
               "gpu_launches": int(launches), "loss": rows[-1]["loss"],
               "rollout_replay_logp_absdiff": {"mean": rows[-1]["logp_gap"][0], "max": rows[-1]["logp_gap"][1]}, "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1),
               "phases_device_ms_last_step": {k: round(v, 2) for k, v in rows[-1]["device_ms"].items()}, "device_span_ms_per_step": span_ms / n_steps}
        print(json.dumps(out))
    trainer.shutdown()
    if world > 1 and dist.is_initialized():
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
