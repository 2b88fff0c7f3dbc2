"""Secondary benchmark: one Flow-DPPO step of the SD3.5-Medium-shaped policy through the public trainer API, device-timed.

Default geometry (per GPU; weak scaling): 4 prompts x 16 samples of 1024 x 1024 (a 128 x 128 x 16 latent, 4096 image tokens),
10-step SDE sampling at noise level 0.7 with guidance 4.5, text conditioning given as random N(0, 1) bf16 embeddings of shape
[333, 4096] plus a pooled [2048] vector (copied from pinned host memory every step), a random-init 4-layer CNN on the latent as the
reward, training on a random subset of 5 of the SDE steps, LoRA rank 64 with LoRA weight sync into a native sampler engine that holds
weights of its own.  On 8 GPUs this is 32 prompts x 16 per step.

    python bench_diffusion.py --steps 1 --warmup 3                       # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_diffusion.py --gpus N

Prints ONE JSON line (rank 0): samples/s over all GPUs (device-timed, max over ranks), seconds per step, the device time of each
phase, the LoRA sync time, the end-to-end value (wall clock around the complete train_step calls, with the bytes copied in and out per
step) and the SM clocks sampled while the timed steps ran.  Synthetic data, random-init weights of the published architecture.
"""

from __future__ import annotations

import argparse
import json
import os
import time

ROOT = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--recipe", default="diffusion/sd35m_flowdppo_lora_native_engine_b200")
    ap.add_argument("--preset", default="sd35-medium", help="random:<preset> architecture (tiny presets run on CPU)")
    ap.add_argument("--prompts-per-gpu", type=int, default=4)
    ap.add_argument("--samples-per-prompt", type=int, default=16)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--resolution", type=int, default=1024)
    ap.add_argument("--inference-steps", type=int, default=10)
    ap.add_argument("--train-timesteps", type=int, default=5, help="SDE steps trained on per rollout (a fresh random subset every step)")
    ap.add_argument("--eta", type=float, default=0.7)
    ap.add_argument("--text-len", type=int, default=333, help="length of the synthetic text embedding sequence (0: encode the recipe's prompts)")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("overrides", nargs="*", help="extra recipe overrides (key=value)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    import sys
    sys.path.insert(0, ROOT)
    from bench import ClockSampler
    from unirl_b200.config.loader import compose
    from unirl_b200.ops._ext import launch_count
    from unirl_b200.trainer.diffusion import DiffusionTrainer
    from unirl_b200.types.conditions import TextEmbedCondition

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    cuda = args.device == "cuda"
    if cuda:
        if not torch.cuda.is_available():
            raise SystemExit("bench_diffusion.py --device cuda needs a CUDA device")
        torch.cuda.set_device(local)
    n_prompts = args.prompts_per_gpu * world
    all_sde = list(range(max(args.inference_steps - 1, 1)))
    ov = [f"num_devices={world}", f"batch_size={n_prompts}", f"bundle.config.pretrained_model_ckpt_path=random:{args.preset}",
          f"sampling.samples_per_prompt={args.samples_per_prompt}", f"sampling.num_inference_steps={args.inference_steps}",
          f"sampling.height={args.resolution}", f"sampling.width={args.resolution}", f"+sampling.eta={args.eta}",
          f"sampling.sde_indices=[{','.join(map(str, all_sde))}]", f"stack.micro_batch_size={args.micro_batch}"]
    ov += ["+pool_backend=spmd" if world > 1 else "+pool_backend=inline"]
    if not cuda:
        ov += ["+pool_device=cpu", "bundle.config.model_precision=fp32", "+bundle.config.autocast_precision=fp32", "+bundle.config.device=cpu",
               "backend.fsdp_cfg.mixed_precision=false", "+reward.backend.device=cpu"]
    probe = compose(args.recipe, overrides=[])
    if probe.get("rollout") is not None and probe.rollout.get("config") is not None:  # an engine with weights of its own follows the bundle's architecture
        ov += [f"rollout.config.pretrained_model_ckpt_path=random:{args.preset}"]
        if not cuda:
            ov += ["rollout.config.model_precision=fp32", "+rollout.config.autocast_precision=fp32", "+rollout.config.device=cpu", "rollout.config.use_cuda_graph=false"]
    cfg = compose(args.recipe, overrides=ov + list(args.overrides))
    tr = DiffusionTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend, rollout_cfg=cfg.rollout,
                          reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack, data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling,
                          sync_cfg=cfg.get("sync"), logging_cfg=None)
    spec_text_dim, spec_pooled = 4096, 2048
    try:
        from unirl_b200.models.dit.config import resolve_family

        t = resolve_family(f"random:{args.preset}").transformer
        spec_text_dim, spec_pooled = int(t.text_dim), int(t.pooled_dim)
    except Exception:  # noqa: BLE001
        pass
    dtype = torch.bfloat16 if cuda else torch.float32
    gen = torch.Generator().manual_seed(1234 + rank)
    h2d = d2h = 0

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def one_step(i: int):
        nonlocal h2d, d2h
        inputs = tr.data_source.get_samples(tr.batch_size)
        # a fresh random subset of the SDE steps to train on this rollout
        sub = sorted(torch.randperm(len(all_sde), generator=torch.Generator().manual_seed(99 + i))[: min(args.train_timesteps, len(all_sde))].tolist())
        tr.sampling_params.sde_indices = [all_sde[k] for k in sub]
        req = tr._build_req(inputs, i)
        if args.text_len > 0:
            n = len(req.sample_ids)
            mk = lambda *shape: torch.randn(*shape, generator=gen).to(dtype).pin_memory() if cuda else torch.randn(*shape, generator=gen).to(dtype)  # noqa: E731
            pos = TextEmbedCondition(embeds=mk(n, args.text_len, spec_text_dim), pooled=mk(n, spec_pooled) if spec_pooled else None,
                                     attn_mask=torch.ones(n, args.text_len, dtype=torch.bool))
            neg = TextEmbedCondition(embeds=mk(n, args.text_len, spec_text_dim), pooled=mk(n, spec_pooled) if spec_pooled else None,
                                     attn_mask=torch.ones(n, args.text_len, dtype=torch.bool))
            req.request_conditions = {"text": pos, "negative_text": neg}
            h2d = 2 * (pos.embeds.numel() * pos.embeds.element_size() + (pos.pooled.numel() * pos.pooled.element_size() if pos.pooled is not None else 0)) // max(1, world)
        result, reward = tr.train_step(req, training_progress=0.0, sync_weights=True, rollout_id=i)
        d2h = 8 + 4 * len(req.sample_ids) // max(1, world)  # the loss and the per-sample rewards come back to the host
        return {"device_ms": dict(tr.phase_timer.device_ms), "loss": float(result.loss), "reward": float(reward),
                "sync_ms": float(getattr(tr, "last_sync_stats", {}).get("sync_ms", 0.0))}

    try:
        for i in range(args.warmup):
            one_step(i)
        barrier()
        sampler = ClockSampler(local)
        if rank == 0 and cuda:
            sampler.start()
        l0 = launch_count()
        if cuda:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        t0 = time.perf_counter()
        rows = [one_step(args.warmup + i) for i in range(args.steps)]
        if cuda:
            ev1.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        clocks = sampler.stop() if rank == 0 and cuda else {}
        span_ms = ev0.elapsed_time(ev1) if cuda else wall_ms
        dev_ms = sum(sum(v for k, v in r["device_ms"].items() if k in ("rollout", "train", "sync", "wake", "sleep", "reward")) for r in rows) or span_ms
        t = torch.tensor([dev_ms, span_ms, wall_ms, max(r["sync_ms"] for r in rows)], dtype=torch.float64, device="cuda" if cuda else "cpu")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dev_ms, span_ms, wall_ms, sync_ms = t.tolist()
        samples = n_prompts * args.samples_per_prompt * args.steps
        if rank == 0:
            print(json.dumps({
                "metric": "flowdppo_samples_per_s", "value": samples / (dev_ms / 1e3), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "s_per_step": dev_ms / 1e3 / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                "dtype": "bf16" if cuda else "fp32",
                "data": "synthetic (random text embeddings, random-init weights of the architecture, random-init latent-CNN reward)", "lora_sync_ms": sync_ms,
                "config": {"model": args.preset, "algorithm": "Flow-DPPO", "prompts": n_prompts, "samples_per_prompt": args.samples_per_prompt,
                           "resolution": args.resolution, "inference_steps": args.inference_steps, "trained_timesteps": min(args.train_timesteps, len(all_sde)),
                           "eta": args.eta, "text_tokens": args.text_len, "micro_batch": args.micro_batch, "lora_rank": 64,
                           "parallelism": f"dp{world} trainer, native sampler engine with weights of its own" if "native" in args.recipe else f"dp{world} trainer, train-side rollout",
                           "l2_policy": "inputs_exceed_l2 (5 GB of bf16 weights and 4429-token activations streamed every forward)"},
                "clocks": clocks,
                "e2e": {"value": samples / (wall_ms / 1e3), "unit": "samples/s", "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                        "s_per_step": wall_ms / 1e3 / args.steps},
                "phases_device_ms_last_step": {k: round(v, 2) for k, v in rows[-1]["device_ms"].items()}, "loss": rows[-1]["loss"], "reward": rows[-1]["reward"],
                "device_span_s_per_step": span_ms / 1e3 / args.steps,
                "gpu_launches": launch_count() - l0, "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1) if cuda else None}), flush=True)
    finally:
        tr.shutdown()
        if world > 1 and dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
