"""Secondary benchmark: one Flow-DPPO step of the SD3.5-Medium-shaped policy (LoRA, 512 x 512, 10 denoising steps, guidance 4.5,
16 samples per prompt, train-side rollout) through the public trainer API, device-timed.

    python bench_diffusion.py --steps 2 --warmup 3                       # 1 GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench_diffusion.py --gpus N

Prints ONE JSON line (rank 0): samples/s over all GPUs, seconds per step, the device time of each phase and the weight-sync
time.  Synthetic prompts, random-init weights of the published architecture, a small latent CNN as the reward.
"""

from __future__ import annotations

import argparse
import json
import os
import time


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--recipe", default="diffusion/sd35m_flowdppo_lora_b200")
    ap.add_argument("--preset", default="sd35-medium", help="random:<preset> architecture (tiny presets run on CPU)")
    ap.add_argument("--prompts-per-gpu", type=int, default=6)  # the published recipe: 48 prompts x 16 samples on 8 GPUs
    ap.add_argument("--samples-per-prompt", type=int, default=16)
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--resolution", type=int, default=512)
    ap.add_argument("--inference-steps", type=int, default=10)
    ap.add_argument("--device", default="cuda")
    ap.add_argument("overrides", nargs="*", help="extra recipe overrides (key=value)")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist

    from unirl_b200.config.loader import compose
    from unirl_b200.ops._ext import launch_count
    from unirl_b200.trainer.diffusion import DiffusionTrainer

    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    cuda = args.device == "cuda"
    if cuda:
        if not torch.cuda.is_available():
            raise SystemExit("bench_diffusion.py --device cuda needs a CUDA device")
        torch.cuda.set_device(local)
    n_prompts = args.prompts_per_gpu * world
    sde = ",".join(str(i) for i in range(max(args.inference_steps - 1, 1)))
    ov = [f"num_devices={world}", f"batch_size={n_prompts}", f"bundle.config.pretrained_model_ckpt_path=random:{args.preset}",
          f"sampling.samples_per_prompt={args.samples_per_prompt}", f"sampling.num_inference_steps={args.inference_steps}",
          f"sampling.height={args.resolution}", f"sampling.width={args.resolution}", f"sampling.sde_indices=[{sde}]", f"stack.micro_batch_size={args.micro_batch}"]
    if world > 1:
        ov += ["+pool_backend=spmd"]
    else:
        ov += ["+pool_backend=inline"]
    if not cuda:
        ov += ["+pool_device=cpu", "bundle.config.model_precision=fp32", "+bundle.config.autocast_precision=fp32", "+bundle.config.device=cpu",
               "backend.fsdp_cfg.mixed_precision=false", "+reward.backend.device=cpu"]
    cfg = compose(args.recipe, overrides=ov + list(args.overrides))
    tr = DiffusionTrainer(cfg=cfg, batch_size=cfg.batch_size, bundle_cfg=cfg.bundle, pipeline_cfg=cfg.pipeline, backend_cfg=cfg.backend, rollout_cfg=cfg.rollout,
                          reward_cfg=cfg.reward, algorithm_cfg=cfg.algorithm, stack_cfg=cfg.stack, data_source_cfg=cfg.data_source, sampling_cfg=cfg.sampling,
                          sync_cfg=cfg.get("sync"), logging_cfg=None)

    def barrier() -> None:
        if world > 1:
            dist.barrier()
        if cuda:
            torch.cuda.synchronize()

    def one_step(i: int):
        inputs = tr.data_source.get_samples(tr.batch_size)
        req = tr._build_req(inputs, i)
        result, reward = tr.train_step(req, training_progress=0.0, sync_weights=True, rollout_id=i)
        return {"device_ms": dict(tr.phase_timer.device_ms), "loss": float(result.loss), "reward": float(reward),
                "sync_ms": float(getattr(tr, "last_sync_stats", {}).get("sync_ms", 0.0))}

    try:
        for i in range(args.warmup):
            one_step(i)
        barrier()
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
        span_ms = ev0.elapsed_time(ev1) if cuda else wall_ms
        t = torch.tensor([span_ms, wall_ms, max(r["sync_ms"] for r in rows)], dtype=torch.float64, device="cuda" if cuda else "cpu")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        span_ms, wall_ms, sync_ms = t.tolist()
        samples = n_prompts * args.samples_per_prompt * args.steps
        if rank == 0:
            print(json.dumps({
                "metric": "flowdppo_samples_per_s", "value": samples / (span_ms / 1e3), "unit": "samples/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "s_per_step": span_ms / 1e3 / args.steps, "higher_is_better": True, "scaling": "weak", "dtype": "bf16" if cuda else "fp32",
                "data": "synthetic (fixed prompt list, random-init weights, latent-CNN reward)", "lora_sync_ms": sync_ms,
                "config": {"model": args.preset, "algorithm": "Flow-DPPO", "prompts": n_prompts, "samples_per_prompt": args.samples_per_prompt,
                           "resolution": args.resolution, "inference_steps": args.inference_steps, "micro_batch": args.micro_batch,
                           "parallelism": f"dp{world} trainer, train-side rollout"},
                "phases_device_ms_last_step": {k: round(v, 2) for k, v in rows[-1]["device_ms"].items()}, "loss": rows[-1]["loss"], "reward": rows[-1]["reward"],
                "gpu_launches": launch_count() - l0, "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1) if cuda else None}), flush=True)
    finally:
        tr.shutdown()
        if world > 1 and dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


if __name__ == "__main__":
    main()
