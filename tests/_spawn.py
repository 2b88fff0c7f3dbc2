"""Helper: run a function on N ranks in child processes (gloo on CPU, or one CUDA device per rank over NCCL) and collect its return values."""
import multiprocessing as mp
import os
import traceback


def _entry(fn, rank, world, port, q, args, cuda=False):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "RANK": str(rank), "WORLD_SIZE": str(world),
                       "LOCAL_RANK": str(rank), "NCCL_NVLS_ENABLE": "0"})
    try:
        import torch
        import torch.distributed as dist

        torch.set_num_threads(2)
        if cuda:
            torch.cuda.set_device(rank)
        dist.init_process_group("cpu:gloo,cuda:nccl" if cuda else "gloo", rank=rank, world_size=world, init_method=f"tcp://127.0.0.1:{port}",
                                **({"device_id": torch.device("cuda", rank)} if cuda else {}))
        out = fn(rank, world, *args)
        dist.barrier()
        dist.destroy_process_group()
        import io

        buf = io.BytesIO()
        torch.save(out, buf)  # tensors travel as bytes (queue hand-off of shared-memory tensors races with child exit)
        q.put((rank, True, buf.getvalue()))
    except BaseException:  # noqa: BLE001
        q.put((rank, False, traceback.format_exc()))


def run_ranks(fn, world, *args, timeout=240, cuda=False):
    from unirl_b200.distributed.utils import free_port

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, q, args, cuda), daemon=True) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, ok, out = q.get(timeout=timeout)
            if not ok:
                raise RuntimeError(f"rank {rank} failed:\n{out}")
            import io

            import torch

            results[rank] = torch.load(io.BytesIO(out), weights_only=False)
    finally:
        for p in procs:
            p.join(10)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
