"""Spawn helper for multi-GPU tests: one process per GPU, NCCL, results returned as plain Python data."""
import os
import socket
import traceback

import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, q, env=None):
    os.environ.update({"RANK": str(rank), "WORLD_SIZE": str(world), "LOCAL_RANK": str(rank),
                       "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0"})
    os.environ.update(env or {})
    import torch
    import torch.distributed as dist
    try:
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
        from b200fw import _native as nv
        nv.set_device(rank)
        out = fn(rank, world, *args)
        torch.cuda.synchronize()
        status = nv.read_status()
        q.put((rank, "ok" if status == 0 else "error", out if status == 0 else f"device status {status}"))
    except Exception:  # noqa: BLE001
        q.put((rank, "error", traceback.format_exc()))
    finally:
        if dist.is_initialized():
            dist.destroy_process_group()


def run_gpu_ranks(fn, world: int, *args, timeout: float = 120.0, env=None):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, q, env)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, status, out = q.get(timeout=timeout)
            if status != "ok":
                raise AssertionError(f"rank {rank} failed:\n{out}")
            results[rank] = out
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.terminate()   # the exact child started above
    return [results[r] for r in range(world)]
