"""Run a function on N spawned ranks (gloo on CPU, nccl on GPUs) and collect results."""
import multiprocessing as mp
import os
import socket
import traceback


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(fn, rank, world, port, backend, args, queue, env):
    try:
        os.environ.update(env or {})
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        import torch
        import torch.distributed as dist

        torch.set_num_threads(1)
        kwargs = {}
        if backend == "nccl":
            torch.cuda.set_device(rank)
            kwargs["device_id"] = torch.device("cuda", rank)
        dist.init_process_group(backend, rank=rank, world_size=world, **kwargs)
        try:
            queue.put((rank, True, fn(rank, world, *args)))
        finally:
            dist.destroy_process_group()
    except BaseException:
        queue.put((rank, False, traceback.format_exc()))


def run_ranks(fn, world, *args, backend="gloo", timeout=180, env=None):
    """Returns the list of per-rank results; raises if any rank failed."""
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_entry, args=(fn, r, world, port, backend, args, queue, env)) for r in range(world)]
    for p in procs:
        p.start()
    results = {}
    try:
        for _ in range(world):
            rank, ok, val = queue.get(timeout=timeout)
            if not ok:
                raise AssertionError(f"rank {rank} failed:\n{val}")
            results[rank] = val
    finally:
        for p in procs:
            p.join(timeout=20)
            if p.is_alive():
                p.kill()
    return [results[r] for r in range(world)]
