"""Helpers to run a function on N CPU ranks (gloo) as child processes."""
import os
import socket
import tempfile
import traceback

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _entry(rank, world, port, fn, args, out_dir, timeout_s):
    try:
        import datetime
        torch.set_num_threads(1)
        dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank,
                                world_size=world, timeout=datetime.timedelta(seconds=timeout_s))
        result = fn(rank, world, *args)
        torch.save(result, os.path.join(out_dir, f"rank{rank}.pt"))
    except BaseException as e:  # noqa: BLE001 - report and re-raise in the parent
        with open(os.path.join(out_dir, f"rank{rank}.err"), "w") as f:
            f.write("".join(traceback.format_exception(type(e), e, e.__traceback__)))
        raise
    finally:
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_ranks(fn, world, *args, timeout_s=120, expect_failure=False):
    """Run ``fn(rank, world, *args)`` on ``world`` gloo ranks; returns the per-rank results
    (or, with ``expect_failure``, the dict rank -> error text of the ranks that raised)."""
    port = free_port()
    with tempfile.TemporaryDirectory() as out_dir:
        ctx = mp.spawn(_entry, args=(world, port, fn, args, out_dir, timeout_s), nprocs=world,
                       join=False)
        failed = False
        try:
            while not ctx.join(timeout=timeout_s + 30):
                pass
        except Exception:
            failed = True
        errors = {}
        for r in range(world):
            p = os.path.join(out_dir, f"rank{r}.err")
            if os.path.exists(p):
                errors[r] = open(p).read()
        if expect_failure:
            return errors
        if failed or errors:
            raise RuntimeError("rank failure:\n" + "\n".join(errors.values()))
        return [torch.load(os.path.join(out_dir, f"rank{r}.pt")) for r in range(world)]
