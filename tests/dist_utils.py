"""Start ``world`` CPU (gloo) ranks of a top-level function and propagate the first failure."""
import os
import socket
import traceback

import torch
import torch.multiprocessing as mp


def _free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


_CTX = None


def _context():
    """Ranks are forked from a server process that has imported torch and the package once (``forkserver`` with
    preloaded modules): a rank then starts in a fraction of a second instead of re-importing torch. The server is a
    fresh interpreter without threads or process groups, so forking from it is as clean as spawning."""
    global _CTX
    if _CTX is None:
        ctx = mp.get_context("forkserver")
        ctx.set_forkserver_preload(["tests._preload"])
        _CTX = ctx
    return _CTX


def _entry(rank, world, port, fn, args, errq, env):
    os.environ.clear()                 # the server's environment is the one it was started with, not the test's
    os.environ.update(env)
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OSLO_B200_BACKEND="gloo")
    torch.set_num_threads(1)
    try:
        fn(rank, world, *args)
    except BaseException:  # noqa: BLE001
        errq.put((rank, traceback.format_exc()))
        raise
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_distributed(fn, world: int, *args, timeout: float = 600.0, fresh: bool = False):
    """``fresh=True`` starts the ranks as new interpreters that have imported nothing yet (for tests that check what a
    rank imports)."""
    ctx = mp.get_context("spawn") if fresh else _context()
    errq = ctx.SimpleQueue()
    port = _free_port()
    env = dict(os.environ)
    procs = [ctx.Process(target=_entry, args=(r, world, port, fn, args, errq, env)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    failed = [p for p in procs if p.exitcode != 0]
    for p in procs:
        if p.is_alive():
            p.kill()
    if failed:
        msgs = []
        while not errq.empty():
            r, tb = errq.get()
            msgs.append(f"--- rank {r} ---\n{tb}")
        raise AssertionError("distributed run failed:\n" + "\n".join(msgs or ["(no traceback; timeout or crash)"]))
