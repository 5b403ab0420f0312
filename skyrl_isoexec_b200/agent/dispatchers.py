"""Scheduling of many agent trajectories through their three stages: set up the environment, run the agent, score the
result (reference: skyrl-agent/skyrl_agent/dispatcher/dispatchers.py:22-170, the ``async_pipeline`` / ``async_batch`` /
``async_fix_pool`` registry, and dispatcher/async_utils.py).

A trajectory is any object with three coroutine methods (names configurable; default ``initialize`` / ``run`` /
``evaluate``). Strategies:

  batch       one task per trajectory runs its three stages back to back; ``max_parallel`` caps the tasks alive
  pipeline    three worker pools joined by queues, so environment set-up of later trajectories overlaps generation of
              earlier ones and scoring has its own cap (``max_eval_parallel``)
  fixed_pool  a fixed set of pre-built environments; a trajectory borrows one for its three stages and returns it

Unlike a bare ``gather``, a failing trajectory does not strand the others: every trajectory runs to its end, failures are
collected, and one ``DispatchError`` listing them is raised afterwards (or returned with ``raise_errors=False``)."""

from __future__ import annotations

import asyncio
import threading
from typing import Any, Awaitable, Callable

DISPATCHERS: dict[str, Callable[..., Awaitable[list]]] = {}


class DispatchError(RuntimeError):
    def __init__(self, failures: list[tuple[Any, BaseException]]):
        self.failures = failures
        super().__init__(f"{len(failures)} trajectories failed: " + "; ".join(f"{k}: {type(e).__name__}: {e}" for k, e in failures[:5]))


def register_dispatcher(name: str):
    def deco(fn):
        DISPATCHERS[name] = fn
        return fn
    return deco


def _keys(trajectories: dict, order: str = "sample_major") -> list[tuple]:
    """(instance, sample) pairs. ``sample_major`` starts the first sample of every instance before any second sample, so a
    run that is cut short still has one result per instance."""
    pairs = [(i, k) for i, per in trajectories.items() for k in per]
    if order == "sample_major":
        rank = {i: n for n, i in enumerate(trajectories)}
        pairs.sort(key=lambda p: (list(trajectories[p[0]]).index(p[1]), rank[p[0]]))
    return pairs


def _finish(failures: list, raise_errors: bool) -> list:
    if failures and raise_errors:
        raise DispatchError(failures)
    return failures


@register_dispatcher("batch")
async def batch_dispatcher(trajectories: dict, max_parallel: int | None = None, stages=("initialize", "run", "evaluate"),
                           raise_errors: bool = True, **_) -> list:
    sem = asyncio.Semaphore(max_parallel) if max_parallel else None
    failures: list = []

    async def one(key):
        t = trajectories[key[0]][key[1]]
        try:
            if sem is not None:
                async with sem:
                    for s in stages:
                        if s:
                            await getattr(t, s)()
            else:
                for s in stages:
                    if s:
                        await getattr(t, s)()
        except Exception as e:  # noqa: BLE001
            failures.append((key, e))

    await asyncio.gather(*[one(k) for k in _keys(trajectories)])
    return _finish(failures, raise_errors)


@register_dispatcher("pipeline")
async def pipeline_dispatcher(trajectories: dict, max_parallel: int = 8, max_eval_parallel: int | None = None,
                              stages=("initialize", "run", "evaluate"), raise_errors: bool = True, **_) -> list:
    keys = _keys(trajectories)
    n = len(keys)
    widths = [min(n, max_parallel), min(n, max_parallel), min(n, max_eval_parallel or max_parallel)]
    queues = [asyncio.Queue() for _ in stages]
    failures: list = []
    for k in keys:
        queues[0].put_nowait(k)

    async def worker(si: int):
        q, nxt = queues[si], queues[si + 1] if si + 1 < len(stages) else None
        while True:
            key = await q.get()
            try:
                if stages[si]:
                    await getattr(trajectories[key[0]][key[1]], stages[si])()
                if nxt is not None:
                    nxt.put_nowait(key)
            except Exception as e:  # noqa: BLE001 -- the trajectory leaves the pipeline here; the others go on
                failures.append((key, e))
            finally:
                q.task_done()

    pools = [[asyncio.create_task(worker(si)) for _ in range(max(1, widths[si]))] for si in range(len(stages))]
    try:
        for q in queues:             # a stage's queue is complete once the stage before it has drained
            await q.join()
    finally:
        for pool in pools:
            for t in pool:
                t.cancel()
        await asyncio.gather(*[t for pool in pools for t in pool], return_exceptions=True)
    return _finish(failures, raise_errors)


@register_dispatcher("fixed_pool")
async def fixed_pool_dispatcher(trajectories: dict, envs: list, stages=("initialize", "run", "evaluate"),
                                raise_errors: bool = True, **_) -> list:
    """Each stage method is called with the borrowed environment: ``await traj.initialize(env)`` and so on."""
    free: asyncio.Queue = asyncio.Queue()
    for e in envs:
        free.put_nowait(e)
    work: asyncio.Queue = asyncio.Queue()
    for k in _keys(trajectories):
        work.put_nowait(k)
    failures: list = []

    async def worker():
        while True:
            key = await work.get()
            env = await free.get()
            try:
                for s in stages:
                    if s:
                        await getattr(trajectories[key[0]][key[1]], s)(env)
            except Exception as e:  # noqa: BLE001
                failures.append((key, e))
            finally:
                free.put_nowait(env)          # the environment goes back to the pool whatever happened
                work.task_done()

    tasks = [asyncio.create_task(worker()) for _ in range(max(1, len(envs)))]
    try:
        await work.join()
    finally:
        for t in tasks:
            t.cancel()
        await asyncio.gather(*tasks, return_exceptions=True)
    return _finish(failures, raise_errors)


async def dispatch(name: str, trajectories: dict, **cfg) -> list:
    if name not in DISPATCHERS:
        raise KeyError(f"unknown dispatcher {name!r}; known: {sorted(DISPATCHERS)}")
    return await DISPATCHERS[name](trajectories, **cfg)


# ----------------------------------------------------------------------------- sync <-> async bridges
async def call_sync_from_async(fn: Callable, *args, **kw):
    """Run a blocking function on the default executor so the event loop keeps serving other trajectories."""
    loop = asyncio.get_running_loop()
    return await loop.run_in_executor(None, lambda: fn(*args, **kw))


def call_async_from_sync(corofn: Callable[..., Awaitable], *args, timeout: float | None = 600.0, **kw):
    """Run a coroutine to its end from synchronous code, whether or not this thread already runs an event loop (then a
    helper thread with its own loop is used). Exceptions and the timeout surface in the caller."""
    async def main():
        return await asyncio.wait_for(corofn(*args, **kw), timeout)

    try:
        asyncio.get_running_loop()
    except RuntimeError:
        return asyncio.run(main())
    box: dict = {}

    def run():
        try:
            box["value"] = asyncio.run(main())
        except BaseException as e:  # noqa: BLE001
            box["error"] = e

    th = threading.Thread(target=run, daemon=True)
    th.start()
    th.join()
    if "error" in box:
        raise box["error"]
    return box["value"]


async def wait_all(coros, timeout: float | None = 600.0) -> list:
    """All results in order; if any failed, every other coroutine still finishes and one ``DispatchError`` names the
    failures; on timeout the stragglers are cancelled."""
    tasks = [asyncio.ensure_future(c) for c in coros]
    if not tasks:
        return []
    done, pending = await asyncio.wait(tasks, timeout=timeout)
    if pending:
        for t in pending:
            t.cancel()
        await asyncio.gather(*pending, return_exceptions=True)
        raise asyncio.TimeoutError(f"{len(pending)} of {len(tasks)} tasks did not finish within {timeout}s")
    failures = [(i, t.exception()) for i, t in enumerate(tasks) if t.exception() is not None]
    if failures:
        raise DispatchError(failures)
    return [t.result() for t in tasks]
