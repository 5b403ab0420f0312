"""Trajectory dispatch strategies: every trajectory passes its three stages, caps hold, stages overlap in the pipeline,
environments are reused in the fixed pool, failures are collected instead of stranding the rest."""

import asyncio

import pytest

from skyrl_isoexec_b200.agent import dispatchers as D


class _Traj:
    live = {"initialize": 0, "run": 0, "evaluate": 0}
    peak = {"initialize": 0, "run": 0, "evaluate": 0}
    log: list = []

    def __init__(self, key, fail_in=None):
        self.key, self.fail_in, self.done = key, fail_in, []

    async def _stage(self, name, env=None):
        c = type(self)
        c.live[name] += 1
        c.peak[name] = max(c.peak[name], c.live[name])
        c.log.append((name, self.key))
        await asyncio.sleep(0.001)
        c.live[name] -= 1
        if self.fail_in == name:
            raise ValueError(f"{name} broke")
        self.done.append((name, env))

    async def initialize(self, env=None):
        await self._stage("initialize", env)

    async def run(self, env=None):
        await self._stage("run", env)

    async def evaluate(self, env=None):
        await self._stage("evaluate", env)


def _fresh(n_inst=4, n_samp=3, fail=None):
    _Traj.live = dict.fromkeys(_Traj.live, 0)
    _Traj.peak = dict.fromkeys(_Traj.peak, 0)
    _Traj.log = []
    return {i: {k: _Traj((i, k), (fail or {}).get((i, k))) for k in range(n_samp)} for i in range(n_inst)}


def _all(tr):
    return [t for per in tr.values() for t in per.values()]


def test_batch_dispatcher_runs_all_stages_under_a_cap_and_collects_failures():
    tr = _fresh()
    assert asyncio.run(D.dispatch("batch", tr, max_parallel=5)) == []
    assert all([s for s, _ in t.done] == ["initialize", "run", "evaluate"] for t in _all(tr))
    assert sum(_Traj.peak.values()) >= 1 and max(_Traj.peak.values()) <= 5
    # sample-major start order: the first sample of every instance starts before any second sample
    starts = [k for s, k in _Traj.log if s == "initialize"]
    assert starts[:4] == [(0, 0), (1, 0), (2, 0), (3, 0)]
    tr = _fresh(fail={(1, 2): "run", (3, 0): "evaluate"})
    with pytest.raises(D.DispatchError) as ei:
        asyncio.run(D.dispatch("batch", tr))
    assert sorted(k for k, _ in ei.value.failures) == [(1, 2), (3, 0)]
    ok = [t for t in _all(tr) if t.fail_in is None]
    assert len(ok) == 10 and all(len(t.done) == 3 for t in ok), "the other trajectories still finished"
    with pytest.raises(KeyError):
        asyncio.run(D.dispatch("nope", tr))


def test_pipeline_dispatcher_overlaps_stages_and_caps_evaluation_separately():
    tr = _fresh(n_inst=6, n_samp=2)
    assert asyncio.run(D.dispatch("pipeline", tr, max_parallel=4, max_eval_parallel=2)) == []
    assert all([s for s, _ in t.done] == ["initialize", "run", "evaluate"] for t in _all(tr))
    assert _Traj.peak["run"] <= 4 and _Traj.peak["initialize"] <= 4 and _Traj.peak["evaluate"] <= 2
    first_run = next(i for i, (s, _) in enumerate(_Traj.log) if s == "run")
    last_init = max(i for i, (s, _) in enumerate(_Traj.log) if s == "initialize")
    assert first_run < last_init, "generation of early trajectories overlaps environment set-up of later ones"
    tr = _fresh(fail={(0, 0): "initialize", (2, 1): "run"})
    failures = asyncio.run(D.dispatch("pipeline", tr, max_parallel=3, raise_errors=False))
    assert sorted(k for k, _ in failures) == [(0, 0), (2, 1)]
    assert tr[0][0].done == [] and [s for s, _ in tr[2][1].done] == ["initialize"]
    assert sum(len(t.done) == 3 for t in _all(tr)) == 10


def test_fixed_pool_dispatcher_reuses_environments_and_returns_them_after_a_failure():
    tr = _fresh(n_inst=5, n_samp=2, fail={(4, 1): "run"})
    envs = ["envA", "envB", "envC"]
    failures = asyncio.run(D.dispatch("fixed_pool", tr, envs=envs, raise_errors=False))
    assert [k for k, _ in failures] == [(4, 1)]
    used = [t.done for t in _all(tr) if t.fail_in is None]
    assert all(len(d) == 3 and len({e for _, e in d}) == 1 and d[0][1] in envs for d in used), "one environment per trajectory"
    assert {d[0][1] for d in used} == set(envs) and max(_Traj.peak.values()) <= 3


def test_sync_async_bridges_and_wait_all():
    import time

    async def add(a, b):
        await asyncio.sleep(0.001)
        return a + b

    assert D.call_async_from_sync(add, 2, 3) == 5

    async def inside_a_loop():
        assert D.call_async_from_sync(add, 4, 5) == 9              # a loop is already running in this thread
        assert await D.call_sync_from_async(lambda x: (time.sleep(0.001), x * 2)[1], 21) == 42
        assert await D.wait_all([add(1, 1), add(2, 2)]) == [2, 4]
        assert await D.wait_all([]) == []

        async def boom():
            raise KeyError("x")

        with pytest.raises(D.DispatchError) as ei:
            await D.wait_all([add(1, 1), boom(), add(3, 3)])
        assert [i for i, _ in ei.value.failures] == [1]
        with pytest.raises(asyncio.TimeoutError):
            await D.wait_all([asyncio.sleep(5)], timeout=0.01)

    asyncio.run(inside_a_loop())
    with pytest.raises(asyncio.TimeoutError):
        D.call_async_from_sync(asyncio.sleep, 5, timeout=0.01)
