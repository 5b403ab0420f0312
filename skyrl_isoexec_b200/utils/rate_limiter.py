"""Limits on how fast and how many trajectories a generator starts (reference: R/train/utils/rate_limiter.py:22-224,
``RateLimiterConfig`` / ``AsyncRateLimiter`` / ``create_rate_limiter``).

Two independent limits, both optional: a start rate (a token bucket whose capacity equals the rate, so a burst of at most
one second's worth of starts passes at once) and a cap on trajectories in flight. ``async with limiter:`` brackets one
trajectory. The clock and the sleep are injectable so tests run on virtual time."""

from __future__ import annotations

import asyncio
import time
from collections.abc import Mapping
from dataclasses import dataclass


@dataclass
class RateLimiterConfig:
    enabled: bool = False
    trajectories_per_second: float | None = None     # >= 1.0: the bucket could never fill to one whole token below that
    max_concurrency: int | None = None

    def __post_init__(self):
        if self.trajectories_per_second is not None and self.trajectories_per_second < 1.0:
            raise ValueError(f"trajectories_per_second must be >= 1.0, got {self.trajectories_per_second}")
        if self.max_concurrency is not None and self.max_concurrency < 1:
            raise ValueError(f"max_concurrency must be >= 1, got {self.max_concurrency}")


class NoOpRateLimiter:
    in_flight = 0

    async def acquire(self) -> None:
        return None

    def release(self) -> None:
        return None

    async def __aenter__(self):
        return self

    async def __aexit__(self, *exc) -> None:
        return None


class AsyncRateLimiter:
    def __init__(self, rate: float | None = None, max_concurrency: int | None = None, clock=time.monotonic, sleep=asyncio.sleep):
        RateLimiterConfig(True, rate, max_concurrency)            # same validation
        self.rate, self.max_concurrency = rate, max_concurrency
        self._clock, self._sleep = clock, sleep
        self._tokens = float(rate or 0.0)
        self._stamp = clock()
        self._bucket_lock: asyncio.Lock | None = None             # made on first use, inside the running loop
        self._slots: asyncio.Semaphore | None = None
        self.in_flight = 0
        self.peak_in_flight = 0
        self.started = 0

    def _refill(self) -> None:
        now = self._clock()
        self._tokens = min(float(self.rate), self._tokens + (now - self._stamp) * self.rate)
        self._stamp = now

    async def _take_token(self) -> None:
        if self._bucket_lock is None:
            self._bucket_lock = asyncio.Lock()
        async with self._bucket_lock:                             # waiters are served in arrival order
            self._refill()
            while self._tokens < 1.0:
                await self._sleep((1.0 - self._tokens) / self.rate)
                self._refill()
            self._tokens -= 1.0

    async def acquire(self) -> None:
        """Wait for a free slot first and a rate token second, so a trajectory that waits for a slot does not hold a token."""
        if self.max_concurrency is not None:
            if self._slots is None:
                self._slots = asyncio.Semaphore(self.max_concurrency)
            await self._slots.acquire()
        try:
            if self.rate is not None:
                await self._take_token()
        except BaseException:
            if self._slots is not None:
                self._slots.release()
            raise
        self.in_flight += 1
        self.started += 1
        self.peak_in_flight = max(self.peak_in_flight, self.in_flight)

    def release(self) -> None:
        self.in_flight -= 1
        if self._slots is not None:
            self._slots.release()

    async def __aenter__(self):
        await self.acquire()
        return self

    async def __aexit__(self, *exc) -> None:
        self.release()


def create_rate_limiter(config) -> NoOpRateLimiter | AsyncRateLimiter:
    """``config``: a ``RateLimiterConfig``, a mapping with its keys, or None. Disabled, or enabled without any limit, gives
    the no-op limiter."""
    if config is None:
        return NoOpRateLimiter()
    if isinstance(config, Mapping):
        config = RateLimiterConfig(bool(config.get("enabled", False)), config.get("trajectories_per_second"), config.get("max_concurrency"))
    if not config.enabled or (config.trajectories_per_second is None and config.max_concurrency is None):
        return NoOpRateLimiter()
    return AsyncRateLimiter(config.trajectories_per_second, config.max_concurrency)
