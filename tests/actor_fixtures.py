"""Picklable service used by the actor tests (must be importable from the spawned child)."""
import asyncio
import os


class Counter:
    def __init__(self, start=0):
        self.value = start

    def add(self, n):
        self.value += n
        return self.value

    async def slow_add(self, n):
        await asyncio.sleep(0.01)
        self.value += n
        return self.value

    async def stream(self, n):
        for i in range(n):
            await asyncio.sleep(0)
            yield {"i": i, "pid": os.getpid()}

    def boom(self):
        raise ValueError("kaboom from child")

    def die(self):
        os._exit(3)
