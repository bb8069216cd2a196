"""Actor runtime: sync / async / async-generator forwarding, error propagation, close, child death."""
import asyncio
import os

import pytest

from art_b200.runtime.actors import move_to_child_process
from tests.actor_fixtures import Counter


def test_proxy_methods_and_streaming():
    proxy = move_to_child_process(Counter(5), process_name="art-b200-test-actor")

    async def main():
        assert await proxy.add(2) == 7
        assert await proxy.slow_add(3) == 10
        items = [x async for x in proxy.stream(4)]
        assert [x["i"] for x in items] == [0, 1, 2, 3]
        assert items[0]["pid"] != os.getpid()
        with pytest.raises(ValueError) as ei:
            await proxy.boom()
        assert "kaboom" in str(ei.value)
        assert "boom" in ei.value.__remote_traceback__
        # concurrent calls
        r = await asyncio.gather(*[proxy.add(1) for _ in range(5)])
        assert sorted(r) == list(range(11, 16))

    try:
        asyncio.run(main())
    finally:
        proxy.close()
    proxy.close()  # idempotent


def test_child_death_is_reported():
    proxy = move_to_child_process(Counter())

    async def main2():
        fut = asyncio.ensure_future(proxy.die())
        await asyncio.sleep(1.0)
        fut.cancel()
        with pytest.raises(RuntimeError):
            await proxy.add(1)

    try:
        asyncio.run(main2())
    finally:
        proxy.close()
