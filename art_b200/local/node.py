"""One model over several GPUs of this machine: a :class:`ModelService` per rank behind one service object.

``engine_args.tensor_parallel_size`` (T) and ``engine_args.data_parallel_size`` (D) of a model's configuration ask for
T x D ranks, one per GPU.  Rank 0 (the leader) is an ordinary model service: it owns the public completion port, the
checkpoints and the metrics.  Every other rank runs the same service class in a child process
(``runtime/actors.py``).  ``NodeService`` is what ``LocalBackend`` holds instead of a single service; it fans every
call out to all ranks:

* ``start_openai_server``: every rank builds its state (the ranks meet in ``torch.distributed``: NCCL on GPUs, gloo
  on CPUs), starts its engine replica and serves it on ``port + rank``; the leader's server spreads incoming
  requests over all replicas (``engine/server.py: OpenAIServer(peers=...)``).
* ``train``: every rank runs the same optimizer steps on its share of the rows (tensor parallel inside groups of T
  ranks, data parallel across the D groups), pausing its own engine first and handing the new adapter to it
  afterwards, device to device; the leader's metrics stream back to the caller while the others are drained.

The reference serves and trains one model from one process on one GPU; its only multi-GPU knobs are pass-through
fields of the inference library (``src/art/dev/engine.py:26-27``, consumed at ``src/art/local/state.py:64-81``).
"""
from __future__ import annotations

import asyncio
import socket
from typing import AsyncIterator

from .. import dev, types
from .pack import DiskPackedTensors
from .service import ModelService


def free_tcp_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


async def _drain(agen) -> int:
    n = 0
    async for _ in agen:
        n += 1
    return n


class NodeService:
    def __init__(self, leader, workers: list):
        self.leader, self.workers = leader, list(workers)

    @property
    def ranks(self) -> list:
        return [self.leader] + self.workers

    async def _all(self, method: str, *args, **kw) -> list:
        """Call ``method`` on every rank at the same time (the ranks rendezvous inside); first error wins."""
        return list(await asyncio.gather(*[getattr(s, method)(*args, **kw) for s in self.ranks]))

    async def start_openai_server(self, config: dev.OpenAIServerConfig | None = None) -> tuple[str, int]:
        await self._all("ready")                  # distributed state first: a rank that fails to build fails everyone
        return (await self._all("start_openai_server", config))[0]

    async def stop_openai_server(self) -> None:
        await self._all("stop_openai_server")

    async def train(self, disk_packed_tensors: DiskPackedTensors, config: types.TrainConfig, _config: dev.TrainConfig,
                    verbose: bool = False) -> AsyncIterator[dict[str, float]]:
        others = [asyncio.ensure_future(_drain(w.train(disk_packed_tensors, config, _config, False))) for w in self.workers]
        lead = self.leader.train(disk_packed_tensors, config, _config, verbose).__aiter__()
        nxt = None
        try:
            while True:
                # the leader's next result races the workers: a rank that failed (its process died, its step raised)
                # is reported at once instead of after the leader's collective has run into its time limit
                nxt = asyncio.ensure_future(lead.__anext__())
                while not nxt.done():
                    await asyncio.wait({nxt, *[t for t in others if not t.done()]}, return_when=asyncio.FIRST_COMPLETED)
                    for t in others:
                        if t.done() and not t.cancelled() and t.exception() is not None:
                            raise t.exception()
                    if all(t.done() for t in others) and not nxt.done():
                        await asyncio.wait({nxt})
                try:
                    metrics = nxt.result()
                except StopAsyncIteration:
                    break
                yield metrics
            await asyncio.gather(*others)
        finally:
            if nxt is not None and not nxt.done():
                nxt.cancel()
            for t in others:
                if not t.done():
                    t.cancel()

    async def flush_checkpoints(self) -> None:
        await self.leader.flush_checkpoints()

    async def shutdown(self) -> None:
        await asyncio.gather(*[s.shutdown() for s in self.ranks], return_exceptions=True)
        self.close()

    def close(self) -> None:
        for s in self.ranks:
            try:
                s.close()
            except Exception:  # noqa: BLE001 - a rank that already went away
                pass


def build_node_service(*, model_name: str, base_model: str, config: dev.InternalModelConfig, output_dir: str, port: int,
                       in_process: bool, log_dir: str | None = None):
    """A plain :class:`ModelService` for a one-GPU model, else a :class:`NodeService` over T x D ranks."""
    from ..runtime.actors import move_to_child_process
    from .service import node_layout

    tp, dp = node_layout(config)
    world = tp * dp
    mk = lambda rank, mport: ModelService(host="localhost", port=port, model_name=model_name, base_model=base_model,  # noqa: E731
                                          config=config, output_dir=output_dir, rank=rank, world=world, tp_size=tp,
                                          master_port=mport)
    log = (lambda name: f"{log_dir}/{name}.log") if log_dir else (lambda name: None)     # noqa: E731
    if world == 1:
        svc = mk(0, 0)
        return svc if in_process else move_to_child_process(svc, log_file=log("model-service"),
                                                            process_name=f"model-service:{model_name}")
    mport = free_tcp_port()
    leader = mk(0, mport)
    if not in_process:
        leader = move_to_child_process(leader, log_file=log("model-service"), process_name=f"model-service:{model_name}")
    workers = [move_to_child_process(mk(r, mport), log_file=log(f"model-service-rank{r}"),
                                     process_name=f"model-service:{model_name}:rank{r}") for r in range(1, world)]
    return NodeService(leader, workers)
