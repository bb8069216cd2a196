"""Model service: the process-local owner of one trainable model (weights, trainer, rollout
engine, completion server).  ``LocalBackend`` talks to it directly (``in_process=True``) or
through the actor proxy in a child process.

Contract parity: reference ``src/art/local/service.py:26-174`` (``start_openai_server``,
``stop_openai_server``, ``train`` as an async generator of per-step metrics, ``_set_lora``) and
``state.py:35-177``.  What differs underneath:

* there is no never-ending trainer loop fed through a queue; ``train`` calls
  ``Trainer.step`` once per optimizer step (in a worker thread so the event loop keeps serving);
* the engine is paused at a step boundary with ``Engine.pause()``; in-flight requests keep their
  KV cache and continue after training under the new adapter;
* the new adapter reaches the engine as a device-to-device copy from the trainer's fp32 master
  buffer; the PEFT checkpoint ``{step:04d}/`` is written from a host copy in a background thread;
* optimizer state is saved next to the adapter (``trainer_state.pt``) so a restarted process
  resumes exactly.
"""
from __future__ import annotations

import asyncio
import os
import threading
import time
from dataclasses import dataclass, field
from typing import AsyncIterator

import torch

from .. import dev, types
from ..models.config import resolve_config
from ..models.peft_io import is_adapter_dir, load_adapter, save_adapter
from ..models.weights import LoraConfig, init_base_weights, init_lora, load_base_weights
from ..utils.get_model_step import get_step_from_dir
from ..utils.output_dirs import get_step_checkpoint_dir
from .checkpoints import get_last_checkpoint_dir
from .pack import DiskPackedTensors, packed_tensors_from_dir
from .tokenizer import load_tokenizer

TRAINER_STATE = "trainer_state.pt"


def shard_rows(packed: dict, keys, start: int, count: int, n_rows: int) -> dict:
    """Rows ``[start, start + count)`` of the packed tensors; positions past ``n_rows`` become copies of row 0 with
    zero weight and no trainable token, which add nothing to loss or gradient."""
    take = list(range(start, min(start + count, n_rows)))
    pad = count - len(take)
    if pad == 0:
        return {k: packed[k][start:start + count] for k in keys}
    idx = torch.tensor(take + [0] * pad, dtype=torch.long)
    rows = {k: packed[k][idx].clone() for k in keys}
    rows["weights"][len(take):] = 0
    rows["assistant_mask"][len(take):] = False
    return rows


def _as_list(x) -> list[str]:
    return [] if not x else ([x] if isinstance(x, str) else list(x))


def node_layout(config: dev.InternalModelConfig) -> tuple[int, int]:
    """(tensor_parallel_size, data_parallel_size) a model's configuration asks for; (1, 1) = one GPU.

    ``engine_args.tensor_parallel_size`` is the knob the reference forwards to its inference library
    (src/art/dev/engine.py:27); here it also sets the trainer's tensor-parallel group size, and
    ``engine_args.data_parallel_size`` the number of such groups.  The service then runs one rank per GPU."""
    ea = config.get("engine_args", {}) or {}
    ta = config.get("trainer_args", {}) or {}
    if int(ea.get("expert_parallel_size") or ta.get("expert_parallel_size") or 1) > 1:
        raise ValueError("expert_parallel_size > 1: the model service lays a model out as (tensor, context or pipeline "
                         "parallel) x data parallel; expert parallel training is reached through trainer.Trainer(ep=) "
                         "(see bench.py --parallel ep), not through LocalBackend yet")
    kind, size = group_layout(config)
    return size, max(1, int(ea.get("data_parallel_size") or 1))


def group_layout(config: dev.InternalModelConfig) -> tuple[str, int]:
    """What the groups of adjacent GPUs of a model split, and how many GPUs a group has: ``("tp", n)`` heads and FFN
    columns (``tensor_parallel_size``), ``("cp", n)`` the tokens of every packed row (``context_parallel_size``), or
    ``("pp", n)`` the layers (``pipeline_parallel_size``).  The sizes are read from the engine arguments, then the
    trainer arguments; at most one of them may exceed 1 (the three do not compose inside the service)."""
    ea, ta = config.get("engine_args", {}) or {}, config.get("trainer_args", {}) or {}
    sizes = {kind: max(1, int(ea.get(key) or ta.get(key) or 1))
             for kind, key in (("tp", "tensor_parallel_size"), ("cp", "context_parallel_size"), ("pp", "pipeline_parallel_size"))}
    big = [k for k, v in sizes.items() if v > 1]
    if len(big) > 1:
        raise ValueError(f"tensor, context and pipeline parallel sizes do not compose in the model service yet: "
                         f"{ {k: sizes[k] for k in big} }")
    return (big[0], sizes[big[0]]) if big else ("tp", 1)


class ModelState:
    """Everything that lives on the device for one model (on one rank of the node, if the model spans several GPUs).

    With ``world > 1`` every rank builds the same state: the trainer is tensor parallel inside groups of ``tp``
    consecutive ranks and data parallel across them (LoRA gradients averaged by the fused all-reduce); the rollout
    engine is one replica per rank over a full copy of the frozen weights, so that after a training step every rank
    hands the new adapter to its own engine without any transfer (all ranks hold identical LoRA masters)."""

    def __init__(self, base_model: str, config: dev.InternalModelConfig, output_dir: str, rank: int = 0, world: int = 1,
                 tp: int = 1, master_port: int = 0):
        from ..engine.engine import Engine
        from ..engine.kv_cache import BlockManager, KVCache
        from ..trainer.trainer import Trainer

        init_args = config.get("init_args", {})
        engine_args = config.get("engine_args", {})
        peft_args = config.get("peft_args", {})
        targs = config.get("trainer_args", {})
        if rank == 0:
            dev.engine.split_engine_args(dict(engine_args))     # names, once each, the keys that have no effect here
            dev.model.warn_ignored(config)
        self.rank, self.world, self.tp_size = rank, world, tp       # tp_size: ranks that share rows (TP or CP group)
        self.group_kind = group_layout(config)[0]
        self.data_index, self.data_ranks = 0, 1
        if world > 1 and rank > 0 and not torch.cuda.is_initialized():
            # a worker rank lives in a process of its own: list its GPU first, so that it is device 0 for every thread of
            # the process (event loop, executor threads, the engine thread) without each of them having to select it;
            # the other GPUs stay visible, as peer mappings of their memory need them to be
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            ids = [v for v in vis.split(",") if v] if vis else [str(i) for i in range(max(world, rank + 1))]
            if len(ids) > rank:
                os.environ["CUDA_VISIBLE_DEVICES"] = ",".join([ids[rank]] + ids[:rank] + ids[rank + 1:])
        has_gpu = torch.cuda.is_available()
        self.device = torch.device("cuda", torch.cuda.current_device()) if has_gpu else torch.device("cpu")
        tp_group = dp_group = None
        self._owns_pg = False
        if world > 1:
            import datetime

            import torch.distributed as dist

            from ..parallel.mesh import ParallelLayout

            if not dist.is_initialized():
                kw = {"device_id": self.device} if has_gpu else {}
                dist.init_process_group("nccl" if has_gpu else "gloo", init_method=f"tcp://127.0.0.1:{master_port}",
                                        rank=rank, world_size=world,
                                        timeout=datetime.timedelta(seconds=float(os.environ.get("ART_B200_DIST_TIMEOUT_S", 600))), **kw)
                self._owns_pg = True
            layout = ParallelLayout(world, tp=tp)
            groups = layout.create_groups(rank)
            tp_group, dp_group = groups["tp"], groups["dp"]
            self.data_index, self.data_ranks = layout.data_shard(rank)
        cp_group = pp_group = None
        if self.group_kind == "cp":      # the same groups of adjacent ranks, used to split rows instead of heads
            tp_group, cp_group = None, tp_group
        elif self.group_kind == "pp":    # ... or to hold consecutive blocks of layers
            tp_group, pp_group = None, tp_group
        self.cfg = resolve_config(base_model, init_args.get("architecture"))
        self.lora_cfg = LoraConfig(r=int(peft_args.get("r", 8)), alpha=float(peft_args.get("lora_alpha", 16)),
                                   target_modules=tuple(peft_args.get("target_modules", LoraConfig().target_modules)),
                                   use_rslora=bool(peft_args.get("use_rslora", False)))
        self.tokenizer = load_tokenizer(base_model, self.cfg.vocab_size)
        seed = int(init_args.get("random_state", 0))
        if os.path.isdir(base_model) and not init_args.get("random_init"):
            base = load_base_weights(base_model, self.cfg, device=self.device)
        else:
            dt = torch.bfloat16 if self.device.type == "cuda" else torch.float32
            base = init_base_weights(self.cfg, seed=seed, dtype=dt, device=self.device,
                                     std=float(init_args.get("init_std", 0.02)))
        # LoRA: resume from the newest checkpoint, else fresh init
        last = get_last_checkpoint_dir(output_dir)
        if last and not is_adapter_dir(last) and int(os.path.basename(last)) > 0:
            # an empty or partial step directory (an interrupted write of an older layout): re-initialising here would
            # silently throw the training away while the step counter carries on
            raise RuntimeError(f"checkpoint directory {last} holds no complete adapter; delete it to resume from the "
                               "step before it")
        if last and is_adapter_dir(last):
            lora, _ = load_adapter(last, self.device)
        else:
            lora = init_lora(self.cfg, self.lora_cfg, seed=int(peft_args.get("random_state", 3407)), device=self.device)
        grad_sync = None
        if self.data_ranks > 1:
            if has_gpu:
                from ..parallel.symm_mem import FusedGradAllReduce

                grad_sync = FusedGradAllReduce(self.device, self.data_ranks, dp_group, wait_ms=20000)
            else:
                from ..parallel.dp import nccl_grad_sync

                grad_sync = nccl_grad_sync(self.data_ranks, dp_group)      # CPU ranks: the library all-reduce on gloo
        if tp > 1 and not has_gpu:
            raise ValueError("tensor- and context-parallel training need GPUs (the CPU path is data parallel only)")
        self.tp_tokens = int(targs.get("tokens_per_microbatch") or 8192 * tp)
        self.trainer = Trainer(self.cfg, base, self.lora_cfg, lora, device=self.device,
                               betas=(float(targs.get("adam_beta1", 0.9)), float(targs.get("adam_beta2", 0.99))),
                               weight_decay=float(targs.get("weight_decay", 0.1)),
                               max_grad_norm=float(targs.get("max_grad_norm", 0.1)),
                               adam_eps=float(targs.get("adam_epsilon", 1e-8)), grad_sync=grad_sync, dp_group=dp_group,
                               tp_group=tp_group, tp_tokens=self.tp_tokens, cp_group=cp_group, pp_group=pp_group)
        if last and os.path.exists(os.path.join(last, TRAINER_STATE)):
            self.trainer.load_trainer_state(torch.load(os.path.join(last, TRAINER_STATE), map_location="cpu"))
        # rollout engine: one replica per rank
        block_size = int(engine_args.get("block_size") or 16)
        max_loras = int(engine_args.get("max_loras", 4))
        max_len = int(engine_args.get("max_model_len") or init_args.get("max_seq_length", 32768))
        if self.device.type == "cuda":
            from ..engine.runner import NativeRunner

            free, total = torch.cuda.mem_get_info(self.device)
            util = float(engine_args.get("gpu_memory_utilization", init_args.get("gpu_memory_utilization", 0.5)))
            per_block = KVCache.bytes_per_block(self.cfg.num_layers, block_size, self.cfg.num_kv_heads, self.cfg.head_dim)
            budget = min(free * 0.6, total * util * 0.5)   # leave room for training activations
            num_blocks = int(engine_args.get("num_gpu_blocks_override") or max(64, int(budget // per_block)))
            # sleep mode frees the cache while the trainer runs: the virtual-memory arena keeps every address stable, so
            # decode graphs captured before a training step stay valid after it
            sleep_mode = bool(engine_args.get("enable_sleep_mode", False))
            try:
                self.kv = KVCache(self.cfg.num_layers, num_blocks, block_size, self.cfg.num_kv_heads, self.cfg.head_dim,
                                  self.device, use_arena=sleep_mode)
            except RuntimeError:   # no VMM support: plain tensors; Engine.sleep() then drops the captured graphs
                self.kv = KVCache(self.cfg.num_layers, num_blocks, block_size, self.cfg.num_kv_heads, self.cfg.head_dim,
                                  self.device)
            if tp_group is not None or pp_group is not None:      # the trainer holds a part of the weights: the replica keeps its own full copy
                runner = NativeRunner(self.cfg, self.lora_cfg, self.kv, base=base, max_loras=max_loras, device=self.device)
            else:           # trainer and engine share the frozen weights
                runner = NativeRunner(self.cfg, self.lora_cfg, self.kv, decoder=self.trainer.model, max_loras=max_loras,
                                      device=self.device)
        else:
            from ..engine.runner import ReferenceRunner

            num_blocks = int(engine_args.get("num_gpu_blocks_override") or 4096)
            self.kv = None
            runner = ReferenceRunner(self.cfg, base, self.lora_cfg, max_loras=max_loras, device=self.device)
        self.engine = Engine(runner, BlockManager(num_blocks, block_size, bool(engine_args.get("enable_prefix_caching", True))),
                             eos_token_id=getattr(self.tokenizer, "eos_token_id", None),
                             max_num_seqs=int(engine_args.get("max_num_seqs") or 256),
                             max_num_batched_tokens=int(engine_args.get("max_num_batched_tokens") or 16384),
                             num_scheduler_steps=int(engine_args.get("num_scheduler_steps", 16)), max_model_len=max_len,
                             max_loras=max_loras, kv_cache=self.kv,
                             enable_chunked_prefill=bool(engine_args.get("enable_chunked_prefill", True)),
                             log_stats_interval=None if engine_args.get("disable_log_stats", init_args.get("disable_log_stats"))
                             else 10.0)
        self.sleep_mode = bool(engine_args.get("enable_sleep_mode", False))

    def close(self) -> None:
        self.engine.shutdown()
        runner = self.engine.runner
        if hasattr(runner, "close"):
            runner.close()
        tpctx = getattr(self.trainer, "tp", None)
        if tpctx is not None:
            tpctx.close()
        if self._owns_pg:
            import torch.distributed as dist

            if dist.is_initialized():
                dist.destroy_process_group()
            self._owns_pg = False


@dataclass
class ModelService:
    host: str
    port: int
    model_name: str
    base_model: str
    config: dev.InternalModelConfig
    output_dir: str
    # this service's place among the ranks of a model that spans several GPUs (rank 0 leads: it owns the public
    # port, the checkpoints and the metrics); see local/node.py
    rank: int = 0
    world: int = 1
    tp_size: int = 1
    master_port: int = 0
    _state: ModelState | None = field(default=None, repr=False, compare=False)
    _pool: object = field(default=None, repr=False, compare=False)
    _server_task: asyncio.Task | None = field(default=None, repr=False, compare=False)
    _ckpt_thread: threading.Thread | None = field(default=None, repr=False, compare=False)
    _ckpt_error: BaseException | None = field(default=None, repr=False, compare=False)

    def __getstate__(self):   # only the configuration crosses the process boundary
        d = dict(self.__dict__)
        d["_state"] = d["_server_task"] = d["_ckpt_thread"] = d["_ckpt_error"] = d["_pool"] = None
        return d

    @property
    def pool(self):
        """Worker threads for blocking device work.  CUDA's current device is per thread and starts at device 0, so
        every thread of this pool selects the model's device when it starts (what matters for a rank other than 0
        living in a process that sees several GPUs)."""
        if self._pool is None:
            from concurrent.futures import ThreadPoolExecutor

            def bind():
                st = self._state
                if st is not None and st.device.type == "cuda":
                    torch.cuda.set_device(st.device)

            self._pool = ThreadPoolExecutor(max_workers=4, thread_name_prefix="art-b200-service", initializer=bind)
        return self._pool

    @property
    def state(self) -> ModelState:
        if self._state is None:
            self._state = ModelState(self.base_model, self.config, self.output_dir, self.rank, self.world, self.tp_size,
                                     self.master_port)
        return self._state

    # -- serving --------------------------------------------------------------------------------------
    async def start_openai_server(self, config: dev.OpenAIServerConfig | None = None) -> tuple[str, int]:
        from ..engine.server import OpenAIServer, route_logs_to_file, serve, serve_kwargs

        st = self.state
        step0 = get_step_checkpoint_dir(self.output_dir, 0)
        if self.rank == 0 and get_last_checkpoint_dir(self.output_dir) is None:
            save_adapter(step0, st.trainer.lora_state_dict(), st.lora_cfg, self.base_model)   # step 0 = untrained adapter
        lora_path = get_last_checkpoint_dir(self.output_dir) or step0
        cfg = dev.get_openai_server_config(self.model_name, self.base_model, f"{self.output_dir}/logs/engine.log",
                                           lora_path, config)
        sargs = cfg.get("server_args", {})
        st.engine.start()
        self._set_lora_in_device()
        for spec in (sargs.get("lora_modules") or []):   # extra adapters served next to the trainable one
            name, path = dev.openai_server.parse_lora_module(spec)
            if name != self.model_name and is_adapter_dir(path):
                st.engine.set_adapter(name, load_adapter(path, st.device)[0])
        host, port0 = sargs.get("host") or "0.0.0.0", int(sargs.get("port", self.port))
        port = port0 + self.rank                # rank r serves its replica on the leader's port + r
        # the leader spreads requests over all replicas (its own included); the others serve what they are sent
        peers = [f"http://127.0.0.1:{port0 + r}" for r in range(1, self.world)] if self.rank == 0 else []
        eargs = cfg.get("engine_args", {})
        server = OpenAIServer.from_server_args(st.engine, st.tokenizer, self.base_model, sargs, peers=peers,
                                               log_requests=eargs.get("disable_log_requests") is False,
                                               stream_per_token=bool(eargs.get("multi_step_stream_outputs", False)),
                                               max_logprobs=int(eargs.get("max_logprobs") or 20),
                                               extra_base_names=_as_list(eargs.get("served_model_name")))
        self._server = server
        await self.stop_openai_server()
        ready = asyncio.Event()
        listener = serve_kwargs(sargs) if self.rank == 0 else {}   # replicas behind the leader are reached over loopback
        listener.setdefault("log_level", "warning")
        if cfg.get("log_file"):
            suffix = f".rank{self.rank}" if self.rank else ""
            listener["log_config"] = route_logs_to_file(cfg["log_file"] + suffix)
        self._server_task = asyncio.create_task(serve(server, host, port, ready=ready, **listener))
        try:
            await asyncio.wait_for(ready.wait(), timeout=30)
        except asyncio.TimeoutError as e:
            raise TimeoutError("completion server did not start within 30 s") from e
        if self._server_task.done():
            self._server_task.result()
        return host, port

    async def stop_openai_server(self) -> None:
        if self._server_task is not None:
            self._server_task.cancel()
            try:
                await self._server_task
            except (asyncio.CancelledError, Exception):
                pass
            self._server_task = None

    def _set_lora_in_device(self) -> None:
        """Hand the trainer's current LoRA to the engine under the model's name (device-to-device)."""
        st = self.state
        st.engine.set_adapter(self.model_name, st.trainer.flat.views)

    async def _set_lora(self, lora_path: str) -> None:
        """Load an adapter directory into the engine (used for externally produced checkpoints)."""
        st = self.state
        state, _ = load_adapter(lora_path, st.device)
        st.engine.pause()
        try:
            st.engine.set_adapter(self.model_name, state)
        finally:
            st.engine.resume()

    # -- training -------------------------------------------------------------------------------------
    async def train(self, disk_packed_tensors: DiskPackedTensors, config: types.TrainConfig, _config: dev.TrainConfig,
                    verbose: bool = False) -> AsyncIterator[dict[str, float]]:
        from ..trainer.trainer import PACKED_KEYS, TrainHyper

        st = self.state
        packed = packed_tensors_from_dir(**disk_packed_tensors)
        hyper = TrainHyper(learning_rate=config.learning_rate, beta=config.beta,
                           epsilon=float(_config.get("epsilon", 0.2)), epsilon_high=_config.get("epsilon_high"),
                           rows_per_optimizer_step=int(_config.get("rows_per_optimizer_step", 1)),
                           tokens_per_microbatch=int(_config.get("tokens_per_microbatch", 8192)),
                           compat_row_positions=bool(_config.get("compat_row_positions", False)),
                           recompute=str(_config.get("activation_recompute")
                                         or self.config.get("init_args", {}).get("activation_recompute", "auto")))
        loop = asyncio.get_running_loop()
        await loop.run_in_executor(self.pool, st.engine.pause)
        slept = False
        try:
            if st.sleep_mode:
                await loop.run_in_executor(self.pool, st.engine.sleep, 1 if st.engine.has_unfinished else 2)
                slept = True
            n_rows = packed["tokens"].shape[0]
            per = max(1, hyper.rows_per_optimizer_step)
            if st.tp_size > 1 and st.group_kind == "tp":      # a tensor-parallel micro-batch has a fixed token count: whole micro-batches per step
                S_row = packed["tokens"].shape[1]
                rows_mb = max(1, st.tp_tokens // S_row)
                per = (per + rows_mb - 1) // rows_mb * rows_mb
                hyper.rows_per_optimizer_step, hyper.tokens_per_microbatch = per, rows_mb * S_row
            elif st.tp_size > 1 and st.group_kind == "pp":    # pipeline micro-batches all have the same number of rows
                rows_mb = max(1, min(per, hyper.tokens_per_microbatch // packed["tokens"].shape[1]))
                per = (per + rows_mb - 1) // rows_mb * rows_mb
                hyper.rows_per_optimizer_step = per
            D, j = st.data_ranks, st.data_index
            t0 = time.monotonic()
            tokens_done = 0
            for start in range(0, n_rows, per * D):
                # data-parallel group j takes the j-th slice of this optimizer step's rows; a slice that runs past the
                # end is filled with weightless copies of the first row, so that every rank still joins the step
                rows = shard_rows(packed, PACKED_KEYS, start + j * per, per, n_rows)
                if st.device.type == "cuda":
                    rows = {k: v.pin_memory() for k, v in rows.items()}
                metrics = await loop.run_in_executor(self.pool, st.trainer.step, rows, hyper)
                tokens_done += rows["tokens"].numel()
                metrics["tokens_per_second"] = tokens_done / max(1e-9, time.monotonic() - t0)
                if verbose:
                    print(f"[train] step {st.trainer.global_step}: {metrics}", flush=True)
                yield metrics
            if self.rank != 0:      # only the leader writes checkpoints; every rank holds the same adapter
                if slept:
                    await loop.run_in_executor(self.pool, st.engine.wake_up)
                    slept = False
                self._set_lora_in_device()
                return
            # new step directory = PEFT adapter (+ optimizer state).  The files are written by a thread while the engine
            # wakes up and takes the new adapter; they go into "{step}.tmp" and are renamed once complete, so a numeric
            # directory always holds a whole checkpoint, and the write has finished (or raised) before train() returns,
            # as in the reference (src/art/local/service.py:150-157: save_model before the generator ends)
            step = get_step_from_dir(self.output_dir) + 1
            ckpt_dir = get_step_checkpoint_dir(self.output_dir, step)
            self._join_checkpoint()
            host_state, tstate = self._host_copies()
            self._start_checkpoint(ckpt_dir, host_state, tstate)
            if slept:
                await loop.run_in_executor(self.pool, st.engine.wake_up)
                slept = False
            self._set_lora_in_device()
            # the adapter of the new step must be on disk before train() returns; the optimizer state (twice its size)
            # may still be in flight: it is joined by the next train / flush / close
            await loop.run_in_executor(self.pool, self._join_adapter)
        finally:
            if slept:
                await loop.run_in_executor(self.pool, st.engine.wake_up)
            st.engine.resume()

    def _host_copies(self) -> tuple[dict, dict]:
        """Host copies of the adapter and of the optimizer state for the checkpoint writer.  The LoRA masters and the
        AdamW moments are three flat fp32 buffers, so this is three device-to-host copies into pinned buffers that are
        kept between steps (the per-tensor dictionary is views of the first)."""
        st = self.state
        flat = st.trainer.flat
        if st.device.type != "cuda":
            return ({k: v.detach().to("cpu", copy=True) for k, v in flat.views.items()}, st.trainer.trainer_state())
        if getattr(self, "_pinned", None) is None or self._pinned[0].numel() != flat.params.numel():
            self._pinned = [torch.empty(flat.params.numel(), dtype=torch.float32).pin_memory() for _ in range(3)]
        hp, hm, hv = self._pinned
        hp.copy_(flat.params.detach(), non_blocking=True)
        hm.copy_(st.trainer.opt.m, non_blocking=True)
        hv.copy_(st.trainer.opt.v, non_blocking=True)
        torch.cuda.current_stream(st.device).synchronize()
        host_state = {k: hp[flat.offsets[k]:flat.offsets[k] + v.numel()].view(v.shape) for k, v in flat.views.items()}
        tstate = {"optimizer": {"m": hm, "v": hv, "step": st.trainer.opt.step_count}, "global_step": st.trainer.global_step}
        return host_state, tstate

    def _start_checkpoint(self, ckpt_dir: str, host_state: dict, tstate: dict) -> None:
        import shutil

        st = self.state
        tmp = ckpt_dir + ".tmp"
        self._ckpt_error = None
        self._adapter_done = threading.Event()

        def write():
            try:
                shutil.rmtree(tmp, ignore_errors=True)
                save_adapter(tmp, host_state, st.lora_cfg, self.base_model)
                os.replace(tmp, ckpt_dir)          # a numeric directory always holds a complete adapter
                self._adapter_done.set()
                part = os.path.join(ckpt_dir, TRAINER_STATE + ".tmp")
                torch.save(tstate, part)
                os.replace(part, os.path.join(ckpt_dir, TRAINER_STATE))
            except BaseException as e:  # noqa: BLE001 - handed to the caller of _join_checkpoint / _join_adapter
                self._ckpt_error = e
            finally:
                self._adapter_done.set()

        self._ckpt_thread = threading.Thread(target=write, daemon=True)
        self._ckpt_thread.start()

    def _join_adapter(self) -> None:
        """Wait until the adapter files of the step being written are in place (or the writer failed)."""
        ev = getattr(self, "_adapter_done", None)
        if ev is not None:
            ev.wait()
        if self._ckpt_error is not None:
            self._join_checkpoint()

    def _join_checkpoint(self) -> None:
        """Wait for the checkpoint writer; an exception it hit (disk full, ...) is raised here, once."""
        t, self._ckpt_thread = self._ckpt_thread, None
        if t is not None:
            t.join()
        err, self._ckpt_error = self._ckpt_error, None
        if err is not None:
            raise RuntimeError("writing the step checkpoint failed") from err

    async def flush_checkpoints(self) -> None:
        await asyncio.get_running_loop().run_in_executor(self.pool, self._join_checkpoint)

    async def shutdown(self) -> None:
        await self.stop_openai_server()
        await self.flush_checkpoints()
        if self._state is not None:
            self._state.close()
            self._state = None

    async def ready(self) -> int:
        """Builds the state (on a multi-GPU model: joins the ranks' rendezvous); returns this service's rank."""
        await asyncio.get_running_loop().run_in_executor(None, lambda: self.state)
        return self.rank

    def close(self) -> None:
        self._join_checkpoint()
        if self._state is not None:
            self._state.close()
            self._state = None
