"""LocalBackend: directory-backed backend that owns model services on this machine.

Parity: reference ``src/art/local/backend.py:53-482``.  Same methods and on-disk layout
(``model.json``, ``{step:04d}/`` adapters, ``trajectories/{split}/{step:04d}.yaml``, ``tensors/``);
additions: metrics are always appended to ``history.jsonl`` (the reference only reads that file,
and only logs to W&B), each model gets its own free port, and starting a model never kills
other processes.
"""
from __future__ import annotations

import asyncio
import json
import math
from datetime import datetime
import os
import random
import socket
from typing import AsyncIterator

from tqdm import auto as tqdm

from .. import dev
from ..backend import Backend
from ..model import Model, TrainableModel
from ..trajectories import Trajectory, TrajectoryGroup
from ..types import TrainConfig
from ..utils import format_message, get_model_step
from ..utils.old_benchmarking.calculate_step_metrics import calculate_step_std_dev
from ..utils.deploy_model import LoRADeploymentJob, LoRADeploymentProvider, deploy_model
from ..utils.output_dirs import get_default_art_path, get_model_dir, get_trajectories_split_dir
from ..utils.s3 import pull_model_from_s3, push_model_to_s3
from ..utils.trajectory_logging import serialize_trajectory_groups
from .checkpoints import delete_checkpoints
from .pack import PackedTensors, packed_tensors_from_tokenized_results, packed_tensors_to_dir, plot_packed_tensors
from .service import ModelService
from .tokenize import tokenize_trajectory_groups
from .tokenizer import load_tokenizer


def _port_is_free(port: int) -> bool:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        try:
            s.bind(("0.0.0.0", port))
            return True
        except OSError:
            return False


def _free_port(preferred: int, span: int = 1) -> int:
    """First port at or after ``preferred`` from which ``span`` consecutive ports are free."""
    for port in range(preferred, preferred + 200):
        if all(_port_is_free(port + i) for i in range(span)):
            return port
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("0.0.0.0", 0))
        return s.getsockname()[1]


def best_step_from_history(path: str, metric: str, smoothing: float) -> int | None:
    """Step with the best exponentially-weighted mean of ``metric`` (alpha = ``smoothing``)."""
    by_step: dict[int, list[float]] = {}
    with open(path) as f:
        for line in f:
            try:
                row = json.loads(line)
            except json.JSONDecodeError:
                continue
            if row.get(metric) is None or "step" not in row:
                continue
            by_step.setdefault(int(row["step"]), []).append(float(row[metric]))
    if not by_step:
        return None
    best, best_v, ewm = None, -math.inf, None
    num = den = 0.0
    for step in sorted(by_step):
        v = sum(by_step[step]) / len(by_step[step])
        num = v + (1 - smoothing) * num    # pandas/polars ewm_mean(adjust=True)
        den = 1 + (1 - smoothing) * den
        ewm = num / den
        if ewm >= best_v:
            best, best_v = step, ewm
    return best


class LocalBackend(Backend):
    def __init__(self, *, in_process: bool = False, path: str | None = None) -> None:
        """``in_process``: run model services inside this process instead of a child process.
        ``path``: storage root, default ``{git root}/.art``."""
        self._in_process = in_process
        self._path = path or get_default_art_path()
        os.makedirs(self._path, exist_ok=True)
        self._services: dict[str, ModelService] = {}
        self._server_configs: dict[str, tuple] = {}     # model name -> (OpenAI server config, (host, port)) of its start
        self.service_restarts: dict[str, int] = {}      # model name -> times its service process was restarted
        self._tokenizers: dict[str, object] = {}
        self._wandb_runs: dict[str, object] = {}
        self._rng = random.Random()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()

    async def __aenter__(self):
        return self

    async def __aexit__(self, *exc):
        self.close()

    def close(self):  # usable both as ``backend.close()`` and ``await backend.close()``
        for service in self._services.values():
            service.close()   # in-process: stops the engine; proxy: shuts the child process down
        self._services.clear()
        return _Done()

    async def register(self, model: Model) -> None:
        out = get_model_dir(model=model, art_path=self._path)
        os.makedirs(out, exist_ok=True)
        with open(f"{out}/model.json", "w") as f:
            json.dump(model.model_dump(), f, default=str)
        if isinstance(model, TrainableModel) and "WANDB_API_KEY" in os.environ:
            self._get_wandb_run(model)

    async def _get_service(self, model: TrainableModel) -> ModelService:
        if model.name not in self._services:
            out = get_model_dir(model=model, art_path=self._path)
            config = dev.get_model_config(base_model=model.base_model, output_dir=out, config=model._internal_config)
            from .node import build_node_service
            from .service import node_layout

            tp, dp = node_layout(config)
            os.makedirs(f"{out}/logs", exist_ok=True)
            # a model over several GPUs serves rank r on port + r: look for that many free ports in a row
            port = _free_port(8000 + 16 * len(self._services), span=tp * dp)
            self._services[model.name] = build_node_service(model_name=model.name, base_model=model.base_model,
                                                            config=config, output_dir=out, port=port,
                                                            in_process=self._in_process, log_dir=f"{out}/logs")
        return self._services[model.name]


    async def _restart_service(self, model: TrainableModel):
        """Replace the model's service process: the new one loads the newest complete checkpoint and serves on the same
        address, so clients that hold the inference URL keep working."""
        old = self._services.pop(model.name, None)
        if old is not None:
            try:
                old.close()          # terminates the child if it is still alive (watchdog case)
            except Exception:  # noqa: BLE001 - the process may be half dead already
                pass
        self.service_restarts[model.name] = self.service_restarts.get(model.name, 0) + 1
        service = await self._get_service(model)
        if model.name in self._server_configs:
            cfg, (_, port) = self._server_configs[model.name]
            cfg = dict(cfg or {})
            cfg["server_args"] = {**cfg.get("server_args", {}), "port": port}
            host, new_port = await service.start_openai_server(config=cfg)
            if new_port != port:
                raise RuntimeError(f"the restarted service of {model.name!r} came up on port {new_port}, not {port}")
        return service

    def _get_packed_tensors(self, model: TrainableModel, trajectory_groups: list[TrajectoryGroup],
                            allow_training_without_logprobs: bool, plot_tensors: bool,
                            seed: int | None = None) -> PackedTensors | None:
        """``seed``: the prompt ids and the two shuffles of this call come from ``random.Random(seed)``, which makes
        the packed rows a function of the trajectories alone; without it the backend's own generator goes on."""
        rng = self._rng if seed is None else random.Random(seed)
        if model.base_model not in self._tokenizers:
            arch = ((model._internal_config or {}).get("init_args", {}) or {}).get("architecture")
            vocab = arch.get("vocab_size") if arch else None
            if vocab is None:
                try:
                    from ..models.config import resolve_config

                    vocab = resolve_config(model.base_model).vocab_size
                except ValueError:
                    vocab = None
            self._tokenizers[model.base_model] = load_tokenizer(model.base_model, vocab)
        tokenizer = self._tokenizers[model.base_model]
        results = list(tokenize_trajectory_groups(tokenizer, trajectory_groups, allow_training_without_logprobs, rng))
        if not results:
            return None
        longest = max(len(r.token_ids) for r in results)
        seq_len = math.ceil(longest / 2048) * 2048
        cap = (model._internal_config or dev.InternalModelConfig()).get("init_args", {}).get("max_seq_length", 32_768)
        seq_len = min(seq_len, cap)
        packed = packed_tensors_from_tokenized_results(results, seq_len, pad_token_id=tokenizer.eos_token_id, rng=rng)
        if not allow_training_without_logprobs and bool(packed["logprobs"].isnan().all()):
            print("There are no assistant logprobs to train on. Did you forget to include at least one Choice in "
                  "Trajectory.messages_and_choices?")
            return None
        if plot_tensors:
            plot_packed_tensors(packed)
        else:
            print(f"Packed {len(results)} trajectories into {packed['tokens'].shape[0]} sequences of length "
                  f"{packed['tokens'].shape[1]}")
        return packed

    async def _get_step(self, model: TrainableModel) -> int:
        return get_model_step(model, self._path)

    async def _delete_checkpoints(self, model: TrainableModel, benchmark: str, benchmark_smoothing: float) -> None:
        out = get_model_dir(model=model, art_path=self._path)
        keep = [get_model_step(model, self._path)]
        try:
            best = best_step_from_history(f"{out}/history.jsonl", benchmark, benchmark_smoothing)
            if best is None:
                print(f'No "{benchmark}" metric found in history')
            else:
                keep.append(best)
        except FileNotFoundError:
            pass
        delete_checkpoints(out, keep)

    async def _prepare_backend_for_training(self, model: TrainableModel,
                                            config: dev.OpenAIServerConfig | None = None) -> tuple[str, str]:
        service = await self._get_service(model)
        host, port = await service.start_openai_server(config=config)
        self._server_configs[model.name] = (config, (host, port))
        server_args = (config or {}).get("server_args", {})
        api_key = server_args.get("api_key", None) or "default"
        shown = "127.0.0.1" if host in ("0.0.0.0", "") else host
        return f"http://{shown}:{port}/v1", api_key

    async def _log(self, model: Model, trajectory_groups: list[TrajectoryGroup], split: str = "val") -> None:
        parent = get_trajectories_split_dir(get_model_dir(model=model, art_path=self._path), split)
        os.makedirs(parent, exist_ok=True)
        step = get_model_step(model, self._path) if isinstance(model, TrainableModel) else 0
        with open(f"{parent}/{step:04d}.yaml", "w") as f:
            f.write(serialize_trajectory_groups(trajectory_groups))
        values: dict[str, list[float]] = {"reward": [], "exception_rate": []}
        for group in trajectory_groups:
            for t in group.trajectories:
                values["exception_rate"].append(0.0)
                values["reward"].append(t.reward)
                for k, v in t.metrics.items():
                    values.setdefault(k, []).append(float(v))
            values["exception_rate"].extend([1.0] * len(group.exceptions))
        averages = {k: sum(v) / len(v) for k, v in values.items() if v}
        averages["reward_std_dev"] = calculate_step_std_dev(trajectory_groups)
        self._log_metrics(model, averages, split)

    def _trajectory_log(self, trajectory: Trajectory) -> str:
        head = f"reward: {trajectory.reward} {' '.join(f'{k}: {v}' for k, v in trajectory.metrics.items())}\n\n"
        body = [format_message(m if isinstance(m, dict) else m.message.model_dump()) for m in trajectory.messages_and_choices]
        return head + "\n".join(body)

    async def _train_model(self, model: TrainableModel, trajectory_groups: list[TrajectoryGroup], config: TrainConfig,
                           dev_config: dev.TrainConfig, verbose: bool = False) -> AsyncIterator[dict[str, float]]:
        service = await self._get_service(model)
        await self._log(model, trajectory_groups, "train")
        packed = self._get_packed_tensors(model, trajectory_groups,
                                          allow_training_without_logprobs=dev_config.get("allow_training_without_logprobs", False),
                                          plot_tensors=False, seed=dev_config.get("packing_seed"))
        if packed is None:
            print("Skipping tuning as there is no suitable data. This can happen when all the trajectories in the same "
                  "group have the same reward and thus no advantage to train on.")
            return
        disk = packed_tensors_to_dir(packed, f"{get_model_dir(model=model, art_path=self._path)}/tensors")
        per = max(1, int(dev_config.get("rows_per_optimizer_step", 1)))
        num_gradient_steps = math.ceil(disk["num_sequences"] / per)
        results: list[dict[str, float]] = []
        bar = tqdm.tqdm(total=num_gradient_steps, desc="train")
        # Supervision: a service process that dies, or a gradient step that exceeds ``step_timeout_s`` (its process is
        # then killed), is replaced by a fresh process that resumes from the last complete checkpoint (adapter +
        # optimizer state), and the call is run again from its first row; ``max_service_restarts`` bounds the retries.
        from ..runtime.actors import ActorDiedError

        max_restarts = 0 if self._in_process else int(dev_config.get("max_service_restarts", 1))
        step_timeout = dev_config.get("step_timeout_s")
        attempt = 0
        try:
            while True:
                agen = service.train(disk, config, dev_config, verbose).__aiter__()
                try:
                    while True:
                        try:
                            result = await asyncio.wait_for(agen.__anext__(), step_timeout) if step_timeout else await agen.__anext__()
                        except StopAsyncIteration:
                            break
                        results.append(result)
                        yield {**result, "num_gradient_steps": num_gradient_steps}
                        bar.update(1)
                        bar.set_postfix(result)
                    break
                except Exception as e:  # noqa: BLE001 - filtered below
                    # a rank whose process is gone may surface as the peers' failed collective rather than as its own
                    # ActorDiedError; anything else (a bug in the step, bad data) is not a case for a restart
                    died = isinstance(e, (ActorDiedError, asyncio.TimeoutError)) or _has_dead_rank(service)
                    if not died or attempt >= max_restarts:
                        raise
                    attempt += 1
                    why = "exceeded step_timeout_s" if isinstance(e, asyncio.TimeoutError) else str(e)
                    print(f"model service of {model.name!r} {why}; restarting it from the last checkpoint "
                          f"(restart {attempt} of {max_restarts})")
                    service = await self._restart_service(model)
                    results.clear()
                    bar.reset()
        finally:
            bar.close()
        keys = {k for d in results for k in d}
        data = {k: sum(d.get(k, 0) for d in results) / sum(1 for d in results if k in d) for k in keys}
        self._log_metrics(model, data, "train", step_offset=-1)

    def _log_metrics(self, model: Model, metrics: dict[str, float], split: str, step_offset: int = 0) -> None:
        metrics = {f"{split}/{k}": v for k, v in metrics.items()} if split else dict(metrics)
        step = (get_model_step(model, self._path) if isinstance(model, TrainableModel) else 0) + step_offset
        out = get_model_dir(model=model, art_path=self._path)
        os.makedirs(out, exist_ok=True)
        with open(f"{out}/history.jsonl", "a") as f:
            # recorded_at lets the benchmark loaders plot metrics against wall-clock time
            f.write(json.dumps({"step": step, "recorded_at": datetime.now().isoformat(), **metrics}) + "\n")
        run = self._get_wandb_run(model)
        if run is not None:
            run.log(metrics, step=step)

    def _get_wandb_run(self, model: Model):
        if "WANDB_API_KEY" not in os.environ:
            return None
        run = self._wandb_runs.get(model.name)
        if run is None or getattr(run, "_is_finished", False):
            import wandb

            run = wandb.init(project=model.project, name=model.name, id=model.name, resume="allow")
            self._wandb_runs[model.name] = run
            try:   # tracing is optional: only when the package is installed
                import weave

                os.environ.setdefault("WEAVE_PRINT_CALL_LINK", "False")
                os.environ.setdefault("WEAVE_LOG_LEVEL", "CRITICAL")
                weave.init(model.project)
            except ImportError:
                pass
        return run

    async def _experimental_pull_from_s3(self, model: Model, step: int | None = None, s3_bucket: str | None = None,
                                         prefix: str | None = None, verbose: bool = False, delete: bool = False) -> None:
        await pull_model_from_s3(model_name=model.name, project=model.project, step=step, s3_bucket=s3_bucket,
                                 prefix=prefix, verbose=verbose, delete=delete, art_path=self._path)

    async def _experimental_push_to_s3(self, model: Model, s3_bucket: str | None = None, prefix: str | None = None,
                                       verbose: bool = False, delete: bool = False) -> None:
        await push_model_to_s3(model_name=model.name, project=model.project, s3_bucket=s3_bucket, prefix=prefix,
                               verbose=verbose, delete=delete, art_path=self._path)

    async def _experimental_deploy(self, deploy_to: LoRADeploymentProvider, model: TrainableModel, step: int | None = None,
                                   s3_bucket: str | None = None, prefix: str | None = None, verbose: bool = False,
                                   pull_s3: bool = True, wait_for_completion: bool = True) -> LoRADeploymentJob:
        return await deploy_model(deploy_to=deploy_to, model=model, step=step, s3_bucket=s3_bucket, prefix=prefix,
                                  verbose=verbose, pull_s3=pull_s3, wait_for_completion=wait_for_completion,
                                  art_path=self._path)


def _has_dead_rank(service) -> bool:
    """True when the service, or a rank of a multi-rank service, lives in a child process that has exited."""
    for r in getattr(service, "ranks", [service]):
        p = getattr(r, "_process", None)
        if p is not None and not p.is_alive():
            return True
    return False


class _Done:
    """Awaitable no-op so that ``await backend.close()`` also works."""

    def __await__(self):
        return iter(())
