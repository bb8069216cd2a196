"""Small helpers of the public surface that the larger tests do not reach."""
import asyncio
import os

import httpx
import pandas as pd
import pytest

import art_b200 as art
from art_b200.errors import (ForbiddenBucketCreationError, LoRADeploymentTimedOutError,
                             UnsupportedBaseModelDeploymentError, UnsupportedLoRADeploymentProviderError)
from art_b200.local.checkpoints import get_last_checkpoint_dir
from art_b200.utils.benchmark_rollout import benchmark_rollout
from art_b200.utils.benchmarking.filter_model_split import filter_rename_model_split
from art_b200.utils.benchmarking.types import BenchmarkModelKey
from art_b200.utils.get_repo_root_path import get_repo_root_path
from art_b200.utils.get_trajectory_messages import get_trajectory_messages
from art_b200.utils.litellm import convert_litellm_choice_to_openai
from art_b200.utils.log_http_errors import log_http_errors
from art_b200.utils.old_benchmarking.calculate_step_metrics import calculate_step_std_dev
from tests.test_api_trajectories import make_choice


def test_litellm_choice_keeps_tool_calls_and_logprobs():
    raw = {"index": 1, "finish_reason": "tool_calls",
           "message": {"content": None, "tool_calls": [{"id": "c1", "function": {"name": "f", "arguments": '{"x": 1}'}}]},
           "logprobs": {"content": [{"token": "token_id:5", "logprob": -0.25, "bytes": [53]}]}}
    ch = convert_litellm_choice_to_openai(raw)
    assert ch.index == 1 and ch.finish_reason == "tool_calls"
    assert ch.message.tool_calls[0].function.name == "f" and ch.message.tool_calls[0].function.arguments == '{"x": 1}'
    assert ch.logprobs.content[0].token == "token_id:5" and ch.logprobs.content[0].logprob == -0.25

    class Obj:                      # attribute-style objects work as well as dictionaries
        index, finish_reason, logprobs = 0, None, None
        message = type("M", (), {"content": "hi", "tool_calls": None})()

    ch = convert_litellm_choice_to_openai(Obj())
    assert ch.message.content == "hi" and ch.finish_reason == "stop" and ch.logprobs is None
    art.Trajectory(messages_and_choices=[{"role": "user", "content": "q"}, ch], reward=1.0)       # usable as a choice


def test_log_http_errors_shows_the_servers_detail():
    req = httpx.Request("POST", "http://h/x")

    @log_http_errors
    async def with_detail():
        raise httpx.HTTPStatusError("boom", request=req, response=httpx.Response(422, json={"detail": "bad rows"}, request=req))

    @log_http_errors
    async def without_json():
        raise httpx.HTTPStatusError("boom", request=req, response=httpx.Response(500, text="<html>", request=req))

    with pytest.raises(Exception, match=r"\[HTTP 422\] http://h/x bad rows"):
        asyncio.run(with_detail())
    with pytest.raises(httpx.HTTPStatusError):
        asyncio.run(without_json())


def test_benchmark_rollout_averages_rewards_and_tolerates_failures():
    async def rollout(model: str, i: int, is_training: bool) -> art.Trajectory:
        assert model == "m" and not is_training
        if i == 2:
            raise RuntimeError("rollout failed")
        return art.Trajectory(messages_and_choices=[{"role": "user", "content": "q"}, make_choice(content="a")], reward=float(i))

    assert asyncio.run(benchmark_rollout("m", 4, rollout)) == pytest.approx((0 + 1 + 3) / 3)


def test_trajectory_messages_and_step_spread():
    t = art.Trajectory(messages_and_choices=[{"role": "user", "content": "q"}, make_choice(content="a")], reward=1.0)
    assert get_trajectory_messages(t) == [{"role": "user", "content": "q"}, {"role": "assistant", "content": "a"}]

    def group(rewards):
        return art.TrajectoryGroup([art.Trajectory(messages_and_choices=[{"role": "user", "content": "q"}, make_choice(content="a")],
                                                   reward=r) for r in rewards])

    # population standard deviation per group, averaged; a single-trajectory group does not count
    assert calculate_step_std_dev([group([0.0, 1.0]), group([1.0, 1.0, 1.0]), group([5.0])]) == pytest.approx(0.25)
    assert calculate_step_std_dev([]) == 0.0


def test_filter_rename_model_split():
    df = pd.DataFrame({"model": ["a", "a", "b", "c"], "split": ["val", "train", "val", "val"], "reward": [1, 2, 3, 4]})
    out = filter_rename_model_split(df, [BenchmarkModelKey("a", "Model A", "val"), BenchmarkModelKey("b")])
    assert out["model"].tolist() == ["Model A", "b"] and out["reward"].tolist() == [1, 3]
    assert filter_rename_model_split(df, BenchmarkModelKey("a", split="train"))["reward"].tolist() == [2]
    assert filter_rename_model_split(df, []).empty and df["model"].tolist() == ["a", "a", "b", "c"]       # input untouched


def test_error_types_carry_their_http_status():
    for cls, code in ((ForbiddenBucketCreationError, 403), (UnsupportedLoRADeploymentProviderError, 400),
                      (UnsupportedBaseModelDeploymentError, 400), (LoRADeploymentTimedOutError, 504)):
        e = cls("why")
        assert e.status_code == code and e.detail == "why"


def test_repo_root_and_last_checkpoint_dir(tmp_path):
    (tmp_path / ".git").mkdir()
    deep = tmp_path / "a" / "b"
    deep.mkdir(parents=True)
    assert get_repo_root_path(str(deep)) == str(tmp_path)
    out = tmp_path / "model"
    assert get_last_checkpoint_dir(str(out)) is None
    for name in ("0000", "0003", "0010", "logs", "0011.tmp"):
        (out / name).mkdir(parents=True)
    assert os.path.basename(get_last_checkpoint_dir(str(out))) == "0010"


def test_settings_without_effect_are_named(caplog):
    import logging

    from art_b200 import dev

    with caplog.at_level(logging.WARNING):
        msgs = dev.model.warn_ignored({"peft_args": {"lora_dropout": 0.1, "bias": "none", "target_modules": ["q_proj", "embed_tokens"]},
                                       "init_args": {"full_finetuning": True}})
    assert len(msgs) == 3 and any("lora_dropout" in m for m in msgs) and any("embed_tokens" in m for m in msgs)
    assert dev.model.warn_ignored(dev.model.get_model_config("x", "/nonexistent/dir", None)) == []      # the defaults are clean
    used, ignored = dev.engine.split_engine_args({"max_model_len": 512, "ray_workers_use_nsight": True})
    assert used == {"max_model_len": 512} and ignored == {"ray_workers_use_nsight": True}


def test_model_service_refuses_layouts_it_does_not_run():
    from art_b200.local.service import node_layout

    assert node_layout({"engine_args": {"tensor_parallel_size": 2, "data_parallel_size": 4}}) == (2, 4)
    assert node_layout({}) == (1, 1)
    assert node_layout({"engine_args": {"context_parallel_size": 4, "data_parallel_size": 2}}) == (4, 2)
    assert node_layout({"trainer_args": {"context_parallel_size": 2}}) == (2, 1)
    assert node_layout({"engine_args": {"pipeline_parallel_size": 2}}) == (2, 1)
    from art_b200.local.service import group_layout
    assert group_layout({"engine_args": {"pipeline_parallel_size": 4}}) == ("pp", 4) and group_layout({}) == ("tp", 1)
    with pytest.raises(ValueError, match="do not compose"):
        node_layout({"engine_args": {"context_parallel_size": 2, "tensor_parallel_size": 2}})
    with pytest.raises(ValueError, match="expert_parallel_size"):
        node_layout({"engine_args": {"expert_parallel_size": 2}})


def test_metrics_go_to_history_and_to_wandb_when_a_key_is_set(tmp_path, monkeypatch):
    """``history.jsonl`` is always written; with ``WANDB_API_KEY`` the same numbers go to a run named after the model
    (a fake ``wandb`` module stands in: there is no network here)."""
    import json
    import sys
    import types

    from art_b200.local import LocalBackend

    calls = {"init": [], "log": []}
    fake = types.ModuleType("wandb")

    class Run:
        _is_finished = False

        def log(self, metrics, step=None):
            calls["log"].append((dict(metrics), step))

    def init(**kw):
        calls["init"].append(kw)
        return Run()

    fake.init = init
    monkeypatch.setitem(sys.modules, "wandb", fake)
    monkeypatch.setitem(sys.modules, "weave", None)          # "not installed": tracing is optional
    model = art.Model(name="prompted", project="proj")
    backend = LocalBackend(in_process=True, path=str(tmp_path))
    monkeypatch.delenv("WANDB_API_KEY", raising=False)
    backend._log_metrics(model, {"reward": 0.25}, "val")
    assert calls["init"] == []
    monkeypatch.setenv("WANDB_API_KEY", "k")
    backend._log_metrics(model, {"reward": 0.5, "exception_rate": 0.0}, "val")
    backend._log_metrics(model, {"reward": 0.75}, "val")
    assert calls["init"] == [{"project": "proj", "name": "prompted", "id": "prompted", "resume": "allow"}]       # one run, reused
    assert calls["log"] == [({"val/reward": 0.5, "val/exception_rate": 0.0}, 0), ({"val/reward": 0.75}, 0)]
    rows = [json.loads(l) for l in open(tmp_path / "proj" / "models" / "prompted" / "history.jsonl")]
    assert [r["val/reward"] for r in rows] == [0.25, 0.5, 0.75] and all("recorded_at" in r for r in rows)


def test_flat_adamw_on_cpu_equals_torch_adamw_with_gradient_clipping():
    import torch

    from art_b200.ops.optim import FlatAdamW

    g = torch.Generator().manual_seed(0)
    p0 = torch.randn(1000, generator=g)
    params, grads = p0.clone(), torch.zeros(1000)
    opt = FlatAdamW(params, grads, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1, max_grad_norm=0.1)
    ref_p = torch.nn.Parameter(p0.clone())
    ref = torch.optim.AdamW([ref_p], lr=1e-3, betas=(0.9, 0.99), eps=1e-8, weight_decay=0.1)
    for step in range(5):
        gr = torch.randn(1000, generator=g) * (0.001 if step == 2 else 1.0)      # one step below the clipping threshold
        grads.copy_(gr)
        ref_p.grad = gr.clone()
        want_norm = torch.nn.utils.clip_grad_norm_([ref_p], 0.1)
        ref.step()
        got_norm = opt.step(1e-3)
        assert float(got_norm) == pytest.approx(float(want_norm), rel=1e-5)
        torch.testing.assert_close(params, ref_p.detach(), rtol=1e-5, atol=1e-7)
