import asyncio
import os

import pytest

from art_b200.utils import format_message, iterate_dataset, limit_concurrency, retry
from art_b200.utils.get_model_step import get_step_from_dir
from art_b200.utils.trajectory_logging import deserialize_trajectory_groups, serialize_trajectory_groups


def test_retry_sync_and_async():
    calls = []

    @retry(max_attempts=3, delay=0.0, on_retry=lambda e, n: calls.append(n))
    def flaky():
        if len(calls) < 2:
            raise ValueError("x")
        return 7

    assert flaky() == 7 and calls == [1, 2]

    @retry(max_attempts=2, delay=0.0, exceptions=(KeyError,))
    async def always():
        raise KeyError("k")

    with pytest.raises(KeyError):
        asyncio.run(always())


def test_iterate_dataset_is_deterministic_and_resumable():
    data = list(range(10))
    full = list(iterate_dataset(data, groups_per_step=3, num_epochs=2, use_tqdm=False))
    assert len(full) == 8 and full[0][1:] == (0, 0, 0) and full[4][1:] == (1, 4, 0)
    assert sorted(sum((b for b, e, *_ in full if e == 0), [])) == data
    resumed = list(iterate_dataset(data, groups_per_step=3, num_epochs=2, initial_step=5, use_tqdm=False))
    assert [r[0] for r in resumed] == [f[0] for f in full[5:]]


def test_limit_concurrency():
    live = peak = 0

    @limit_concurrency(2)
    async def work():
        nonlocal live, peak
        live += 1
        peak = max(peak, live)
        await asyncio.sleep(0.005)
        live -= 1

    async def main():
        await asyncio.gather(*[work() for _ in range(6)])

    asyncio.run(main())
    assert peak == 2


def test_format_message_and_step_dir(tmp_path):
    m = {"role": "assistant", "content": "hi", "tool_calls": [{"function": {"name": "f", "arguments": "{}"}}]}
    assert format_message(m) == "Assistant:\nhi\nf({})"
    assert get_step_from_dir(str(tmp_path)) == 0
    os.makedirs(tmp_path / "0003")
    os.makedirs(tmp_path / "notes")
    assert get_step_from_dir(str(tmp_path)) == 3


def test_trajectory_yaml_round_trip():
    from tests.test_api_trajectories import traj
    import art_b200 as art

    groups = [art.TrajectoryGroup([traj(0.5, metrics={"a": 1}), traj(1.0)], metadata={"scenario": "s"})]
    text = serialize_trajectory_groups(groups)
    assert "logprobs" not in text
    back = deserialize_trajectory_groups(text)
    assert back[0].metadata == {"scenario": "s"} and [t.reward for t in back[0]] == [0.5, 1.0]
    assert back[0].trajectories[0].messages()[1]["content"] == "abc"


def test_s3_paths_and_sync_commands(monkeypatch):
    from art_b200.utils import s3

    assert s3.build_s3_path(model_name="m", project="p", step=3, s3_bucket="b", prefix="/x/") == "s3://b/x/p/models/m/0003"
    assert s3.build_s3_zipped_step_path(model_name="m", project="p", step=3, s3_bucket="b").endswith("zipped-steps/0003.zip")
    seen = []

    async def fake_run(cmd, **kw):
        seen.append(cmd)
        return (1 if "head-bucket" in cmd else 0), "https://signed", ""

    monkeypatch.setattr(s3, "_run", fake_run)
    asyncio.run(s3.ensure_bucket_exists("b"))
    assert seen[1][-3:] == ["create-bucket", "--bucket", "b"]
    asyncio.run(s3.s3_sync("/tmp", "s3://b/x", delete=True))
    assert seen[-1][:4] == ["aws", "s3", "sync", "--delete"]


def test_deploy_model_reuses_running_job(monkeypatch, tmp_path):
    import art_b200 as art
    from art_b200.utils import deploy_model as dm

    model = art.TrainableModel(name="m", project="p", base_model="Qwen/Qwen2.5-14B-Instruct")
    calls = []

    async def fake_request(method, url, body=None):
        calls.append((method, url))
        if url.endswith("/jobs"):
            return {"data": [{"job_id": "j1", "updated_at": 1, "args": {"modelName": "acct/p-m-2"}}]}
        if "/jobs/" in url:
            return {"status": "Complete", "status_updates": [{"message": "ok"}], "args": {"modelName": "acct/p-m-2"}}
        raise AssertionError("should not upload again")

    async def fake_presign(**kw):
        return "https://signed"

    monkeypatch.setattr(dm, "_request", fake_request)
    monkeypatch.setattr(dm, "archive_and_presign_step_url", fake_presign)
    job = asyncio.run(dm.deploy_model(dm.LoRADeploymentProvider.TOGETHER, model, step=2, pull_s3=False, art_path=str(tmp_path)))
    assert job.status == dm.LoRADeploymentJobStatus.COMPLETE and job.job_id == "j1"
    assert dm.convert_together_job_status("Retry Queued") == dm.LoRADeploymentJobStatus.QUEUED


def test_phase_timer_and_chrome_trace(tmp_path):
    import json
    import time

    from art_b200.utils.profiling import ChromeTrace, PhaseTimer, nvtx_range

    t = PhaseTimer("cpu")
    with t.phase("a"):
        time.sleep(0.01)
    with t.phase("a"):
        time.sleep(0.01)
    with t.phase("b"), nvtx_range("inner"):
        pass
    rec = t.dump_jsonl(str(tmp_path / "phases.jsonl"), extra={"step": 3})
    assert rec["step"] == 3 and rec["phases_ms"]["a"] >= 15 and "b" in rec["phases_ms"]
    assert t.summary() == {}                                   # reset after the dump
    off = PhaseTimer("cpu", enabled=False)
    with off.phase("x"):
        pass
    assert off.summary() == {}
    tr = ChromeTrace("test")
    with tr.span("engine.step", running=2):
        tr.counter("sequences", running=2, waiting=1)
    tr.instant("preempt", seq=7)
    tr.save(str(tmp_path / "trace.json"))
    ev = json.load(open(tmp_path / "trace.json"))["traceEvents"]
    assert {e["ph"] for e in ev} == {"M", "X", "C", "i"} and any(e.get("dur", 0) >= 0 and e["name"] == "engine.step" for e in ev)


def test_truncated_adapter_checkpoint_fails_cleanly(tmp_path):
    """A checkpoint cut short by a crash must raise on load (and never be mistaken for a usable adapter)."""
    import pytest
    import torch

    from art_b200.models import peft_io
    from art_b200.models.config import PRESETS
    from art_b200.models.weights import LoraConfig, init_lora

    cfg, lcfg = PRESETS["tiny"], LoraConfig()
    lora = init_lora(cfg, lcfg)
    d = tmp_path / "0001"
    peft_io.save_adapter(str(d), lora, lcfg, "tiny")
    back, lcfg_back = peft_io.load_adapter(str(d))
    assert lcfg_back.r == lcfg.r and set(back) == set(lora) and all(torch.equal(back[k], lora[k]) for k in lora)
    f = d / "adapter_model.safetensors"
    raw = f.read_bytes()
    f.write_bytes(raw[: len(raw) // 2])
    with pytest.raises(Exception):
        peft_io.load_adapter(str(d))


def test_small_m_gemm_plan_fills_one_wave_only():
    """The split-K planner never asks for more work items than the GPU has CTAs (or CTA pairs): a second,
    nearly empty wave would double the time of a weight-streaming GEMM."""
    from art_b200.ops.gemm import plan_small_m

    for M in (8, 64, 128, 256, 512):
        for N in (64, 128, 576, 3648, 4736, 18944, 37888, 152064):
            for K in (64, 1024, 3584, 18944):
                bn, splits = plan_small_m(M, N, K)
                tiles = ((M + 127) // 128) * ((N + bn - 1) // bn)
                assert splits >= 1 and (splits == 1 or tiles * splits <= 148), (M, N, K, bn, splits)
                assert splits <= max(1, ((K + 63) // 64) // 4) or splits == 1
                if M % 256 == 0 and N >= 256:
                    bn2, sp2 = plan_small_m(M, N, K, pair=True)
                    units = (M // 256) * ((N + 255) // 256)
                    assert bn2 == 256 and (sp2 == 1 or units * sp2 <= 74), (M, N, K, sp2)


def test_deploy_model_command_pulls_then_deploys(tmp_path, monkeypatch):
    """``deploy-model``: with ``--step latest`` every checkpoint is pulled and the newest local step is deployed; with a
    number only that step is pulled; a failed job raises."""
    import asyncio

    from art_b200.utils import deploy_cli
    from art_b200.utils.deploy_model import LoRADeploymentJob, LoRADeploymentJobStatus

    calls = []

    async def fake_pull(**kw):
        calls.append(("pull", kw.get("step")))
        d = tmp_path / kw["project"] / "models" / kw["model_name"]
        for s in ((3, 7) if kw.get("step") is None else (kw["step"],)):
            (d / f"{s:04d}").mkdir(parents=True, exist_ok=True)

    async def fake_deploy(**kw):
        calls.append(("deploy", kw["step"], kw["pull_s3"], kw["deploy_to"]))
        ok = kw["step"] != 5
        return LoRADeploymentJob(status=LoRADeploymentJobStatus.COMPLETE if ok else LoRADeploymentJobStatus.FAILED,
                                 job_id="job-1", model_name="acct/agent-001", failure_reason=None if ok else "quota")

    monkeypatch.setenv("BACKUP_BUCKET", "bucket")
    base = ["--project", "p", "--model", "agent-001", "--base-model", "random:tiny", "--art-path", str(tmp_path)]
    job = asyncio.run(deploy_cli.deploy(deploy_cli.parse_args(base), pull=fake_pull, deploy_fn=fake_deploy))
    assert job.model_name == "acct/agent-001" and calls == [("pull", None), ("deploy", 7, False, "together")]
    calls.clear()
    asyncio.run(deploy_cli.deploy(deploy_cli.parse_args(base + ["--step", "3"]), pull=fake_pull, deploy_fn=fake_deploy))
    assert calls == [("pull", 3), ("deploy", 3, False, "together")]
    with pytest.raises(RuntimeError, match="quota"):
        asyncio.run(deploy_cli.deploy(deploy_cli.parse_args(base + ["--step", "5"]), pull=fake_pull, deploy_fn=fake_deploy))
    monkeypatch.delenv("BACKUP_BUCKET")
    with pytest.raises(SystemExit):
        asyncio.run(deploy_cli.deploy(deploy_cli.parse_args(base), pull=fake_pull, deploy_fn=fake_deploy))


def test_adapter_writer_fast_path_matches_the_generic_writer(tmp_path):
    """Views that lie back to back in the trainer's flat buffer are written as header + one buffer; the file loads to the
    same tensors as the generic writer's, and any other layout falls back to the generic writer."""
    import torch
    from safetensors.torch import load_file

    from art_b200.models import peft_io
    from art_b200.models.config import PRESETS
    from art_b200.models.native import LoraFlat
    from art_b200.models.weights import LoraConfig, init_lora

    cfg, lcfg = PRESETS["tiny"], LoraConfig()
    lora = init_lora(cfg, lcfg, seed=0)
    g = torch.Generator().manual_seed(0)
    lora = {k: torch.randn(v.shape, generator=g) for k, v in lora.items()}
    flat = LoraFlat(cfg, lcfg, lora, "cpu")
    views = dict(flat.views)
    assert peft_io._write_consecutive_views(str(tmp_path / "probe.safetensors"), views, torch.float32)
    assert not peft_io._write_consecutive_views(str(tmp_path / "probe2.safetensors"), lora, torch.float32)       # separate tensors
    assert not peft_io._write_consecutive_views(str(tmp_path / "probe3.safetensors"), views, torch.bfloat16)     # needs a cast
    peft_io.save_adapter(str(tmp_path / "fast"), views, lcfg, "random:tiny")
    peft_io.save_adapter(str(tmp_path / "generic"), lora, lcfg, "random:tiny")
    a = load_file(str(tmp_path / "fast" / "adapter_model.safetensors"))
    b = load_file(str(tmp_path / "generic" / "adapter_model.safetensors"))
    assert a.keys() == b.keys() and all(torch.equal(a[k], b[k]) for k in a)
    st, got_cfg = peft_io.load_adapter(str(tmp_path / "fast"))
    assert got_cfg.r == lcfg.r and all(torch.equal(st[k], lora[k]) for k in lora)
