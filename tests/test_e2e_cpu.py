"""End-to-end on CPU with the tiny model: register -> rollouts over HTTP -> train -> new adapter
is served; PEFT checkpoint layout; resume; remote Backend <-> CLI app round trip."""
import asyncio
import json
import os

import httpx
import pytest
import torch

import art_b200 as art
from art_b200.local import LocalBackend

ARCH = dict(name="tiny", vocab_size=1024, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
            intermediate_size=384)


def make_model(name="agent-001"):
    return art.TrainableModel(name=name, project="proj", base_model="random:tiny",
                              _internal_config={"init_args": {"architecture": ARCH, "max_seq_length": 2048},
                                                "engine_args": {"num_scheduler_steps": 4, "max_model_len": 512}})


async def rollout(model, prompt: str, i: int) -> art.Trajectory:
    client = model.openai_client()
    messages = [{"role": "user", "content": prompt}]
    resp = await client.chat.completions.create(model=model.get_inference_name(), messages=messages, max_tokens=6, seed=i)
    choice = resp.choices[0]
    return art.Trajectory(messages_and_choices=[*messages, choice], reward=float(i % 2))


def test_full_loop(tmp_path):
    async def main():
        backend = LocalBackend(in_process=True, path=str(tmp_path))
        model = make_model()
        try:
            await model.register(backend)
            assert await model.get_step() == 0
            out = tmp_path / "proj" / "models" / "agent-001"
            assert (out / "0000" / "adapter_model.safetensors").exists() and (out / "model.json").exists()
            groups = await art.gather_trajectory_groups(
                (art.TrajectoryGroup(rollout(model, f"q{g}", i) for i in range(4)) for g in range(2)), pbar_desc=None)
            assert all(len(g) == 4 for g in groups)
            ch = groups[0].trajectories[0].messages_and_choices[-1]
            assert ch.logprobs.content[0].token.startswith("token_id:")
            await model.log(groups, split="val")
            before = await rollout(model, "q0", 0)
            await model.train(groups, config=art.TrainConfig(learning_rate=1e-2), _config={"rows_per_optimizer_step": 1})
            assert await model.get_step() == 1
            service = backend._services["agent-001"]
            await service.flush_checkpoints()
            cfg = json.load(open(out / "0001" / "adapter_config.json"))
            assert cfg["peft_type"] == "LORA" and cfg["r"] == 8 and "q_proj" in cfg["target_modules"]
            from safetensors.torch import load_file
            sd = load_file(str(out / "0001" / "adapter_model.safetensors"))
            k = "base_model.model.model.layers.0.self_attn.q_proj.lora_B.weight"
            assert sd[k].shape == (128, 8) and sd[k].abs().sum() > 0
            assert (out / "0001" / "trainer_state.pt").exists()
            hist = [json.loads(l) for l in open(out / "history.jsonl")]
            assert any("train/loss" in h for h in hist) and any("val/reward" in h for h in hist)
            assert (out / "trajectories" / "train" / "0000.yaml").exists()
            # the engine now serves the trained adapter: same seed, different log-probs
            after = await rollout(model, "q0", 0)
            lp0 = [t.logprob for t in before.messages_and_choices[-1].logprobs.content]
            lp1 = [t.logprob for t in after.messages_and_choices[-1].logprobs.content]
            assert lp0 != lp1
            # base model is still served untouched under its own name
            r = await model.openai_client().chat.completions.create(model="random:tiny", messages=[{"role": "user", "content": "q0"}], max_tokens=2)
            assert len(r.choices[0].logprobs.content) == 2
            assert (out / "logs" / "engine.log").exists()           # engine and listener write their log here
            await model.delete_checkpoints()      # val/reward was logged at step 0: best (0) and latest (1) are kept
            assert sorted(d for d in os.listdir(out) if d.isdigit()) == ["0000", "0001"]
            await model.delete_checkpoints(best_checkpoint_metric="val/none")   # unknown metric: only the latest stays
            assert sorted(d for d in os.listdir(out) if d.isdigit()) == ["0001"]
        finally:
            await model.openai_client().close()
            for s in backend._services.values():
                await s.shutdown()
            backend.close()

    asyncio.run(main())


def test_resume_from_checkpoint(tmp_path):
    from art_b200.local.service import ModelState
    from art_b200.models.peft_io import save_adapter
    from art_b200.models.weights import LoraConfig, init_lora
    from art_b200.models.config import ModelConfig

    cfg = ModelConfig(**ARCH)
    lora = init_lora(cfg, LoraConfig())
    for k in lora:
        if "lora_B" in k:
            lora[k] = torch.full_like(lora[k], 0.25)
    out = tmp_path / "m"
    save_adapter(str(out / "0003"), lora, LoraConfig(), "random:tiny")
    st = ModelState("random:tiny", art.dev.get_model_config("random:tiny", str(out), {"init_args": {"architecture": ARCH}}), str(out))
    k = "base_model.model.model.layers.1.mlp.down_proj.lora_B.weight"
    assert torch.allclose(st.trainer.flat.views[k], torch.full_like(st.trainer.flat.views[k], 0.25))


def test_remote_backend_round_trip(tmp_path):
    from art_b200.backend import Backend
    from art_b200.cli import build_app

    class FakeBackend:
        def __init__(self):
            self.calls = []

        async def register(self, model):
            self.calls.append(("register", type(model).__name__, model._internal_config if hasattr(model, "_internal_config") else None))

        async def _get_step(self, model):
            return 7

        async def _prepare_backend_for_training(self, model, config):
            return "http://127.0.0.1:8000/v1", "default"

        async def _log(self, model, groups, split):
            self.calls.append(("log", len(groups), split))

        async def _train_model(self, model, groups, config, dev_config, verbose):
            for i in range(3):
                yield {"loss": 1.0 / (i + 1), "num_gradient_steps": 3}

        async def _delete_checkpoints(self, model, benchmark, smoothing):
            self.calls.append(("delete", benchmark, smoothing))

        def close(self):
            self.calls.append(("close",))

    fake = FakeBackend()
    remote = Backend(base_url="http://art")
    remote._client = httpx.AsyncClient(transport=httpx.ASGITransport(app=build_app(fake)), base_url="http://art")

    async def main():
        model = make_model()
        await model.register(remote)
        assert model.inference_base_url.endswith("/v1") and model.inference_model_name == "agent-001"
        assert fake.calls[0][:2] == ("register", "TrainableModel") and fake.calls[0][2]["init_args"]["architecture"]["hidden_size"] == 128
        assert await model.get_step() == 7
        from tests.test_api_trajectories import traj
        groups = [art.TrajectoryGroup([traj(1.0), traj(0.0)])]
        await model.log(groups)
        seen = [m async for m in remote._train_model(model, groups, art.TrainConfig(), {}, False)]
        assert len(seen) == 3 and seen[0]["loss"] == 1.0
        await model.delete_checkpoints()
        await remote.close()
        assert ("log", 1, "val") in fake.calls and ("delete", "val/reward", 1.0) in fake.calls and ("close",) in fake.calls

    asyncio.run(main())


def test_service_process_is_restarted_from_the_last_checkpoint(tmp_path):
    """Supervision: the model service runs in a child process; it is killed between two train calls (a failure made on
    the host) and the second call restarts it from the newest checkpoint, on the same inference address."""
    async def main():
        backend = LocalBackend(in_process=False, path=str(tmp_path))
        model = make_model("agent-sup")
        try:
            await model.register(backend)
            groups = await art.gather_trajectory_groups(
                (art.TrajectoryGroup(rollout(model, f"q{g}", i) for i in range(4)) for g in range(2)), pbar_desc=None)
            await model.train(groups, config=art.TrainConfig(learning_rate=1e-2), _config={"rows_per_optimizer_step": 1})
            assert await model.get_step() == 1
            svc = backend._services["agent-sup"]
            await svc.flush_checkpoints()
            svc._process.kill()
            svc._process.join(10)
            await model.train(groups, config=art.TrainConfig(learning_rate=1e-2), _config={"rows_per_optimizer_step": 1})
            assert backend.service_restarts == {"agent-sup": 1}
            assert await model.get_step() == 2
            out = tmp_path / "proj" / "models" / "agent-sup"
            await backend._services["agent-sup"].flush_checkpoints()
            assert (out / "0002" / "adapter_model.safetensors").exists()
            # the restarted process serves on the address the client already holds
            t = await rollout(model, "q0", 3)
            assert len(t.messages_and_choices[-1].logprobs.content) == 6
            # watchdog: a gradient step that exceeds its time limit ends the call (no restart budget here)
            with pytest.raises(asyncio.TimeoutError):
                await model.train(groups, config=art.TrainConfig(learning_rate=1e-2),
                                  _config={"rows_per_optimizer_step": 1, "step_timeout_s": 1e-4, "max_service_restarts": 0})
            # no restart budget: the failure surfaces
            backend._services["agent-sup"]._process.kill()
            backend._services["agent-sup"]._process.join(10)
            from art_b200.runtime.actors import ActorDiedError
            with pytest.raises(ActorDiedError):
                await model.train(groups, config=art.TrainConfig(learning_rate=1e-2),
                                  _config={"rows_per_optimizer_step": 1, "max_service_restarts": 0})
        finally:
            await model.openai_client().close()
            backend.close()

    asyncio.run(main())


def test_two_rank_service_recovers_from_a_dead_worker(tmp_path):
    """A model over two data-parallel ranks (gloo, CPU), each in its own process: one worker is killed between two
    train calls (a host-made failure); the failure is seen at once, every rank is replaced, and training goes on from
    the last checkpoint."""
    async def main():
        backend = LocalBackend(in_process=False, path=str(tmp_path))
        model = art.TrainableModel(name="agent-dp", project="proj", base_model="random:tiny",
                                   _internal_config={"init_args": {"architecture": ARCH, "max_seq_length": 2048},
                                                     "engine_args": {"num_scheduler_steps": 4, "max_model_len": 512,
                                                                     "data_parallel_size": 2}})
        try:
            await model.register(backend)
            groups = await art.gather_trajectory_groups(
                (art.TrajectoryGroup(rollout(model, f"q{g}", i) for i in range(4)) for g in range(2)), pbar_desc=None)
            await model.train(groups, config=art.TrainConfig(learning_rate=1e-2), _config={"rows_per_optimizer_step": 2})
            assert await model.get_step() == 1
            svc = backend._services["agent-dp"]
            await svc.flush_checkpoints()
            worker = svc.workers[0]
            worker._process.kill()
            worker._process.join(10)
            import time
            t0 = time.monotonic()
            await model.train(groups, config=art.TrainConfig(learning_rate=1e-2), _config={"rows_per_optimizer_step": 2})
            assert backend.service_restarts == {"agent-dp": 1} and await model.get_step() == 2
            assert time.monotonic() - t0 < 120          # noticed through the dead process, not through a collective's time limit
            t = await rollout(model, "q0", 3)
            assert len(t.messages_and_choices[-1].logprobs.content) == 6
        finally:
            await model.openai_client().close()
            backend.close()

    asyncio.run(main())
