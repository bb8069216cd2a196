"""SkyPilot backend and helpers against a fake ``sky`` module (the real package is optional and needs a cloud)."""
import asyncio
import types

import pytest

from art_b200.skypilot import utils as su
from art_b200.skypilot.backend import SERVER_COMMAND, SkyPilotBackend
from art_b200.skypilot.stop_server import stop_server


class FakeResources:
    def __init__(self, accelerators=None, ports=None):
        self.accelerators, self.ports = accelerators, list(ports or [])

    def copy(self, **kw):
        r = FakeResources(self.accelerators, self.ports)
        for k, v in kw.items():
            setattr(r, k, v)
        return r


class FakeTask:
    def __init__(self, name=None, run=None, setup=None):
        self.name, self.run, self.setup, self.envs, self.resources, self.workdir = name, run, setup, {}, None, None

    def update_envs(self, envs):
        self.envs.update(envs)

    def set_resources(self, r):
        self.resources = r


def fake_sky(cluster_up=False, jobs=None, start_after=0):
    """``start_after``: the server task reports SETTING_UP for that many queue polls before RUNNING."""
    sky = types.SimpleNamespace()
    sky.calls = []
    sky.jobs = list(jobs or [])
    sky.cluster_up = cluster_up
    sky.polls = 0
    sky.Resources, sky.Task = FakeResources, FakeTask
    sky.ClusterStatus = types.SimpleNamespace(UP="UP", STOPPED="STOPPED")
    sky.JobStatus = types.SimpleNamespace(RUNNING="RUNNING", PENDING="PENDING", SETTING_UP="SETTING_UP", INIT="INIT",
                                          FAILED="FAILED", CANCELLED="CANCELLED")

    def status(cluster_names=None):
        return [{"name": cluster_names[0], "status": "UP"}] if sky.cluster_up else []

    def launch(task, cluster_name=None, retry_until_up=False):
        sky.calls.append(("launch", cluster_name, task.setup, task.resources.ports))
        sky.cluster_up = True

    def queue(cluster_name):
        sky.polls += 1
        out = []
        for j in sky.jobs:
            j = dict(j)
            if j["job_name"] == su.SERVER_TASK and j["status"] == "SETTING_UP" and sky.polls > start_after:
                j["status"] = "RUNNING"
            out.append(j)
        return out

    def exec_(task=None, cluster_name=None, detach_run=False):
        sky.calls.append(("exec", cluster_name, task.run, dict(task.envs)))
        sky.jobs.insert(0, {"job_name": task.name, "status": "SETTING_UP"})

    def cancel(cluster_name=None, all=False):
        sky.calls.append(("cancel", cluster_name, all))
        sky.jobs = []

    def endpoints(cluster, port):
        return {port: f"10.0.0.5:{30000 + port}"}

    def down(cluster_name=None):
        sky.calls.append(("down", cluster_name))
        sky.cluster_up = False

    sky.status, sky.launch, sky.queue, sky.cancel, sky.endpoints, sky.down = status, launch, queue, cancel, endpoints, down
    setattr(sky, "exec", exec_)
    return sky


def test_task_status_helpers_and_start_wait():
    sky = fake_sky(cluster_up=True, jobs=[{"job_name": "art_server", "status": "SETTING_UP"}], start_after=3)

    async def main():
        assert await su.get_task_status("c", "nope", sky) is None
        assert not await su.is_task_created("c", "nope", sky)
        assert await su.is_task_created("c", "art_server", sky)
        await su.wait_for_task_to_start("c", "art_server", sky, attempts=10, interval=0)
        assert su._state_name(await su.get_task_status("c", "art_server", sky)) == "RUNNING"
        with pytest.raises(ValueError, match="not found"):
            await su.wait_for_task_to_start("c", "other", sky, attempts=2, interval=0)
        assert await su.get_art_server_base_url("c", sky) == "http://10.0.0.5:37999"
        assert await su.get_vllm_base_url("c", sky) == "http://10.0.0.5:38000/v1"

    asyncio.run(main())
    # a task that never leaves SETTING_UP times out; one that failed is reported as such
    slow = fake_sky(cluster_up=True, jobs=[{"job_name": "art_server", "status": "SETTING_UP"}], start_after=10 ** 6)
    with pytest.raises(ValueError, match="failed to start"):
        asyncio.run(su.wait_for_task_to_start("c", "art_server", slow, attempts=3, interval=0))
    dead = fake_sky(cluster_up=True, jobs=[{"job_name": "art_server", "status": "FAILED"}])
    with pytest.raises(ValueError, match="FAILED"):
        asyncio.run(su.wait_for_task_to_start("c", "art_server", dead, attempts=3, interval=0))


def test_health_wait_retries_then_gives_up():
    answers = iter([ConnectionError("boot"), 503, 200])

    async def get(url):
        a = next(answers)
        if isinstance(a, Exception):
            raise a
        return a

    asyncio.run(su.wait_for_healthcheck("http://x", attempts=5, interval=0, get=get))

    async def never(url):
        return 500

    with pytest.raises(TimeoutError):
        asyncio.run(su.wait_for_healthcheck("http://x", attempts=3, interval=0, get=never))


def test_backend_launches_cluster_runs_server_and_points_at_it(tmp_path):
    env = tmp_path / ".env"
    env.write_text("WANDB_API_KEY=abc\n# comment\nEMPTY=\n")
    sky = fake_sky(cluster_up=False, start_after=2)

    async def healthy(url):
        return 200

    async def main():
        b = await SkyPilotBackend.initialize_cluster(cluster_name="c1", gpu="B200", env_path=str(env), sky_module=sky,
                                                     health_get=healthy)
        assert b._base_url == "http://10.0.0.5:37999"
        kinds = [c[0] for c in sky.calls]
        assert kinds == ["launch", "exec"]
        assert sky.calls[0][3] == ["7999", "8000"]                      # both service ports opened
        assert sky.calls[1][2] == SERVER_COMMAND and sky.calls[1][3]["WANDB_API_KEY"] == "abc"
        # a second initialisation re-uses the running server
        b2 = await SkyPilotBackend.initialize_cluster(cluster_name="c1", gpu="B200", sky_module=sky, health_get=healthy)
        assert [c[0] for c in sky.calls] == ["launch", "exec"] and b2._base_url == b._base_url
        # force_restart cancels and starts it again
        await SkyPilotBackend.initialize_cluster(cluster_name="c1", gpu="B200", sky_module=sky, health_get=healthy,
                                                 force_restart=True)
        assert [c[0] for c in sky.calls] == ["launch", "exec", "cancel", "exec"]
        await b.down()
        assert sky.calls[-1] == ("down", "c1")

    asyncio.run(main())
    with pytest.raises(ValueError, match="gpu or resources"):
        asyncio.run(SkyPilotBackend.initialize_cluster(cluster_name="c", sky_module=sky))


def test_stop_server_checks_cluster_and_task_then_cancels():
    sky = fake_sky(cluster_up=False)
    with pytest.raises(ValueError, match="is not running"):
        asyncio.run(stop_server("c", sky, close_backend=False))
    sky = fake_sky(cluster_up=True)
    with pytest.raises(ValueError, match="task"):
        asyncio.run(stop_server("c", sky, close_backend=False))
    sky = fake_sky(cluster_up=True, jobs=[{"job_name": "art_server", "status": "RUNNING"}])
    asyncio.run(stop_server("c", sky, close_backend=False))
    assert sky.calls == [("cancel", "c", True)]
