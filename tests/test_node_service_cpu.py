"""A model over several ranks of one machine (``local/node.py``) on CPU: two gloo ranks, data parallel.

Rank 0 lives in the test process, rank 1 in a spawned child.  Checked: both replicas serve requests sent to the one
public port, a training call runs one optimizer step across the ranks and yields the same adapter as a single rank
that sees all rows, every replica serves the new adapter afterwards, and the shard helper pads with weightless rows."""
import asyncio
import os

import httpx
import pytest
import torch

import art_b200 as art
from art_b200 import dev
from art_b200.local.node import NodeService, build_node_service
from art_b200.local.pack import packed_tensors_to_dir
from art_b200.local.service import node_layout, shard_rows
from art_b200.trainer.trainer import PACKED_KEYS

ARCH = dict(name="tiny", vocab_size=1024, hidden_size=128, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=32,
            intermediate_size=384)


def _packed(R, S, seed=1):
    g = torch.Generator().manual_seed(seed)
    seg = S // 4
    tok = torch.randint(0, 1024, (R, S), generator=g)
    gid = torch.empty(R, S, dtype=torch.long)
    pid = torch.empty(R, S, dtype=torch.long)
    pos = torch.empty(R, S, dtype=torch.long)
    mask = torch.zeros(R, S, dtype=torch.bool)
    adv, w = torch.zeros(R, S), torch.zeros(R, S)
    lp = torch.full((R, S), float("nan"))
    for r in range(R):
        p = 100 * r
        gid[r, :seg] = p
        pid[r] = p
        pos[r, :seg] = torch.arange(seg)
        for c in range(3):
            o = seg * (c + 1)
            gid[r, o:o + seg] = p + c + 1
            pos[r, o:o + seg] = torch.arange(seg, 2 * seg)
            mask[r, o:o + seg] = True
            adv[r, o:o + seg] = 1.0 if (c + r) % 2 == 0 else -1.0
            w[r, o:o + seg] = 1.0
            lp[r, o:o + seg] = -6.5 - torch.rand(seg, generator=g)
    return dict(tokens=tok, group_ids=gid, parent_ids=pid, input_pos=pos, assistant_mask=mask, logprobs=lp, advantages=adv,
                weights=w)


def _config(out, dp):
    return dev.get_model_config("random:tiny", out, {"init_args": {"architecture": ARCH, "max_seq_length": 1024},
                                                     "engine_args": {"num_scheduler_steps": 2, "max_model_len": 256,
                                                                     "data_parallel_size": dp}})


def test_layout_and_row_sharding():
    assert node_layout({}) == (1, 1)
    assert node_layout({"engine_args": {"tensor_parallel_size": 2, "data_parallel_size": 4}}) == (2, 4)
    p = _packed(3, 16)
    full = shard_rows(p, PACKED_KEYS, 0, 2, 3)
    assert torch.equal(full["tokens"], p["tokens"][:2])
    tail = shard_rows(p, PACKED_KEYS, 2, 2, 3)                # one real row, one weightless filler
    assert torch.equal(tail["tokens"][0], p["tokens"][2]) and tail["weights"][1].abs().sum() == 0
    assert not tail["assistant_mask"][1].any() and p["weights"][0].abs().sum() > 0     # the source is untouched
    empty = shard_rows(p, PACKED_KEYS, 4, 2, 3)
    assert empty["tokens"].shape == (2, 16) and empty["weights"].abs().sum() == 0


def test_two_rank_node_serves_and_trains_like_one_rank(tmp_path):
    from safetensors.torch import load_file

    packed = _packed(2, 64)

    async def run(dp: int, out: str, rows_per_step: int):
        disk = packed_tensors_to_dir(packed, f"{out}/tensors")
        port = 18200 + 10 * dp + (os.getpid() % 50) * 20
        svc = build_node_service(model_name="m", base_model="random:tiny", config=_config(out, dp), output_dir=out,
                                 port=port, in_process=True)
        assert isinstance(svc, NodeService) == (dp > 1)
        seen = {}
        try:
            host, p0 = await svc.start_openai_server(None)
            assert p0 == port
            async with httpx.AsyncClient(headers={"Authorization": "Bearer default"}, timeout=60) as c:
                async def ask(seed):
                    r = await c.post(f"http://127.0.0.1:{port}/v1/chat/completions",
                                     json={"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 4,
                                           "seed": seed, "temperature": 1.0})
                    assert r.status_code == 200, r.text
                    return [e["logprob"] for e in r.json()["choices"][0]["logprobs"]["content"]]

                before = await asyncio.gather(*[ask(s) for s in range(6)])
                if dp > 1:       # the public port spread the six requests over both replicas
                    m1 = (await c.get(f"http://127.0.0.1:{port + 1}/metrics")).json()
                    m0 = (await c.get(f"http://127.0.0.1:{port}/metrics")).json()
                    assert m1["generated_tokens"] >= 8 and m0["generated_tokens"] >= 8
                    assert m0["replica_load"] == [0, 0]
                    streamed = []
                    async with c.stream("POST", f"http://127.0.0.1:{port}/v1/chat/completions",
                                        json={"model": "m", "messages": [{"role": "user", "content": "hi"}], "max_tokens": 3,
                                              "stream": True}) as r:
                        async for line in r.aiter_lines():
                            if line.startswith("data: "):
                                streamed.append(line)
                    assert streamed[-1] == "data: [DONE]" and len(streamed) >= 4
                steps = [m async for m in svc.train(disk, art.TrainConfig(learning_rate=1e-2),
                                                    {"rows_per_optimizer_step": rows_per_step})]
                assert len(steps) == 1 and steps[0]["grad_norm"] > 0
                seen["loss"] = steps[0]["loss"]
                after = await asyncio.gather(*[ask(s) for s in range(6)])
                assert all(a != b for a, b in zip(after, before))            # every replica serves the new adapter
        finally:
            await svc.shutdown()
        seen["adapter"] = load_file(f"{out}/0001/adapter_model.safetensors")
        return seen

    one = asyncio.run(run(1, str(tmp_path / "one"), 2))
    two = asyncio.run(run(2, str(tmp_path / "two"), 1))
    assert abs(one["loss"] - two["loss"]) < 1e-5 * max(1.0, abs(one["loss"]))
    for k, v in one["adapter"].items():
        assert torch.allclose(v, two["adapter"][k], atol=1e-6), k
    assert not torch.distributed.is_initialized()
