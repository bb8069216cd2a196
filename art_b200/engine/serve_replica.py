"""OpenAI-compatible completion server over a tensor-parallel engine replica.

Launch one process per GPU of the replica:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        -m art_b200.engine.serve_replica --model qwen2.5-32b [--weights /path/to/hf_dir] --port 8000

Rank 0 runs the HTTP server on a :class:`~art_b200.engine.replica.ReplicaEngine`; the other ranks mirror
it (``follow()``).  Collectives of the model run over NCCL, the control traffic of the replica over a
gloo group of the same ranks.  ``--reference`` swaps in the PyTorch reference runner on CPU (gloo only),
which is how the control path is tested without GPUs.  Adapters: ``--lora name=/path/to/adapter_dir``
(PEFT layout), repeatable.

The reference reaches this through ``vllm serve --tensor-parallel-size`` (src/art/vllm/server.py).
"""
from __future__ import annotations

import argparse
import asyncio
import os

import torch
import torch.distributed as dist


def build_replica(args):
    from ..local.tokenizer import load_tokenizer
    from ..models.config import PRESETS, ModelConfig
    from ..models.weights import LoraConfig, init_base_weights, load_base_weights
    from .kv_cache import BlockManager, KVCache
    from .replica import ReplicaEngine

    rank, world = dist.get_rank(), dist.get_world_size()
    if args.weights:
        cfg = ModelConfig.from_hf_dict(__import__("json").load(open(os.path.join(args.weights, "config.json"))),
                                       name=args.model)
    else:
        cfg = PRESETS[args.model]
    lcfg = LoraConfig()
    ctrl = dist.new_group(list(range(world)), backend="gloo")
    bs = args.block_size
    if args.reference:
        from .runner import ReferenceRunner

        dev = torch.device("cpu")
        base = (load_base_weights(args.weights, cfg, dtype=torch.float32, device=dev) if args.weights
                else init_base_weights(cfg, seed=args.seed))
        runner, kv = ReferenceRunner(cfg, base, lcfg, max_loras=args.max_loras), None
    else:
        from .runner import NativeRunner

        dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
        base = (load_base_weights(args.weights, cfg, device=dev) if args.weights
                else init_base_weights(cfg, seed=args.seed, dtype=torch.bfloat16, device=dev))
        kv = KVCache(cfg.num_layers, args.num_blocks, bs, cfg.num_kv_heads // world, cfg.head_dim, dev)
        runner = NativeRunner(cfg, lcfg, kv, base=base, max_loras=args.max_loras, device=dev,
                              tp_group=dist.group.WORLD if world > 1 else None)
        del base
        torch.cuda.empty_cache()
    tok = load_tokenizer(args.tokenizer or args.weights or f"byte-chat:{args.model}", cfg.vocab_size)
    eng = ReplicaEngine(runner, BlockManager(args.num_blocks, bs, True), ctrl_group=ctrl,
                        eos_token_id=getattr(tok, "eos_token_id", None), max_num_seqs=args.max_num_seqs,
                        max_num_batched_tokens=args.max_num_batched_tokens, num_scheduler_steps=args.num_scheduler_steps,
                        max_model_len=args.max_model_len, max_loras=args.max_loras, kv_cache=kv)
    return eng, tok, dev


async def _lead(eng, tok, args, dev) -> None:
    from ..models.peft_io import load_adapter
    from .server import OpenAIServer, serve

    for spec in args.lora or []:
        name, path = spec.split("=", 1)
        state, _ = load_adapter(path, dev)
        eng.set_adapter(name, state)
    eng.start()
    srv = OpenAIServer(eng, tok, args.served_model_name or args.model, api_key=args.api_key)
    try:
        await serve(srv, args.host, args.port)
    finally:
        eng.shutdown()


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--model", default="qwen2.5-7b", help="architecture preset (or a name for --weights)")
    ap.add_argument("--weights", default=None, help="Hugging Face directory with config.json and *.safetensors")
    ap.add_argument("--tokenizer", default=None)
    ap.add_argument("--served-model-name", default=None)
    ap.add_argument("--lora", action="append", help="name=adapter_dir, repeatable")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=8000)
    ap.add_argument("--api-key", default="default")
    ap.add_argument("--num-blocks", type=int, default=16384)
    ap.add_argument("--block-size", type=int, default=16)
    ap.add_argument("--max-loras", type=int, default=4)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-num-batched-tokens", type=int, default=16384)
    ap.add_argument("--num-scheduler-steps", type=int, default=16)
    ap.add_argument("--max-model-len", type=int, default=32768)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--reference", action="store_true", help="PyTorch reference runner on CPU (control-path testing)")
    args = ap.parse_args(argv)
    if args.reference:
        dist.init_process_group("gloo")
    else:
        local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    eng, tok, dev = build_replica(args)
    try:
        if eng.is_leader:
            try:
                asyncio.run(_lead(eng, tok, args, dev))
            except KeyboardInterrupt:
                pass
        else:
            eng.follow()
    finally:
        close = getattr(eng.runner, "close", None)
        if close is not None:
            close()                      # captured graphs go before the communicator does
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
