#!/usr/bin/env python
"""Headline benchmark: GRPO LoRA training throughput on the Qwen2.5-7B architecture.

    python bench.py --gpus N --steps K --warmup W            (N == 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
           --master-port P bench.py --gpus N --steps K --warmup W

One "step" is one GRPO optimizer step over the per-GPU share of the batch the baseline
configuration names (32 groups x 8 rollouts of 2048 tokens over 8 GPUs = 32 packed rows of
2048 tokens per GPU, 512 shared-prompt tokens + 3 x 512... see ``synthetic_rows``), i.e.
forward, fused log-prob/GRPO loss, backward, LoRA-gradient all-reduce across the data-parallel
ranks, gradient clipping and AdamW.  On one GPU the model is whole; on N >= 2 GPUs the default
layout is the one that configuration names, tensor-parallel pairs x data parallel (TP2 x DP N/2:
fused all-gather->GEMM / GEMM->reduce-scatter inside a pair, fused LoRA-gradient all-reduce
across pairs); a pair shares its rows, so it gets the rows of two GPUs and the per-GPU work stays
the same at every N.  ``--parallel dp`` is plain data parallelism; with ``--extra-dp 1`` that
number is measured too and printed beside the headline as ``extra``.  Weights are random-initialised bf16 of the named
architecture and token ids are uniform random (no datasets or checkpoints are available).

Timing: ``W`` warm-up steps, then exactly ``K`` steps between CUDA events, bracketed by a
barrier and a device synchronise; the reported time is the maximum over ranks.  ``value`` is
tokens/s summed over all GPUs with the step inputs already resident on the device;
``e2e.value`` repeats the measurement through ``Trainer.train_packed`` with the packed
tensors in pinned host memory, so every step includes their host-to-device copy and the
device-to-host read of the step's loss and gradient norm.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "library"])
    ap.add_argument("--model", default="qwen2.5-7b")
    ap.add_argument("--rows-per-gpu", type=int, default=32)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--micro-tokens", type=int, default=16384)
    ap.add_argument("--lora-rank", type=int, default=8)
    ap.add_argument("--attn", default=None)
    ap.add_argument("--grad-sync", default="auto", choices=["auto", "nccl", "fused"])
    ap.add_argument("--parallel", default="auto", choices=["auto", "dp", "cp", "ep", "tp", "pp"],
                    help="auto: tp with --tp-size 2 on two or more GPUs (dense presets; ep for MoE presets); "
                         "dp: rows split over GPUs; cp: every row sharded over GPUs (long context); "
                         "ep: experts sharded over GPUs (MoE presets); tp: tensor-parallel groups of --tp-size "
                         "GPUs, data parallel across the groups; pp: layers split over the GPUs, 1F1B pipeline")
    ap.add_argument("--tp-size", type=int, default=2)
    ap.add_argument("--ep-capacity", default="2.0",
                    help="--parallel ep: receive capacity of an expert owner as a multiple of one rank's rows; "
                         "'dropless' sizes for the worst case (no row can be dropped; world/2 times the memory)")
    ap.add_argument("--rollout", type=int, default=1, help="also measure rollout decode tokens/s (reported beside the headline)")
    ap.add_argument("--rollout-new-tokens", type=int, default=1536,
                    help="sampled tokens per sequence in the rollout measurement (the configuration: up to 1536)")
    ap.add_argument("--e2e", default="service", choices=["service", "trainer"],
                    help="end-to-end number through the model service (default) or through Trainer.step on pinned rows")
    ap.add_argument("--extra-dp", type=int, default=0,
                    help="after a tensor-parallel run also measure plain data parallelism on the same GPUs (reported as `extra`)")
    return ap.parse_args()


def synthetic_rows(cfg, rows: int, S: int, seed: int):
    """Packed rows shaped like the baseline configuration: each 2048-token row holds one shared
    prompt of S/4 tokens followed by three sibling completions of S/4 tokens each (all trainable,
    prompt masked), uniform-random token ids, +-1 advantages, sampled-policy log-probs given."""
    import torch

    g = torch.Generator().manual_seed(seed)
    seg = S // 4
    tok = torch.randint(0, cfg.vocab_size, (rows, S), generator=g)
    gid = torch.empty(rows, S, dtype=torch.long)
    pid = torch.empty(rows, S, dtype=torch.long)
    pos = torch.empty(rows, S, dtype=torch.long)
    mask = torch.zeros(rows, S, dtype=torch.bool)
    adv = torch.zeros(rows, S)
    w = torch.zeros(rows, S)
    lp = torch.full((rows, S), float("nan"))
    nid = seed * 1_000_003
    for r in range(rows):
        p_id = nid
        nid += 1
        gid[r, :seg] = p_id
        pid[r, :] = p_id
        pos[r, :seg] = torch.arange(seg)
        for c in range(3):
            o = seg * (c + 1)
            gid[r, o:o + seg] = nid
            nid += 1
            pos[r, o:o + seg] = torch.arange(seg, 2 * seg)
            mask[r, o:o + seg] = True
            adv[r, o:o + seg] = 1.0 if (c + r) % 2 == 0 else -1.0
            w[r, o:o + seg] = 1.0
            lp[r, o:o + seg] = -11.0 - torch.rand(seg, generator=g)
    return dict(tokens=tok, group_ids=gid, parent_ids=pid, input_pos=pos, assistant_mask=mask, logprobs=lp,
                advantages=adv, weights=w)


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.2):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples: list[int] = []
        self.reasons: set[str] = set()
        self.max_mhz = 0
        self._stop_evt = threading.Event()

    def run(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {
                nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap",
                nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                nv.nvmlClocksThrottleReasonHwPowerBrakeSlowdown: "hw_power_brake_slowdown",
            }
            while not self._stop_evt.is_set():
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
                self._stop_evt.wait(self.period)
        except Exception as e:  # NVML unavailable: report that instead of clocks
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def stop(self) -> dict:
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz or None,
                "reasons": sorted(self.reasons), "samples": len(s)}


def nvml_index(local_rank: int) -> int:
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except (ValueError, IndexError):
            pass
    return local_rank


def main():
    args = parse_args()
    if args.impl == "reference":
        # The reference cannot be installed offline: its build backend (hatchling) and its pinned
        # runtime stack (unsloth, trl, peft, bitsandbytes, vllm 0.8.5) are absent from the wheelhouse.
        print(json.dumps({"impl": "reference", "unavailable":
                          "pip install of the reference fails offline: build backend hatchling and the pinned "
                          "unsloth/trl/peft/bitsandbytes/vllm==0.8.5.post1 stack are not in the image or wheelhouse"}))
        return 0

    import torch
    import torch.distributed as dist

    from art_b200.models.config import PRESETS
    from art_b200.models.weights import LoraConfig, init_base_weights, init_lora
    from art_b200.ops import _lib
    from art_b200.trainer.trainer import TrainHyper, Trainer

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(f"bench.py: --gpus {args.gpus} needs torch.distributed.run with that many ranks", file=sys.stderr)
            return 2
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    cfg = PRESETS[args.model]
    lcfg = LoraConfig(r=args.lora_rank, alpha=2.0 * args.lora_rank)
    impl = "native" if args.impl == "native" else "reference"
    attn_impl = args.attn or ("native" if impl == "native" else "sdpa")
    par = args.parallel if world > 1 else "dp"
    if par == "auto":
        par = "ep" if cfg.is_moe else "tp"
    S = args.seq_len

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def measure(par: str, steps: int, warmup: int, keep_base: bool):
        """Build the trainer for one layout, time it; returns a dict (and the base weights if ``keep_base``)."""
        base = init_base_weights(cfg, seed=0, dtype=torch.bfloat16, device=dev, scale_residual_out=cfg.is_moe)
        grad_sync = None
        sync_name = "none"
        R, micro = args.rows_per_gpu, args.micro_tokens
        ep = cp_group = tp_group = pp_group = None
        expert_range = None
        data_ranks, data_index = world, rank        # how many ranks hold different rows, and which share this one has
        label = f"{par}{world}"
        if world > 1 and par == "dp":
            from art_b200.parallel.dp import make_grad_sync

            grad_sync, sync_name = make_grad_sync(args.grad_sync, dev, world)
        elif par == "cp":
            cp_group, sync_name = dist.group.WORLD, "fused-p2p-allreduce(sum over cp)"
            data_ranks, data_index = 1, 0
        elif par == "pp":
            pp_group, sync_name = dist.group.WORLD, "fused-p2p-allreduce(sum over pp) + NCCL p2p activations"
            data_ranks, data_index = 1, 0
        elif par == "tp":
            T = args.tp_size
            if world % T:
                raise SystemExit("bench.py: --tp-size must divide the number of GPUs")
            from art_b200.parallel.mesh import ParallelLayout

            layout = ParallelLayout(world, tp=T)                # TP innermost: ranks (2i, 2i+1) share activations
            groups = layout.create_groups(rank)                 # every rank creates every group, in the same order
            tp_group, dp_group = groups["tp"], groups["dp"]
            data_index, data_ranks = layout.data_shard(rank)
            # a tensor-parallel group shares its rows: it takes the rows of all its GPUs (the micro-batch stays: its
            # tokens are split over the group, and the all-token activations of the local heads / columns grow with it)
            R = R * T
            label = f"tp{T}xdp{data_ranks}"
            sync_name = f"fused-p2p-allreduce(sum over tp{T})"
            if data_ranks > 1:
                from art_b200.parallel.symm_mem import FusedGradAllReduce

                grad_sync = FusedGradAllReduce(dev, data_ranks, dp_group, wait_ms=20000)
                sync_name += f" + fused-p2p-allreduce(mean over dp{data_ranks})"
        elif par == "ep":
            from art_b200.parallel.ep import ExpertParallel

            if not cfg.is_moe:
                raise SystemExit("bench.py: --parallel ep needs a mixture-of-experts preset (e.g. --model qwen3-30b-a3b)")
            ep = ExpertParallel(dev, None, micro, cfg.num_experts_per_tok, cfg.num_experts, cfg.hidden_size,
                                capacity_factor=None if args.ep_capacity == "dropless" else float(args.ep_capacity),
                                drop_overflow=args.ep_capacity != "dropless")
            El = cfg.num_experts // world
            expert_range, sync_name = (rank * El, (rank + 1) * El), "nccl-allreduce(shared factors) + 1/world(experts)"
            # this rank keeps only its experts' frozen weights
            base = {k: v for k, v in base.items()
                    if ".mlp.experts." not in k or expert_range[0] <= int(k.split(".experts.")[1].split(".")[0]) < expert_range[1]}
        lora = init_lora(cfg, lcfg, seed=3407, device=dev, expert_range=expert_range)
        trainer = Trainer(cfg, base, lcfg, lora, device=dev, impl=impl, attn_impl=attn_impl, grad_sync=grad_sync, ep=ep,
                          cp_group=cp_group, tp_group=tp_group, tp_tokens=micro, pp_group=pp_group)
        if not keep_base:
            base = None
        hyper = TrainHyper(learning_rate=1e-5, rows_per_optimizer_step=R, tokens_per_microbatch=micro)
        # cp: all ranks work on the SAME rows (each holds 1/world of every row); dp / ep: every rank has its own rows
        host_rows = {k: v.pin_memory() for k, v in synthetic_rows(cfg, R, S, seed=data_index + 1).items()}
        dev_rows = {k: v.to(dev) for k, v in host_rows.items()}
        tokens_per_step = R * S * data_ranks

        def timed(rows, n):
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            l0 = _lib.LAUNCHES
            e0.record()
            last = None
            for _ in range(n):
                last = trainer.step(rows, hyper)
            e1.record()
            barrier()
            ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            return float(ms.item()), _lib.LAUNCHES - l0, last

        for _ in range(warmup):
            trainer.step(dev_rows, hyper)
        if ep is not None:
            ep.dropped_rows()   # reset the counter: warm-up does not count
        sampler = ClockSampler(nvml_index(local_rank))
        sampler.start()
        ms, launches, last = timed(dev_rows, steps)
        clocks = sampler.stop()
        ep_drop = None
        if ep is not None:
            # share of dispatched (token, expert) rows that found their expert's owner over capacity, forward + backward
            n = torch.tensor([float(ep.dropped_rows())], device=dev)
            dist.all_reduce(n)
            sent = 2.0 * steps * tokens_per_step * cfg.num_experts_per_tok * cfg.num_layers
            ep_drop = round(float(n.item()) / sent, 6)
        trainer.step(host_rows, hyper)  # warm the host-input path
        ms_e2e, _, _ = timed(host_rows, steps)
        if os.environ.get("ARTB_PROFILE_STEP"):
            # one extra step between cudaProfilerStart/Stop for `ncu --profile-from-start off`
            torch.cuda.synchronize()
            torch.cuda.profiler.start()
            trainer.step(dev_rows, hyper)
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
        if os.environ.get("ARTB_PHASE_TIMING") == "1" and rank == 0:
            print("phases(ms):", json.dumps(trainer.phase_summary()), file=sys.stderr, flush=True)
        _lib.check_status(dev)
        if trainer.tp is not None:
            trainer.tp.close()
        del trainer
        torch.cuda.empty_cache()
        return {"label": label, "ms": ms, "ms_e2e": ms_e2e, "launches": launches, "last": last, "clocks": clocks,
                "tokens_per_step": tokens_per_step, "global_batch": R * data_ranks, "micro": micro, "sync": sync_name,
                "ep_drop": ep_drop, "h2d": sum(v.numel() * v.element_size() for v in host_rows.values()), "base": base}

    def measure_service(par: str, steps: int, warmup: int):
        """The same optimizer step through the product's service layer: packed rows on disk (the memory-mapped files the
        backend writes after tokenising and packing) -> ``ModelService.train`` on every rank, i.e. per step: pin and
        copy this rank's rows to the device, pause the engine, train, write the PEFT step checkpoint from a host copy
        of the adapter, hand the adapter to the rollout engine device to device, resume.  One ``train`` call = one
        optimizer step over ``rows_per_gpu`` rows per GPU.  Returns (ms per step, h2d bytes, d2h bytes) or raises."""
        import asyncio
        import shutil
        import tempfile

        from art_b200 import dev as artdev
        from art_b200 import types as arttypes
        from art_b200.local.pack import packed_tensors_to_dir
        from art_b200.local.service import ModelService

        T = args.tp_size if par == "tp" else 1
        D = world // T
        R = args.rows_per_gpu * T
        box = [tempfile.mkdtemp(prefix="artb_bench_") if rank == 0 else None]
        if world > 1:
            dist.broadcast_object_list(box, src=0)
        root = box[0]
        out = f"{root}/model"
        disk = {"dir": f"{root}/tensors", "num_sequences": D * R, "sequence_length": S}
        if rank == 0:
            parts = [synthetic_rows(cfg, R, S, seed=j + 1) for j in range(D)]
            disk = packed_tensors_to_dir({k: torch.cat([p[k] for p in parts]) for k in parts[0]}, disk["dir"])
        barrier()
        config = artdev.get_model_config(f"random:{cfg.name}", out, {
            "init_args": {"random_init": True},
            "peft_args": {"r": lcfg.r, "lora_alpha": lcfg.alpha},
            "engine_args": {"tensor_parallel_size": T, "data_parallel_size": D, "enable_sleep_mode": False,
                            "num_gpu_blocks_override": 4096, "max_model_len": 4096},
            "trainer_args": {"tokens_per_microbatch": args.micro_tokens}})
        svc = ModelService(host="127.0.0.1", port=0, model_name="bench", base_model=f"random:{cfg.name}", config=config,
                           output_dir=out, rank=rank, world=world, tp_size=T)
        try:
            st = svc.state            # every rank builds trainer + engine on the launcher's process group
            barrier()
            tcfg = arttypes.TrainConfig(learning_rate=1e-5)
            dcfg = {"rows_per_optimizer_step": R, "tokens_per_microbatch": args.micro_tokens}

            async def calls(n: int):
                last = None
                for _ in range(n):
                    async for met in svc.train(disk, tcfg, dcfg, False):
                        last = met
                return last

            asyncio.run(calls(warmup))
            barrier()
            t0 = time.perf_counter()
            asyncio.run(calls(steps))
            barrier()
            ms = torch.tensor([(time.perf_counter() - t0) * 1e3], device=dev)      # total of the timed calls
            if world > 1:
                dist.all_reduce(ms, op=dist.ReduceOp.MAX)
            per_tok = sum(torch.empty((), dtype=v.dtype).element_size() for v in synthetic_rows(cfg, 1, 8, seed=0).values())
            h2d = args.rows_per_gpu * T * S * per_tok
            d2h = 12 + (st.trainer.flat.numel * 4 if rank == 0 else 0)
            _lib.check_status(dev)
            return float(ms.item()), h2d, d2h
        finally:
            svc.close()
            torch.cuda.empty_cache()
            barrier()
            if rank == 0:
                shutil.rmtree(root, ignore_errors=True)

    want_rollout = bool(args.rollout and impl == "native" and not cfg.is_moe)
    m = measure(par, args.steps, args.warmup, keep_base=want_rollout)
    rollout_base = m.pop("base")
    extra = None
    if args.extra_dp and world > 1 and par == "tp":
        x = measure("dp", max(2, args.steps // 2), max(3, args.warmup // 2), keep_base=False)
        extra = {"parallelism": x["label"], "value": round(x["tokens_per_step"] * max(2, args.steps // 2) / (x["ms"] / 1e3), 1),
                 "unit": "tokens/s", "note": "plain data parallelism on the same GPUs, same per-GPU rows"}
    ms, ms_e2e, launches, last, clocks = m["ms"], m["ms_e2e"], m["launches"], m["last"], m["clocks"]
    tokens_per_step, sync_name, ep_drop, h2d = m["tokens_per_step"], m["sync"], m["ep_drop"], m["h2d"]
    e2e_api, d2h = "art_b200.trainer.Trainer.step on pinned host tensors", 12
    e2e_note = None
    if args.e2e == "service" and impl == "native" and par in ("dp", "tp") and not cfg.is_moe:
        try:
            ms_e2e, h2d, d2h = measure_service(par, args.steps, max(3, args.warmup))
            e2e_api = ("art_b200.local.service.ModelService.train (what LocalBackend.train drives) on packed rows on disk: "
                       "pin + H2D, engine pause, optimizer step, PEFT checkpoint, adapter hand-off; one call per step")
        except Exception as e:  # noqa: BLE001 - keep the trainer-level number, say why
            e2e_note = f"service path failed ({type(e).__name__}: {e}); value is Trainer.step on pinned host tensors"
            if world > 1:      # a rank that failed alone would leave the others in a collective
                raise

    rollout = None
    if rollout_base is not None:
        # rollout half of the headline metric: decode tokens/s of the inference engine on the same weights
        # (one engine replica per GPU, 256 sequences over 4 LoRA adapters), outside the timed training region
        try:
            from art_b200.engine.bench_decode import measure_decode

            rollout = measure_decode(cfg, dev, base=rollout_base, new_tokens=args.rollout_new_tokens)
            del rollout_base
            agg = torch.tensor([rollout["decode_tok_s"]], device=dev)
            if world > 1:
                dist.all_reduce(agg)
            rollout["decode_tok_s_all_gpus"] = round(float(agg.item()), 1)
        except Exception as e:  # the training number stands on its own
            rollout = {"error": f"{type(e).__name__}: {e}"}
            if world > 1:
                dist.all_reduce(torch.zeros(1, device=dev))

    # frozen weights resident per GPU (W and W^T of the layer stack, bf16), for the note on L2
    shard = args.tp_size if m["label"].startswith("tp") else (world if par in ("pp", "ep") else 1)
    emb = cfg.vocab_size * cfg.hidden_size * (1 if cfg.tie_word_embeddings else 2)
    weight_gb = 2 * 2 * (cfg.num_params() - emb) / shard / 1e9
    value = tokens_per_step * args.steps / (ms / 1e3)
    e2e = tokens_per_step * args.steps / (ms_e2e / 1e3)      # ms_e2e: total of the timed steps
    if rank == 0:
        out = {
            "metric": ("GRPO train tokens/s, Qwen2.5-7B-arch LoRA" if cfg.name == "qwen2.5-7b"
                       else f"GRPO train tokens/s, {cfg.name}-arch LoRA"),
            "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 2), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None,     # the reference publishes no throughput for this model / hardware
            "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
            "impl": args.impl,
            "config": {"model": cfg.name, "global_batch": m["global_batch"], "seq_len": S, "parallelism": m["label"],
                       "lora_rank": lcfg.r, "tokens_per_step": tokens_per_step, "micro_tokens": m["micro"],
                       "attention": attn_impl, "grad_sync": sync_name, "optimizer_steps_per_step": 1,
                       **({"ep_capacity_factor": args.ep_capacity, "ep_dropped_row_share": ep_drop} if ep_drop is not None else {}),
                       "l2": f"inputs larger than L2: each step streams the bf16 weights (W and W^T, "
                             f"{weight_gb:.0f} GB on this GPU for {cfg.name}) plus activations"},
            "clocks": clocks,
            "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": e2e_api, **({"note": e2e_note} if e2e_note else {})},
            "gpu_launches": launches,
            "loss": last["loss"] if last else None,
            "rollout": rollout,
        }
        if extra is not None:
            out["extra"] = extra
        print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
