"""Kernel micro-benchmarks: ``python -m art_b200.ops.microbench gemm --m 8192 --n 3584 --k 3584``.

Times one op with CUDA events on the launching stream after warm-up (inputs larger than L2 by
default, or pass ``--flush`` to write a 256 MB buffer between iterations) and prints one JSON line
with the achieved TFLOP/s or GB/s next to the library baseline.  The same entry point is what the
profiler is pointed at when a single kernel is captured (``--iters 1 --warmup 1 --no-baseline``).
"""
from __future__ import annotations

import argparse
import json

import torch


def _time(fn, iters: int, warmup: int, flush: torch.Tensor | None) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    return total / iters


def bench_gemm(a) -> dict:
    from . import _lib
    from .gemm import gemm_tn

    dev = "cuda"
    x = torch.randn(a.m, a.k, device=dev).bfloat16()
    w = (torch.randn(a.n, a.k, device=dev) * 0.02).bfloat16()
    out = torch.empty(a.m, 2 * a.n if a.epilogue == "swiglu_bwd" else a.n, device=dev, dtype=torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush else None
    two = None if a.two_cta < 0 else bool(a.two_cta)
    kw = {}
    if a.epilogue == "resid":
        kw["residual"] = torch.randn(a.m, a.n, device=dev).bfloat16()
    elif a.epilogue == "swiglu":
        kw["swiglu_out"] = torch.empty(a.m, a.n // 2, device=dev, dtype=torch.bfloat16)
    elif a.epilogue == "swiglu_bwd":
        kw["swiglu_bwd_gu"] = torch.randn(a.m, 2 * a.n, device=dev).bfloat16()
    ms = _time(lambda: gemm_tn(x, w, out=out, bn=a.bn, two_cta=two, **kw), a.iters, a.warmup, flush)
    _lib.check_status()
    fl = 2.0 * a.m * a.n * a.k
    res = {"op": "gemm_tn", "m": a.m, "n": a.n, "k": a.k, "bn": a.bn, "two_cta": a.two_cta, "epilogue": a.epilogue, "ms": round(ms, 4),
           "tflops": round(fl / ms / 1e9, 1)}
    if not a.no_baseline:
        ms_b = _time(lambda: torch.matmul(x, w.t(), out=out), a.iters, a.warmup, flush)
        res["cublas_ms"] = round(ms_b, 4)
        res["cublas_tflops"] = round(fl / ms_b / 1e9, 1)
    return res


def _sustained(fn, seconds: float = 0.6, warm: int = 5, agree=None) -> float:
    """Milliseconds per call with the calls issued back to back (no host sync, no flush) for about ``seconds``: the
    rate a kernel holds inside a long training step, under the power cap.  ``agree`` (int -> int) makes several ranks
    settle on ONE repetition count: a call that contains a collective must run equally often everywhere."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    fn()
    e1.record()
    torch.cuda.synchronize()
    reps = max(10, int(seconds * 1e3 / max(1e-3, e0.elapsed_time(e1))))
    if agree is not None:
        reps = agree(reps)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def bench_gemm_layer(a) -> dict:
    """The eight projection / data-gradient GEMMs of one decoder layer at ``--tokens`` rows, each with the epilogue and
    the LoRA extra-K block the trainer uses, sustained (back to back), next to cuBLAS on the plain product."""
    from ..models.config import PRESETS
    from . import _lib
    from .gemm import gemm_tn

    cfg = PRESETS[a.model]
    dev, bf = "cuda", torch.bfloat16
    M, d, q, kv, F = a.tokens, cfg.hidden_size, cfg.q_size, cfg.kv_size, cfg.intermediate_size
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, sc=1.0: (torch.randn(*s, device=dev, generator=g) * sc).to(bf)      # noqa: E731
    # name, N, K, epilogue
    shapes = [("qkv", q + 2 * kv, d, "bias" if cfg.qkv_bias else "plain"), ("o", d, q, "resid"), ("gate_up", 2 * F, d, "swiglu"),
              ("down", d, F, "resid"), ("d_down", F, d, "swiglu_bwd"), ("d_gate_up", d, 2 * F, "plain"), ("d_o", q, d, "plain"),
              ("d_qkv", d, q + 2 * kv, "plain")]
    rows, tot_ms, tot_lib, tot_fl = [], 0.0, 0.0, 0.0
    for name, N, K, epi in shapes:
        x, w = rnd(M, K), rnd(N, K, sc=0.02)
        t, b2 = rnd(M, 64, sc=0.1), rnd(N, 64, sc=0.02)
        kw: dict = {"a2": t, "b2": b2}
        if epi == "resid":
            kw["residual"] = rnd(M, N)
        elif epi == "bias":
            kw["bias"] = torch.randn(N, device=dev, generator=g)
        elif epi == "swiglu":
            kw["swiglu_out"] = torch.empty(M, N // 2, device=dev, dtype=bf)
        elif epi == "swiglu_bwd":
            kw["swiglu_bwd_gu"] = rnd(M, 2 * N)
        out = torch.empty(M, 2 * N if epi == "swiglu_bwd" else N, device=dev, dtype=bf)
        plain = torch.empty(M, N, device=dev, dtype=bf)
        fl = 2.0 * M * N * K
        row = {"gemm": name, "n": N, "k": K, "epilogue": epi}
        ms = _sustained(lambda: gemm_tn(x, w, out=out, **kw), a.seconds)
        row["ms"], row["tflops"] = round(ms, 4), round(fl / ms / 1e9, 1)
        if a.ablate:      # what the LoRA extra-K block and the epilogue cost: the same product without them
            ms_p = _sustained(lambda: gemm_tn(x, w, out=plain), a.seconds)
            row["plain_tflops"] = round(fl / ms_p / 1e9, 1)
            ms_e = _sustained(lambda: gemm_tn(x, w, out=out, **{k: v for k, v in kw.items() if k not in ("a2", "b2")}), a.seconds)
            row["no_lora_tflops"] = round(fl / ms_e / 1e9, 1)
        if a.try_bn:
            for bn in a.try_bn:
                try:
                    ms_b = _sustained(lambda: gemm_tn(x, w, out=out, bn=bn, two_cta=True, **kw), a.seconds)
                    row[f"bn{bn}_tflops"] = round(fl / ms_b / 1e9, 1)
                except Exception as e:  # noqa: BLE001 - a tile width this epilogue does not support
                    row[f"bn{bn}_tflops"] = f"{type(e).__name__}"
        if not a.no_baseline:
            ms_l = _sustained(lambda: torch.matmul(x, w.t(), out=plain), a.seconds)
            row["cublas_tflops"] = round(fl / ms_l / 1e9, 1)
            tot_lib += ms_l
        tot_ms += ms
        tot_fl += fl
        rows.append(row)
        del x, w, out, plain, kw
    _lib.check_status()
    res = {"op": "gemm_layer", "model": cfg.name, "tokens": M, "layer_ms": round(tot_ms, 3),
           "layer_tflops": round(tot_fl / tot_ms / 1e9, 1), "gemms": rows}
    if tot_lib:
        res["cublas_layer_ms"] = round(tot_lib, 3)
        res["cublas_layer_tflops"] = round(tot_fl / tot_lib / 1e9, 1)
    return res


def bench_tp_layer(a) -> dict:
    """The eight fused tensor-parallel GEMMs of one decoder layer (run under torchrun, one rank per GPU): all-gather->GEMM
    for the column-parallel products, GEMM->reduce-scatter for the row-parallel ones, each sustained, next to (a) the
    same product as a plain local GEMM without communication (the compute floor of this kernel family), (b) the bare
    library pair NCCL collective + cuBLAS (no LoRA term, no element-wise work) and (c) library calls that compute what the
    fused kernel computes (both gathers, LoRA as ``addmm_``, SwiGLU forward / backward as eager tensor ops, residual
    add).  Times are the maximum over ranks."""
    import os

    import torch.distributed as dist

    from ..models.config import PRESETS
    from ..parallel.tp import TPContext, unfused_ag_gemm, unfused_gemm_rs
    from . import _lib
    from .gemm import gemm_tn

    rank, local = int(os.environ["RANK"]), int(os.environ.get("LOCAL_RANK", os.environ["RANK"]))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    import datetime

    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=60))
    P = dist.get_world_size()
    cfg = PRESETS[a.model]
    bf = torch.bfloat16
    M, d, q, kv, F = a.tokens, cfg.hidden_size, cfg.q_size // P, cfg.kv_size // P, cfg.intermediate_size // P
    m_seg = M // P
    g = torch.Generator(device=dev).manual_seed(rank)
    rnd = lambda *s, sc=1.0: (torch.randn(*s, device=dev, generator=g) * sc).to(bf)      # noqa: E731
    ctx = TPContext(dev, None, m_seg, k_max=d, n_max=d, kt=64)

    def mx(ms: float) -> float:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    def agree(reps: int) -> int:
        t = torch.tensor([reps], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        return int(t)

    def sustained(fn):
        dist.barrier()
        return mx(_sustained(fn, a.seconds, agree=agree))

    rows = []
    # all-gather -> GEMM: gathered K = d; name, local N, epilogue
    for name, N, epi in (("qkv", q + 2 * kv, "plain"), ("gate_up", 2 * F, "swiglu"), ("d_down", F, "swiglu_bwd"), ("d_o", q, "plain")):
        x_shard, w, b2 = rnd(m_seg, d), rnd(N, d, sc=0.02), rnd(N, 64, sc=0.02)
        t_shard = rnd(m_seg, 64, sc=0.1)
        kw = {}
        if epi == "swiglu":
            kw["swiglu_out"] = torch.empty(M, N // 2, device=dev, dtype=bf)
        elif epi == "swiglu_bwd":
            kw["swiglu_bwd_gu"] = rnd(M, 2 * N)
        out = torch.empty(M, 2 * N if epi == "swiglu_bwd" else N, device=dev, dtype=bf)

        def fused():
            ctx.ag_input(d).copy_(x_shard)
            ctx.ag_t_input().copy_(t_shard)
            ctx.ag_gemm(d, w, b2=b2, out=out, **kw)

        x_full, t_full = rnd(M, d), rnd(M, 64, sc=0.1)
        fl = 2.0 * M * N * d
        ms_f = sustained(fused)
        ms_l = sustained(lambda: gemm_tn(x_full, w, a2=t_full, b2=b2, out=out, **kw))
        ms_u = sustained(lambda: unfused_ag_gemm(x_shard, w))

        def library_same_math():
            # what the fused kernel computes, from library calls: both gathers, the LoRA term, the element-wise pass
            y = unfused_ag_gemm(x_shard, w)
            t_all = torch.empty(M, 64, device=dev, dtype=bf)
            dist.all_gather_into_tensor(t_all, t_shard)
            y.addmm_(t_all, b2.t())
            if epi == "swiglu":
                return torch.nn.functional.silu(y[:, : N // 2]) * y[:, N // 2:]
            if epi == "swiglu_bwd":
                gu = kw["swiglu_bwd_gu"]
                g, u = gu[:, :N], gu[:, N:]
                sg = torch.sigmoid(g)
                return torch.cat([y * u * sg * (1 + g * (1 - sg)), y * g * sg], dim=1)
            return y

        ms_s = sustained(library_same_math)
        rows.append({"op": "ag_gemm", "gemm": name, "n": N, "k": d, "epilogue": epi, "fused_ms": round(ms_f, 4),
                     "fused_tflops": round(fl / ms_f / 1e9, 1), "local_gemm_ms": round(ms_l, 4), "nccl_cublas_ms": round(ms_u, 4),
                     "library_same_math_ms": round(ms_s, 4),
                     "nvlink_mb_in": round((P - 1) * m_seg * (d + 64) * 2 / 1e6, 1)})
        del x_shard, w, b2, out, x_full, kw
    # GEMM -> reduce-scatter: N = d; name, local K
    for name, K in (("o", q), ("down", F), ("d_gate_up", 2 * F), ("d_qkv", q + 2 * kv)):
        x, w = rnd(M, K), rnd(d, K, sc=0.02)
        t, b2 = rnd(M, 64, sc=0.1), rnd(d, 64, sc=0.02)
        res = rnd(m_seg, d)
        out = torch.empty(m_seg, d, device=dev, dtype=bf)
        full = torch.empty(M, d, device=dev, dtype=bf)
        fl = 2.0 * M * d * K
        ms_f = sustained(lambda: ctx.gemm_rs(x, w, a2=t, b2=b2, residual=res, out=out))
        ms_l = sustained(lambda: gemm_tn(x, w, a2=t, b2=b2, out=full))
        ms_u = sustained(lambda: unfused_gemm_rs(x, w).add_(res))

        def library_same_math():
            part = (x @ w.t()).addmm_(t, b2.t())
            o = torch.empty(m_seg, d, device=dev, dtype=bf)
            dist.reduce_scatter_tensor(o, part)
            return o.add_(res)

        ms_s = sustained(library_same_math)
        rows.append({"op": "gemm_rs", "gemm": name, "n": d, "k": K, "fused_ms": round(ms_f, 4),
                     "fused_tflops": round(fl / ms_f / 1e9, 1), "local_gemm_ms": round(ms_l, 4), "nccl_cublas_ms": round(ms_u, 4),
                     "library_same_math_ms": round(ms_s, 4),
                     "nvlink_mb_out": round((P - 1) * m_seg * d * 2 / 1e6, 1)})
        del x, w, t, b2, res, out, full
    torch.cuda.synchronize()
    _lib.check_status(dev)
    ctx.close()
    res = {"op": "tp_layer", "model": cfg.name, "tokens": M, "tp": P, "fused_layer_ms": round(sum(r["fused_ms"] for r in rows), 3),
           "local_gemm_layer_ms": round(sum(r["local_gemm_ms"] for r in rows), 3),
           "nccl_cublas_layer_ms": round(sum(r["nccl_cublas_ms"] for r in rows), 3),
           "library_same_math_layer_ms": round(sum(r["library_same_math_ms"] for r in rows), 3), "gemms": rows}
    dist.barrier()
    dist.destroy_process_group()
    return res if rank == 0 else {}


def bench_attn(a) -> dict:
    """Tree-masked attention forward + backward on the benchmark mask (prompt + 3 sibling completions per row)."""
    from . import _lib, attn_native
    from . import attention as A

    dev = "cuda"
    rows, S, Hq, Hkv, hd = a.rows, a.seq, a.hq, a.hkv, a.hd
    M = rows * S
    g = torch.Generator(device=dev).manual_seed(0)
    qkv = (torch.randn(M, (Hq + 2 * Hkv) * hd, device=dev, generator=g) * 0.5).bfloat16()
    do = (torch.randn(M, Hq * hd, device=dev, generator=g) * 0.5).bfloat16()
    seg = S // 4
    gid = torch.empty(rows, S, dtype=torch.int32)
    pid = torch.empty(rows, S, dtype=torch.int32)
    for r in range(rows):
        p = 100 * r
        gid[r, :seg] = p
        pid[r] = p
        for c in range(3):
            gid[r, seg * (c + 1): seg * (c + 2)] = p + c + 1
    gid, pid = gid.reshape(-1).to(dev), pid.reshape(-1).to(dev)
    plan = A.make_plan(gid, pid, S, "native")
    density = (plan.state.float() > 0).float().mean().item()
    fl = 4.0 * rows * S * S * hd * Hq * density
    res = {"op": "tree_attention", "rows": rows, "seq": S, "heads": f"{Hq}/{Hkv}x{hd}", "tile_density": round(density, 3)}
    for name, tc in (("tcgen05", True), ("mma_sync", False)):
        if a.no_baseline and not tc:
            continue
        attn_native.USE_TC = attn_native.USE_TC_BWD = tc
        box = {}

        def fwd():
            box["o"], box["saved"] = attn_native.forward(qkv, Hq, Hkv, hd, plan)

        tf = _time(fwd, a.iters, a.warmup, None)
        tb = _time(lambda: attn_native.backward(do, box["saved"], plan), a.iters, a.warmup, None)
        res[name] = {"fwd_ms": round(tf, 4), "bwd_ms": round(tb, 4), "fwd_tflops": round(fl / tf / 1e9, 1),
                     "bwd_tflops": round(2.5 * fl / tb / 1e9, 1)}
    attn_native.USE_TC = attn_native.USE_TC_BWD = True
    _lib.check_status()
    return res


def bench_moe(a) -> dict:
    """Router + gather + grouped gate|up GEMM (SwiGLU epilogue) + grouped down GEMM + combine at a sparse-model shape."""
    from . import _lib, moe

    dev = "cuda"
    M, E, k, d, F = a.tokens, a.experts, a.topk, a.d_model, a.ffn
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.randn(M, d, device=dev, generator=g).bfloat16()
    logits = torch.randn(M, E, device=dev, generator=g)
    wgu = (torch.randn(E * 2 * F, d, device=dev, generator=g) * 0.02).bfloat16()
    wd = (torch.randn(E * d, F, device=dev, generator=g) * 0.02).bfloat16()
    plan = moe.route(logits, k, True)
    xp = moe.gather(x, plan)
    h = torch.empty(plan.cap_rows, F, device=dev, dtype=torch.bfloat16)
    gu = torch.empty(plan.cap_rows, 2 * F, device=dev, dtype=torch.bfloat16)
    y = torch.empty(plan.cap_rows, d, device=dev, dtype=torch.bfloat16)
    t_route = _time(lambda: moe.route(logits, k, True), a.iters, a.warmup, None)
    t_gather = _time(lambda: moe.gather(x, plan, out=xp), a.iters, a.warmup, None)
    t_gu = _time(lambda: moe.grouped_gemm(xp, wgu, plan, 2 * F, swiglu_out=h, out=gu), a.iters, a.warmup, None)
    t_dn = _time(lambda: moe.grouped_gemm(h, wd, plan, d, out=y), a.iters, a.warmup, None)
    t_comb = _time(lambda: moe.combine(y, plan, weighted=True, residual=x), a.iters, a.warmup, None)
    _lib.check_status()
    rows = M * k
    res = {"op": "moe_layer_fwd", "tokens": M, "experts": E, "topk": k, "d_model": d, "ffn": F, "rows": rows,
           "route_ms": round(t_route, 4), "gather_ms": round(t_gather, 4), "combine_ms": round(t_comb, 4),
           "gate_up_ms": round(t_gu, 4), "gate_up_tflops": round(2.0 * rows * 2 * F * d / t_gu / 1e9, 1),
           "down_ms": round(t_dn, 4), "down_tflops": round(2.0 * rows * d * F / t_dn / 1e9, 1)}
    if not a.no_baseline:
        seg = plan.seg_off.tolist()

        def loop():
            for e in range(E):
                r = slice(seg[e], seg[e + 1])
                if seg[e + 1] > seg[e]:
                    torch.matmul(xp[r], wgu[e * 2 * F:(e + 1) * 2 * F].t(), out=gu[r])

        t_loop = _time(loop, max(1, a.iters // 4), 1, None)
        res["cublas_loop_gate_up_ms"] = round(t_loop, 4)
        res["cublas_loop_gate_up_tflops"] = round(2.0 * rows * 2 * F * d / t_loop / 1e9, 1)
    return res


def bench_sampler(a) -> dict:
    """LM head + sampling for one decode step: the fused Gumbel-max epilogue against the top-k / top-p path (fp32
    logits GEMM + radix-select kernel) and, as the library baseline, cuBLAS logits + torch softmax / multinomial."""
    from . import _lib, paged
    from .gemm import gemm_tn

    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    M, K, V = a.rows, a.k, a.vocab
    hid = (torch.randn(M, K, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    head = (torch.randn(V, K, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    it = torch.ones(M, device=dev)
    sd = torch.arange(M, dtype=torch.int32, device=dev)
    tk = torch.full((M,), a.top_k, dtype=torch.int32, device=dev)
    tp = torch.full((M,), a.top_p, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if a.flush else None
    logits = gemm_tn(hid, head, out_dtype=torch.float32)
    out = {"op": "sampler", "rows": M, "k": K, "vocab": V, "top_k": a.top_k, "top_p": a.top_p,
           "fused_ms": round(_time(lambda: paged.sample(hid, head, it, sd), a.iters, a.warmup, flush), 4),
           "restricted_ms": round(_time(lambda: paged.sample_restricted(hid, head, it, sd, tk, tp), a.iters, a.warmup, flush), 4),
           "select_kernel_ms": round(_time(lambda: paged.sample_from_logits(logits, it, sd, tk, tp), a.iters, a.warmup, flush), 4)}
    if not a.no_baseline:
        def lib():
            p = torch.softmax((hid @ head.t()).float(), -1)
            return torch.multinomial(p, 1)
        out["cublas_softmax_multinomial_ms"] = round(_time(lib, a.iters, a.warmup, flush), 4)
    _lib.check_status(dev)
    return out


def bench_paged_decode(a) -> dict:
    """Decode attention over a paged KV cache at a rollout-engine shape: ``seqs`` sequences of ``ctx`` cached tokens,
    ``layers`` distinct caches visited round-robin (together larger than L2, so every launch reads its keys and values
    from HBM, as in a real step where 28 layers follow one another).  Reports the K+V bytes per second."""
    from . import _lib, paged

    dev = "cuda"
    bs = 16
    nblk = (a.ctx + bs - 1) // bs
    g = torch.Generator(device=dev).manual_seed(0)
    caches = []
    for _ in range(a.layers):
        k = (torch.randn(a.seqs * nblk, bs, a.hkv, a.hd, device=dev, generator=g) * 0.5).bfloat16()
        v = (torch.randn(a.seqs * nblk, bs, a.hkv, a.hd, device=dev, generator=g) * 0.5).bfloat16()
        caches.append((k, v))
    perm = torch.randperm(a.seqs * nblk, device=dev, generator=g).to(torch.int32)
    width = 64
    while width < nblk:
        width *= 2
    bt = torch.zeros(a.seqs, width, dtype=torch.int32, device=dev)
    bt[:, :nblk] = perm.view(a.seqs, nblk)
    ctx = torch.full((a.seqs,), a.ctx, dtype=torch.int32, device=dev)
    q = (torch.randn(a.seqs, a.hq * a.hd, device=dev, generator=g) * 0.5).bfloat16()
    out = torch.empty_like(q)
    splits = a.splits
    ws = torch.empty(a.seqs * a.hq * splits * (a.hd + 2), dtype=torch.float32, device=dev) if splits > 1 else None

    def run():                    # one launch per cache, back to back, as the layers of a step follow one another
        for k, v in caches:
            paged.paged_decode(q, k, v, bt, ctx, a.hq, a.hkv, a.hd, out, splits, ws)

    ms = _time(run, a.iters, a.warmup, None) / a.layers
    _lib.check_status()
    kv_bytes = 2.0 * a.seqs * a.ctx * a.hkv * a.hd * 2
    return {"op": "paged_decode", "seqs": a.seqs, "ctx": a.ctx, "hq": a.hq, "hkv": a.hkv, "hd": a.hd, "splits": splits,
            "layers": a.layers, "ms": round(ms, 4), "kv_mb": round(kv_bytes / 1e6, 1), "kv_gb_s": round(kv_bytes / ms / 1e6, 1)}


def bench_wgrad(a) -> dict:
    """LoRA factor gradient ``acc[C, 64] += P[M, C]^T Q[M, 64]``: reads the wide operand once, so the figure of merit is
    bytes of P (+ Q) per second against the copy bandwidth.  Several P buffers are visited round-robin (> L2 together)."""
    from . import _lib, wgrad

    dev = "cuda"
    g = torch.Generator(device=dev).manual_seed(0)
    n_buf = max(2, int(400e6 // (a.m * a.c * 2)) + 1)
    Ps = [(torch.randn(a.m, a.c, device=dev, generator=g) * 0.5).bfloat16() for _ in range(n_buf)]
    Q = (torch.randn(a.m, 64, device=dev, generator=g) * 0.5).bfloat16()
    acc = torch.zeros(a.c, 64, device=dev)

    def run():
        for P in Ps:
            wgrad.accumulate(acc, P, Q, False)

    ms = _time(run, a.iters, a.warmup, None) / n_buf
    _lib.check_status()
    nbytes = a.m * (a.c + 64) * 2.0
    return {"op": "lora_wgrad", "m": a.m, "c": a.c, "ms": round(ms, 4), "mb": round(nbytes / 1e6, 1),
            "gb_s": round(nbytes / ms / 1e6, 1)}


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="op", required=True)
    g = sub.add_parser("gemm")
    g.add_argument("--m", type=int, default=8192)
    g.add_argument("--n", type=int, default=3584)
    g.add_argument("--k", type=int, default=3584)
    g.add_argument("--bn", type=int, default=0)
    g.add_argument("--two-cta", type=int, default=-1, help="-1 auto, 0 one CTA per tile, 1 CTA pairs")
    g.add_argument("--epilogue", default="plain", choices=["plain", "resid", "swiglu", "swiglu_bwd"])
    t = sub.add_parser("attn")
    t.add_argument("--rows", type=int, default=4)
    t.add_argument("--seq", type=int, default=2048)
    t.add_argument("--hq", type=int, default=28)
    t.add_argument("--hkv", type=int, default=4)
    t.add_argument("--hd", type=int, default=128)
    m = sub.add_parser("moe")
    m.add_argument("--tokens", type=int, default=8192)
    m.add_argument("--experts", type=int, default=128)
    m.add_argument("--topk", type=int, default=8)
    m.add_argument("--d-model", type=int, default=2048)
    m.add_argument("--ffn", type=int, default=768)
    sp = sub.add_parser("sampler")
    sp.add_argument("--rows", type=int, default=256)
    sp.add_argument("--k", type=int, default=3584)
    sp.add_argument("--vocab", type=int, default=152064)
    sp.add_argument("--top-k", type=int, default=50)
    sp.add_argument("--top-p", type=float, default=0.9)
    pd = sub.add_parser("paged-decode")
    pd.add_argument("--seqs", type=int, default=256)
    pd.add_argument("--ctx", type=int, default=640)
    pd.add_argument("--hq", type=int, default=28)
    pd.add_argument("--hkv", type=int, default=4)
    pd.add_argument("--hd", type=int, default=128)
    pd.add_argument("--splits", type=int, default=1)
    pd.add_argument("--layers", type=int, default=8, help="distinct caches visited round-robin (8 x 335 MB at the defaults)")
    wg = sub.add_parser("wgrad")
    wg.add_argument("--m", type=int, default=8192)
    wg.add_argument("--c", type=int, default=3584)
    gl = sub.add_parser("gemm-layer")
    gl.add_argument("--model", default="qwen2.5-7b")
    gl.add_argument("--tokens", type=int, default=8192)
    gl.add_argument("--seconds", type=float, default=0.5, help="length of each back-to-back timing run")
    gl.add_argument("--try-bn", type=int, nargs="*", default=[], help="also time CTA-pair tiles of these widths (224)")
    gl.add_argument("--ablate", action="store_true", help="also time each product without LoRA / without its epilogue")
    tl = sub.add_parser("tp-layer", help="run under torchrun: one rank per GPU of the tensor-parallel group")
    tl.add_argument("--model", default="qwen2.5-7b")
    tl.add_argument("--tokens", type=int, default=16384)
    tl.add_argument("--seconds", type=float, default=0.4)
    for p in (g, t, m, sp, gl, tl, pd, wg):
        p.add_argument("--iters", type=int, default=20)
        p.add_argument("--warmup", type=int, default=3)
        p.add_argument("--flush", action="store_true")
        p.add_argument("--no-baseline", action="store_true")
    a = ap.parse_args()
    res = {"attn": bench_attn, "moe": bench_moe, "gemm": bench_gemm, "sampler": bench_sampler,
           "gemm-layer": bench_gemm_layer, "tp-layer": bench_tp_layer, "paged-decode": bench_paged_decode,
           "wgrad": bench_wgrad}[a.op](a)
    if res:
        print(json.dumps(res))


if __name__ == "__main__":
    main()
