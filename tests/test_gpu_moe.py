"""Mixture-of-experts kernels and the sparse decoder against PyTorch oracles."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device=DEV).manual_seed(seed)
    return (torch.randn(*shape, device=DEV, generator=g) * scale).to(torch.bfloat16)


def rel_err(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    yield
    from art_b200.ops import _lib

    torch.cuda.synchronize()
    _lib.check_status()


@pytest.mark.parametrize("M,E,k,norm", [(300, 8, 2, True), (1000, 128, 8, True), (257, 64, 6, False)])
def test_router_plan_gather_combine(M, E, k, norm):
    from art_b200.ops import moe

    D = 256
    g = torch.Generator(device=DEV).manual_seed(1)
    logits = torch.randn(M, E, device=DEV, generator=g) * 2
    plan = moe.route(logits, k, norm)
    ti, tw = moe.reference_route(logits, k, norm)
    assert torch.equal(plan.topi.long().sort(-1).values, ti.sort(-1).values)
    order = plan.topi.long().argsort(-1)
    assert torch.allclose(plan.topw.gather(-1, order), tw.gather(-1, ti.argsort(-1)), atol=1e-5)
    counts = torch.bincount(ti.reshape(-1), minlength=E)
    assert torch.equal(plan.counts.long(), counts)
    seg = plan.seg_off.long()
    assert torch.equal(seg[1:] - seg[:-1], (counts + 127) // 128 * 128)
    total = int(seg[-1])
    te = plan.tile_expert.long()
    assert (te[total // 128:] == -1).all()
    for t in range(total // 128):
        e = int(te[t])
        assert seg[e] <= t * 128 < seg[e + 1]
    # every (token, slot) owns a distinct row inside its expert's segment
    pos = plan.pos.long()
    assert pos.unique().numel() == M * k
    assert ((pos >= seg[plan.topi.long()]) & (pos < seg[plan.topi.long()] + counts[plan.topi.long()])).all()
    assert torch.equal(plan.row_token.long()[pos.reshape(-1)], torch.arange(M, device=DEV).repeat_interleave(k))
    x = bf(M, D, seed=2)
    xp = moe.gather(x, plan)
    assert torch.equal(xp[pos.reshape(-1)], x.repeat_interleave(k, 0))
    pad = plan.row_token[:total] < 0
    assert (xp[:total][pad] == 0).all()
    # combine with weights + residual, and the routing-weight gradient dots
    yp = bf(plan.cap_rows, D, seed=3)
    res = bf(M, D, seed=4)
    gout = bf(M, D, seed=5)
    out, dots = moe.combine(yp, plan, weighted=True, residual=res, grad_for_dots=gout)
    ref = res.float() + (yp[pos].float() * plan.topw.unsqueeze(-1)).sum(1)
    assert rel_err(out, ref) < 1e-2
    assert torch.allclose(dots, (yp[pos].float() * gout.float().unsqueeze(1)).sum(-1), rtol=2e-3, atol=2e-2)
    # router backward against autograd
    l32 = logits.clone().requires_grad_(True)
    p = l32.softmax(-1)
    w = p.gather(-1, plan.topi.long())
    if norm:
        w = w / w.sum(-1, keepdim=True)
    dw = torch.randn(M, k, device=DEV, generator=g)
    (w * dw).sum().backward()
    dl = moe.router_bwd(logits, plan, dw, norm, (E + 7) // 8 * 8)
    assert rel_err(dl[:, :E], l32.grad) < 1e-2


def test_grouped_gemm_and_wgrad():
    from art_b200.ops import moe

    M, E, k, K, N = 700, 8, 2, 192, 320
    g = torch.Generator(device=DEV).manual_seed(1)
    plan = moe.route(torch.randn(M, E, device=DEV, generator=g), k, True)
    x = bf(M, K, seed=2)
    xp = moe.gather(x, plan)
    W = bf(E * N, K, scale=0.05, seed=3)
    A = bf(E * 64, K, scale=0.05, seed=4)
    B = bf(E * N, 64, scale=0.05, seed=5)
    T = moe.grouped_gemm(xp, A, plan, 64)
    h = torch.empty(plan.cap_rows, N // 2, dtype=torch.bfloat16, device=DEV)
    y = moe.grouped_gemm(xp, W, plan, N, a2=T, b2=B, swiglu_out=h)
    seg = plan.seg_off.tolist()
    acc = torch.zeros(E, K, 64, dtype=torch.float32, device=DEV)
    dT = bf(plan.cap_rows, 64, seed=6)
    moe.grouped_wgrad(acc, xp, dT, plan)
    for e in range(E):
        rows = slice(seg[e], seg[e + 1])
        xe = xp[rows].float()
        Te = xe @ A[e * 64:(e + 1) * 64].float().t()
        assert rel_err(T[rows], Te) < 1e-2
        ye = xe @ W[e * N:(e + 1) * N].float().t() + T[rows].float() @ B[e * N:(e + 1) * N].float().t()
        assert rel_err(y[rows], ye) < 1e-2
        ge = y[rows].float().view(-1, N // 32, 2, 16)
        assert rel_err(h[rows], (torch.nn.functional.silu(ge[:, :, 0]) * ge[:, :, 1]).reshape(-1, N // 2)) < 1e-2
        assert rel_err(acc[e], xe.t() @ dT[rows].float()) < 1e-2


def test_native_moe_trainer_matches_autograd_reference():
    from art_b200.models.config import ModelConfig
    from art_b200.models.weights import LoraConfig, init_base_weights, init_lora
    from art_b200.trainer.trainer import TrainHyper, Trainer
    from tests.test_gpu_model import _packed

    cfg = ModelConfig(name="small-moe", family="qwen3_moe", vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4,
                      num_kv_heads=2, head_dim=64, intermediate_size=0, qkv_bias=False, qk_norm=True, num_experts=8,
                      num_experts_per_tok=2, moe_intermediate_size=128)
    base = init_base_weights(cfg, seed=0)
    for k_ in base:                      # spread the router so that bf16 rounding does not flip the top-k
        if k_.endswith("mlp.gate.weight"):
            base[k_] = base[k_] * 8
    lcfg = LoraConfig()
    lora = init_lora(cfg, lcfg)
    g = torch.Generator().manual_seed(5)
    for k_ in lora:
        if "lora_B" in k_:
            lora[k_] = torch.randn(lora[k_].shape, generator=g) * 0.05
    packed = _packed(cfg, 2, 256)
    hy = TrainHyper(learning_rate=1e-4, beta=0.0, rows_per_optimizer_step=2)
    ref = Trainer(cfg, base, lcfg, {k_: v.clone() for k_, v in lora.items()}, device=DEV, impl="reference")
    nat = Trainer(cfg, base, lcfg, {k_: v.clone() for k_, v in lora.items()}, device=DEV, impl="native")
    mr, mn = ref.step(packed, hy), nat.step(packed, hy)
    assert abs(mr["loss"] - mn["loss"]) < 1e-2 * max(1.0, abs(mr["loss"]))
    keys = sorted(ref.flat.grad_views)
    gr = torch.cat([ref.flat.grad_views[k_].reshape(-1) for k_ in keys])
    gn = torch.cat([nat.flat.grad_views[k_].reshape(-1) for k_ in keys])
    assert torch.nn.functional.cosine_similarity(gr, gn, dim=0) > 0.98
    ge = torch.cat([ref.flat.grad_views[k_].reshape(-1) for k_ in keys if "experts" in k_])
    gne = torch.cat([nat.flat.grad_views[k_].reshape(-1) for k_ in keys if "experts" in k_])
    assert torch.nn.functional.cosine_similarity(ge, gne, dim=0) > 0.97
    assert abs(mr["grad_norm"] - mn["grad_norm"]) < 6e-2 * mr["grad_norm"]


def test_native_engine_serves_a_sparse_model_like_the_reference_runner():
    """Router + grouped experts inside the rollout engine (prefill and captured multi-step decode), base model and
    adapter rows in one batch, against the plain-PyTorch runner."""
    from art_b200.engine.engine import Engine, SamplingParams
    from art_b200.engine.kv_cache import BlockManager, KVCache
    from art_b200.engine.runner import NativeRunner, ReferenceRunner
    from art_b200.models.config import ModelConfig
    from art_b200.models.weights import LoraConfig, init_base_weights, init_lora

    cfg = ModelConfig(name="small-moe", family="qwen3_moe", vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4,
                      num_kv_heads=2, head_dim=64, intermediate_size=0, qkv_bias=False, qk_norm=True, num_experts=8,
                      num_experts_per_tok=2, moe_intermediate_size=128)
    base = init_base_weights(cfg, seed=0)
    for k_ in base:                      # spread the router so that bf16 rounding does not flip the top-k
        if k_.endswith("mlp.gate.weight"):
            base[k_] = base[k_] * 8
    lcfg = LoraConfig()
    lora = init_lora(cfg, lcfg)
    g = torch.Generator().manual_seed(5)
    for k_ in lora:
        if "lora_B" in k_:
            lora[k_] = torch.randn(lora[k_].shape, generator=g) * 0.05
    base_bf = {k: v.to(torch.bfloat16) for k, v in base.items()}
    kv = KVCache(cfg.num_layers, 128, 16, cfg.num_kv_heads, cfg.head_dim, torch.device(DEV))
    nat = Engine(NativeRunner(cfg, lcfg, kv, base=base_bf, max_loras=1, device=DEV), BlockManager(128, 16, True),
                 eos_token_id=None, max_loras=1, num_scheduler_steps=4, kv_cache=kv)
    ref = Engine(ReferenceRunner(cfg, base_bf, lcfg, max_loras=1, device=DEV), BlockManager(128, 16, True),
                 eos_token_id=None, max_loras=1, num_scheduler_steps=4)
    for e in (nat, ref):
        e.set_adapter("a", {k: v.to(DEV) for k, v in lora.items()})
    prompts = [list(range(5, 40)), list(range(100, 117)), [7, 8, 9], list(range(300, 330))]
    adapters = [None, "a", "a", None]                   # one batch mixes base-model rows and adapter rows
    p = SamplingParams(max_tokens=12, temperature=0.0)
    sn = [nat.add_request(pr, p, ad) for pr, ad in zip(prompts, adapters)]
    sr = [ref.add_request(pr, p, ad) for pr, ad in zip(prompts, adapters)]
    while not all(s.finished for s in sn):
        nat.step()
    while not all(s.finished for s in sr):
        ref.step()
    for a, b in zip(sn, sr):
        agree = sum(x == y for x, y in zip(a.output_ids, b.output_ids))
        assert a.output_ids[0] == b.output_ids[0] and agree >= 8, (a.output_ids, b.output_ids)
        assert abs(a.logprobs[0] - b.logprobs[0]) < 0.05
    # the adapter changes what the experts compute: same prompt, different continuation or log-prob
    s_base = nat.generate_sync(prompts[1], p, None)
    assert s_base.output_ids != sn[1].output_ids or abs(s_base.logprobs[0] - sn[1].logprobs[0]) > 1e-3
