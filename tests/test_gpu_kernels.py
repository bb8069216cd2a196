"""Numerics of every CUDA kernel against a plain PyTorch fp32 restatement of the same op."""
import math

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


@pytest.mark.parametrize("M,N,K,K2,bn", [(128, 64, 64, 0, 64), (256, 512, 512, 0, 256), (200, 264, 328, 0, 0),
                                         (1024, 1024, 1024, 64, 0), (4096, 4608, 3584, 8, 0), (77, 3584, 128, 16, 64),
                                         (2048, 3584, 512, 64, 0), (512, 3584, 256, 0, 224), (300, 600, 320, 16, 192)])
def test_gemm_tn(M, N, K, K2, bn):
    from art_b200.ops.gemm import gemm_tn, reference_gemm_tn

    a, b = bf(M, K, seed=1), bf(N, K, scale=0.05, seed=2)
    a2 = bf(M, K2, seed=3) if K2 else None
    b2 = bf(N, K2, scale=0.05, seed=4) if K2 else None
    r = bf(M, N, seed=5)
    bias = torch.randn(N, device=DEV)
    out = gemm_tn(a, b, a2=a2, b2=b2, residual=r, bias=bias, bn=bn)
    ref = reference_gemm_tn(a, b, a2, b2, r, bias)
    assert rel_err(out, ref) < 5e-3
    out32 = gemm_tn(a, b, out_dtype=torch.float32, bn=bn)
    assert rel_err(out32, reference_gemm_tn(a, b)) < 1e-3


def test_gemm_two_cta_224_tiles():
    from art_b200.ops.gemm import gemm_tn, reference_gemm_tn

    a, b = bf(1024, 512, seed=1), bf(3584, 512, scale=0.05, seed=2)
    out = gemm_tn(a, b, bn=224, two_cta=True)
    assert rel_err(out, reference_gemm_tn(a, b)) < 5e-3


@pytest.mark.parametrize("M,N,K", [(256, 2112, 512), (300, 600, 320), (512, 37952, 256)])
def test_gemm_two_cta_tails_and_partial_residual(M, N, K):
    """Pair tiles with M and N tails, and a residual that covers only the first columns (the decode-time
    ``[W ; A_all]`` product: base columns get the residual, the shrink columns do not)."""
    from art_b200.ops.gemm import gemm_tn, reference_gemm_tn

    a, b = bf(M, K, seed=1), bf(N, K, scale=0.05, seed=2)
    bias = torch.randn(N, device=DEV)
    rc = N - 64
    r = bf(M, rc, seed=5)
    out = gemm_tn(a, b, residual=r, res_cols=rc, bias=bias, two_cta=True)
    ref = reference_gemm_tn(a, b, None, None, None, bias)
    ref[:, :rc] += r.float()
    assert rel_err(out, ref) < 5e-3


@pytest.mark.parametrize("pair,M,N,K", [(False, 256, 512, 1024), (True, 256, 512, 1024), (True, 512, 3584, 2304),
                                        (True, 256, 4608, 3584)])
def test_splitk_finalize_applies_the_adapter_slot_mask(pair, M, N, K):
    from art_b200.ops.gemm import gemm_splitk_, plan_small_m, reference_gemm_tn, splitk_finalize

    kpad, cols = 64, 16
    a, b = bf(M, K, seed=1), bf(N + kpad, K, scale=0.05, seed=2)
    r = bf(M, N, seed=3)
    adapter = (torch.arange(M, device=DEV, dtype=torch.int32) % 5) - 1          # -1 .. 3
    bn, splits = plan_small_m(M, N + kpad, K, pair=pair)
    units = ((M + 255) // 256) * ((N + kpad + 255) // 256) if pair else ((M + 127) // 128) * ((N + kpad + bn - 1) // bn)
    assert splits > 1 and units * splits <= (74 if pair else 148)
    ws = torch.zeros(M, N + kpad, dtype=torch.float32, device=DEV)
    out = torch.empty(M, N + kpad, dtype=torch.bfloat16, device=DEV)
    gemm_splitk_(ws, a, b, bn, splits, two_cta=pair)
    splitk_finalize(ws, out, None, r, N, adapter, N, cols)
    ref = reference_gemm_tn(a, b)
    ref[:, :N] += r.float()
    col = torch.arange(kpad, device=DEV).unsqueeze(0)
    lo = (adapter.long() * cols).unsqueeze(1)
    keep = (adapter.unsqueeze(1) >= 0) & (col >= lo) & (col < lo + cols)
    ref[:, N:] *= keep
    assert rel_err(out, ref) < 5e-3
    assert (out[:, N:][~keep] == 0).all() and float(ws.abs().max()) == 0.0


def test_gemm_swiglu_epilogue():
    from art_b200.ops import elementwise as ew
    from art_b200.ops.gemm import gemm_tn

    M, K, F = 300, 256, 384
    x, wg, wu = bf(M, K, seed=1), bf(F, K, scale=0.1, seed=2), bf(F, K, scale=0.1, seed=3)
    h = torch.empty(M, F, dtype=torch.bfloat16, device=DEV)
    gu = gemm_tn(x, ew.interleave_gate_up(wg, wu), swiglu_out=h)
    g, u = ew.deinterleave_gate_up(gu)
    assert rel_err(g, x.float() @ wg.float().t()) < 5e-3 and rel_err(u, x.float() @ wu.float().t()) < 5e-3
    assert rel_err(h, torch.nn.functional.silu(g.float()) * u.float()) < 1e-2
    assert rel_err(ew.swiglu_fwd(gu), h) < 1e-2
    dh = bf(M, F, seed=4)
    g32, u32 = g.float().requires_grad_(True), u.float().requires_grad_(True)
    (torch.nn.functional.silu(g32) * u32).backward(dh.float())
    dg, du = ew.deinterleave_gate_up(ew.swiglu_bwd(dh, gu))
    assert rel_err(dg, g32.grad) < 1e-2 and rel_err(du, u32.grad) < 1e-2
    # the same backward fused into the epilogue of the GEMM that produces dh = dy @ Wd
    for Mf, two in ((M, False), (1024, True)):
        xf = bf(Mf, K, seed=11)
        guf = gemm_tn(xf, ew.interleave_gate_up(wg, wu))
        dy, wd = bf(Mf, 128, seed=5), bf(128, F, scale=0.1, seed=6)       # down-proj weight [d, F]; dh = dy @ wd
        dh_ref = gemm_tn(dy, wd.t().contiguous())
        fused = gemm_tn(dy, wd.t().contiguous(), swiglu_bwd_gu=guf, two_cta=two)
        assert rel_err(fused, ew.swiglu_bwd(dh_ref, guf)) < 1e-2


@pytest.mark.parametrize("M,D", [(64, 128), (300, 3584), (17, 5120)])
def test_rmsnorm_fwd_bwd(M, D):
    from art_b200.ops import elementwise as ew

    x, w, dy, dres = bf(M, D, seed=1), bf(D, scale=0.5, seed=2) + 1, bf(M, D, seed=3), bf(M, D, seed=4)
    y, rstd = ew.rmsnorm_fwd(x, w, 1e-6)
    assert rel_err(y, ew.rmsnorm_reference(x, w, 1e-6)) < 5e-3
    x32 = x.float().requires_grad_(True)
    (x32 * torch.rsqrt(x32.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()).backward(dy.float())
    dx = ew.rmsnorm_bwd(dy, x, w, rstd, dres=dres)
    assert rel_err(dx, x32.grad + dres.float()) < 1e-2


def test_rope_forward_inverse_and_headnorm():
    from art_b200.ops import elementwise as ew

    M, Hq, Hkv, hd = 100, 4, 2, 64
    buf = bf(M, (Hq + 2 * Hkv) * hd, seed=1)
    orig = buf.clone()
    pos = torch.randint(0, 5000, (M,), device=DEV, dtype=torch.int32)
    ew.rope_(buf, pos, 0, Hq + Hkv, hd, 1e6)
    ref = ew.rope_reference(orig[:, :(Hq + Hkv) * hd].view(M, Hq + Hkv, hd), pos, 1e6).reshape(M, -1)
    assert rel_err(buf[:, :(Hq + Hkv) * hd], ref) < 5e-3
    assert torch.equal(buf[:, (Hq + Hkv) * hd:], orig[:, (Hq + Hkv) * hd:])       # v untouched
    ew.rope_(buf, pos, 0, Hq + Hkv, hd, 1e6, inverse=True)
    assert rel_err(buf, orig) < 1e-2
    w = bf(hd, scale=0.2, seed=3) + 1
    x = orig.clone()
    rstd = ew.headnorm_fwd_(x, w, 0, Hq, hd, 1e-6)
    q = orig[:, :Hq * hd].float().view(M, Hq, hd)
    refn = (q * torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6)) * w.float()
    assert rel_err(x[:, :Hq * hd], refn.reshape(M, -1)) < 5e-3
    q32 = q.clone().requires_grad_(True)
    dy = bf(M, (Hq + 2 * Hkv) * hd, seed=5)
    ((q32 * torch.rsqrt(q32.pow(2).mean(-1, keepdim=True) + 1e-6)) * w.float()).backward(dy[:, :Hq * hd].float().view(M, Hq, hd))
    d = dy.clone()
    ew.headnorm_bwd_(d, orig, w, rstd, 0, Hq, hd)
    assert rel_err(d[:, :Hq * hd], q32.grad.reshape(M, -1)) < 1e-2


def test_gather_scatter_advnorm():
    from art_b200.local.tokenize import group_advantages
    from art_b200.ops import elementwise as ew

    table = bf(50, 64, seed=1)
    idx = torch.tensor([3, 49, 0, 7], device=DEV)
    assert torch.equal(ew.gather_rows(table, idx), table[idx])
    out = torch.zeros(50, 64, dtype=torch.bfloat16, device=DEV)
    ew.scatter_rows_(table[:4].contiguous(), idx, out)
    assert torch.equal(out[idx], table[:4]) and out.abs().sum() == table[:4].abs().sum()
    rewards = [[1.0, 0.0, 0.0, 1.0], [0.5, 0.5], [3.0, 1.0, 2.0]]
    flat = torch.tensor(sum(rewards, []), device=DEV)
    offs = torch.tensor([0, 4, 6, 9], device=DEV, dtype=torch.int32)
    adv, keep = ew.adv_norm(flat, offs)
    ref = sum((group_advantages(r) for r in rewards), [])
    assert torch.allclose(adv.cpu(), torch.tensor(ref), atol=1e-5)
    assert keep.tolist() == [a != 0 for a in ref]


def test_lora_wgrad():
    from art_b200.ops import wgrad

    M, C = 1000, 392
    p, q = bf(M, C, seed=1), bf(M, 64, seed=2)
    acc = torch.ones(C, 64, device=DEV)
    wgrad.accumulate(acc, p, q)
    assert rel_err(acc, 1 + p.float().t() @ q.float()) < 2e-3


def test_flat_adamw_matches_torch():
    from art_b200.ops.optim import FlatAdamW

    n = 10_000
    p0 = torch.randn(n, device=DEV)
    p_ref = p0.clone().requires_grad_(True)
    opt_ref = torch.optim.AdamW([p_ref], lr=1e-3, betas=(0.9, 0.99), weight_decay=0.1, eps=1e-8)
    p, g = p0.clone(), torch.zeros(n, device=DEV)
    opt = FlatAdamW(p, g, max_grad_norm=0.1)
    for step in range(3):
        grad = torch.randn(n, device=DEV, generator=torch.Generator(device=DEV).manual_seed(step))
        g.copy_(grad)
        p_ref.grad = grad.clone()
        norm_ref = torch.nn.utils.clip_grad_norm_([p_ref], 0.1)
        opt_ref.step()
        norm = opt.step(1e-3)
        assert abs(float(norm) - float(norm_ref)) < 1e-3 * float(norm_ref)
    assert torch.allclose(p, p_ref.detach(), atol=1e-6, rtol=1e-5)


def test_restricted_sampler_matches_oracle_and_fused_sampler():
    from art_b200.ops import paged

    dev = torch.device(DEV)
    g = torch.Generator(device=dev).manual_seed(5)
    M, V = 96, 5003
    logits = (torch.randn(M, V, device=dev, generator=g) * 3).contiguous()
    temps = [0.0, 0.7, 1.0, 1.5]
    ks = [-1, 1, 5, 50, 4000]
    ps = [1.0, 0.9, 0.5, 0.05]
    cfgs = [(temps[i % 4], ks[(i // 4) % 5], ps[(i // 20) % 4]) for i in range(M)]
    inv_t = torch.tensor([0.0 if t <= 0 else 1.0 / t for t, _, _ in cfgs], dtype=torch.float32, device=dev)
    tk = torch.tensor([k for _, k, _ in cfgs], dtype=torch.int32, device=dev)
    tp = torch.tensor([p for _, _, p in cfgs], dtype=torch.float32, device=dev)
    seeds = torch.arange(M, dtype=torch.int32, device=dev) * 7919 + 13
    tok, lp = paged.sample_from_logits(logits, inv_t, seeds, tk, tp)
    torch.cuda.synchronize()
    for i, (t, k, p) in enumerate(cfgs):
        x = logits[i] * (1.0 if t <= 0 else 1.0 / t)
        full = torch.log_softmax(x.float(), -1)
        ti = int(tok[i])
        assert abs(float(lp[i]) - float(full[ti])) < 2e-3, (i, t, k, p)
        if t <= 0 or k == 1:
            assert ti == int(x.argmax()), (i, t, k, p)
            continue
        keep = paged.reference_restrict(x, k, p)
        if not bool(keep[ti]):      # only a token sitting on the threshold may differ (summation order)
            thr = full[keep].min()
            assert float(full[ti]) > float(thr) - 1e-3, (i, t, k, p, float(full[ti]), float(thr))
    # the empirical distribution over many seeds is the renormalised restricted one
    V2, n = 64, 40000
    row = torch.randn(V2, device=dev, generator=g) * 2
    lg = row.unsqueeze(0).expand(n, V2).contiguous()
    one = torch.ones(n, dtype=torch.float32, device=dev)
    for k, p, mp in ((10, 1.0, 0.0), (-1, 0.8, 0.0), (20, 0.6, 0.0), (-1, 1.0, 0.15), (8, 0.9, 0.05)):
        tok2, _ = paged.sample_from_logits(lg, one, torch.arange(n, dtype=torch.int32, device=dev),
                                           torch.full((n,), k, dtype=torch.int32, device=dev), one * p, one * mp)
        keep = paged.reference_restrict(row, k, p, mp)
        want = torch.softmax(row.float(), -1) * keep
        want = want / want.sum()
        got = torch.bincount(tok2.long(), minlength=V2).float() / n
        assert float((got - want).abs().max()) < 0.012, (k, p, mp, float((got - want).abs().max()))
        assert float(got[~keep].sum()) < 1e-3
    # nothing restricted: the same tokens as the fused LM-head sampler (same noise, same statistics)
    hid = (torch.randn(48, 256, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    head = (torch.randn(3008, 256, device=dev, generator=g) * 0.2).to(torch.bfloat16)
    it = torch.full((48,), 1.0 / 0.8, dtype=torch.float32, device=dev)
    it[::5] = 0.0
    sd = torch.arange(48, dtype=torch.int32, device=dev) + 1000
    t_f, lp_f = paged.sample(hid, head, it, sd)
    t_r, lp_r = paged.sample_restricted(hid, head, it, sd, torch.zeros(48, dtype=torch.int32, device=dev),
                                        torch.ones(48, dtype=torch.float32, device=dev))
    assert int((t_f == t_r).sum()) >= 46
    same = t_f == t_r
    assert float((lp_f[same] - lp_r[same]).abs().max()) < 5e-3


def test_logit_edit_and_top_logprobs_kernels_match_pytorch():
    from art_b200.engine.runner import LogitProc
    from art_b200.ops import paged

    M, V = 5, 3001
    g = torch.Generator(device="cuda").manual_seed(4)
    logits = torch.randn(M, V, device="cuda", generator=g) * 3
    procs = [None,
             (LogitProc(3, repetition_penalty=1.7), [5, 9, 5, 2000, 9]),
             (LogitProc(2, presence_penalty=0.5, frequency_penalty=0.25, logit_bias={7: 4.0, 3000: -100.0}), [1, 2, 7, 7, 8]),
             None,
             (LogitProc(0, repetition_penalty=0.5, frequency_penalty=1.0), [10, 10, 10])]
    edits = paged.build_logit_edits(procs)
    want = paged.logit_adjust_(logits.cpu().clone(), edits)            # the PyTorch restatement
    got = paged.logit_adjust_(logits.clone(), edits)
    assert torch.allclose(got.cpu(), want, atol=1e-6)
    x = logits.cpu()
    assert torch.isclose(want[1, 5], x[1, 5] / 1.7 if x[1, 5] > 0 else x[1, 5] * 1.7)
    assert torch.isclose(want[2, 7], x[2, 7] - (0.25 * 2 + 0.5) + 4.0) and torch.isclose(want[2, 8], x[2, 8] - 0.75)
    assert want[2, 1] == x[2, 1] and torch.equal(want[0], x[0])       # prompt tokens carry no frequency / presence penalty
    inv_t = torch.tensor([1.0, 0.5, 0.0, 2.0, 1.0], device="cuda")
    ti, tl = paged.top_logprobs(got, inv_t, 6)
    ri, rl = paged.top_logprobs(want, inv_t.cpu(), 6)
    assert torch.equal(ti.cpu(), ri) and torch.allclose(tl.cpu(), rl, atol=1e-4)


@pytest.mark.parametrize("with_lora", [False, True])
def test_decode_finalize_kernels_match_pytorch(with_lora):
    """The fused finish of a decode-time split-K projection (bias + residual + LoRA expand of the row's slot + RMSNorm,
    and bias + LoRA expand + RoPE + cache write for q|k|v) against plain fp32 tensor code."""
    from art_b200.ops import paged

    g = torch.Generator(device=DEV).manual_seed(5)
    M, N, slots, cols = 40, 1536, 3, 16
    kpad = 64
    ldw = N + kpad + 24
    ws = torch.randn(M, ldw, device=DEV, generator=g)
    ws0 = ws.clone()
    bias = torch.randn(N, device=DEV, generator=g)
    R = bf(M, N, seed=1)
    B_all = bf(kpad, N, scale=0.3, seed=2)          # scaled LoRA B, transposed: [shrink column, output feature]
    adapter = torch.randint(-1, slots, (M,), device=DEV, generator=g, dtype=torch.int32)
    nw = (1 + 0.1 * torch.randn(N, device=DEV, generator=g)).bfloat16()
    x_out, h_out = torch.empty(M, N, device=DEV, dtype=torch.bfloat16), torch.empty(M, N, device=DEV, dtype=torch.bfloat16)
    paged.decode_finalize_norm(ws, M, N, kpad, x_out, bias=bias, residual=R, adapter=adapter if with_lora else None,
                               B_all=B_all if with_lora else None, cols=cols if with_lora else 0, norm_w=nw, eps=1e-6, h_out=h_out)

    def lora_term(w0, n_main, bt):
        out = torch.zeros(M, n_main, device=DEV)
        if with_lora:
            for m in range(M):
                a = int(adapter[m])
                if a >= 0:
                    t = w0[m, n_main + a * cols:n_main + (a + 1) * cols]
                    out[m] = t @ bt[a * cols:(a + 1) * cols].float()
        return out

    want = ws0[:, :N] + bias + R.float() + lora_term(ws0, N, B_all)
    assert rel_err(x_out, want) < 5e-3
    xr = x_out.float()
    hn = (xr * torch.rsqrt((xr * xr).mean(-1, keepdim=True) + 1e-6)).bfloat16().float() * nw.float()
    assert rel_err(h_out, hn) < 5e-3
    assert float(ws[:, :N].abs().max()) == 0.0
    if with_lora:
        assert float(ws[:, N:N + kpad].abs().max()) == 0.0
    assert torch.equal(ws[:, N + kpad:], ws0[:, N + kpad:])

    # q|k|v
    Hq, Hkv, hd, bs, blocks = 6, 2, 128, 16, 8
    qs, kvs = Hq * hd, Hkv * hd
    Nq = qs + 2 * kvs
    ldw = Nq + kpad
    ws = torch.randn(M, ldw, device=DEV, generator=g)
    ws0 = ws.clone()
    bias = torch.randn(Nq, device=DEV, generator=g)
    B_all = bf(kpad, Nq, scale=0.3, seed=3)
    pos = torch.randint(0, 5000, (M,), device=DEV, generator=g, dtype=torch.int32)
    slot = torch.randperm(blocks * bs, device=DEV, generator=g)[:M].to(torch.int32)
    slot[3] = -1
    kc = torch.zeros(blocks, bs, Hkv, hd, device=DEV, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    q_out = torch.empty(M, qs, device=DEV, dtype=torch.bfloat16)
    paged.decode_finalize_qkv(ws, M, Hq, Hkv, hd, kpad, pos, 1e6, slot, kc, vc, q_out, bias=bias,
                              adapter=adapter if with_lora else None, B_all=B_all if with_lora else None,
                              cols=cols if with_lora else 0)
    y = ws0[:, :Nq] + bias + lora_term(ws0, Nq, B_all)

    def rope(t, heads):
        t = t.view(M, heads, hd)
        i = torch.arange(hd // 2, device=DEV, dtype=torch.float32)
        ang = pos.float()[:, None] * torch.exp2(-torch.log2(torch.tensor(1e6)) * 2 * i / hd)[None]
        c, s_ = ang.cos()[:, None], ang.sin()[:, None]
        a, b = t[..., :hd // 2], t[..., hd // 2:]
        return torch.cat([a * c - b * s_, b * c + a * s_], -1).reshape(M, heads * hd)

    assert rel_err(q_out, rope(y[:, :qs], Hq)) < 5e-3
    kw, vw = rope(y[:, qs:qs + kvs], Hkv), y[:, qs + kvs:]
    ok = slot >= 0
    assert rel_err(kc.view(-1, kvs)[slot[ok].long()], kw[ok]) < 5e-3
    assert rel_err(vc.view(-1, kvs)[slot[ok].long()], vw[ok]) < 5e-3
    assert float(ws[:, :Nq].abs().max()) == 0.0
