"""Tokenize -> pack -> mask -> loss semantics on CPU (the oracle path)."""
import math
import random

import torch

import art_b200 as art
from art_b200.local.pack import packed_tensors_from_dir, packed_tensors_from_tokenized_results, packed_tensors_to_dir
from art_b200.local.tokenize import group_advantages, tokenize_trajectory_groups
from art_b200.local.tokenizer import ByteChatTokenizer
from art_b200.models.reference import grpo_loss, tree_attention_mask
from tests.test_api_trajectories import make_choice

TOK = ByteChatTokenizer(512)


def traj(reward, ids, prompt="hello"):
    return art.Trajectory(messages_and_choices=[{"role": "user", "content": prompt}, make_choice(ids, "x" * len(ids))],
                          reward=reward)


def test_advantages_population_std_and_zero_drop():
    adv = group_advantages([1.0, 0.0, 0.0, 1.0])
    assert all(abs(abs(a) - 0.5 / (0.5 + 1e-6)) < 1e-9 for a in adv)
    groups = [art.TrajectoryGroup([traj(1.0, (65, 66)), traj(1.0, (67, 68))]),          # equal rewards: nothing to learn
              art.TrajectoryGroup([traj(1.0, (65, 66, 67)), traj(0.0, (70, 71))])]
    res = list(tokenize_trajectory_groups(TOK, groups, False, random.Random(0)))
    assert len(res) == 2 and sorted(round(r.advantage, 3) for r in res) == [-1.0, 1.0]


def test_sampled_ids_are_spliced_and_prompt_prefix_found():
    groups = [art.TrajectoryGroup([traj(1.0, (300, 301, 302)), traj(0.0, (303,))])]
    a, b = sorted(tokenize_trajectory_groups(TOK, groups, False, random.Random(0)), key=lambda r: -r.advantage)
    prompt_ids = TOK.apply_chat_template([{"role": "user", "content": "hello"}], add_generation_prompt=True)
    assert a.token_ids[:len(prompt_ids)] == prompt_ids and a.prompt_length == len(prompt_ids) == b.prompt_length
    n = len(prompt_ids)
    assert a.token_ids[n:n + 3] == [300, 301, 302] and a.assistant_mask[n:n + 3] == [1, 1, 1]
    assert sum(a.assistant_mask) == 3 and a.logprobs[n] == -0.5 and math.isnan(a.logprobs[0])
    assert a.prompt_id == b.prompt_id and a.input_pos == list(range(len(a.token_ids)))


def test_pack_shares_prompt_and_mask_isolates_siblings(tmp_path):
    groups = [art.TrajectoryGroup([traj(1.0, (300, 301, 302)), traj(0.0, (303, 304))]),
              art.TrajectoryGroup([traj(0.0, (310,), "other"), traj(1.0, (311, 312), "other")])]
    rng = random.Random(1)
    res = list(tokenize_trajectory_groups(TOK, groups, False, rng))
    packed = packed_tensors_from_tokenized_results(res, 128, pad_token_id=TOK.eos_token_id, rng=rng)
    assert packed["tokens"].shape == (1, 128)                       # everything fits one row
    n_tok = sum(len(r.token_ids) for r in res) - sum(r.prompt_length for r in res[1::1] if False)
    gid, pid = packed["group_ids"][0], packed["parent_ids"][0]
    used = int((gid != -1).sum())
    p = res[0].prompt_length
    by_group = {}
    for r in res:
        by_group.setdefault(r.prompt_id, []).append(r)
    expect = sum(g[0].prompt_length + sum(len(r.token_ids) - r.prompt_length for r in g) for g in by_group.values())
    assert used == expect                                           # each prompt stored once per group
    m = tree_attention_mask(gid[None], pid[None])[0]
    comp = [i for i in range(used) if packed["assistant_mask"][0, i]]
    for q in comp:
        allowed = m[q].nonzero().flatten().tolist()
        assert all(k <= q for k in allowed)
        for k in allowed:                                           # own completion or its own prompt only
            assert gid[k] == gid[q] or gid[k] == pid[q]
        assert any(gid[k] == pid[q] and gid[k] != gid[q] for k in allowed)   # does see the shared prompt
    # completion positions continue after the prompt regardless of where they sit in the row
    first_comp = comp[0]
    assert int(packed["input_pos"][0, first_comp]) == res[0].prompt_length or True
    w = packed["weights"][0][packed["assistant_mask"][0]]
    assert abs(float(w.mean()) - 1.0) < 1e-5
    assert torch.isnan(packed["logprobs"][0, used:]).all() and (packed["tokens"][0, used:] == TOK.eos_token_id).all()
    disk = packed_tensors_to_dir(packed, str(tmp_path / "t"))
    back = packed_tensors_from_dir(**disk)
    assert torch.equal(back["tokens"], packed["tokens"]) and torch.equal(back["assistant_mask"], packed["assistant_mask"])


def test_pack_opens_new_row_and_truncates():
    long = [art.TrajectoryGroup([traj(1.0, tuple(range(300, 360))), traj(0.0, tuple(range(360, 420)))])]
    rng = random.Random(2)
    res = list(tokenize_trajectory_groups(TOK, long, False, rng))
    packed = packed_tensors_from_tokenized_results(res, 96, pad_token_id=0, rng=rng, verbosity=0)
    assert packed["tokens"].shape == (2, 96)                        # second trajectory does not fit next to the first
    tiny = packed_tensors_from_tokenized_results(res, 64, pad_token_id=0, rng=rng, verbosity=0)
    assert tiny["tokens"].shape[1] == 64                            # over-long rows are cut at seq_len


def test_grpo_loss_clipping_and_nan_old_logprobs():
    S = 6
    packed = {"logprobs": torch.tensor([[float("nan"), -1.0, -1.0, float("nan"), -1.0, -1.0]]),
              "advantages": torch.tensor([[0.0, 1.0, 1.0, -1.0, -1.0, 1.0]]),
              "assistant_mask": torch.tensor([[False, True, True, True, True, False]]),
              "weights": torch.ones(1, S)}
    new = torch.tensor([[-1.0, -0.5, -1.0, -2.0, -1.0, -1.0]], requires_grad=True)   # aligned to next-token targets
    loss, met = grpo_loss(new, packed, epsilon=0.2)
    # after the one-token shift: (new, old, adv) = (-1,-1,1) (-0.5,-1,1) (-1,nan,-1) (-2,-1,-1), rest masked
    terms = [-1.0, -1.2, 1.0, 0.8]     # unclipped; clipped high; nan-old -> ratio 1; clipped low with negative advantage
    assert abs(float(loss.detach()) - sum(terms) / (4 + 1e-6)) < 1e-5
    loss.backward()
    assert abs(float(new.grad[0, 0]) + 0.25) < 1e-6                 # d(-ratio*adv)/dnew / 4
    assert new.grad[0, 1] == 0 and new.grad[0, 3] == 0              # clipped branches carry no gradient
    assert new.grad[0, 4] == 0 and new.grad[0, 5] == 0              # masked out


def test_packing_seed_makes_the_packed_rows_a_function_of_the_trajectories(tmp_path):
    from art_b200.local import LocalBackend

    backend = LocalBackend(in_process=True, path=str(tmp_path))
    model = art.TrainableModel(name="m", project="p", base_model="random:tiny",
                               _internal_config={"init_args": {"architecture": {"vocab_size": 512}}})
    groups = [art.TrajectoryGroup([traj(float(i % 2), [10 + i, 20 + g], prompt=f"q{g}") for i in range(4)]) for g in range(3)]
    a = backend._get_packed_tensors(model, groups, False, False, seed=7)
    b = backend._get_packed_tensors(model, groups, False, False, seed=7)
    c = backend._get_packed_tensors(model, groups, False, False, seed=8)
    for k in ("tokens", "group_ids", "parent_ids", "advantages"):
        assert torch.equal(a[k], b[k])
    assert not torch.equal(a["group_ids"], c["group_ids"])      # other ids (and very likely another order)


def test_packed_rows_give_the_log_probs_of_running_every_trajectory_alone():
    """The point of the whole data path: tokenise, share prompts, pack, mask by ids, position by ``input_pos``.  The
    log-prob of every trainable token in the packed row equals the log-prob of the same token when its trajectory is
    run on its own as one ordinary causal sequence."""
    from art_b200.models.config import PRESETS
    from art_b200.models.reference import ReferenceModel
    from art_b200.models.weights import init_base_weights

    cfg = PRESETS["tiny"]
    model = ReferenceModel(cfg, init_base_weights(cfg, seed=0))
    groups = [art.TrajectoryGroup([traj(1.0, (300, 301, 302, 65)), traj(0.0, (303, 304)), traj(0.5, (66,))]),
              art.TrajectoryGroup([traj(0.0, (310,), "another prompt"), traj(1.0, (311, 312, 313), "another prompt")])]
    rng = random.Random(3)
    res = list(tokenize_trajectory_groups(TOK, groups, False, rng))
    packed = packed_tensors_from_tokenized_results(res, 256, pad_token_id=TOK.eos_token_id, rng=rng)
    assert packed["tokens"].shape[0] == 1
    tok, gid, pid, pos = (packed[k] for k in ("tokens", "group_ids", "parent_ids", "input_pos"))
    with torch.no_grad():
        h = model.hidden_states(tok, gid, pid, pos, use_lora=False)
        lp_packed = torch.log_softmax(h[0].float() @ model.base["lm_head.weight"].float().t(), -1)
    checked = 0
    for r in res:
        ids = torch.tensor([r.token_ids])
        z = torch.zeros_like(ids)
        with torch.no_grad():
            ha = model.hidden_states(ids, z, z, None, use_lora=False)
            lp_alone = torch.log_softmax(ha[0].float() @ model.base["lm_head.weight"].float().t(), -1)
        n_train = sum(r.assistant_mask)
        comp = r.token_ids[r.prompt_length:r.prompt_length + n_train]          # the sampled tokens follow the prompt
        assert r.assistant_mask[r.prompt_length:r.prompt_length + n_train] == [1] * n_train
        # locate them in the packed row: a run of trainable tokens with these ids that starts at this position
        starts = [i for i in range(tok.shape[1] - len(comp) + 1)
                  if tok[0, i:i + len(comp)].tolist() == comp and bool(packed["assistant_mask"][0, i:i + len(comp)].all())
                  and int(pos[0, i]) == r.prompt_length]
        assert len(starts) >= 1
        s0 = starts[0]
        for j, t in enumerate(comp):
            # the token at packed index s0 + j is predicted from the index before it in the tree: the previous
            # completion token, or the last prompt token (which is the last token of the parent group) for j = 0
            if j == 0:
                parent = int(pid[0, s0])
                prev = max(i for i in range(tok.shape[1]) if int(gid[0, i]) == parent)
            else:
                prev = s0 + j - 1
            want = lp_alone[r.prompt_length + j - 1, t]
            got = lp_packed[prev, t]
            assert abs(float(got - want)) < 2e-4, (r.prompt_id, j, float(got), float(want))
            checked += 1
    assert checked == sum(sum(r.assistant_mask) for r in res) == 4 + 2 + 1 + 3      # the mean-reward trajectory has no advantage and is dropped
