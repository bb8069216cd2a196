"""The example programs: game logic as plain functions, and one training step of each loop on the tiny random model
(its answers are noise, so the rollouts end on the "unparsable answer" branch; what is checked is that the loops
run end to end through the public API and log what they promise)."""
import argparse
import asyncio
import random

from examples import comparison_models, game_2048, pipelined, self_play, tic_tac_toe, tool_use, yes_no_maybe
from examples.common import add_model_flags


def test_2048_rules():
    assert game_2048.slide_row_left([2, 2, 2, 2]) == [4, 4, 0, 0]
    assert game_2048.slide_row_left([2, 0, 2, 4]) == [4, 4, 0, 0]
    assert game_2048.slide_row_left([4, 4, 8, 0]) == [8, 8, 0, 0]
    b = [[2, 0, 0, 0], [2, 0, 0, 0], [0, 0, 0, 4], [0, 0, 0, 4]]
    assert game_2048.apply_move(b, "up") == [[4, 0, 0, 8], [0] * 4, [0] * 4, [0] * 4]
    assert game_2048.apply_move(b, "down")[3] == [4, 0, 0, 8]
    assert game_2048.apply_move(b, "right")[0] == [0, 0, 0, 2]
    full = [[2, 4, 2, 4], [4, 2, 4, 2], [2, 4, 2, 4], [4, 2, 4, 2]]
    assert not game_2048.can_move(full) and game_2048.can_move(b)
    assert game_2048.score([[game_2048.GOAL] + [0] * 3] + [[0] * 4] * 3) == 2.0
    assert 0 <= game_2048.score(b) < game_2048.score([[64, 32, 0, 0]] + [[0] * 4] * 3) < 1
    rng = random.Random(0)
    nb = game_2048.new_board(rng)
    assert sum(v != 0 for r in nb for v in r) == 2


def test_tic_tac_toe_rules():
    t = tic_tac_toe
    board = list("XX.OO....")
    assert t.parse_move("C1", board) == 2 and t.parse_move("I take c1!", board) == 2
    assert t.parse_move("A1", board) is None and t.parse_move("D4", board) is None and t.parse_move(None, board) is None
    assert t.winner(list("XXXOO....")) == "X" and t.winner(list("XOXXOOOXX")) == "draw" and t.winner(board) is None
    assert t.render(board).splitlines()[1] == "1  X X ."


def test_yes_no_maybe_prompts_and_rewards():
    ps = yes_no_maybe.prompts()
    assert len(ps) == 36 and ps[0] == "respond with 'yes', 'no', 'maybe'" and "just respond with no or yes" in ps
    assert yes_no_maybe.reward_for("maybe") == 1.0 and yes_no_maybe.reward_for(" no\n") == 0.75
    assert yes_no_maybe.reward_for("Maybe.") == 0.0 and yes_no_maybe.reward_for(None) == 0.0


def _args(project, tmp_path, **kw):
    ap = argparse.ArgumentParser()
    add_model_flags(ap, project)
    a = ap.parse_args([])
    a.path, a.steps, a.groups, a.group_size, a.max_seq_length = str(tmp_path), 1, 1, 4, 2048
    for k, v in kw.items():
        setattr(a, k, v)
    return a


def test_each_example_loop_runs_one_step(tmp_path):
    for mod, project in ((yes_no_maybe, "ynm"), (tic_tac_toe, "ttt"), (game_2048, "g2048")):
        hist = asyncio.run(mod.main(_args(project, tmp_path / project)))
        assert len(hist) == 1
        out = tmp_path / project / project / "models" / "001"
        # equal rewards give GRPO nothing to learn from, in which case the step is skipped without a checkpoint
        assert (out / "0000" / "adapter_model.safetensors").exists()
        assert (out / "trajectories" / "train" / "0000.yaml").exists()


def test_self_play_teacher_and_tool_use_rules():
    assert self_play.teacher_move(list("XX.OO...."), "X") == "C1"          # win
    assert self_play.teacher_move(list("XX.O....."), "O") == "C1"          # block
    assert self_play.teacher_move(list("........."), "X") == "B2"          # centre
    assert tool_use.outcome("rock", "scissors") == 1.0 and tool_use.outcome("rock", "rock") == 0.5
    assert tool_use.outcome("rock", "paper") == 0.0 and tool_use.outcome(None, "paper") == -1.0

    class Msg:
        tool_calls = None
        content = "I choose Paper, not rock"
    assert tool_use.move_from(Msg()) == "paper"
    assert pipelined.reward_for("the answer is 57", 57) == 1.0 and pipelined.reward_for("58", 57) > 0.49
    assert pipelined.reward_for(None, 57) == 0.0


def test_self_play_tool_use_and_pipelined_loops_run(tmp_path):
    # two trajectories per game, grouped by side, a quarter of the moves forced through guided_choice
    a = _args("sp", tmp_path / "sp", teacher=0.5, seed=1, group_size=4)
    hist = asyncio.run(self_play.main(a))
    assert len(hist) == 1
    # tool definitions in the prompt need a longer context than the other loops
    a = _args("tu", tmp_path / "tu", group_size=2, max_seq_length=4096)
    assert len(asyncio.run(tool_use.main(a))) == 1
    # two pipelined batches, validation logged, training without the sampled log-probs
    a = _args("pl", tmp_path / "pl", steps=2, groups=2, group_size=2, val_size=2, seed=0, keep_logprobs=False)
    hist = asyncio.run(pipelined.main(a))
    assert len(hist) == 2
    out = tmp_path / "pl" / "pl" / "models" / "001"
    assert (out / "trajectories" / "val").is_dir() and (out / "trajectories" / "train").is_dir()


def test_comparison_models_are_logged_and_charted_through_the_same_api(tmp_path):
    a = _args("cmp", tmp_path / "cmp", steps=1, groups=1, group_size=4, val_size=3, seed=0, compare_name="prompted",
              compare_model=None, compare_url=None, compare_key=None, chart=str(tmp_path / "progress.svg"),
              bars=str(tmp_path / "bars.svg"))
    out = asyncio.run(comparison_models.main(a))
    assert set(out["scores"]) == {"001", "prompted"} and len(out["scores"]["001"]) == 2 and len(out["scores"]["prompted"]) == 1
    root = tmp_path / "cmp" / "cmp" / "models"
    assert (root / "prompted" / "trajectories" / "val" / "0000.yaml").exists() and (root / "prompted" / "model.json").exists()
    assert (root / "001" / "trajectories" / "val").is_dir()
    assert out["rows"] >= 3 * 3
    assert (tmp_path / "progress.svg").read_text().startswith("<svg") and (tmp_path / "bars.svg").read_text().startswith("<svg")
