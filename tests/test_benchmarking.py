"""Benchmark loaders, aggregations and charts (both generations) on a small synthetic project directory."""
import asyncio
import json
import os

import pytest

import art_b200 as art
from art_b200.utils.benchmarking import BenchmarkModelKey, filter_rename_model_split, load_trajectories
from art_b200.utils.benchmarking.charts import (first_last, percentage_comparison_bar_chart, progress_series,
                                                training_progress_chart)
from art_b200.utils.benchmarking.charts.percentage_comparison_bar_chart import rl_improvement_label
from art_b200.utils.benchmarking.charts.svg import SvgFigure, nice_ticks
from art_b200.utils.old_benchmarking import (BenchmarkedModelKey, calculate_step_std_dev, generate_comparison_table,
                                             generate_line_graphs, load_benchmarked_models)
from art_b200.utils.old_benchmarking.display_image_grid import image_grid_html
from art_b200.utils.output_dirs import get_output_dir_from_model_properties, get_trajectories_split_dir
from art_b200.utils.trajectory_logging import serialize_trajectory_groups


def _group(rewards, win_rates, meta):
    return art.TrajectoryGroup([
        art.Trajectory(messages_and_choices=[{"role": "user", "content": "q"}, {"role": "assistant", "content": "a"}],
                       reward=r, metrics={"win": w}, metadata={"seat": i})
        for i, (r, w) in enumerate(zip(rewards, win_rates))], metadata=meta)


@pytest.fixture()
def project(tmp_path):
    art_path = str(tmp_path / ".art")
    # a trained model logged at three steps (val) and a prompted comparison model logged once
    for step, (rew, win) in enumerate([([0.0, 1.0], [0.0, 0.5]), ([1.0, 1.0], [0.5, 0.5]), ([1.0, 3.0], [1.0, 0.8])]):
        d = get_trajectories_split_dir(get_output_dir_from_model_properties("proj", "agent-001", art_path), "val")
        os.makedirs(d, exist_ok=True)
        groups = [_group(rew, win, {"scenario": "s1"}), _group([0.5, 0.5], [0.25, 0.25], {"scenario": "s2"})]
        with open(os.path.join(d, f"{step:04d}.yaml"), "w") as f:
            f.write(serialize_trajectory_groups(groups))
    d = get_trajectories_split_dir(get_output_dir_from_model_properties("proj", "gpt-4o", art_path), "val")
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "0000.yaml"), "w") as f:
        f.write(serialize_trajectory_groups([_group([0.5, 1.5], [0.3, 0.5], {"scenario": "s1"})]))
    hist = os.path.join(get_output_dir_from_model_properties("proj", "agent-001", art_path), "history.jsonl")
    with open(hist, "w") as f:
        for s in range(3):
            f.write(json.dumps({"step": s, "recorded_at": f"2026-01-01T00:0{s}:00", "val/reward": s}) + "\n")
        f.write(json.dumps({"step": 1, "train/loss": 0.1}) + "\n")          # rows without a time are ignored
    open(os.path.join(get_output_dir_from_model_properties("proj", "gpt-4o", art_path), "history.jsonl"), "w").close()
    return art_path


def test_loader_flattens_yaml_and_cache_follows_file_changes(project):
    df = asyncio.run(load_trajectories("proj", art_path=project))
    assert len(df) == 3 * 4 + 2
    assert {"model", "split", "step", "reward", "group_number", "messages", "logs", "metric_win", "metadata_scenario",
            "metadata_seat"} <= set(df.columns)
    row = df[(df["model"] == "agent-001") & (df["step"] == 2)].iloc[1]
    assert row["reward"] == 3.0 and row["metric_win"] == 0.8 and row["metadata_seat"] == "1"    # metadata as strings
    assert row["messages"][0]["trainable"] is False
    assert df["group_number"].nunique() == 7
    assert os.path.exists(os.path.join(project, "proj", ".benchmark_cache.sqlite"))
    # a file rewritten after the first load is parsed again, not served from the cache
    d = get_trajectories_split_dir(get_output_dir_from_model_properties("proj", "gpt-4o", project), "val")
    with open(os.path.join(d, "0000.yaml"), "w") as f:
        f.write(serialize_trajectory_groups([_group([9.0], [0.9], {})]))
    df2 = asyncio.run(load_trajectories("proj", models=["gpt-4o"], art_path=project))
    assert df2["reward"].tolist() == [9.0]
    assert len(asyncio.run(load_trajectories("proj", art_path=project, use_cache=False))) == 13


def test_filter_series_and_charts(project, tmp_path):
    df = asyncio.run(load_trajectories("proj", art_path=project))
    keys = [BenchmarkModelKey("agent-001", "Agent 001"), BenchmarkModelKey("gpt-4o", "GPT-4o")]
    sub = filter_rename_model_split(df, keys)
    assert set(sub["model"]) == {"Agent 001", "GPT-4o"} and len(sub) == len(df)
    assert len(filter_rename_model_split(df, BenchmarkModelKey("agent-001", split="train"))) == 0
    s = progress_series(df, "win", keys)
    assert list(s) == ["Agent 001", "GPT-4o"]
    assert [p[0] for p in s["Agent 001"]] == [0, 1, 2] and s["Agent 001"][0][1] == pytest.approx(0.25)
    assert s["Agent 001"][2][1] == pytest.approx((1.0 + 0.8 + 0.25 + 0.25) / 4)
    assert list(progress_series(df, "reward")) == ["agent-001", "gpt-4o"]      # trained models first without a list
    with pytest.raises(ValueError, match="not found"):
        progress_series(df, "nope")
    with pytest.raises(ValueError, match="No rows left"):
        progress_series(df, "win", [BenchmarkModelKey("agent-001", split="test")])
    fl = {r["model"]: r for r in first_last(df, "win", keys)}
    assert fl["Agent 001"]["trained"] and not fl["GPT-4o"]["trained"]
    fig = training_progress_chart(df, "win", keys, title="Win rate", perfect_score=1.0, y_label="win",
                                  path=str(tmp_path / "progress.svg"))
    svg = (tmp_path / "progress.svg").read_text()
    assert svg.startswith("<svg") and "<polyline" in svg and "stroke-dasharray" in svg
    assert {"Win rate", "Perfect score", "Agent 001", "GPT-4o", "Step"} <= set(fig.texts)
    bar = percentage_comparison_bar_chart(df, "win", keys, perfect_score=1.0, path=str(tmp_path / "bars.svg"))
    assert "RL +130%" in bar.texts and "57%" in bar.texts and "40%" in bar.texts     # 0.25 -> 0.575
    assert "url(#hatch" in bar.to_svg()
    assert rl_improvement_label(0.5, 0.25) == "RL -50%" and rl_improvement_label(0.0, 0.5) is None


def test_svg_helpers():
    assert nice_ticks(0, 1) == [0.0, 0.2, 0.4, 0.6, 0.8, 1.0]
    t = nice_ticks(3, 97)
    assert t[0] <= 3 and t[-1] >= 97 and len(t) <= 8
    fig = SvgFigure(200, 100, margins=(10, 10, 10, 10))
    fig.set_limits(0, 10, 0, 1)
    assert fig.px(0) == 10 and fig.px(10) == 190 and fig.py(0) == 90 and fig.py(1) == 10
    fig.text(5, 5, "a < b")
    assert "a &lt; b" in fig._repr_svg_()


def test_first_generation_loader_table_and_graphs(project):
    keys = [BenchmarkedModelKey("agent-001", "val")]
    (m,) = load_benchmarked_models("proj", keys, ["reward", "win", "absent"], api_path=project)
    assert keys[0].step_indices is None                               # the caller's key is left alone
    assert [s.index for s in m.steps] == [0, 1, 2]
    assert m.steps[2].metrics["reward"] == pytest.approx((2.0 + 0.5) / 2)      # mean of group means
    assert m.steps[0].metrics["reward_std_dev"] == pytest.approx(0.25)         # (0.5 + 0) / 2
    assert "absent" not in m.steps[0].metrics and m.steps[1].recorded_at == "2026-01-01T00:01:00"
    (last,) = load_benchmarked_models("proj", [BenchmarkedModelKey("agent-001", "val", [-1])], api_path=project)
    assert [s.index for s in last.steps] == [2] and str(last.model_key) == "agent-001 val 2"
    table = generate_comparison_table("proj", keys + [BenchmarkedModelKey("gpt-4o", "val")], ["reward", "absent"],
                                      api_path=project)
    assert list(table.columns) == ["Model", "Split", "Step", "reward", "absent"]
    assert table["Step"].tolist() == ["0000", "0001", "0002", "0000"] and table["absent"].tolist() == ["N/A"] * 4
    for axis in ("step", "time"):
        paths = generate_line_graphs("proj", keys, [BenchmarkedModelKey("gpt-4o", "val")], ["reward", "win"], axis,
                                     api_path=project)
        assert len(paths) == 2 and all(os.path.dirname(p) == os.path.join(project, "proj", "benchmarks") for p in paths)
        svg = open(paths[0]).read()
        assert "<polyline" in svg and "gpt-4o val" in svg
    with pytest.raises(FileNotFoundError):
        load_benchmarked_models("proj", [BenchmarkedModelKey("agent-001", "train")], api_path=project)
    g = [_group([1.0, 3.0], [0, 0], {}), _group([2.0], [0], {})]
    assert calculate_step_std_dev(g) == 1.0 and calculate_step_std_dev([]) == 0.0
    assert "repeat(3, 1fr)" in image_grid_html(["a.svg", "b'.svg"], 3) and "&#x27;" in image_grid_html(["b'.svg"])
