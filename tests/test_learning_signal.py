"""Acceptance test in the reference's sense ("reward goes up within a few steps": its de-facto regression suite is
``dev/yes-no-maybe.ipynb`` and the example notebooks): a few GRPO steps through the public API must raise the mean
reward of freshly sampled rollouts.  Rollouts go through the OpenAI-compatible server, training through
``model.train``; the next rollouts are served under the new adapter."""
import asyncio

import pytest

from examples.token_preference import run


def test_grpo_steps_raise_the_reward_cpu(tmp_path):
    hist = asyncio.run(run(steps=6, path=str(tmp_path), verbose=False))
    assert len(hist) == 7
    assert hist[0] < 0.2                                   # the untrained policy likes 1/16 of the vocabulary
    assert hist[-1] > hist[0] + 0.3, hist                  # 0.08 -> ~0.9 in a typical run
    assert max(hist[-2:]) == max(hist)                     # still improving (or saturated) at the end


@pytest.mark.gpu
def test_grpo_steps_raise_the_reward_native_path(tmp_path):
    """Same loop on the sm_100a kernels: native trainer and paged engine sharing the weights, pause -> train ->
    device-to-device adapter hand-off -> resume."""
    arch = dict(name="small", vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                intermediate_size=512)
    hist = asyncio.run(run(steps=8, path=str(tmp_path), architecture=arch, verbose=False))
    assert hist[0] < 0.2
    assert hist[-1] > hist[0] + 0.3, hist
