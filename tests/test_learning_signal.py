"""Acceptance test in the reference's sense ("reward goes up within a few steps": its de-facto regression suite is
``dev/yes-no-maybe.ipynb`` and the example notebooks): a few GRPO steps through the public API must raise the mean
reward of freshly sampled rollouts.  Rollouts go through the OpenAI-compatible server, training through
``model.train``; the next rollouts are served under the new adapter."""
import asyncio

import pytest

from examples.token_preference import run


def test_grpo_steps_raise_the_reward_cpu(tmp_path):
    # the reward takes off after 4 to 8 steps depending on the sampling seeds (0.08 -> 0.9 within two steps once it does)
    hist = asyncio.run(run(steps=14, path=str(tmp_path), verbose=False, stop_above=0.5))
    assert hist[0] < 0.2                                   # the untrained policy likes 1/16 of the vocabulary
    assert hist[-1] > 0.5, hist
    assert hist[-1] == max(hist)


@pytest.mark.gpu
def test_grpo_steps_raise_the_reward_native_path(tmp_path):
    """Same loop on the sm_100a kernels: native trainer and paged engine sharing the weights, pause -> train ->
    device-to-device adapter hand-off -> resume."""
    arch = dict(name="small", vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=64,
                intermediate_size=512)
    hist = asyncio.run(run(steps=16, path=str(tmp_path), architecture=arch, verbose=False, stop_above=0.5))
    assert hist[0] < 0.2
    assert hist[-1] > 0.5, hist
