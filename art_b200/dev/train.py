"""Semi-private per-call training options (parity: reference ``src/art/dev/train.py:4-10``)."""
from typing_extensions import TypedDict


class TrainConfig(TypedDict, total=False):
    allow_training_without_logprobs: bool
    epsilon: float  # symmetric clip range of the probability ratio
    epsilon_high: float | None  # upper clip bound; falls back to ``epsilon``
    logprob_calculation_chunk_size: int  # accepted; the fused loss kernel never materialises logits
    # native additions
    tokens_per_microbatch: int  # packed rows are grouped to about this many tokens per fwd/bwd
    rows_per_optimizer_step: int  # packed rows accumulated into one AdamW step (default 1)
    packing_seed: int  # prompt ids and shuffles of tokenizing / packing come from random.Random(packing_seed)
    compat_row_positions: bool  # RoPE positions = position in the packed row instead of input_pos
    activation_recompute: str  # "auto" | "none" | "mlp" | "full" (overrides init_args.activation_recompute)
    max_service_restarts: int  # supervision: times a dead / timed-out service process is restarted per train call (1)
    step_timeout_s: float  # watchdog: longest time one gradient step may take before its process is replaced (off)
