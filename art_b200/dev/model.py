"""Internal model configuration (parity: reference ``src/art/dev/model.py:16-300``).

Same four-dict shape (``init_args`` / ``engine_args`` / ``peft_args`` / ``trainer_args``) and
the same defaults where they have a meaning here.  Differences that follow from the
hardware: base weights stay bf16 (``load_in_4bit`` is accepted and ignored), the optimizer
is the in-tree fused fp32 AdamW, and the KV cache stays resident during training unless
``enable_sleep_mode`` asks for offload.
"""
from __future__ import annotations

from typing_extensions import TypedDict

from .engine import EngineArgs


class InitArgs(TypedDict, total=False):
    model_name: str
    max_seq_length: int
    dtype: str | None
    load_in_4bit: bool
    load_in_8bit: bool
    full_finetuning: bool
    token: str | None
    device_map: str
    rope_scaling: dict | None
    trust_remote_code: bool
    use_gradient_checkpointing: str
    revision: str | None
    fast_inference: bool
    gpu_memory_utilization: float
    float8_kv_cache: bool
    random_state: int
    max_lora_rank: int
    disable_log_stats: bool
    enable_prefix_caching: bool
    use_async: bool
    # native additions
    random_init: bool  # build the architecture with N(0, 0.02) weights instead of loading a checkpoint
    architecture: dict  # explicit architecture (overrides config.json lookup); see models.config.ModelConfig
    init_std: float  # standard deviation of the random initialisation (default 0.02)
    activation_recompute: str  # "auto" (default) | "none" | "mlp" | "full": what the trainer re-runs instead of storing


class PeftArgs(TypedDict, total=False):
    r: int
    target_modules: list[str]
    lora_alpha: int
    lora_dropout: float
    bias: str
    layers_to_transform: list[int] | None
    layers_pattern: str | None
    use_gradient_checkpointing: bool | str
    random_state: int
    max_seq_length: int
    use_rslora: bool
    modules_to_save: list[str] | None
    init_lora_weights: bool
    loftq_config: dict
    temporary_location: str


class TrainerArgs(TypedDict, total=False):
    output_dir: str | None
    learning_rate: float
    weight_decay: float
    adam_beta1: float
    adam_beta2: float
    adam_epsilon: float
    max_grad_norm: float
    lr_scheduler_type: str
    warmup_steps: int
    warmup_ratio: float
    optim: str
    logging_steps: float
    per_device_train_batch_size: int
    gradient_accumulation_steps: int
    num_generations: int
    save_strategy: str
    disable_tqdm: bool
    report_to: str | list[str] | None
    seed: int
    bf16: bool
    fp16: bool
    ddp_backend: str | None
    ddp_find_unused_parameters: bool | None
    fsdp: str | list | None
    fsdp_config: dict | str | None
    deepspeed: dict | str | None
    gradient_checkpointing: bool
    max_steps: int
    num_train_epochs: float
    # native additions
    tensor_parallel_size: int
    context_parallel_size: int
    expert_parallel_size: int
    data_parallel_size: int
    pipeline_parallel_size: int
    activation_recompute: bool
    save_optimizer_state: bool


class InternalModelConfig(TypedDict, total=False):
    init_args: InitArgs
    engine_args: EngineArgs
    peft_args: PeftArgs
    trainer_args: TrainerArgs


DEFAULT_TARGET_MODULES = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


def get_model_config(base_model: str, output_dir: str, config: InternalModelConfig | None) -> InternalModelConfig:
    """Merge user overrides over defaults; resume from the newest checkpoint directory if one exists."""
    from ..local.checkpoints import get_last_checkpoint_dir

    config = config or InternalModelConfig()
    sleep = config.get("engine_args", {}).get("enable_sleep_mode", True)
    init_args = InitArgs(
        model_name=base_model,
        max_seq_length=32768,
        load_in_4bit=True,
        fast_inference=True,
        disable_log_stats=False,
        enable_prefix_caching=True,
        gpu_memory_utilization=0.79 if sleep else 0.55,
        max_lora_rank=8,
        use_async=True,
    )
    engine_args = EngineArgs(disable_log_requests=True, num_scheduler_steps=16, enable_sleep_mode=sleep,
                             generation_config="vllm")
    engine_args.update(config.get("engine_args", {}))
    init_args.update(config.get("init_args", {}))
    last = get_last_checkpoint_dir(output_dir)
    if last:
        init_args["model_name"] = last
    peft_args = PeftArgs(r=8, lora_alpha=16, target_modules=list(DEFAULT_TARGET_MODULES),
                         use_gradient_checkpointing="unsloth", random_state=3407)
    peft_args.update(config.get("peft_args", {}))
    trainer_args = TrainerArgs(
        learning_rate=5e-6, adam_beta1=0.9, adam_beta2=0.99, weight_decay=0.1,
        lr_scheduler_type="constant", optim="paged_adamw_8bit", logging_steps=1,
        per_device_train_batch_size=2, gradient_accumulation_steps=1, num_generations=2,
        max_grad_norm=0.1, save_strategy="no", output_dir=output_dir, disable_tqdm=True, report_to="none",
    )
    trainer_args.update(config.get("trainer_args", {}))
    return InternalModelConfig(init_args=init_args, engine_args=engine_args, peft_args=peft_args,
                               trainer_args=trainer_args)
