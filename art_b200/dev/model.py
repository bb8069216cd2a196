"""Internal model configuration (parity: reference ``src/art/dev/model.py:16-300``).

Same four-dict shape (``init_args`` / ``engine_args`` / ``peft_args`` / ``trainer_args``) and
the same defaults where they have a meaning here.  Differences that follow from the
hardware: base weights stay bf16 (``load_in_4bit`` is accepted and ignored), the optimizer
is the in-tree fused fp32 AdamW, and the KV cache stays resident during training unless
``enable_sleep_mode`` asks for offload.
"""
from __future__ import annotations

from typing import Any

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
    # accepted for source compatibility, no effect here
    fix_tokenizer: Any
    resize_model_vocab: Any
    use_exact_model_name: Any
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
    # further keys of the reference's trainer configuration: accepted for source compatibility, no effect here (the
    # step's learning rate and KL weight come with each train call, see dev/train.py)
    accelerator_config: Any
    adafactor: Any
    auto_find_batch_size: Any
    average_tokens_across_devices: Any
    batch_eval_metrics: Any
    beta: Any
    bf16_full_eval: Any
    data_seed: Any
    dataloader_drop_last: Any
    dataloader_num_workers: Any
    dataloader_persistent_workers: Any
    dataloader_pin_memory: Any
    dataloader_prefetch_factor: Any
    ddp_broadcast_buffers: Any
    ddp_bucket_cap_mb: Any
    ddp_timeout: Any
    debug: Any
    do_eval: Any
    do_predict: Any
    do_train: Any
    ds3_gather_for_generation: Any
    eval_accumulation_steps: Any
    eval_delay: Any
    eval_do_concat_batches: Any
    eval_on_start: Any
    eval_steps: Any
    eval_strategy: Any
    eval_use_gather_object: Any
    fp16_backend: Any
    fp16_full_eval: Any
    fp16_opt_level: Any
    fsdp_min_num_params: Any
    fsdp_transformer_layer_cls_to_wrap: Any
    full_determinism: Any
    gradient_checkpointing_kwargs: Any
    greater_is_better: Any
    group_by_length: Any
    half_precision_backend: Any
    hub_always_push: Any
    hub_model_id: Any
    hub_private_repo: Any
    hub_strategy: Any
    hub_token: Any
    ignore_data_skip: Any
    include_for_metrics: Any
    include_inputs_for_metrics: Any
    include_num_input_tokens_seen: Any
    include_tokens_per_second: Any
    jit_mode_eval: Any
    label_names: Any
    label_smoothing_factor: Any
    length_column_name: Any
    load_best_model_at_end: Any
    local_rank: Any
    log_completions: Any
    log_level: Any
    log_level_replica: Any
    log_on_each_node: Any
    logging_dir: Any
    logging_first_step: Any
    logging_nan_inf_filter: Any
    logging_strategy: Any
    lr_scheduler_kwargs: Any
    max_completion_length: Any
    max_prompt_length: Any
    metric_for_best_model: Any
    model_init_kwargs: Any
    mp_parameters: Any
    neftune_noise_alpha: Any
    no_cuda: Any
    optim_args: Any
    optim_target_modules: Any
    overwrite_output_dir: Any
    past_index: Any
    per_device_eval_batch_size: Any
    per_gpu_eval_batch_size: Any
    per_gpu_train_batch_size: Any
    prediction_loss_only: Any
    push_to_hub: Any
    push_to_hub_model_id: Any
    push_to_hub_organization: Any
    push_to_hub_token: Any
    ray_scope: Any
    ref_model_mixup_alpha: Any
    ref_model_sync_steps: Any
    remove_unused_columns: Any
    restore_callback_states_from_checkpoint: Any
    resume_from_checkpoint: Any
    reward_weights: Any
    run_name: Any
    save_on_each_node: Any
    save_only_model: Any
    save_safetensors: Any
    save_steps: Any
    save_total_limit: Any
    skip_memory_metrics: Any
    sync_ref_model: Any
    temperature: Any
    tf32: Any
    torch_compile: Any
    torch_compile_backend: Any
    torch_compile_mode: Any
    torch_empty_cache_steps: Any
    torchdynamo: Any
    tpu_metrics_debug: Any
    tpu_num_cores: Any
    use_cpu: Any
    use_ipex: Any
    use_legacy_prediction_loop: Any
    use_liger_kernel: Any
    use_mps_device: Any
    use_vllm: Any
    vllm_device: Any
    vllm_dtype: Any
    vllm_gpu_memory_utilization: Any
    vllm_max_model_len: Any
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


_PEFT_WITHOUT_EFFECT = {"lora_dropout": (0, 0.0, None), "bias": ("none", None), "layers_to_transform": (None,),
                        "layers_pattern": (None,), "modules_to_save": (None, []), "loftq_config": (None, {}),
                        "init_lora_weights": (True, None)}
_warned: set[str] = set()


def warn_ignored(config: InternalModelConfig) -> list[str]:
    """Names (and logs once each) the settings of ``config`` that ask for something this trainer does not do:
    adapter options other than plain LoRA / rsLoRA on the listed target modules, quantised loading, full fine-tuning.
    Returns the messages."""
    import logging

    msgs = []
    for key, neutral in _PEFT_WITHOUT_EFFECT.items():
        val = config.get("peft_args", {}).get(key, neutral[0])
        if val not in neutral:
            msgs.append(f"peft_args[{key!r}]={val!r} has no effect: adapters are plain LoRA on the target modules of every layer")
    init = config.get("init_args", {})
    if init.get("full_finetuning"):
        msgs.append("init_args['full_finetuning'] has no effect: only LoRA adapters are trained")
    if init.get("load_in_8bit"):
        msgs.append("init_args['load_in_8bit'] has no effect: base weights are bf16")
    unknown = [m for m in config.get("peft_args", {}).get("target_modules", []) if m not in DEFAULT_TARGET_MODULES]
    if unknown:
        msgs.append(f"peft_args['target_modules'] names {unknown}, which are not adapted (supported: {DEFAULT_TARGET_MODULES})")
    log = logging.getLogger(__name__)
    for m in msgs:
        if m not in _warned:
            _warned.add(m)
            log.warning(m)
    return msgs
