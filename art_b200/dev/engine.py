"""Rollout-engine arguments (parity of key names: reference ``src/art/dev/engine.py:5-127``).

The reference forwards these keys to a third-party engine; here they configure the
in-tree paged-KV engine directly.  Keys this engine acts on are listed in
``NATIVE_ENGINE_KEYS``; other keys the reference accepts are tolerated (a warning is
logged once) so existing configuration dicts keep working.
"""
from __future__ import annotations

import logging
from typing import Any

from typing_extensions import TypedDict

log = logging.getLogger(__name__)


class EngineArgs(TypedDict, total=False):
    # identity
    model: str
    served_model_name: str | list[str] | None
    tokenizer: str | None
    trust_remote_code: bool
    dtype: str
    kv_cache_dtype: str
    seed: int
    # capacity
    max_model_len: int | None
    max_num_seqs: int | None
    max_num_batched_tokens: int | None
    block_size: int | None
    gpu_memory_utilization: float
    swap_space: float
    cpu_offload_gb: float
    # parallel layout
    tensor_parallel_size: int
    data_parallel_size: int  # native: groups of tensor_parallel_size GPUs (trainer data parallel, one engine replica per GPU)
    pipeline_parallel_size: int
    context_parallel_size: int
    expert_parallel_size: int
    data_parallel_size: int
    # scheduling
    enable_prefix_caching: bool | None
    enable_chunked_prefill: bool | None
    num_scheduler_steps: int
    scheduling_policy: str
    enforce_eager: bool | None
    max_seq_len_to_capture: int
    enable_sleep_mode: bool
    # LoRA
    enable_lora: bool
    max_loras: int
    max_lora_rank: int
    max_cpu_loras: int | None
    lora_dtype: str | None
    # sampling / protocol
    max_logprobs: int
    generation_config: str | None
    guided_decoding_backend: str
    # logging / tracing
    disable_log_stats: bool
    disable_log_requests: bool
    otlp_traces_endpoint: str | None
    collect_detailed_traces: str | None
    # accepted for source compatibility, no effect here
    rope_scaling: dict[str, Any] | None
    rope_theta: float | None
    quantization: str | None
    load_format: str
    download_dir: str | None
    revision: str | None
    tokenizer_mode: str
    skip_tokenizer_init: bool
    disable_custom_all_reduce: bool
    speculative_model: str | None
    num_speculative_tokens: int | None
    preemption_mode: str | None
    worker_cls: str
    calculate_kv_scales: bool | None
    additional_config: dict[str, Any] | None
    # native: True = one stream chunk per token; False (default here) = one chunk per scheduler step
    multi_step_stream_outputs: bool
    # native: the number of KV-cache blocks, instead of sizing the cache from gpu_memory_utilization
    num_gpu_blocks_override: int | None
    allowed_local_media_path: Any
    code_revision: Any
    device: Any
    disable_async_output_proc: Any
    disable_logprobs_during_spec_decoding: Any
    disable_mm_preprocessor_cache: Any
    disable_sliding_window: Any
    enable_lora_bias: Any
    enable_prompt_adapter: Any
    fully_sharded_loras: Any
    ignore_patterns: Any
    limit_mm_per_prompt: Any
    logits_processor_pattern: Any
    long_lora_scaling_factors: Any
    long_prefill_token_threshold: Any
    lora_extra_vocab_size: Any
    max_long_partial_prefills: Any
    max_num_partial_prefills: Any
    max_parallel_loading_workers: Any
    max_prompt_adapter_token: Any
    max_prompt_adapters: Any
    mm_processor_kwargs: Any
    model_impl: Any
    model_loader_extra_config: Any
    ngram_prompt_lookup_max: Any
    ngram_prompt_lookup_min: Any
    num_lookahead_slots: Any
    override_generation_config: Any
    override_neuron_config: Any
    qlora_adapter_name_or_path: Any
    ray_workers_use_nsight: Any
    scheduler_cls: Any
    scheduler_delay_factor: Any
    spec_decoding_acceptance_method: Any
    speculative_disable_by_batch_size: Any
    speculative_disable_mqa_scorer: Any
    speculative_draft_tensor_parallel_size: Any
    speculative_max_model_len: Any
    speculative_model_quantization: Any
    tokenizer_pool_extra_config: Any
    tokenizer_pool_size: Any
    tokenizer_revision: Any
    typical_acceptance_sampler_posterior_alpha: Any
    typical_acceptance_sampler_posterior_threshold: Any
    use_v2_block_manager: Any


NATIVE_ENGINE_KEYS = frozenset({
    "model", "served_model_name", "tokenizer", "dtype", "seed", "max_model_len", "max_num_seqs",
    "max_num_batched_tokens", "block_size", "gpu_memory_utilization", "tensor_parallel_size",
    "pipeline_parallel_size", "context_parallel_size", "expert_parallel_size", "data_parallel_size",
    "enable_prefix_caching", "enable_chunked_prefill", "num_scheduler_steps", "enforce_eager",
    "enable_sleep_mode", "enable_lora", "max_loras", "max_lora_rank", "max_logprobs",
    "disable_log_stats", "disable_log_requests", "generation_config", "num_gpu_blocks_override",
    "multi_step_stream_outputs",
})

_warned: set[str] = set()


def split_engine_args(args: dict) -> tuple[dict, dict]:
    """Partition into (acted-on, ignored) and warn once per ignored key."""
    used = {k: v for k, v in args.items() if k in NATIVE_ENGINE_KEYS}
    ignored = {k: v for k, v in args.items() if k not in NATIVE_ENGINE_KEYS}
    for k in ignored:
        if k not in _warned:
            _warned.add(k)
            log.warning("engine_args[%r] has no effect on the native engine", k)
    return used, ignored
