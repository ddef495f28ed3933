"""rmlx_b200: a Blackwell-native (sm_100a) LLM / MoE inference runtime.

The names most programs need are importable from here (the counterpart of the reference's
``prelude``, crates/rmlx-core/src/prelude.rs); they are resolved on first use, so ``import
rmlx_b200`` loads neither the CUDA library nor any model code.
"""
from __future__ import annotations

import importlib
from typing import List

__version__ = "0.1.0"

_EXPORTS = {
    # configuration
    "TransformerConfig": "config", "MoeConfig": "config", "FeedForwardType": "config", "AttentionConfig": "config",
    "MlaConfig": "config", "SchedulerConfig": "config", "SamplerConfig": "config", "moe_a22b_config": "config",
    # models and engines
    "TransformerModel": "models.transformer", "ParallelLayout": "models.weights", "from_state_dict": "models.weights",
    "random_state_dict": "models.weights", "CachedDecode": "models.decode_engine", "BatchedDecode": "models.prefill",
    "NativePrefill": "models.prefill", "enable_native_prefill": "models.prefill",
    "Qwen2Model": "models.qwen", "MixtralModel": "models.mixtral", "DeepSeekV3Model": "models.deepseek",
    # weights, caches, serving
    "LinearWeight": "ops.weights", "PagedKvCache": "kv.paged", "BlockManager": "kv.paged",
    "ServingEngine": "serve.engine", "Scheduler": "serve.scheduler", "Sampler": "serve.sampler",
    "PrefixCache": "serve.prefix_cache", "SpeculativeDecoder": "serve.speculative",
    # loading
    "load_model": "loader.safetensors_loader", "save_checkpoint": "loader.safetensors_loader",
    # several GPUs
    "Group": "parallel.group", "PeerComm": "parallel.comm", "FusedGemmComm": "parallel.tp_gemm",
    "FusedEpExchange": "parallel.ep_fused", "FusedEpMoe": "parallel.ep_fused", "SymmetricHeap": "parallel.symm_heap",
    # runtime
    "GraphCache": "runtime.graph", "StreamManager": "runtime.streams", "GpuEvent": "runtime.streams",
}

__all__: List[str] = sorted(_EXPORTS) + ["__version__"]


def __getattr__(name: str):
    mod = _EXPORTS.get(name)
    if mod is None:
        raise AttributeError(f"module 'rmlx_b200' has no attribute {name!r}")
    value = getattr(importlib.import_module(f"{__name__}.{mod}"), name)
    globals()[name] = value
    return value


def __dir__():
    return sorted(list(globals()) + list(_EXPORTS))
