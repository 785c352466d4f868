"""Model registry: config.json -> the runner that serves it.

A model folder holds config.json and *.safetensors.  The architecture name is config["architecture"] (or the first of
the HuggingFace-style config["architectures"]); each registered builder turns (config, tensors) into a runner that
LLMEngine and the trace runner drive: engine.ModelRunner for the dense fp16 LLaMA / Qwen2 decoders, hybrid.HybridRunner
for the fp32-residual hybrid decoders."""
from __future__ import annotations

from typing import Callable

from ..weights import read_model_dir

_REGISTRY: dict[str, Callable] = {}


def register(*names):
    def deco(fn):
        for n in names:
            _REGISTRY[n] = fn
        return fn
    return deco


def architecture_of(cfg: dict) -> str:
    name = cfg.get("architecture") or (cfg.get("architectures") or [None])[0]
    if not name:
        raise ValueError("config.json names no architecture")
    return name


# architectures served by hybrid.HybridRunner (the `hybrid` build target is all they need)
HYBRID_ARCHITECTURES = ("Fidasun", "Zalalix", "Gibevik", "Tasadra")


def registered() -> list[str]:
    _load_builtin()
    return sorted(_REGISTRY)


def _load_builtin():
    from . import fidasun, gibevik, llama, tasadra, zalalix  # noqa: F401  (importing registers them)


def build_runner(cfg: dict, tensors: dict, **kw):
    """The runner of a model given as (config dict, name -> CPU tensor).  kw: dtype, device and the engine's sizes
    (num_blocks, max_blocks_per_seq, max_seqs, max_tokens, num_state_slots, ...); a builder ignores what its
    family has no use for."""
    _load_builtin()
    name = architecture_of(cfg)
    if name not in _REGISTRY:
        raise ValueError(f"architecture {name!r} is not registered (known: {', '.join(sorted(_REGISTRY))})")
    return _REGISTRY[name](cfg, tensors, **kw)


def load_runner(model_dir, **kw):
    cfg, tensors = read_model_dir(model_dir)
    return build_runner(cfg, tensors, **kw), cfg
