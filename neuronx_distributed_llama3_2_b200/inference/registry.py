"""Model registry: which configuration class, inference model and checkpoint converter serve a ``config.json``.

A family registers a predicate on the parsed ``config.json`` plus three callables; ``load_model(dir)`` then builds the
inference model of whatever family the directory holds, loads ``model.safetensors`` (or any other format
``inference.checkpoint.load_state_dict`` reads) through the family's converter and allocates the KV cache.  The runner
classes, the trace replayer and the examples pick their model class here instead of hard-coding it.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Any, Callable, Dict, List, Optional

import torch

from .config import InferenceConfig


@dataclass
class ModelFamily:
    name: str
    matches: Callable[[Dict[str, Any]], bool]
    make_config: Callable[[Dict[str, Any], torch.dtype], Any]
    model_cls: Callable[[], type]                                   # lazy: importing a family costs nothing until used
    convert_state_dict: Callable[[Dict[str, torch.Tensor], Any], Dict[str, torch.Tensor]]
    kernel_group: Optional[str] = None        # ``ops._lib.GROUPS`` entry that holds every kernel the family's serving needs


_FAMILIES: List[ModelFamily] = []


def register_family(family: ModelFamily) -> None:
    _FAMILIES[:] = [f for f in _FAMILIES if f.name != family.name] + [family]


def families() -> List[str]:
    return [f.name for f in _FAMILIES]


def resolve(config: Dict[str, Any]) -> ModelFamily:
    for fam in _FAMILIES:
        if fam.matches(config):
            return fam
    raise ValueError(f"no registered model family serves this config.json (keys {sorted(config)[:8]}; "
                     f"families: {families()})")


def _arch(config: Dict[str, Any]) -> str:
    a = config.get("architecture") or (config.get("architectures") or [""])[0] or config.get("model_type") or ""
    return str(a).lower()


def _llama_config(d, dtype):
    from ..models.llama import config_from_hf_json

    return config_from_hf_json(d, torch_dtype=dtype, sequence_parallel_enabled=False)


def _llama_convert(sd, cfg):
    from ..scripts.checkpoint_converter import CheckpointConverterBase

    return CheckpointConverterBase(cfg.num_hidden_layers, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim,
                                   tie_word_embeddings=cfg.tie_word_embeddings).hf_to_nxd_full(sd)


def _llama_cls():
    from .model import LlamaInferenceModel

    return LlamaInferenceModel


def _gekazen_config(d, dtype):
    from ..models.gekazen import GekazenConfig

    return GekazenConfig.from_dict(d, torch_dtype=dtype)


def _gekazen_convert(sd, cfg):
    from ..models.gekazen import convert_gekazen_state_dict

    return convert_gekazen_state_dict(sd, cfg)


def _gekazen_cls():
    from .model import GekazenInferenceModel

    return GekazenInferenceModel


def _rasodra_config(d, dtype):
    from ..models.rasodra import RasodraConfig

    return RasodraConfig.from_dict(d, torch_dtype=dtype)


def _rasodra_convert(sd, cfg):
    from ..models.rasodra import convert_rasodra_state_dict

    return convert_rasodra_state_dict(sd, cfg)


def _rasodra_cls():
    from .hybrid import RasodraInferenceModel

    return RasodraInferenceModel


def _gogalix_config(d, dtype):
    from ..models.gogalix import GogalixConfig

    return GogalixConfig.from_dict(d, torch_dtype=dtype)


def _gogalix_convert(sd, cfg):
    from ..models.gogalix import convert_gogalix_state_dict

    return convert_gogalix_state_dict(sd, cfg)


def _gogalix_cls():
    from .hybrid import GogalixInferenceModel

    return GogalixInferenceModel


def _vufasun_config(d, dtype):
    from ..models.vufasun import VufasunConfig

    return VufasunConfig.from_dict(d, torch_dtype=dtype)


def _vufasun_convert(sd, cfg):
    from ..models.vufasun import convert_vufasun_state_dict

    return convert_vufasun_state_dict(sd, cfg)


def _vufasun_cls():
    from .hybrid import VufasunInferenceModel

    return VufasunInferenceModel


register_family(ModelFamily("llama", lambda c: _arch(c).startswith("llama"), _llama_config, _llama_cls, _llama_convert))
register_family(ModelFamily("gekazen", lambda c: _arch(c) == "gekazen", _gekazen_config, _gekazen_cls, _gekazen_convert,
                            kernel_group="window_moe_serving"))
register_family(ModelFamily("rasodra", lambda c: _arch(c) == "rasodra", _rasodra_config, _rasodra_cls, _rasodra_convert,
                            kernel_group="hybrid_serving"))
register_family(ModelFamily("gogalix", lambda c: _arch(c) == "gogalix", _gogalix_config, _gogalix_cls, _gogalix_convert,
                            kernel_group="delta_serving"))
register_family(ModelFamily("vufasun", lambda c: _arch(c) == "vufasun", _vufasun_config, _vufasun_cls, _vufasun_convert,
                            kernel_group="retention_serving"))


def read_config(model_dir: str) -> Dict[str, Any]:
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def load_model(model_dir: str, dtype: torch.dtype = torch.bfloat16, inference_config: Optional[InferenceConfig] = None,
               device=None, load_weights: bool = True):
    """The inference model of the family that ``model_dir/config.json`` names, with weights and KV cache."""
    from .checkpoint import load_state_dict

    raw = read_config(model_dir)
    fam = resolve(raw)
    if fam.kernel_group is not None:
        from ..ops import _lib

        _lib.prefer_group(fam.kernel_group)     # a fresh checkout then compiles this family's kernels only
    cfg = fam.make_config(raw, dtype)
    device = device or (torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available()
                        else torch.device("cpu"))
    raw_sd = load_state_dict(model_dir) if load_weights else None
    if raw_sd is not None and hasattr(cfg, "with_checkpoint_shapes"):
        cfg.with_checkpoint_shapes(raw_sd)         # sizes that only the tensors' shapes tell (a low-rank inner size)
    model = fam.model_cls()(cfg, inference_config, device=device)
    if load_weights:
        sd = fam.convert_state_dict(raw_sd, cfg)
        missing, unexpected = model.load_state_dict(sd, strict=False)
        missing = [k for k in missing if not k.endswith("slopes")]
        if missing or unexpected:
            raise KeyError(f"{fam.name}: checkpoint does not fit the model (missing {missing[:4]}, "
                           f"unexpected {list(unexpected)[:4]})")
    model.init_kv_cache(device=device)
    return model
