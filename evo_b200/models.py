"""`Evo` front door and checkpoint ingest: the reference's evo/models.py (Evo :21-62,
load_checkpoint :73-152) re-expressed for the evo_b200 engine.  Checkpoint key names after
the 'backbone.' strip, the tied unembed, strict loading and the bf16-except-poles/residues
dtype policy are the contract (evo/models.py:124-148)."""
from __future__ import annotations

import json
import os
from typing import Optional

import torch
import yaml

from .configs import MODEL_NAMES, MODELS, get_config
from .stripedhyena import StripedHyena, dotdict
from .tokenizer import CharLevelTokenizer

HF_MODEL_NAME_MAP = {name: spec[1] for name, spec in MODELS.items()}


def _read_safetensors(model_dir: str) -> dict:
    from safetensors.torch import load_file
    index = os.path.join(model_dir, "model.safetensors.index.json")
    single = os.path.join(model_dir, "model.safetensors")
    if os.path.exists(index):
        with open(index) as f:
            shards = sorted(set(json.load(f)["weight_map"].values()))
        tensors = {}
        for shard in shards:
            tensors.update(load_file(os.path.join(model_dir, shard)))
        return tensors
    if os.path.exists(single):
        return load_file(single)
    raise FileNotFoundError(f"No safetensors files found in {model_dir}. Expected model.safetensors.index.json or model.safetensors.")


# the reference resolves config_path relative to its package (pkgutil.get_data, evo/models.py:141); those two names
# map to the built-in dicts of evo_b200/configs.py, which hold the same keys and values
_PACKAGE_CONFIGS = {"evo-1-8k-base_inference.yml": "evo-1-8k-base", "evo-1-131k-base_inference.yml": "evo-1-131k-base"}


def _resolve_config(model_name: str, config_path: Optional[str]) -> dict:
    if config_path is None:
        return get_config(model_name)
    if os.path.isfile(config_path):
        with open(config_path) as f:
            return yaml.safe_load(f)
    base = os.path.basename(config_path)
    if base in _PACKAGE_CONFIGS and os.path.dirname(config_path) in ("configs", "evo/configs"):
        return get_config(_PACKAGE_CONFIGS[base])
    raise FileNotFoundError(f"config file {config_path!r} does not exist (and is not one of the package configs "
                            f"{sorted('configs/' + k for k in _PACKAGE_CONFIGS)})")


def load_checkpoint(model_name: str = "evo-1-8k-base", config_path: Optional[str] = None, device: str = None,
                    model_dir: Optional[str] = None, random_init: bool = False, seed: int = 0, streaming: bool = True, *args, **kwargs):
    """HF snapshot -> safetensors -> StripedHyena on `device`.

    model_dir: use an already-downloaded snapshot directory instead of huggingface_hub.
    random_init: skip the checkpoint (benchmarks / tests on boxes without network) and keep the
    constructor's random initialisation, seeded.
    streaming: True (default) = tensor-by-tensor ingest straight into the device layouts; False = the reference's
    host-state-dict sequence (kept as the comparator for the ingest tests)."""
    cfg = dotdict(_resolve_config(model_name, config_path))

    if random_init:
        # build straight on the target device: no 26 GB fp32 host copy of a 7B model
        torch.manual_seed(seed)
        with torch.device(device if device is not None else "cpu"):
            model = StripedHyena(cfg)
        model.to_bfloat16_except_poles_residues()
        return model if device is None else model.to(device)
    if model_dir is None:
        from huggingface_hub import snapshot_download
        _, repo, revision = MODELS[model_name]
        model_dir = snapshot_download(repo, revision=revision)
    if not streaming:
        # the reference's own sequence (evo/models.py:96-150): host state dict -> strict load -> bf16 -> device
        state = {}
        for key, value in _read_safetensors(model_dir).items():
            state[key[len("backbone."):] if key.startswith("backbone.") else key] = value
        if "unembed.weight" not in state and "embedding_layer.weight" in state:
            state["unembed.weight"] = state["embedding_layer.weight"]
        model = StripedHyena(cfg)
        model.load_state_dict(state, strict=True)
        model.to_bfloat16_except_poles_residues()
        return model if device is None else model.to(device)
    # streaming ingest: parameters are allocated once, on the target device, in their final dtype and layout;
    # each checkpoint tensor goes mmap -> pinned staging -> device and is cast / packed there (evo_b200/ingest.py)
    from .ingest import load_streaming
    dev = torch.device(device) if device is not None else torch.device("cpu")
    with torch.device("meta"):
        model = StripedHyena(cfg)
    model.to_bfloat16_except_poles_residues()
    model = model.to_empty(device=dev)
    model.ingest_stats = load_streaming(model, model_dir, dev)
    return model


def _load_flat(family, model_dir: str, config: dict, device, dtype):
    """Families described by a flat table of checkpoint tensors (StreamDecoder subclasses)."""
    from .ingest import load_named_tensors
    cls, cfg_cls = family()
    model = cls(cfg_cls.from_dict(config), dtype=dtype or torch.bfloat16)
    dev = torch.device(device) if device is not None else torch.device("cpu")
    shapes = {k: tuple(v.shape) for k, v in model.weights.items()}
    tensors, model.ingest_stats = load_named_tensors(model_dir, dev, shapes, type(model).__name__, ignorable=getattr(model.config, "unused_tensor_names", ()))
    for name, t in tensors.items():
        model.weights[name] = t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)
    model._invalidate()
    return model


def _load_zaverax(model_dir: str, config: dict, device, dtype, **kwargs):
    def family():
        from .zaverax import Zaverax, ZaveraxConfig
        return Zaverax, ZaveraxConfig
    return _load_flat(family, model_dir, config, device, dtype)


def _load_movalorn(model_dir: str, config: dict, device, dtype, **kwargs):
    def family():
        from .movalorn import Movalorn, MovalornConfig
        return Movalorn, MovalornConfig
    return _load_flat(family, model_dir, config, device, dtype)


def _load_nelovik(model_dir: str, config: dict, device, dtype, **kwargs):
    def family():
        from .nelovik import Nelovik, NelovikConfig
        return Nelovik, NelovikConfig
    return _load_flat(family, model_dir, config, device, dtype)


def _load_gakupel(model_dir: str, config: dict, device, dtype, **kwargs):
    def family():
        from .gakupel import Gakupel, GakupelConfig
        return Gakupel, GakupelConfig
    return _load_flat(family, model_dir, config, device, dtype)


def _load_stripedhyena(model_dir: str, config: dict, device, dtype, model_name: str = "evo-1-8k-base", **kwargs):
    if dtype not in (None, torch.bfloat16):
        raise NotImplementedError("StripedHyena runs in bfloat16 (fp32 poles and residues) only")
    return load_checkpoint(model_name=model_name, device=device, model_dir=model_dir, **kwargs)


# config.json "architecture" -> (loader, activation dtypes the model class can run in)
ARCHITECTURES = {
    "Zaverax": (_load_zaverax, (torch.bfloat16, torch.float32)),
    "Movalorn": (_load_movalorn, (torch.bfloat16, torch.float32)),
    "Nelovik": (_load_nelovik, (torch.bfloat16, torch.float32)),
    "Gakupel": (_load_gakupel, (torch.bfloat16, torch.float32)),
    "StripedHyena": (_load_stripedhyena, (torch.bfloat16,)),
    "StripedHyenaModelForCausalLM": (_load_stripedhyena, (torch.bfloat16,)),
}


def read_architecture(model_dir: str):
    """(architecture name, config dict) of a checkpoint folder; the name selects the model class."""
    with open(os.path.join(model_dir, "config.json")) as f:
        config = json.load(f)
    arch = config.get("architecture") or (config.get("architectures") or [None])[0]
    if arch not in ARCHITECTURES:
        raise ValueError(f"{model_dir}: architecture {arch!r} is not one of {sorted(ARCHITECTURES)}")
    return arch, config


def load_model_dir(model_dir: str, device: str = None, dtype: Optional[torch.dtype] = None, **kwargs):
    """Checkpoint folder (config.json + safetensors) -> model on `device`; the model class is chosen by config.json."""
    arch, config = read_architecture(model_dir)
    loader, dtypes = ARCHITECTURES[arch]
    if dtype is not None and dtype not in dtypes:
        raise NotImplementedError(f"{arch} does not run in {dtype}")
    return loader(model_dir, config, device, dtype, **kwargs)


class Evo:
    """Evo('evo-1-8k-base') -> .model (StripedHyena protocol), .tokenizer."""

    def __init__(self, model_name: str = "evo-1-8k-base", device: str = None, **load_kwargs):
        if model_name not in MODEL_NAMES:
            raise ValueError(f"Invalid model name {model_name}. Should be one of: {', '.join(MODEL_NAMES)}.")
        self.device = device
        model_dir = load_kwargs.get("model_dir")
        if model_dir is not None and os.path.exists(os.path.join(model_dir, "config.json")):
            # a checkpoint folder that names its own architecture (config.json): the registry picks the model class
            load_kwargs = {k: v for k, v in load_kwargs.items() if k not in ("model_dir", "random_init")}
            self.model = load_model_dir(model_dir, device=device, model_name=model_name, **load_kwargs)
        else:
            self.model = load_checkpoint(model_name=model_name, device=device, **load_kwargs)
        self.tokenizer = CharLevelTokenizer(512)
