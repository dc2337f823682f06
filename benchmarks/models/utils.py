"""One place for the model options of the benchmark scripts.

Counterpart of the reference's ``benchmarks/models/utils.py``: every script that builds a
``FullTransformer`` / ``ChainTransformer`` (or, here, a Llama-family model) gets the same flags,
the same ``--config-file`` handling and the same precedence — a value given on the command line
wins over the file, the file wins over the built-in default.

    parser = argparse.ArgumentParser()
    add_transformer_args(parser)
    args = parser.parse_args()
    model, dtype = build_model_from_args(args)

The config file is JSON or YAML with a ``model`` section whose keys are the option names with
``-`` or ``_`` (``hidden_dim``, ``n_blocks``, ``num_heads``, ``num_kv_heads``, ``ffn_dim``, ``seq_len``,
``vocab_size``/``input_dim``, ``dropout``, ``dtype``, ``sdp_backend``, ``architecture``, ``name``).
"""

from __future__ import annotations

import argparse
import json
import logging
from pathlib import Path
from typing import Any, Dict, Tuple

import torch

__all__ = ["add_transformer_args", "model_config_from_args", "build_model_from_args", "get_dtype", "get_sdpa", "load_config_file"]

logger = logging.getLogger("benchmarks.models")

ARCHITECTURES = ("full", "chain", "llama")
_DTYPES = {"float16": torch.float16, "fp16": torch.float16, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}
_SDPA = {"none": None, "naive": "naive", "math": "MATH", "flash": "FLASH_ATTENTION", "efficient": "EFFICIENT_ATTENTION", "cudnn": "CUDNN_ATTENTION", "fatt3": "fatt3", "native": "native"}

# option name -> (type, built-in default); ``None`` defaults are filled in by ``model_config_from_args``
_OPTIONS = {
    "architecture": (str, "full"),
    "name": (str, "llama3-8b"),
    "input_dim": (int, 32000),
    "hidden_dim": (int, 1024),
    "n_blocks": (int, 8),
    "seq_len": (int, 1024),
    "num_heads": (int, 16),
    "num_kv_heads": (int, None),
    "ffn_dim": (int, None),
    "dropout": (float, 0.0),
    "dtype": (str, "float32"),
    "sdp_backend": (str, "none"),
}
_ALIASES = {"vocab_size": "input_dim", "nblocks": "n_blocks", "num_blocks": "n_blocks", "n_heads": "num_heads", "n_kv_heads": "num_kv_heads", "model": "name"}


def get_dtype(name) -> torch.dtype:
    if isinstance(name, torch.dtype):
        return name
    try:
        return _DTYPES[str(name).lower()]
    except KeyError:
        raise ValueError(f"Invalid data type: {name!r} (choose from {sorted(_DTYPES)})") from None


def get_sdpa(name):
    """Map the command-line spelling (``none, naive, math, flash, efficient, cudnn, fatt3, native``)
    to what the attention modules of ``elf_b200.models.simple`` take."""
    try:
        return _SDPA[str(name).lower()]
    except KeyError:
        raise ValueError(f"Invalid SDPA implementation: {name!r} (choose from {sorted(_SDPA)})") from None


def load_config_file(path: str) -> Dict[str, Any]:
    """The ``model`` section of a JSON / YAML file, keys normalised to option names."""
    p = Path(path)
    text = p.read_text()
    if p.suffix.lower() in (".yaml", ".yml"):
        import yaml

        data = yaml.safe_load(text)
    else:
        data = json.loads(text)
    if not isinstance(data, dict) or not isinstance(data.get("model"), dict):
        raise ValueError(f"{path}: expected a mapping with a 'model' section")
    out = {}
    for key, value in data["model"].items():
        key = key.replace("-", "_")
        key = _ALIASES.get(key, key)
        if key not in _OPTIONS:
            logger.warning("%s: unknown model option %r ignored", path, key)
            continue
        out[key] = value
    return out


def add_transformer_args(parser: argparse.ArgumentParser) -> None:
    """Add the model flags.  Every default is ``None`` so that "given on the command line" can be
    told apart from "left alone" when a config file is merged in."""
    g = parser.add_argument_group("model")
    g.add_argument("--config-file", help="JSON/YAML file with a 'model' section; command-line flags win over it")
    g.add_argument("--architecture", choices=ARCHITECTURES, default=None)
    g.add_argument("--name", "--model", dest="name", default=None, help="llama architecture: one of elf_b200.models.llama.LLAMA_CONFIGS")
    g.add_argument("--input-dim", "--vocab-size", dest="input_dim", type=int, default=None)
    g.add_argument("--hidden-dim", type=int, default=None)
    g.add_argument("--n-blocks", "--nblocks", "--num-blocks", dest="n_blocks", type=int, default=None)
    g.add_argument("--seq-len", type=int, default=None)
    g.add_argument("--num-heads", "--n-heads", dest="num_heads", type=int, default=None)
    g.add_argument("--num-kv-heads", "--n-kv-heads", dest="num_kv_heads", type=int, default=None)
    g.add_argument("--ffn-dim", type=int, default=None)
    g.add_argument("--dropout", type=float, default=None)
    g.add_argument("--dtype", choices=sorted(_DTYPES), default=None)
    g.add_argument("--sdp-backend", choices=sorted(_SDPA), default=None)


def model_config_from_args(args: argparse.Namespace) -> Dict[str, Any]:
    """Merged options: built-in defaults < config file < command line.  ``dtype`` and
    ``sdp_backend`` come back resolved (``torch.dtype``, back-end name or ``None``)."""
    cfg = {k: default for k, (_, default) in _OPTIONS.items()}
    if getattr(args, "config_file", None):
        cfg.update(load_config_file(args.config_file))
    for key in _OPTIONS:
        value = getattr(args, key, None)
        if value is not None:
            cfg[key] = value
    for key, (typ, _) in _OPTIONS.items():
        if cfg[key] is not None and typ is not str:
            cfg[key] = typ(cfg[key])
    if cfg["architecture"] not in ARCHITECTURES:
        raise ValueError(f"unknown architecture {cfg['architecture']!r}")
    if cfg["ffn_dim"] is None:
        cfg["ffn_dim"] = 4 * cfg["hidden_dim"]
    cfg["dtype"] = get_dtype(cfg["dtype"])
    cfg["sdp_backend"] = get_sdpa(cfg["sdp_backend"])
    return cfg


def build_model_from_args(args: argparse.Namespace, device=None) -> Tuple[torch.nn.Module, torch.dtype]:
    """Instantiate the requested model (on ``device`` if given, which may be ``"meta"``) in its
    dtype; returns ``(model, dtype)``.  ``llama`` builds the whole decoder as one flat
    ``nn.Sequential`` of fused blocks (``elf_b200.models.llama.build_llama``)."""
    cfg = model_config_from_args(args)
    dtype = cfg["dtype"]
    arch = cfg["architecture"]
    if arch == "llama":
        from elf_b200.models.llama import LLAMA_CONFIGS, build_llama

        if cfg["name"] not in LLAMA_CONFIGS:
            raise ValueError(f"unknown llama shape {cfg['name']!r}; choose from {sorted(LLAMA_CONFIGS)}")
        return build_llama(LLAMA_CONFIGS[cfg["name"]], device=device, dtype=dtype), dtype
    from elf_b200.models.simple import ChainTransformer, FullTransformer

    kw = {k: cfg[k] for k in ("hidden_dim", "n_blocks", "seq_len", "num_heads", "num_kv_heads", "ffn_dim", "dropout", "sdp_backend")}
    ctx = torch.device(device) if device is not None else None
    if arch == "full":
        kw["input_dim"] = cfg["input_dim"]
    cls = FullTransformer if arch == "full" else ChainTransformer
    if ctx is not None:
        with ctx:
            model = cls(**kw)
    else:
        model = cls(**kw)
    return model.to(dtype), dtype
