"""Model registry: which host class serves a checkpoint.

calm's own models come as one `.calm` file whose metadata names the architecture (llama, mixtral, qwen2, ... all served
by the single-sequence engine behind lib.DeviceModel).  Layer-list models come as a folder with config.json and
model.safetensors; config["architecture"] picks the loader."""
from __future__ import annotations

import json
import os
from typing import Callable, Dict

SEQ_LOADERS: Dict[str, Callable] = {}


def register(architecture: str, loader: Callable) -> None:
    SEQ_LOADERS[architecture] = loader


def _defaults() -> None:
    from . import bovinex, sopepel, vimulorn, zazilix

    register(vimulorn.ARCHITECTURE, vimulorn.load)
    register(bovinex.ARCHITECTURE, bovinex.load)
    register(zazilix.ARCHITECTURE, zazilix.load)
    register(sopepel.ARCHITECTURE, sopepel.load)


def architecture_of(path: str) -> str:
    if os.path.isdir(path):
        with open(os.path.join(path, "config.json")) as f:
            return json.load(f).get("architecture", "")
    from . import container

    _, meta = container.read_tensors(path)
    return meta.get("arch", "calm")


def load_model(path: str, **kw):
    """A folder -> the layer-list runtime (seqlib.SeqDeviceModel); a `.calm` file -> the calm engine (lib.DeviceModel is
    built by its callers from a ModelSpec: the drop-in binary is that family's command line)."""
    if not SEQ_LOADERS:
        _defaults()
    if not os.path.isdir(path):
        raise ValueError(f"{path}: single-file calm checkpoints are served by the drop-in `run` binary / lib.DeviceModel")
    arch = architecture_of(path)
    if arch not in SEQ_LOADERS:
        raise ValueError(f"{path}: architecture {arch!r} is not registered (known: {sorted(SEQ_LOADERS)})")
    return SEQ_LOADERS[arch](path, **kw)
