"""Model registry: which graph of the native engine serves a model file or folder.

Two kinds of source: a GGUF file (`general.architecture` names the graph, today "llama": quantised blocks through
the mat-vec / tcgen05 GEMM path of engine.cu) and a folder with `config.json` + `model.safetensors`
(`architecture` names the graph; layer-list designs go through layered.cu). A family knows how to read its
hyper-parameters, how to describe itself to the C ABI and which engine class runs it.

The reference loads exactly one kind of file through llama-cpp-python (/root/reference/api.py:24-28); the registry
is what lets `Llama(model_path=...)`, the scheduler and the trace runner take either without knowing which.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional

FAMILIES: Dict[str, "Family"] = {}


@dataclass
class Family:
    name: str                       # architecture string in the file
    source: str                     # "gguf" | "folder"
    open_engine: Callable           # (source, **engine kwargs) -> engine object with the common engine interface


def register(family: Family) -> Family:
    FAMILIES[family.name] = family
    return family


@dataclass
class ModelSource:
    path: str
    family: Family
    gguf: object = None             # GGUFFile for "gguf" sources
    config: Optional[dict] = None   # parsed config.json for "folder" sources
    weights: object = None          # SafetensorsFile for "folder" sources
    metadata: Optional[dict] = None


def architectures() -> List[str]:
    _load_builtin()
    return sorted(FAMILIES)


def _load_builtin():
    from . import dibesun, goponex, llama_family, nafelix, vazunex  # noqa: F401  (each registers itself on import)


def open_model(path: str) -> ModelSource:
    """Look at `path` and pick the family. Raises ValueError for an unknown architecture."""
    _load_builtin()
    if os.path.isdir(path):
        cfg_path = os.path.join(path, "config.json")
        if not os.path.exists(cfg_path):
            raise ValueError(f"{path}: a model folder needs config.json")
        with open(cfg_path) as f:
            cfg = json.load(f)
        arch = cfg.get("architecture")
        fam = FAMILIES.get(arch)
        if fam is None or fam.source != "folder":
            raise ValueError(f"unsupported architecture {arch!r}; known: {architectures()}")
        from .safetensors_file import SafetensorsFile
        st = SafetensorsFile(os.path.join(path, "model.safetensors"))
        return ModelSource(path=path, family=fam, config=cfg, weights=st, metadata={})
    from .gguf_file import GGUFFile
    g = GGUFFile(path)
    arch = g.metadata.get("general.architecture", "llama")
    fam = FAMILIES.get(arch)
    if fam is None or fam.source != "gguf":
        raise ValueError(f"unsupported architecture {arch!r}: known: {architectures()}")
    return ModelSource(path=path, family=fam, gguf=g, metadata=g.metadata)


def open_engine(src: ModelSource, **kw):
    return src.family.open_engine(src, **kw)
