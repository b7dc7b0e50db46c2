"""Config / checkpoint round-trip shared by every module of the transcoder.

Mirrors the reference's ``SerializableModule`` surface
(crosslayer_transcoder/model/serializable_module.py:15-69): ``to_config`` returns
``{"class_path", "init_args"}``, ``from_config`` rebuilds nested modules from such
dicts, ``save_pretrained`` / ``from_pretrained`` write and read ``config.yaml`` +
``checkpoint.safetensors``.
"""
from __future__ import annotations

import importlib
from pathlib import Path
from typing import Any, Dict, Union

import yaml
from torch import nn


_OWN_PACKAGE = "crosslayer_transcoder_b200"
_REFERENCE_PACKAGE = "crosslayer_transcoder"

#: when set (``save_pretrained(..., reference_class_paths=True)``), configs name the reference's classes
#: (``crosslayer_transcoder.model...``) so that the reference's own ``from_pretrained`` can read them
_emit_reference_paths = False


def _class_path(obj) -> str:
    mod = type(obj).__module__
    if _emit_reference_paths and mod.startswith(_OWN_PACKAGE + "."):
        mod = _REFERENCE_PACKAGE + mod[len(_OWN_PACKAGE):]
    return f"{mod}.{type(obj).__name__}"


def _resolve(path: str):
    """Class named by a config's ``class_path``.  Paths into the reference package
    (``crosslayer_transcoder.model.clt.Encoder`` ...), as written by the reference's ``save_pretrained``,
    resolve to this package's classes of the same name, so its checkpoints load here unchanged."""
    mod, _, name = path.rpartition(".")
    if mod == _REFERENCE_PACKAGE or mod.startswith(_REFERENCE_PACKAGE + "."):
        mod = _OWN_PACKAGE + mod[len(_REFERENCE_PACKAGE):]
    return getattr(importlib.import_module(mod), name)


class SerializableModule(nn.Module):
    #: names of the constructor arguments written to the config
    _config_fields: tuple = ()

    def _init_args(self) -> Dict[str, Any]:
        return {k: getattr(self, k) for k in self._config_fields}

    def to_config(self) -> Dict[str, Any]:
        return {"class_path": _class_path(self), "init_args": self._init_args()}

    @classmethod
    def from_config(cls, config: Dict[str, Any]):
        kwargs = {}
        for key, val in (config.get("init_args") or {}).items():
            if isinstance(val, dict) and "class_path" in val:
                val = _resolve(val["class_path"]).from_config(val)
            kwargs[key] = val
        return cls(**kwargs)

    def config_for_export(self, reference_class_paths: bool = False) -> Dict[str, Any]:
        """``to_config()``; with ``reference_class_paths`` every ``class_path`` names the reference's class."""
        global _emit_reference_paths
        prev = _emit_reference_paths
        _emit_reference_paths = bool(reference_class_paths)
        try:
            return self.to_config()
        finally:
            _emit_reference_paths = prev

    def save_pretrained(self, directory: Union[Path, str], reference_class_paths: bool = False) -> None:
        from safetensors.torch import save_file

        directory = Path(directory)
        directory.mkdir(parents=True, exist_ok=True)
        (directory / "config.yaml").write_text(yaml.dump({"model": self.config_for_export(reference_class_paths)}))
        save_file({k: v.contiguous() for k, v in self.state_dict().items()}, directory / "checkpoint.safetensors")

    @classmethod
    def from_pretrained(cls, directory: Union[Path, str]):
        from safetensors.torch import load_file

        directory = Path(directory)
        full = yaml.safe_load((directory / "config.yaml").read_text())
        cfg = full.get("model")
        if cfg is None:
            raise ValueError("Model config not found in config.yaml", full)
        model = cls.from_config(cfg)
        model.load_state_dict(load_file(directory / "checkpoint.safetensors"))
        model._is_folded = cfg.get("is_folded", False)
        return model
