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


def _class_path(obj) -> str:
    return f"{type(obj).__module__}.{type(obj).__name__}"


def _resolve(path: str):
    mod, _, name = path.rpartition(".")
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

    def save_pretrained(self, directory: Union[Path, str]) -> None:
        from safetensors.torch import save_file

        directory = Path(directory)
        directory.mkdir(parents=True, exist_ok=True)
        (directory / "config.yaml").write_text(yaml.dump({"model": self.to_config()}))
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
