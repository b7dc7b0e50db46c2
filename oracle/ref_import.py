"""Import the unmodified reference modules for pinning the oracle.  TEST INFRASTRUCTURE ONLY.

The reference's package ``__init__`` files pull in its data pipeline and
Lightning, which are not installed here.  Registering empty parent packages
whose ``__path__`` points at the reference directories lets
``crosslayer_transcoder/model/{clt,jumprelu,topk,standardize}.py`` import
exactly as they are; three small stand-in modules (``lightning``,
``torchmetrics``, ``nnsight``) are enough for
``crosslayer_transcoder/model/clt_lightning.py`` too.

Used by ``tests/golden/make_golden.py``, ``tests/test_oracle_vs_reference.py`` and the benchmark's
reference arm (``oracle/ref_step.py``); the sources come from the reference tree, or from the
unmodified mirror ``oracle/make_ref.py`` makes of it.
"""
from __future__ import annotations

import importlib
import os
import sys
import types
from pathlib import Path

import torch

def _find_root() -> Path:
    """The reference tree itself where it exists, else the unmodified mirror of its model package that
    ``oracle/make_ref.py`` leaves under ``oracle/_ref/`` (which travels to machines without the tree)."""
    cands = [Path(os.environ.get("CLT_REFERENCE_ROOT", "/root/reference")), Path(__file__).resolve().parent / "_ref"]
    for c in cands:
        if (c / "crosslayer_transcoder" / "model" / "clt.py").exists():
            return c
    return cands[0]


REF_ROOT = _find_root()


def available() -> bool:
    return (REF_ROOT / "crosslayer_transcoder" / "model" / "clt.py").exists()


def _pkg(name: str, path: Path) -> types.ModuleType:
    m = types.ModuleType(name)
    m.__path__ = [str(path)]
    sys.modules[name] = m
    return m


def _shim_lightning():
    if "lightning" in sys.modules:
        return
    L = types.ModuleType("lightning")

    class _Trainer:
        max_steps = 1
        num_devices = 1

    class LightningModule(torch.nn.Module):
        def __init__(self, *a, **k):
            super().__init__()
            self.trainer = _Trainer()
            self.global_step = 0
            self.logger = None
            self.logged = {}

        def log(self, name, value, *a, **k):
            self.logged[name] = value

        def save_hyperparameters(self, *a, **k):
            pass

        def lr_schedulers(self):
            return None

    class Callback:
        pass

    class LightningDataModule:
        pass

    L.LightningModule = LightningModule
    L.Callback = Callback
    L.LightningDataModule = LightningDataModule
    sys.modules["lightning"] = L

    tm = types.ModuleType("torchmetrics")

    class Metric(torch.nn.Module):
        def __init__(self, *a, **k):
            super().__init__()

        def add_state(self, name, default, dist_reduce_fx=None):
            self.register_buffer(name, default)

    tm.Metric = Metric
    sys.modules["torchmetrics"] = tm
    sys.modules.setdefault("nnsight", types.ModuleType("nnsight"))
    if "wandb" not in sys.modules:
        try:
            import wandb  # noqa: F401
        except Exception:
            w = types.ModuleType("wandb")
            w.wandb_run = types.SimpleNamespace(Run=type("Run", (), {}))
            sys.modules["wandb"] = w


_loaded = {}


def load(with_lightning: bool = False) -> types.SimpleNamespace:
    """Return a namespace with the reference's model modules (``clt``, ``jumprelu``,
    ``topk``, ``standardize`` and, optionally, ``clt_lightning``)."""
    if not available():
        raise RuntimeError(f"reference tree not found at {REF_ROOT}")
    key = bool(with_lightning)
    if key in _loaded:
        return _loaded[key]
    base = REF_ROOT / "crosslayer_transcoder"
    if "crosslayer_transcoder" not in sys.modules:
        _pkg("crosslayer_transcoder", base)
        _pkg("crosslayer_transcoder.model", base / "model")
        _pkg("crosslayer_transcoder.metrics", base / "metrics")
        utils = _pkg("crosslayer_transcoder.utils", base / "utils")
        uu = types.ModuleType("crosslayer_transcoder.utils.utils")
        uu.get_webtext_dataloader = lambda *a, **k: None
        sys.modules["crosslayer_transcoder.utils.utils"] = uu
        utils.utils = uu
    ns = types.SimpleNamespace()
    for name in ("serializable_module", "standardize", "jumprelu", "topk", "clt"):
        setattr(ns, name, importlib.import_module(f"crosslayer_transcoder.model.{name}"))
    if with_lightning:
        _shim_lightning()
        ns.clt_lightning = importlib.import_module("crosslayer_transcoder.model.clt_lightning")
    _loaded[key] = ns
    return ns


def load_shared_memory():
    """The reference's ``crosslayer_transcoder/data/shared_memory.py`` as a stand-alone module (it imports
    only torch, numpy and the standard library), or None where neither the tree nor the mirror has it."""
    import importlib.util

    if "ref_shared_memory" in sys.modules:
        return sys.modules["ref_shared_memory"]
    path = REF_ROOT / "crosslayer_transcoder" / "data" / "shared_memory.py"
    if not path.exists():
        return None
    spec = importlib.util.spec_from_file_location("ref_shared_memory", path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules["ref_shared_memory"] = mod
    spec.loader.exec_module(mod)
    return mod
