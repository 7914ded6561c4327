"""Name -> class registry for datasets (``teletron/datasets/registry.py:17-63``, ``build.py:1-12``)."""

from __future__ import annotations

from typing import Callable, Dict, Optional


class Registry:
    def __init__(self, name: str):
        self._name = name
        self._modules: Dict[str, type] = {}

    @property
    def name(self) -> str:
        return self._name

    def __len__(self):
        return len(self._modules)

    def __contains__(self, key):
        return key in self._modules

    def get(self, key: str) -> Optional[type]:
        return self._modules.get(key)

    def register_module(self, name: Optional[str] = None, force: bool = False, module: Optional[type] = None):
        def _register(cls):
            key = name or cls.__name__
            if key in self._modules and not force:
                raise KeyError(f"{key} is already registered in {self._name}")
            self._modules[key] = cls
            return cls
        if module is not None:
            return _register(module)
        return _register

    def build(self, cfg, **default_args):
        if isinstance(cfg, str):
            cfg = {"type": cfg}
        cfg = dict(cfg)
        kind = cfg.pop("type")
        cls = self.get(kind) if isinstance(kind, str) else kind
        if cls is None:
            raise KeyError(f"{kind} is not registered in {self._name}; known: {sorted(self._modules)}")
        for k, v in default_args.items():
            cfg.setdefault(k, v)
        return cls(**cfg)


DATASETS = Registry("dataset")


def build_dataset(cfg, **default_args):
    """``build_dataset("FakeDataset", num_frames=33, ...)`` or ``build_dataset({"type": ..., ...})``."""
    return DATASETS.build(cfg, **default_args)


def build_module(cfg, registry: Registry, default_args: Optional[dict] = None):
    return registry.build(cfg, **(default_args or {}))
