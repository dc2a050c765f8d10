"""One registry: architecture name -> how to build its model.

After zllm src/backend/arch.rs:21-64: one table, a lookup that ignores case
(``spec_for``), and a hard error that names the unknown architecture
(``detect``: ``unsupported GGUF architecture "x"``).  An entry carries the
typed-config reader and the function that turns a configuration into a
``ModelSpec`` (layers listed part by part); no other file needs to know the
name.  Architectures defined outside the package come in as plug-in modules
named in ``ZLLM_PLUGINS``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict

from ..errors import ConfigError


@dataclass(frozen=True)
class ArchEntry:
    name: str
    read_config: Callable[[dict], object]      # raw config.json dict -> typed config
    build_spec: Callable[[object], object]     # typed config -> ModelSpec


_ARCHS: Dict[str, ArchEntry] = {}


def register_architecture(name: str, read_config, build_spec) -> ArchEntry:
    entry = ArchEntry(name, read_config, build_spec)
    _ARCHS[name.lower()] = entry
    return entry


def architecture(name: str) -> ArchEntry:
    _ensure_builtin()
    entry = _ARCHS.get(str(name).lower())
    if entry is None:
        known = ", ".join(sorted(e.name for e in _ARCHS.values()))
        raise ConfigError(f"unsupported architecture {name!r} (known: {known})")
    return entry


def known_architectures():
    _ensure_builtin()
    return sorted(e.name for e in _ARCHS.values())


def architecture_of(config_json: dict) -> ArchEntry:
    """The entry named by ``architectures[0]`` of a raw config.json dictionary."""
    archs = config_json.get("architectures")
    if not archs or not isinstance(archs, (list, tuple)):
        raise ConfigError("config.json: missing key 'architectures' (a list with the model class name)")
    return architecture(archs[0])


_plugins_loaded = False


def _ensure_builtin():
    """The built-in architectures register themselves on import.  So do plug-ins: every module
    named in the environment variable ZLLM_PLUGINS (comma-separated, importable from sys.path) is
    imported once; a plug-in registers its parts and its architecture with the ``register_*``
    functions, and the command line, ``bin/trace_run`` and the Python entry points then take its
    model folders like any other."""
    global _plugins_loaded
    from ..models import llama  # noqa: F401
    if not _plugins_loaded:
        _plugins_loaded = True
        import importlib
        import os
        for mod in filter(None, (m.strip() for m in os.environ.get("ZLLM_PLUGINS", "").split(","))):
            try:
                importlib.import_module(mod)
            except ImportError as e:
                raise ConfigError(f"ZLLM_PLUGINS names {mod!r}, which cannot be imported: {e}") from e
