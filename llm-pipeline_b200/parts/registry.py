"""Registries of part kinds. A configuration names parts by kind (``PartSpec.kind``); the model
builder looks the class up here and constructs it with ``PartSpec.args`` and the tensor-name
prefix. Registering a new kind needs no change to the framework's files::

    from llm_pipeline_b200.parts import register_mixer, Mixer

    @register_mixer("my_mixer")
    class MyMixer(Mixer):
        def __init__(self, prefix, **sizes): ...
"""

from __future__ import annotations

from typing import Callable, Dict

_FAMILIES: Dict[str, Dict[str, type]] = {name: {} for name in (
    "mixer", "feed_forward", "norm", "position", "block", "embedding", "head")}


def _register(family: str, kind: str) -> Callable[[type], type]:
    def decorate(cls: type) -> type:
        _FAMILIES[family][kind] = cls
        return cls
    return decorate


def register_mixer(kind: str):
    return _register("mixer", kind)


def register_feed_forward(kind: str):
    return _register("feed_forward", kind)


def register_norm(kind: str):
    return _register("norm", kind)


def register_position(kind: str):
    return _register("position", kind)


def register_block(kind: str):
    return _register("block", kind)


def register_embedding(kind: str):
    return _register("embedding", kind)


def register_head(kind: str):
    return _register("head", kind)


def lookup(family: str, kind: str) -> type:
    table = _FAMILIES[family]
    if kind not in table:
        raise KeyError(f"no {family} part of kind {kind!r} is registered; known: {sorted(table)}")
    return table[kind]


def kinds(family: str):
    return sorted(_FAMILIES[family])
