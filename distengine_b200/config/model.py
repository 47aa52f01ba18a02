"""What every architecture's configuration gives the engine: layer specs, a run plan, sizes.

A model is described as data:

* ``PartSpec``  - the kind of one part ("attention", "gated_mlp", "rmsnorm", "rope", ...) and its
  sizes and constants.  The kind is looked up in the part registries of
  ``distengine_b200.parts.base``; the parameters become the part's constructor arguments.
* ``LayerSpec`` - one layer: the block arrangement, its mixer, its feed-forward, its norm and the
  prefixes under which its tensors are stored.  Layers of one model may differ.
* ``PlanEntry`` - one execution of a layer.  The plan is the order in which layers run; it may name
  a layer twice (each run that writes has a cache of its own) or let a run read the cache that an
  earlier run wrote (``reads_cache_of``), in which case it writes nothing.

The reference builds one fixed stack (src/models/llama.py:112-124) and loops over it
(:183-189); it has no layer specs and no plan.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


class ConfigError(ValueError):
    """A config.json that this engine cannot run; the message names the key."""


def _freeze(params: Mapping[str, Any]) -> tuple[tuple[str, Any], ...]:
    return tuple(sorted(params.items()))


@dataclass(frozen=True)
class PartSpec:
    kind: str
    items: tuple[tuple[str, Any], ...] = ()

    @staticmethod
    def of(kind: str, **params: Any) -> "PartSpec":
        return PartSpec(kind, _freeze(params))

    @property
    def params(self) -> dict[str, Any]:
        return dict(self.items)


@dataclass(frozen=True)
class LayerSpec:
    block: str                      # arrangement kind, e.g. "prenorm"
    mixer: PartSpec
    feed_forward: PartSpec
    norm: PartSpec                  # built twice: before the mixer and before the feed-forward
    # where this layer's tensors live in the weight file: part role -> name prefix
    prefixes: tuple[tuple[str, str], ...] = ()

    def prefix(self, role: str) -> str:
        return dict(self.prefixes)[role]


@dataclass(frozen=True)
class PlanEntry:
    layer: int
    reads_cache_of: int | None = None     # index of an earlier plan entry


@dataclass(frozen=True)
class ModelConfig:
    """Base of the typed configurations.  Subclasses parse their own config.json keys."""

    architecture: str = field(default="", kw_only=True)

    # -- sizes the generic model needs
    @property
    def width(self) -> int:
        raise NotImplementedError

    @property
    def vocabulary(self) -> int:
        raise NotImplementedError

    @property
    def max_positions(self) -> int:
        raise NotImplementedError

    @property
    def tied_output(self) -> bool:
        raise NotImplementedError

    # -- the model as data
    def layer_specs(self) -> list[LayerSpec]:
        raise NotImplementedError

    def plan(self) -> list[PlanEntry]:
        return [PlanEntry(i) for i in range(len(self.layer_specs()))]

    def final_norm(self) -> PartSpec:
        raise NotImplementedError

    def tensor_names(self) -> dict[str, str]:
        """role -> tensor name of the tensors outside the layers."""
        raise NotImplementedError

    def to_json(self) -> dict[str, Any]:
        """The config.json that parses back to this configuration."""
        raise NotImplementedError


def require(data: Mapping[str, Any], key: str, kind: type | tuple[type, ...]) -> Any:
    if key not in data or data[key] is None:
        raise ConfigError(f"config.json: key '{key}' is missing")
    value = data[key]
    if kind is float and isinstance(value, int) and not isinstance(value, bool):
        value = float(value)
    if isinstance(value, bool) and kind is not bool or not isinstance(value, kind):
        raise ConfigError(f"config.json: key '{key}' must be {getattr(kind, '__name__', kind)}, "
                          f"got {value!r}")
    return value


def positive(name: str, value: int) -> int:
    if value <= 0:
        raise ConfigError(f"config.json: '{name}' must be positive, got {value}")
    return value
