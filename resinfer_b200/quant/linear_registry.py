"""Registry of named linear implementations.

Same public surface as the reference's quant/linear_registry.py:12-70: ``register(name)`` (decorator;
the class must provide a ``from_linear`` classmethod), ``get``, ``list``, ``is_registered``, ``clear``, and
the pre-registered passthrough ``TorchLinear``.
"""
from __future__ import annotations

from typing import Type

import torch.nn as nn


class LinearRegistry:
    """Global mapping from string identifiers to linear implementation classes."""

    _registry: dict[str, Type[nn.Module]] = {}

    @classmethod
    def register(cls, name: str):
        """Class decorator: register a linear class under ``name``."""

        def decorator(linear_cls: Type[nn.Module]):
            if not hasattr(linear_cls, "from_linear"):
                raise TypeError(
                    f"{linear_cls.__name__} must implement from_linear() class method\n"
                    "Signature: @classmethod from_linear(cls, linear: nn.Module, **kwargs) -> nn.Module")
            if name in cls._registry:
                print(f"Warning: Overwriting registered Linear type '{name}'")
            cls._registry[name] = linear_cls
            return linear_cls

        return decorator

    @classmethod
    def get(cls, name: str) -> Type[nn.Module]:
        try:
            return cls._registry[name]
        except KeyError:
            raise KeyError(
                f"Linear type {name!r} not registered.\n"
                f"Available types: {list(cls._registry.keys())}\n"
                "Did you forget to import and register the implementation?") from None

    @classmethod
    def list(cls) -> list[str]:
        return sorted(cls._registry)

    @classmethod
    def is_registered(cls, name: str) -> bool:
        return name in cls._registry

    @classmethod
    def clear(cls) -> None:
        """Clear all registrations. Intended for tests."""
        cls._registry.clear()


@LinearRegistry.register("TorchLinear")
class TorchLinearWrapper(nn.Linear):
    """Passthrough wrapper for standard ``torch.nn.Linear``."""

    @classmethod
    def from_linear(cls, linear: nn.Module, **kwargs) -> nn.Module:
        return linear


__all__ = ["LinearRegistry", "TorchLinearWrapper"]
