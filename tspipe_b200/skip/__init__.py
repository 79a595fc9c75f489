"""Skip connections across pipeline stages (``@skippable``, ``stash``, ``pop``, ``Namespace``)."""
from .layout import SkipLayout, inspect_skip_layout
from .namespace import Namespace
from .skippable import Skippable, SkipSequential, pop, skippable, stash, verify_skippables, wrap_partitions

__all__ = ["skippable", "stash", "pop", "verify_skippables", "Namespace", "Skippable", "SkipSequential",
           "SkipLayout", "inspect_skip_layout", "wrap_partitions"]
