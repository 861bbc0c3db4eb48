"""Tools for multi-turn rollouts: base classes and parser (``base``), built-in sandbox / search
tools (``builtin``, imported here so that their registered names resolve), the turn loop
(``multi_turn``)."""
from . import base, builtin  # noqa: F401
