"""B200-native persistent decode megakernel behind TileMega's serving-plan ABI."""
from .build import LIBRARY, build_library  # noqa: F401
from .planbuild import emit_plan  # noqa: F401

__all__ = ["LIBRARY", "build_library", "emit_plan"]
