from .presets import PRESETS, MoEShape, get_preset  # noqa: F401
