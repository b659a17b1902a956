from .adamw import FusedAdamW  # noqa: F401
