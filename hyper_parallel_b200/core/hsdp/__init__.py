from .api import HSDPCell, hsdp, hsdp_sync_stream  # noqa: F401
