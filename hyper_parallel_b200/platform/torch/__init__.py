"""Module paths of the reference's torch backend (``hyper_parallel/platform/torch/...``), kept so
that imports written against it keep working; the implementations live under ``core``."""
