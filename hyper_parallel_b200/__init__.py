"""hyper_parallel_b200: a Blackwell-native hybrid-parallel training framework."""
__version__ = "0.1.0"
