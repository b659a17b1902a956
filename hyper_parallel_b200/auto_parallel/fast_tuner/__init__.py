"""Fast-Tuner: rule + memory + cost driven search of hybrid-parallel strategies."""
from .config import ModelSpec, Strategy, TunerConfig  # noqa: F401
from .parallel_tool import main, taylor_search_tool  # noqa: F401
from .pipeline_tool import pipeline_search_tool  # noqa: F401
