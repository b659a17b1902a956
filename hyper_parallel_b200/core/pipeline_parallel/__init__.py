from .scheduler import (MetaStep, MetaStepType, PipelineScheduleRuntime, Schedule1F1B, ScheduleGPipe,  # noqa: F401
                        ScheduleInterleaved1F1B, add_send_recv, validate_pipeline_execution)
from .stage import PipelineStage, SharedParameterInfo  # noqa: F401
from .utils import BatchDimSpec  # noqa: F401
