"""Parts a model is put together from; importing this package registers the built-in kinds."""
from . import attention, block, embedding, mlp, norm, rotary  # noqa: F401  (registration)
from .base import Part, StepContext, TensorWant, build_part, register_part  # noqa: F401
from .plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry  # noqa: F401
