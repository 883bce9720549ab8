from .model import DecoderModel, build_model  # noqa: F401
from .step import Runner, StepError, StepItem  # noqa: F401
