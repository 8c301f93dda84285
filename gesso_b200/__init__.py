"""gesso_b200: a small, whole LFM2 inference engine for one NVIDIA B200."""
from . import config as _config  # noqa: F401  (registers the built-in architecture)
from . import parts as _parts    # noqa: F401  (registers the built-in parts)
from .api import load, random_model, run_dtype
from .errors import ErrorCode, GessoError
from .engine.session import BatchRequest, BatchResult, Session, generate
from .sampling.sampler import SamplingParams

__all__ = ["load", "random_model", "run_dtype", "ErrorCode", "GessoError", "BatchRequest", "BatchResult",
           "Session", "generate", "SamplingParams"]
__version__ = "0.1.0"
