"""gibbs_b200: a small, whole inference engine for one B200.

From a model folder (config.json + safetensors) to generated tokens: typed
configuration and architecture registry (``config``), weights by tensor name
(``weights``), models put together from parts (``parts``), a paged cache with
block tables and fixed-size state slots (``cache``), one step function over
ragged batches, a scheduler and entry points (``engine``), sampling
(``sampling``) and the CUDA kernels for sm_100a (``csrc``, bound in ``ops``).
"""
from .config import Lfm2Config, ModelPlan, parse_config, register_architecture
from .parts import register_part
from .engine import Engine, Generator, Scheduler, StepEntry, load_model, random_model
from .sampling import Sampler, SamplingParams
from .weights import write_random_model

__version__ = "0.1.0"
__all__ = ["Lfm2Config", "ModelPlan", "parse_config", "register_architecture", "register_part", "Engine", "Generator", "Scheduler", "Sampler", "SamplingParams",
           "StepEntry", "load_model", "random_model", "write_random_model"]
