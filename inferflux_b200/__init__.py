"""inferflux_b200: a single-GPU inference engine for the Qwen2.5 dense decoder,
written for B200 (sm_100a).

    from inferflux_b200 import Engine, SamplingParams
    engine = Engine("path/to/model", dtype="bfloat16")
    results = engine.generate([[1, 2, 3]], SamplingParams(temperature=0.0), max_tokens=16)
"""
__version__ = "0.1.0"

from .config import Qwen2Config, load_config
from .engine import Engine, GenerationResult, ModelLoadSpec
from .sampling import SamplingParams

__all__ = ["Engine", "GenerationResult", "ModelLoadSpec", "SamplingParams", "Qwen2Config", "load_config"]
