"""sleuth_b200: a small generation library for the Qwen3 dense decoder on one NVIDIA B200.

    import sleuth_b200 as sb
    engine = sb.load("model-dir", dtype="bf16")
    out = sb.generate(engine, [1, 2, 3], max_new_tokens=16, sampling=sb.SamplingConfig(temperature=0))

Importing the package needs no GPU; loading a model does.
"""

from .config import ConfigError, Qwen3Config, parse_config, register_architecture
from .sampling.config import SamplingConfig

__version__ = "0.1.0"


def load(*args, **kwargs):
    from .engine.engine import load as _load
    return _load(*args, **kwargs)


def generate(*args, **kwargs):
    from .engine.engine import generate as _generate
    return _generate(*args, **kwargs)


def write_random_model(*args, **kwargs):
    from .weights.random_init import write_random_model as _w
    return _w(*args, **kwargs)


__all__ = ["ConfigError", "Qwen3Config", "parse_config", "register_architecture", "SamplingConfig", "load",
           "generate", "write_random_model", "__version__"]
