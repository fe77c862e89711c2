"""redline_b200: a small, whole inference engine for one GPU (NVIDIA B200, sm_100a).

    from redline_b200 import Engine
    engine = Engine("path/to/model_dir", max_seqs=8)
    outs = engine.generate([[1, 2, 3]], max_new_tokens=16)

See ``redline_b200.runtime`` for the entry point in the reference's manner.
"""

from .config import EngineConfig, LlamaConfig, ModelConfig, load_config
from .sampling import SamplingParams

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "ModelRunner"):
        from . import engine as _engine
        return getattr(_engine, name)
    raise AttributeError(name)
