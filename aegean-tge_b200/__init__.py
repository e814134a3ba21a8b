"""A small, whole inference engine for one B200, from token ids to next token: the Qwen2.5 dense decoder, the
Lepizen decoder (parallel blocks, attention with sinks and normalised projections, capped logits) and the Mozepel
decoder (layers that normalise after the sum, decayed linear attention with a state per request, a window attention
with pooled blocks).

Public entry points:

* :class:`Engine` - load a model folder (or random weights) and generate;
* :class:`SamplingParams` - sampling controls;
* :func:`write_random_model` - a model folder from a configuration and a seed;
* ``bin/tge`` and ``bin/trace_run`` - the command line and trace replay.
"""
from . import models as _models  # noqa: F401  (registers architectures)
from . import parts as _parts    # noqa: F401  (registers parts)
from .config import ConfigError, LepizenConfig, MozepelConfig, Qwen2Config
from .registry import architecture_of, register_architecture, registered_architectures
from .sampling import SamplingParams
from .weights import WeightError, write_random_model

__version__ = "0.1.0"


def __getattr__(name):
    # The engine pulls in the CUDA bindings; keep `import aegean_tge_b200` light for host-only use.
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)


__all__ = ["Engine", "SamplingParams", "ConfigError", "LepizenConfig", "MozepelConfig", "Qwen2Config", "WeightError", "write_random_model",
           "architecture_of", "register_architecture", "registered_architectures", "__version__"]
