"""oracle_engine_b200: a small, whole inference library for the Llama dense decoder on one
NVIDIA B200 (sm_100a), modelled on what Titouan935/oracle-engine does on the CPU.

Public entry points:
    Engine.from_pretrained(folder, dtype=..., max_tokens=...)   load a model folder
    Engine.from_config(config, seed)                            seeded random weights
    engine.generate(prompts, GenParams(...))                    token ids in, token ids out
    engine.step([...])                                          the step function itself
    write_model_folder(folder, config, seed)                    random-weights model folder
"""
from .config.base import ConfigError, load_config, register_architecture     # noqa: F401
from .config.llama import LlamaConfig, RopeScaling                            # noqa: F401
from .engine.batch import SequenceStep                                        # noqa: F401
from .sampling.params import GenParams                                        # noqa: F401
from .weights.safetensors_io import WeightError                               # noqa: F401
from .weights.random_init import write_model_folder                           # noqa: F401
from . import models                                                          # noqa: F401


def __getattr__(name):
    if name == "Engine":
        from .engine.engine import Engine
        return Engine
    raise AttributeError(name)
