"""chibillm_b200: a small inference engine for one NVIDIA B200.

Python entry point::

    import chibillm_b200
    llm = chibillm_b200.LLM("path/to/model", dtype="bfloat16")
    tokens = llm.generate([[1, 2, 3]], max_tokens=16)           # greedy
    tokens = llm.generate([[1, 2, 3]], max_tokens=16, temperature=0.7, seed=1)

Command line: ``python -m chibillm_b200 --help``.
"""
from . import config, parts  # noqa: F401  (registers the built-in architecture and parts)
from .api import LLM, generate
from .sampling import SamplingParams

__all__ = ["LLM", "generate", "SamplingParams"]
__version__ = "0.1.0"
