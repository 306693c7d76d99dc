"""safetyraise-lmengine_b200: a single-GPU inference engine for the Qwen3 dense
decoder on NVIDIA B200 (sm_100a), built after the engine of
QianYan-Art/SafetyRAISE-LMEngine (``rsinfer``).

Public entry points: ``Engine`` (the step function), ``LLM`` (generation through
the scheduler), ``SamplingParams``, and the command line
``python -m safetyraise_lmengine_b200 inspect|run|benchmark|replay``.
"""
from .config import qwen3 as _qwen3
from .config.registry import ARCHITECTURES, register_architecture, spec_from_config  # noqa: F401
from .errors import *  # noqa: F401,F403


def _build_decoder(spec, mctx, source):
    from .parts import attention, block, feedforward, norm, position  # noqa: F401  (register the parts)
    from .parts.model import DecoderModel
    return DecoderModel(spec, mctx, source)


register_architecture(_qwen3.ARCHITECTURE, _qwen3.read_spec, _build_decoder, _qwen3.adapt_source)

__version__ = "0.1.0"


def __getattr__(name):
    if name in ("Engine", "StepEntry"):
        from .engine import step
        return getattr(step, name)
    if name in ("LLM", "GenerationRequest", "EngineConfig"):
        from .engine import llm
        return getattr(llm, name)
    if name == "SamplingParams":
        from .sampling.params import SamplingParams
        return SamplingParams
    raise AttributeError(name)
