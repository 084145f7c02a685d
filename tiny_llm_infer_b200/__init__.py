"""A small, whole, single-GPU inference engine for NVIDIA B200 (sm_100a): model folder in,
next tokens out.  The importable name of this package is ``tiny_llm_infer_b200``.

Sub-packages: ``config`` (typed configurations, architecture registry), ``weights``
(safetensors by name, random-weights mode), ``parts`` (mixers, feed-forwards, norms,
position encodings, block arrangements), ``models`` (architectures as data, model
assembly), ``cache`` (paged keys and values, per-request state slots), ``engine`` (step
function, scheduler, LLMEngine), ``sampling``, ``ops`` and ``csrc`` (the CUDA kernels).
"""
__version__ = "0.1.0"


def __getattr__(name):
    # the public names, resolved lazily so that importing the package stays cheap
    if name in ("LLM", "LLMEngine", "EngineConfig", "GenerationResult", "SchedulerConfig"):
        from . import engine
        return getattr(engine, name)
    if name == "SamplingParams":
        from .sampling import SamplingParams
        return SamplingParams
    raise AttributeError(name)
