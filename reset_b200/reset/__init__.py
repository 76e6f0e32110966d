"""ReSET step-aware temperature processor on the GPU - same names as the reference's
``reset`` package (reset/reset/__init__.py:9-23)."""

from .logits_processor import (ReSETRequest, entropy_of, get_newline_token_ids,
                               scale_by_temperature)

__all__ = ["ReSETRequest", "ReSETBatchProcessor", "ReSETAdapter", "entropy_of",
           "scale_by_temperature", "get_newline_token_ids"]


def __getattr__(name):
    # ReSETAdapter and ReSETBatchProcessor subclass vLLM classes (vLLM only accepts
    # subclasses of its LogitsProcessor): they are built when asked for, so the package
    # imports without vLLM (the GPU kernels themselves do not need it).
    if name == "ReSETAdapter":
        from .logits_processor import make_adapter_class
        return make_adapter_class()
    if name == "ReSETBatchProcessor":
        from .logits_processor import make_batch_processor_class
        return make_batch_processor_class()
    raise AttributeError(name)
