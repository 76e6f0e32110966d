"""ReSET step-aware temperature processor on the GPU - same names as the reference's
``reset`` package (reset/reset/__init__.py:9-23)."""

from .logits_processor import (ReSETBatchProcessor, ReSETRequest, entropy_of,
                               get_newline_token_ids, scale_by_temperature)

__all__ = ["ReSETRequest", "ReSETBatchProcessor", "ReSETAdapter", "entropy_of",
           "scale_by_temperature", "get_newline_token_ids"]


def __getattr__(name):
    # ReSETAdapter subclasses a vLLM class: build it only when asked for, so the
    # package imports without vLLM (as the GPU kernels themselves do not need it).
    if name == "ReSETAdapter":
        from .logits_processor import make_adapter_class
        return make_adapter_class()
    raise AttributeError(name)
