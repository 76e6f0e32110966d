"""reset_b200 - B200-native (sm_100a) implementation of the NVFP4 W4A4 small-M decode
path and the ReSET step-aware temperature processor.

Sub-modules
-----------
``capi``    tensor-level wrappers over the C ABI (``include/nvfp4r_b200.h``)
``nvfp4r``  mirror of the reference's ``nvfp4r`` Python package
            (``torch.ops.nvfp4r.*``, ``enable/disable/configure/status``)
``reset``   mirror of the reference's ``reset`` logits-processor package
``build``   in-tree build of the native libraries

Nothing here falls back to a CPU or plain-PyTorch implementation: without the built
CUDA library every call raises.
"""

__version__ = "0.1.0"
