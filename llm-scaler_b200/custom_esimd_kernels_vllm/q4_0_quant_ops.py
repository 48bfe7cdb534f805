"""Importing this module registers torch.ops.custom_esimd_kernels_vllm.q4_0_quantize, as importing the reference's
extension module of the same name does (csrc/xpu/torch_extension_q4_0.cc:86)."""
from . import _register  # noqa: F401
