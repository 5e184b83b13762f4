"""B200-native kernels behind the reference's quantized-LoRA modules.

``b2g._lib`` loads the C-ABI library (``csrc/libb2g.so``); ``b2g.ops`` wraps it as
PyTorch operators with autograd.  There is no CPU or PyTorch fallback: importing works
anywhere, calling an operator without the built library or without a CUDA device raises.
"""
