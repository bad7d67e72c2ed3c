"""B200-native fused decode-in-matmul for QVB8 / QVB8R weight packs.

Hand-written sm_100a CUDA kernels behind a C-ABI library (``csrc/``), reached from Python through thin
extension objects that expose the entry points of the reference's ``qvb8_cuda`` / ``qvb8r_cuda`` modules.
"""
__version__ = "0.1.0"
