"""kernelcodegen_b200 — sm_100a kernels behind the KernelCodeGen operator API.

``kernelcodegen_b200.ops`` calls the C ABI (include/kcg_kernels.h) on torch CUDA tensors;
``kernelcodegen_b200.build`` compiles the native libraries in-tree.
"""
__all__ = ["ops", "build", "shard"]
