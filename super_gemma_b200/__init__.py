"""B200-native attention and KV kernels behind super-gemma's ``sg-gpu`` kernel interface.

The product is ``libsgattn.so`` (CUDA for sm_100a, C ABI in ``include/sgattn.h``); this package
is the thin host-side mirror of the reference's Rust API that tests and benchmarks drive it with.
"""
from .gpu import (ABI, LIB_PATH, Bounds, Buffer, BufferBinding, CommandGraph, CudaError, GpuContext, GpuError, GpuTimer,
                  Kernel, KernelBlob, NoDevice, State, StepState, Timeout, UnknownKernel, Validation, kernel_blob, kernels,
                  lib)

__all__ = ["ABI", "LIB_PATH", "Bounds", "Buffer", "BufferBinding", "CommandGraph", "CudaError", "GpuContext", "GpuError",
           "GpuTimer", "Kernel", "KernelBlob", "NoDevice", "State", "StepState", "Timeout", "UnknownKernel", "Validation",
           "kernel_blob", "kernels", "lib"]
