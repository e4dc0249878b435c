"""Python faces of the hand-written CUDA kernels.  Each function checks shapes and types,
then calls one C entry point on the current CUDA stream.  Nothing here computes on the CPU
or calls a library kernel, except ``linear`` where it says so."""
from dispec_b200.ops.attention import paged_attention
from dispec_b200.ops.elementwise import embed, feed_tokens, fill_normal, rms_norm, rope_kv_store, swiglu
from dispec_b200.ops.gemm import linear
from dispec_b200.ops.library import KernelError, device_error, raise_on_device_error
from dispec_b200.ops.sampling import argmax, sample

__all__ = ["paged_attention", "embed", "feed_tokens", "fill_normal", "rms_norm", "rope_kv_store", "swiglu", "linear",
           "KernelError", "device_error", "raise_on_device_error", "argmax", "sample"]
