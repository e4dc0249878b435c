"""y = x W^T (+ bias) (+ residual): the one matrix product the model uses.

float32: the FMA kernel (``dsp_gemm_simt``), always; no tensor cores, no reduced-precision
mode, one FMA chain per output so that a row does not depend on its batch.
bfloat16: the weight-streaming tensor-core kernel for up to 64 rows (decoding and the
rows whose logits are wanted); above that the tcgen05/TMA kernel of this package
(``LARGE_BACKEND = "tcgen05"``).  ``"library"`` selects the library matrix product instead
(cuBLAS through torch.mm), which is where the reference engine itself calls a library
(puneethgv/DiSpec dispec/engine/model_runner.py:132,158,225-226,231); it is kept for
comparison and is not on the default path.
"""
from __future__ import annotations

import torch

from dispec_b200.ops import library as L

SKINNY_MAX_ROWS = 64  # rows the weight-streaming kernel takes
SKINNY_TARGET_CTAS = 148 * 2  # resident CTA slots a weight-streaming launch may fill by splitting K
LARGE_BACKEND = "tcgen05"  # "tcgen05" | "library" | "simt"


def _simt(x, w, bias, residual, out):
    M, K = x.shape
    N = w.shape[0]
    L.check(L.core().dsp_gemm_simt(
        L.ptr(x), L.i64(x.stride(0)), L.ptr(w), L.ptr(bias), L.ptr(residual),
        L.i64(residual.stride(0) if residual is not None else 0), L.ptr(out), L.i64(out.stride(0)),
        M, N, K, L.dtype_code(x.dtype), L.dtype_code(out.dtype), L.stream_handle()))
    return out


PRO_NONE, PRO_RMSNORM = 0, 1
EPI_PLAIN, EPI_SWIGLU = 0, 1
SWIGLU_BLOCK = 16  # gate/up rows alternate in blocks of this many for the fused epilogue
FUSED_MAX_ROWS = 16  # rows up to which the weight-streaming kernel can fuse a prologue


def _skinny(x, w, bias, residual, out, target_ctas=None, prologue=PRO_NONE, gain=None, eps=0.0,
            epilogue=EPI_PLAIN):
    M = x.shape[0]
    N, K = w.shape
    L.check(L.skinny().dsp_gemm_skinny(
        L.ptr(x), L.i64(x.stride(0)), L.ptr(w), L.ptr(bias), L.ptr(residual),
        L.i64(residual.stride(0) if residual is not None else 0), L.ptr(out), L.i64(out.stride(0)),
        M, N, K, L.dtype_code(out.dtype), SKINNY_TARGET_CTAS if target_ctas is None else target_ctas,
        prologue, L.ptr(gain), L.f32(eps), epilogue, L.stream_handle()))
    return out


TCGEN05_PAIRS = True  # CTA pairs (cta_group::2) for the tensor-core product


def _tcgen05(x, w, bias, residual, out, pairs=None, epilogue=0):
    M, K = x.shape
    N = w.shape[0]
    L.check(L.core().dsp_gemm_tcgen05(
        L.ptr(x), L.i64(x.stride(0)), L.ptr(w), L.ptr(bias), L.ptr(residual),
        L.i64(residual.stride(0) if residual is not None else 0), L.ptr(out), L.i64(out.stride(0)),
        M, N, K, L.dtype_code(out.dtype), int(TCGEN05_PAIRS if pairs is None else pairs), epilogue,
        L.stream_handle()))
    return out


def tcgen05_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def skinny_supported(M: int, N: int, K: int, x: torch.Tensor, w: torch.Tensor) -> bool:
    return (M <= SKINNY_MAX_ROWS and K % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def fused_prologue_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether ``linear_rms_norm`` / ``linear_swiglu`` may be used for these operands."""
    M = x.shape[0]
    return (x.dtype == torch.bfloat16 and 0 < M <= FUSED_MAX_ROWS and w.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and x.stride(1) == 1 and x.data_ptr() % 16 == 0)


def linear_rms_norm(x, gain, eps, w, bias=None, residual=None, out_dtype=None, out=None):
    """linear(rms_norm(x, gain, eps), w, ...) in one kernel (bfloat16, at most 16 rows)."""
    assert fused_prologue_supported(x, w) and x.shape[1] == w.shape[1]
    assert gain.dtype == x.dtype and gain.shape == (x.shape[1],) and gain.is_contiguous()
    out_dtype = out_dtype or (out.dtype if out is not None else x.dtype)
    if out is None:
        out = torch.empty((x.shape[0], w.shape[0]), dtype=out_dtype, device=x.device)
    return _skinny(x, w, bias, residual, out, prologue=PRO_RMSNORM, gain=gain, eps=eps)


STREAM_BACKEND = "tcgen05"  # weight streaming for up to 64 rows: "tcgen05" (TMA + tensor memory) | "mma"


def _stream(x, w, bias, residual, out, epilogue=EPI_PLAIN, target_ctas=0):
    M = x.shape[0]
    N, K = w.shape
    L.check(L.core().dsp_gemm_stream(
        L.ptr(x), L.i64(x.stride(0)), L.ptr(w), L.ptr(bias), L.ptr(residual),
        L.i64(residual.stride(0) if residual is not None else 0), L.ptr(out), L.i64(out.stride(0)),
        M, N, K, L.dtype_code(out.dtype), target_ctas, epilogue, L.stream_handle()))
    return out


def gate_up_swiglu_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    """Whether silu(gate) * up can be formed in the epilogue of the gate/up product."""
    M, K = x.shape
    if x.dtype != torch.bfloat16 or w.shape[0] % 32:
        return False
    if M <= SKINNY_MAX_ROWS:
        return skinny_supported(M, w.shape[0], K, x, w)
    return LARGE_BACKEND == "tcgen05" and tcgen05_supported(x, w)


def linear_gate_up_swiglu(x, w_interleaved, norm=None, out=None):
    """silu(x Wg^T) * (x Wu^T) in one kernel: ``w_interleaved`` holds 16 gate rows, the 16 up
    rows of the same outputs, the next 16 gate rows, ...  Returns [M, N/2].  ``norm`` = (gain, eps)
    applies an RMSNorm to x on the way in (at most 16 rows)."""
    assert gate_up_swiglu_supported(x, w_interleaved)
    M, N = x.shape[0], w_interleaved.shape[0]
    if out is None:
        out = torch.empty((M, N // 2), dtype=x.dtype, device=x.device)
    if M > SKINNY_MAX_ROWS:
        assert norm is None
        return _tcgen05(x, w_interleaved, None, None, out, epilogue=EPI_SWIGLU)
    if norm is not None:
        return _skinny(x, w_interleaved, None, None, out, prologue=PRO_RMSNORM, gain=norm[0], eps=norm[1],
                       epilogue=EPI_SWIGLU)
    if STREAM_BACKEND == "tcgen05":
        return _stream(x, w_interleaved, None, None, out, epilogue=EPI_SWIGLU)
    return _skinny(x, w_interleaved, None, None, out, epilogue=EPI_SWIGLU)


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None, backend: str | None = None) -> torch.Tensor:
    """x [M, K] (row stride free, unit column stride), w [N, K] contiguous, bias [N],
    residual [M, N] of the output type.  Output type: ``out_dtype`` (default: x's);
    bfloat16 inputs may produce float32 (logits)."""
    if not (x.is_cuda and w.is_cuda):
        raise L.KernelError("linear: CUDA tensors only (there is no CPU path)")
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1], (x.shape, w.shape)
    assert x.stride(1) == 1 and w.is_contiguous() and x.dtype == w.dtype
    M, K = x.shape
    N = w.shape[0]
    out_dtype = out_dtype or (out.dtype if out is not None else x.dtype)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype == out_dtype
    if bias is not None:
        assert bias.shape == (N,) and bias.dtype == x.dtype and bias.is_contiguous()
    if residual is not None:
        assert residual.shape == (M, N) and residual.dtype == out_dtype and residual.stride(1) == 1
    if M == 0:
        return out
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32
        return _simt(x, w, bias, residual, out)
    if backend is None:
        if skinny_supported(M, N, K, x, w):
            backend = "skinny"
        elif M > SKINNY_MAX_ROWS and (out_dtype == torch.bfloat16 or LARGE_BACKEND == "tcgen05"):
            backend = LARGE_BACKEND
        else:
            backend = "simt"
    if backend == "skinny":
        if STREAM_BACKEND == "tcgen05":
            return _stream(x, w, bias, residual, out)
        return _skinny(x, w, bias, residual, out)
    if backend == "stream":
        return _stream(x, w, bias, residual, out)
    if backend == "mma":
        return _skinny(x, w, bias, residual, out)
    if backend == "tcgen05":
        if tcgen05_supported(x, w):
            return _tcgen05(x, w, bias, residual, out)
        backend = "library" if out_dtype == torch.bfloat16 else "simt"
    if backend == "library":
        # the library matrix product; bias and residual are folded in by the library as well
        assert out_dtype == torch.bfloat16
        if residual is not None:
            if out.data_ptr() != residual.data_ptr():
                out.copy_(residual)
            out.addmm_(x, w.t())
            if bias is not None:
                out.add_(bias)
        elif bias is not None:
            torch.addmm(bias, x, w.t(), out=out)
        else:
            torch.mm(x, w.t(), out=out)
        return out
    return _simt(x, w, bias, residual, out)
