"""y = x W^T (+ bias) (+ residual): the one matrix product the model uses.

float32: the FMA kernel (``dsp_gemm_simt``), always; no tensor cores, no reduced-precision
mode, one FMA chain per output so that a row does not depend on its batch.
bfloat16: the weight-streaming tcgen05 kernel for up to 128 rows (decoding and the rows whose
logits are wanted); above that the persistent tcgen05/TMA kernel of this package, except that a
narrow product with a long K at a few hundred rows runs the weight-streaming kernel once per
128 rows where ``tuning.rows_in_chunks_is_faster`` says so (the many-row kernel does not split K).  Operands
those kernels cannot take (a width that is no multiple of 8) go to the FMA kernel when there
are at most 64 rows or 32-bit logits are wanted, and otherwise to the library matrix product
(cuBLAS through torch.mm), which is where the reference engine itself calls a library
(puneethgv/DiSpec dispec/engine/model_runner.py:132,158,225-226,231).  ``backend=`` names a kernel outright (tests and
comparisons).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from dispec_b200.ops import library as L
from dispec_b200.ops import tuning

STREAM_MAX_ROWS = 128  # rows the weight-streaming kernel takes
NORM_SPLIT_MAX_ROWS = 64  # rows up to which a norm is split over two products


@dataclass
class NormedRows:
    """The input of a product, given as a norm that is still to be applied:
    weight * (source * rsqrt(mean(source^2) + eps)).  ``scaled`` = round(source) * weight in the
    storage type, if the product that wrote ``source`` stored it as well: then a few-row product
    multiplies ``scaled`` by its matrix and its result rows by the rsqrt factors (which it forms
    itself from ``source`` while the matrix streams), and the norm needs no kernel of its own.
    Every other consumer calls ``materialize()``, which runs the norm kernel."""
    source: torch.Tensor
    weight: torch.Tensor
    eps: float
    scaled: torch.Tensor | None = None

    @property
    def shape(self):
        return self.source.shape

    @property
    def dtype(self):
        return self.source.dtype

    @property
    def device(self):
        return self.source.device

    def materialize(self) -> torch.Tensor:
        from dispec_b200.ops.elementwise import rms_norm
        return rms_norm(self.source, self.weight, self.eps)

    def splittable(self, w: torch.Tensor) -> bool:
        """Whether the few-row kernel can take this norm apart (see the class text)."""
        x = self.scaled
        M, K = self.source.shape
        return (x is not None and x.dtype == torch.bfloat16 and M <= NORM_SPLIT_MAX_ROWS
                and self.source.stride(1) == 1 and self.source.stride(0) % 8 == 0
                and self.source.data_ptr() % 16 == 0 and stream_supported(M, K, x, w))
EPI_PLAIN, EPI_SWIGLU = 0, 1
SWIGLU_BLOCK = 16  # gate/up rows alternate in blocks of this many for the fused epilogue


def _simt(x, w, bias, residual, out):
    M, K = x.shape
    N = w.shape[0]
    L.check(L.core().dsp_gemm_simt(
        L.ptr(x), L.i64(x.stride(0)), L.ptr(w), L.ptr(bias), L.ptr(residual),
        L.i64(residual.stride(0) if residual is not None else 0), L.ptr(out), L.i64(out.stride(0)),
        M, N, K, L.dtype_code(x.dtype), L.dtype_code(out.dtype), L.stream_handle()))
    return out


def _tcgen05(x, w, bias, residual, out, pairs: bool = True, epilogue=EPI_PLAIN):
    """The many-row product; ``pairs``: CTA pairs (cta_group::2), the default, or single CTAs."""
    M, K = x.shape
    N = w.shape[0]
    L.check(L.core().dsp_gemm_tcgen05(
        L.ptr(x), L.i64(x.stride(0)), L.ptr(w), L.ptr(bias), L.ptr(residual),
        L.i64(residual.stride(0) if residual is not None else 0), L.ptr(out), L.i64(out.stride(0)),
        M, N, K, L.dtype_code(out.dtype), int(pairs), epilogue, L.stream_handle()))
    return out


def _stream(x, w, bias, residual, out, epilogue=EPI_PLAIN, target_ctas: int | None = None,
            norm: NormedRows | None = None, scaled_out: tuple | None = None):
    """The few-row product; ``target_ctas``: resident CTA slots the launch may fill by splitting K
    over a cluster (default: one per SM of the device).  ``norm``: x is ``norm.scaled`` and the
    result rows take the norm's rsqrt factors.  ``scaled_out`` = (gain, out2): out2 = out * gain."""
    M = x.shape[0]
    N, K = w.shape
    if target_ctas is None:
        target_ctas = tuning.stream_target_ctas(x.device)
    src = norm.source if norm is not None else None
    gain2, out2 = scaled_out if scaled_out is not None else (None, None)
    L.check(L.core().dsp_gemm_stream(
        L.ptr(x), L.i64(x.stride(0)), L.ptr(w), L.ptr(bias), L.ptr(residual),
        L.i64(residual.stride(0) if residual is not None else 0), L.ptr(out), L.i64(out.stride(0)),
        M, N, K, L.dtype_code(out.dtype), target_ctas, epilogue,
        L.i64(tuning.STREAM_LATE_TRIGGER_BYTES), L.ptr(src), L.i64(src.stride(0) if src is not None else 0),
        ctypes.c_float(norm.eps if norm is not None else 0.0), L.ptr(gain2), L.ptr(out2),
        L.i64(out2.stride(0) if out2 is not None else 0), L.stream_handle()))
    return out


def tcgen05_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def stream_supported(M: int, K: int, x: torch.Tensor, w: torch.Tensor) -> bool:
    return (M <= STREAM_MAX_ROWS and K % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gate_up_swiglu_supported(x, w: torch.Tensor) -> bool:
    """Whether silu(gate) * up can be formed in the epilogue of the gate/up product."""
    M, K = x.shape
    if x.dtype != torch.bfloat16 or w.shape[0] % 32:
        return False
    if isinstance(x, NormedRows):
        x = x.scaled if x.splittable(w) else x.source
    if M <= STREAM_MAX_ROWS:
        return stream_supported(M, K, x, w)
    return tcgen05_supported(x, w)


def linear_gate_up_swiglu(x, w_interleaved, out=None):
    """silu(x Wg^T) * (x Wu^T) in one kernel: ``w_interleaved`` holds 16 gate rows, the 16 up
    rows of the same outputs, the next 16 gate rows, ...  Returns [M, N/2].  ``x``: a tensor or
    ``NormedRows``."""
    assert gate_up_swiglu_supported(x, w_interleaved)
    norm = None
    if isinstance(x, NormedRows):
        if x.splittable(w_interleaved):
            norm, x = x, x.scaled
        else:
            x = x.materialize()
    M, N = x.shape[0], w_interleaved.shape[0]
    if out is None:
        out = torch.empty((M, N // 2), dtype=x.dtype, device=x.device)
    if M > STREAM_MAX_ROWS:
        return _tcgen05(x, w_interleaved, None, None, out, epilogue=EPI_SWIGLU)
    return _stream(x, w_interleaved, None, None, out, epilogue=EPI_SWIGLU, norm=norm)


def _library(x, w, bias, residual, out):
    """The library matrix product; bias and residual are folded in by the library as well."""
    assert out.dtype == torch.bfloat16
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


def linear(x, w: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None, out_dtype: torch.dtype | None = None,
           out: torch.Tensor | None = None, backend: str | None = None, then_norm=None):
    """x [M, K] (row stride free, unit column stride), w [N, K] contiguous, bias [N],
    residual [M, N] of the output type.  Output type: ``out_dtype`` (default: x's);
    bfloat16 inputs may produce float32 (logits).  ``backend``: "stream", "tcgen05", "library"
    or "simt" instead of the choice described at the top of this file.

    ``x`` may be ``NormedRows`` (a norm still to be applied): the few-row kernel takes it apart
    where it can, otherwise the norm kernel runs first.  ``then_norm`` = (weight, eps) of the
    norm that follows this product: the call returns (out, NormedRows of out), with the scaled
    copy filled in where the few-row kernel wrote it."""
    norm = None
    if isinstance(x, NormedRows):
        if backend in (None, "stream") and x.splittable(w):
            norm, x, backend = x, x.scaled, "stream"
        elif (backend is None and x.scaled is not None and x.scaled.dtype == torch.bfloat16
              and x.source.shape[0] > STREAM_MAX_ROWS and x.source.stride(1) == 1 and x.source.stride(0) % 8 == 0
              and x.source.data_ptr() % 16 == 0 and stream_supported(STREAM_MAX_ROWS, x.source.shape[1], x.scaled, w)
              and tuning.rows_in_chunks_is_faster(x.source.shape[0], w.shape[0], x.source.shape[1], w.device, STREAM_MAX_ROWS)):
            norm, x, backend = x, x.scaled, "stream_chunks"
        else:
            x = x.materialize()
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

    def result(scaled=None):
        if then_norm is None:
            return out
        return out, NormedRows(out, then_norm[0], then_norm[1], scaled)

    if M == 0:
        return result()
    if x.dtype == torch.float32:
        assert out_dtype == torch.float32
        _simt(x, w, bias, residual, out)
        return result()
    if backend is None:
        if stream_supported(M, K, x, w):
            backend = "stream"
        elif (M > STREAM_MAX_ROWS and stream_supported(STREAM_MAX_ROWS, K, x, w)
              and tuning.rows_in_chunks_is_faster(M, N, K, x.device, STREAM_MAX_ROWS)):
            backend = "stream_chunks"
        elif M > STREAM_MAX_ROWS and tcgen05_supported(x, w):
            backend = "tcgen05"
        elif M > STREAM_MAX_ROWS and out_dtype == torch.bfloat16:
            backend = "library"
        else:
            backend = "simt"
    if backend == "stream_chunks":
        # a narrow product with a long K at a few hundred rows: the few-row kernel per 128 rows
        # (see tuning.rows_in_chunks_is_faster); norms around it run as kernels
        for r in range(0, M, STREAM_MAX_ROWS):
            rows = slice(r, min(M, r + STREAM_MAX_ROWS))
            _stream(x[rows], w, bias, None if residual is None else residual[rows], out[rows])
        return result()
    if backend == "stream":
        scaled = None
        if (then_norm is not None and M <= NORM_SPLIT_MAX_ROWS and out_dtype == torch.bfloat16
                and then_norm[0].dtype == torch.bfloat16):
            scaled = torch.empty((M, N), dtype=out_dtype, device=x.device)
        _stream(x, w, bias, residual, out, norm=norm,
                scaled_out=(then_norm[0], scaled) if scaled is not None else None)
        return result(scaled)
    if backend == "tcgen05":
        _tcgen05(x, w, bias, residual, out)
    elif backend == "library":
        _library(x, w, bias, residual, out)
    elif backend == "simt":
        _simt(x, w, bias, residual, out)
    else:
        raise ValueError(f"unknown backend {backend!r}")
    return result()
