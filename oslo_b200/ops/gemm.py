"""GEMM on the tcgen05 tensor cores (bf16 / fp16 in, fp32 accumulate in tensor memory).

``gemm(a, b, ...)`` computes ``a @ b.T``-style products where each operand is
given by its *logical* ``[rows, K]`` matrix: a row-major tensor is passed
"K-major", a transposed view (``x.t()``) is passed "MN-major" — no copy is made
in either case.  ``linear`` is the autograd function used by every Linear layer of
this package on CUDA; on CPU (or for dtypes/shapes the kernel does not take) it
falls back to ``torch.nn.functional.linear``.

Kernel: ``csrc/gemm_sm100a.cu``.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch
import torch.nn.functional as F

from . import _lib

_EPI = {None: 0, "none": 0, "bias": 1, "gelu": 2, "gelu_grad": 3}

#: use the two-CTA kernel (256 x 256 tile on a CTA pair) automatically for large products; OSLO_B200_GEMM_2CTA=0 turns it
#: off.  Measured against the one-CTA kernel it is 7 - 12 % faster from K = 2048 up and slower at K = 256.
AUTO_TWO_CTA = __import__("os").environ.get("OSLO_B200_GEMM_2CTA", "1") == "1"


def _operand(t: torch.Tensor):
    """Classify an operand ``[.., rows, K]``: returns (tensor, mn_major, ld, inner_stride, outer_stride)."""

    def batch_strides(u):
        if u.dim() == 2:
            return 0, 0
        if u.dim() == 3:
            return u.stride(0), 0
        return u.stride(1), u.stride(0)

    rows, k = t.shape[-2], t.shape[-1]
    if t.stride(-1) == 1 and (rows == 1 or t.stride(-2) >= k):
        return (t, 0, t.stride(-2) if rows > 1 else k) + batch_strides(t)
    if t.stride(-2) == 1 and (k == 1 or t.stride(-1) >= rows):
        return (t, 1, t.stride(-1) if k > 1 else rows) + batch_strides(t)
    t = t.contiguous()
    return (t, 0, t.stride(-2)) + batch_strides(t)


def supported(a: torch.Tensor, b: torch.Tensor) -> bool:
    if not (a.is_cuda and b.is_cuda and _lib.has_cuda_kernels()):
        return False
    if a.dtype not in (torch.bfloat16, torch.float16) or a.dtype != b.dtype:
        return False
    return True


def gemm(
    a: torch.Tensor,
    b: torch.Tensor,
    bias: Optional[torch.Tensor] = None,
    epilogue: Optional[str] = None,
    out: Optional[torch.Tensor] = None,
    accumulate: bool = False,
    aux: Optional[torch.Tensor] = None,
    block_n: int = 0,
    causal: int = 0,
    two_cta: Optional[bool] = None,
) -> torch.Tensor:
    """``out[.., M, N] = epilogue(a[.., M, K] @ b[.., N, K]^T (+ bias))`` on tcgen05.

    Operands are 2-D, or 3-D / 4-D with one / two leading batch dims (any strides);
    ``a`` / ``b`` may be transposed views (MN-major) — nothing is copied.  ``aux``
    (optional, same layout as ``out``) receives the pre-activation ``acc + bias``
    when ``epilogue="gelu"``.  ``causal`` selects triangular work skipping for
    attention products (see ``csrc/gemm_sm100a.cu``).  ``two_cta`` picks the kernel in which an SM pair shares one
    256 x 256 tile (``csrc/gemm2cta_sm100a.cu``); ``None`` = automatically for products with at least one such tile
    per SM pair.
    """
    assert a.dim() == b.dim() and a.dim() in (2, 3, 4), "gemm takes 2-D or batched 3-D / 4-D operands"
    M, K = a.shape[-2], a.shape[-1]
    N = b.shape[-2]
    assert b.shape[-1] == K, f"K mismatch {tuple(a.shape)} x {tuple(b.shape)}"
    nd = a.dim()
    b_in = a.shape[-3] if nd >= 3 else 1
    b_out = a.shape[0] if nd == 4 else 1
    a, a_mn, lda, sa, osa = _operand(a)
    b, b_mn, ldb, sb, osb = _operand(b)
    if out is None:
        assert not accumulate
        out = torch.empty(tuple(a.shape[:-2]) + (M, N), dtype=a.dtype, device=a.device)
    assert out.stride(-1) == 1 and out.dim() == nd
    ldc = out.stride(-2) if M > 1 else N
    sc = out.stride(-3) if nd >= 3 else 0
    osc = out.stride(0) if nd == 4 else 0
    if aux is not None:
        assert aux.stride() == out.stride()
    from oslo_b200.transformers import profiler as _prof

    if _prof._ACTIVE is not None:
        _prof.report_gemm_flops(M, N, K, b_in * b_out)
    lib = _lib.cuda_lib()
    status = _lib.status_word(a.device)
    use_epi = _EPI[epilogue] if (bias is not None or epilogue in ("gelu", "gelu_grad")) else 0
    if use_epi == 3:
        # ``aux`` is an INPUT here: the product is multiplied by gelu_tanh'(aux) element by element
        assert aux is not None and bias is None and not accumulate, "gelu_grad takes aux (the pre-activation) and nothing else"
    if two_cta is None and block_n == 0 and causal == 0:
        from . import gemm_algo

        tuned = gemm_algo.lookup(M, N, K, a_mn, b_mn, a.dtype, b_in * b_out)  # offline search results, when a map is loaded
        if tuned is not None:
            two_cta, block_n = tuned.two_cta, tuned.block_n
    if two_cta is None:
        pairs = _lib.num_sms() // 2
        tiles = b_in * b_out * ((M + 255) // 256) * ((N + 255) // 256)
        two_cta = AUTO_TWO_CTA and causal == 0 and block_n == 0 and M >= 256 and N >= 256 and K >= 1024 and tiles >= pairs
    if two_cta:
        rc = lib.oslo_gemm_tcgen05_2cta(
            _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(aux),
            ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(b_in),
            ctypes.c_longlong(lda), ctypes.c_longlong(ldb), ctypes.c_longlong(ldc),
            ctypes.c_longlong(sa), ctypes.c_longlong(sb), ctypes.c_longlong(sc),
            ctypes.c_int(a_mn), ctypes.c_int(b_mn), ctypes.c_int(1 if a.dtype == torch.bfloat16 else 0),
            ctypes.c_int(use_epi), ctypes.c_int(1 if accumulate else 0), ctypes.c_int(_lib.num_sms()), _lib.ptr(status),
            _lib.stream_ptr(), ctypes.c_int(b_out), ctypes.c_longlong(osa), ctypes.c_longlong(osb), ctypes.c_longlong(osc))
        if rc == 0:
            return out
        if rc != -8:  # -8: shape too small for a 256-wide tile, use the one-CTA kernel below
            raise RuntimeError(f"oslo_gemm_tcgen05_2cta failed with code {rc} for {tuple(a.shape)} x {tuple(b.shape)}")
    rc = lib.oslo_gemm_tcgen05(
        _lib.ptr(a), _lib.ptr(b), _lib.ptr(out), _lib.ptr(bias), _lib.ptr(aux),
        ctypes.c_int(M), ctypes.c_int(N), ctypes.c_int(K), ctypes.c_int(b_in),
        ctypes.c_longlong(lda), ctypes.c_longlong(ldb), ctypes.c_longlong(ldc),
        ctypes.c_longlong(sa), ctypes.c_longlong(sb), ctypes.c_longlong(sc),
        ctypes.c_int(a_mn), ctypes.c_int(b_mn), ctypes.c_int(1 if a.dtype == torch.bfloat16 else 0),
        ctypes.c_int(use_epi), ctypes.c_int(1 if accumulate else 0), ctypes.c_int(block_n),
        ctypes.c_int(_lib.num_sms()), _lib.ptr(status), _lib.stream_ptr(),
        ctypes.c_int(b_out), ctypes.c_longlong(osa), ctypes.c_longlong(osb), ctypes.c_longlong(osc),
        ctypes.c_int(causal),
    )
    if rc != 0:
        raise RuntimeError(
            f"oslo_gemm_tcgen05 failed with code {rc} for {tuple(a.shape)} (strides {a.stride()}) x "
            f"{tuple(b.shape)} (strides {b.stride()})"
        )
    return out


def _aligned(*dims) -> bool:
    return all(d % 8 == 0 for d in dims)


class _LinearFn(torch.autograd.Function):
    """y = x W^T (+ b); dX = dY W; dW = dY^T x; db = column sum — three tcgen05 GEMMs."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        # allocate the result in its final shape: returning a view made here would forbid in-place ops on it
        y = torch.empty(*x.shape[:-1], weight.shape[0], dtype=x.dtype, device=x.device)
        gemm(x2, weight, bias=bias, epilogue="bias" if bias is not None else None, out=y.view(-1, weight.shape[0]))
        ctx.save_for_backward(x2, weight)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return y

    @staticmethod
    def backward(ctx, gy):
        x2, weight = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dX[M, K] = dY[M, N] x (W^T)[K, N]^T : B operand is W viewed [K, N] -> MN-major
            gx = torch.empty(ctx.x_shape, dtype=gy2.dtype, device=gy2.device)
            gemm(gy2, weight.t(), out=gx.view(-1, weight.shape[1]))
        if ctx.needs_input_grad[1]:
            # dW[N, K] = (dY^T)[N, M] x (x^T)[K, M]^T : both operands MN-major
            gw = gemm(gy2.t(), x2.t())
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .activation import colsum

            gb = colsum(gy2)
        return gx, gw, gb


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Drop-in for ``F.linear`` that runs the tcgen05 kernel on CUDA bf16/fp16 inputs."""
    if supported(x, weight) and _aligned(x.shape[-1], weight.shape[0], x.numel() // x.shape[-1]):
        if bias is not None and bias.dtype != x.dtype:
            bias = bias.to(x.dtype)
        return _LinearFn.apply(x, weight, bias)
    return F.linear(x, weight, bias)


def gelu_backward(gy: torch.Tensor, pre: torch.Tensor) -> torch.Tensor:
    """``gy * gelu_tanh'(pre)`` (no autograd): one pass of the bias-GELU backward kernel, or torch elsewhere."""
    from . import activation as act

    if act._cuda_ok(pre) and gy.dtype == pre.dtype:
        gy = gy.contiguous()
        dx = torch.empty_like(pre)
        rc = _lib.cuda_lib().oslo_bias_gelu_backward(
            _lib.ptr(gy), _lib.ptr(pre), None, _lib.ptr(dx), ctypes.c_longlong(pre.numel()), ctypes.c_int(pre.shape[-1]),
            ctypes.c_int(act._DT[pre.dtype]), ctypes.c_int(_lib.num_sms()), _lib.stream_ptr())
        if rc:
            raise RuntimeError(f"oslo_bias_gelu_backward failed ({rc})")
        return dx
    with torch.enable_grad():
        p = pre.detach().float().requires_grad_(True)
        y = F.gelu(p, approximate="tanh")
    (g,) = torch.autograd.grad(y, p, gy.float())
    return g.to(pre.dtype)


def gemm_bias_gelu(x2: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor]):
    """``(gelu_tanh(x2 W^T + b), x2 W^T + b)`` (no autograd): on tcgen05 both come out of ONE GEMM, whose epilogue writes
    the pre-activation as a second output and applies the GELU before the first."""
    if supported(x2, weight) and _aligned(x2.shape[-1], weight.shape[0], x2.shape[0]) and (bias is None or bias.dtype == x2.dtype):
        pre = torch.empty(x2.shape[0], weight.shape[0], dtype=x2.dtype, device=x2.device)
        h = gemm(x2, weight, bias=bias, epilogue="gelu", aux=pre)
        return h, pre
    pre = F.linear(x2, weight, bias)
    return F.gelu(pre, approximate="tanh"), pre


class _LinearGeluFn(torch.autograd.Function):
    """y = gelu_tanh(x W^T + b) with the bias and the activation in the GEMM epilogue; backward: one GELU-derivative
    pass, a column sum, and the two gradient GEMMs."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        x2 = x.reshape(-1, x.shape[-1])
        h, pre = gemm_bias_gelu(x2, weight, bias)
        ctx.save_for_backward(x2, weight, pre)
        ctx.has_bias = bias is not None
        ctx.x_shape = x.shape
        return h.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, weight, pre = ctx.saved_tensors
        dpre = gelu_backward(gy.reshape(-1, gy.shape[-1]), pre)
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            gx = matmul_nt(dpre, weight.t()).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            gw = matmul_nt(dpre.t(), x2.t())
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .activation import colsum

            gb = colsum(dpre)
        return gx, gw, gb


class _MLPGeluFn(torch.autograd.Function):
    """``y = gelu_tanh(x W1^T + b1) W2^T``.  Forward: bias + GELU in the first GEMM's epilogue.  Backward: the GEMM that
    brings the gradient back through W2 multiplies by ``gelu'(pre)`` in ITS epilogue, so the activation's backward costs no
    pass of its own over the ``[tokens, 4 hidden]`` tensor."""

    @staticmethod
    def forward(ctx, x, w1, b1, w2):
        x2 = x.reshape(-1, x.shape[-1])
        h, pre = gemm_bias_gelu(x2, w1, b1)
        y = matmul_nt(h, w2)
        ctx.save_for_backward(x2, w1, w2, pre, h)
        ctx.has_bias = b1 is not None
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w2.shape[0])

    @staticmethod
    def backward(ctx, gy):
        x2, w1, w2, pre, h = ctx.saved_tensors
        gy2 = gy.reshape(-1, gy.shape[-1])
        if not gy2.is_contiguous():
            gy2 = gy2.contiguous()
        if supported(gy2, w2.t()) and _aligned(gy2.shape[-1], w2.shape[1], gy2.shape[0]):
            dpre = gemm(gy2, w2.t(), epilogue="gelu_grad", aux=pre)
        else:
            dpre = gelu_backward(matmul_nt(gy2, w2.t()), pre)
        gx = gw1 = gb1 = gw2 = None
        if ctx.needs_input_grad[0]:
            gx = matmul_nt(dpre, w1.t()).view(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            gw1 = matmul_nt(dpre.t(), x2.t())
        if ctx.has_bias and ctx.needs_input_grad[2]:
            from .activation import colsum

            gb1 = colsum(dpre)
        if ctx.needs_input_grad[3]:
            gw2 = matmul_nt(gy2.t(), h.t())
        return gx, gw1, gb1, gw2


def mlp_gelu(x: torch.Tensor, w1: torch.Tensor, b1: Optional[torch.Tensor], w2: torch.Tensor) -> torch.Tensor:
    """``gelu_tanh(F.linear(x, w1, b1)) @ w2^T`` (the second bias is left to the caller) with both element-wise steps folded
    into GEMM epilogues, forward and backward."""
    if b1 is not None and b1.dtype != x.dtype:
        b1 = b1.to(x.dtype)
    return _MLPGeluFn.apply(x, w1, b1, w2)


def linear_gelu(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``gelu_tanh(F.linear(x, weight, bias))`` as one fused GEMM on CUDA bf16/fp16."""
    if bias is not None and bias.dtype != x.dtype:
        bias = bias.to(x.dtype)
    return _LinearGeluFn.apply(x, weight, bias)


def matmul_nt(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """``a @ b.transpose(-1, -2)`` (no autograd) with tcgen05 when possible."""
    if supported(a, b) and a.dim() in (2, 3, 4) and a.dim() == b.dim():
        return gemm(a, b)
    return torch.matmul(a, b.transpose(-1, -2))
