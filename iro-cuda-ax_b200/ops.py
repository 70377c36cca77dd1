"""Host-side operators over the C-ABI: torch tensors in, launches on the current
CUDA stream.  PyTorch is used for device memory and streams only; the arithmetic
runs in the sm_100a kernels of ``libaxp_sm100.so``.

Tensors: E4M3 operands are ``torch.float8_e4m3fn`` or ``torch.uint8``; bf16
operands ``torch.bfloat16``; scales and LSE ``torch.float32``.
"""
from __future__ import annotations

import ctypes

import torch

from . import capi

_status = {}


def status_word(device: torch.device) -> torch.Tensor:
    """The per-device status word the kernels OR error codes into."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
    return _status[idx]


def check_status(device: torch.device | None = None) -> None:
    """Synchronise and raise if any kernel's bounded wait ran out since the last check."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    st = status_word(device)
    value = int(st.item()) & 0xFFFFFFFF
    if value != 0:
        st.zero_()
        raise capi.AxpError(capi.AXP_ERR_TIMEOUT, f"device status word 0x{value:08x} (a bounded wait ran out)")


def _ptr(t: torch.Tensor | None):
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need_cuda(*ts):
    for t in ts:
        if t is not None and not t.is_cuda:
            raise ValueError("device tensors required (the kernels have no CPU path)")


def _is_fp8(t: torch.Tensor) -> bool:
    return t.dtype in (torch.float8_e4m3fn, torch.uint8)


def _check_bias(bias, N):
    if bias is None:
        return
    if bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous():
        raise ValueError("bias must be contiguous float32 of N elements")


def gemm_fp8_blockscaled(A, B, sA, sB, out=None, n_range=None, bias=None, act: int = capi.AXP_ACT_NONE):
    """C[:, n0:n1] = bf16(sum_kb sA[m,kb] sB[n/128,kb] (A_kb . B_kb^T)); A [M,K], B [N,K] E4M3."""
    _need_cuda(A, B, sA, sB, out)
    if not (_is_fp8(A) and _is_fp8(B)):
        raise TypeError("A and B must be float8_e4m3fn (or uint8 bytes)")
    if sA.dtype != torch.float32 or sB.dtype != torch.float32:
        raise TypeError("scales must be float32")
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or A.stride(1) != 1 or B.stride(1) != 1:
        raise ValueError("A [M,K] and B [N,K] must be K-contiguous with equal K")
    if tuple(sA.shape) != (M, K // 128) or tuple(sB.shape) != ((N + 127) // 128, K // 128):
        raise ValueError("sA must be [M,K/128] and sB [ceil(N/128),K/128]")
    if not (sA.is_contiguous() and sB.is_contiguous()):
        raise ValueError("scales must be contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    n0, n1 = n_range if n_range is not None else (0, N)
    _check_bias(bias, N)
    if bias is not None:
        _need_cuda(bias)
        capi.check(capi.lib().axp_sm100_gemm_fp8_blockscaled_bias_act(
            _ptr(A), _ptr(B), _ptr(sA), _ptr(sB), _ptr(bias), _ptr(out), M, N, K, A.stride(0), B.stride(0), out.stride(0),
            n0, n1, int(act), _stream(), _ptr(status_word(A.device))))
        return out
    capi.check(capi.lib().axp_sm100_gemm_fp8_blockscaled(
        _ptr(A), _ptr(B), _ptr(sA), _ptr(sB), _ptr(out), M, N, K, A.stride(0), B.stride(0), out.stride(0),
        n0, n1, _stream(), _ptr(status_word(A.device))))
    return out


def gemm_bf16(A, B, out=None, n_range=None, bias=None, act: int = capi.AXP_ACT_NONE):
    """C[:, n0:n1] = bf16(act(A . B^T + bias)) with fp32 accumulate; A [M,K], B [N,K] bf16; bias f32 [N] optional."""
    _need_cuda(A, B, out)
    if A.dtype != torch.bfloat16 or B.dtype != torch.bfloat16:
        raise TypeError("A and B must be bfloat16")
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or A.stride(1) != 1 or B.stride(1) != 1:
        raise ValueError("A [M,K] and B [N,K] must be K-contiguous with equal K")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    n0, n1 = n_range if n_range is not None else (0, N)
    _check_bias(bias, N)
    if bias is not None:
        _need_cuda(bias)
        capi.check(capi.lib().axp_sm100_gemm_bf16_bias_act(
            _ptr(A), _ptr(B), _ptr(bias), _ptr(out), M, N, K, A.stride(0), B.stride(0), out.stride(0), n0, n1, int(act),
            _stream(), _ptr(status_word(A.device))))
        return out
    capi.check(capi.lib().axp_sm100_gemm_bf16(
        _ptr(A), _ptr(B), _ptr(out), M, N, K, A.stride(0), B.stride(0), out.stride(0), n0, n1, _stream(),
        _ptr(status_word(A.device))))
    return out


def gemm_lincomb(A, B, C_in, alpha: float, beta: float, sA=None, sB=None, out=None, n_range=None):
    """D[:, n0:n1] = bf16(alpha * (A . B^T) + beta * C_in): the linear-combination epilogue.  bf16 operands, or E4M3
    operands with block scales ``sA`` / ``sB``; ``out`` may be ``C_in`` (in-place update)."""
    _need_cuda(A, B, C_in, sA, sB, out)
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or A.stride(1) != 1 or B.stride(1) != 1:
        raise ValueError("A [M,K] and B [N,K] must be K-contiguous with equal K")
    if C_in.dtype != torch.bfloat16 or C_in.shape != (M, N) or C_in.stride(1) != 1:
        raise ValueError("C_in must be bf16 [M,N] with contiguous rows")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=A.device)
    n0, n1 = n_range if n_range is not None else (0, N)
    cf = ctypes.c_float
    if sA is None:
        if A.dtype != torch.bfloat16 or B.dtype != torch.bfloat16:
            raise TypeError("A and B must be bfloat16 (or pass sA, sB for E4M3 operands)")
        capi.check(capi.lib().axp_sm100_gemm_bf16_lincomb(
            _ptr(A), _ptr(B), _ptr(C_in), _ptr(out), cf(alpha), cf(beta), M, N, K, A.stride(0), B.stride(0), C_in.stride(0),
            out.stride(0), n0, n1, _stream(), _ptr(status_word(A.device))))
    else:
        if not (_is_fp8(A) and _is_fp8(B)):
            raise TypeError("A and B must be float8_e4m3fn (or uint8 bytes) when scales are given")
        capi.check(capi.lib().axp_sm100_gemm_fp8_blockscaled_lincomb(
            _ptr(A), _ptr(B), _ptr(sA), _ptr(sB), _ptr(C_in), _ptr(out), cf(alpha), cf(beta), M, N, K, A.stride(0), B.stride(0),
            C_in.stride(0), out.stride(0), n0, n1, _stream(), _ptr(status_word(A.device))))
    return out


def gemm_bf16_swiglu(X, Wg, Wu, out=None, n_range=None):
    """H[:, n0:n1] = bf16(SiLU(X . Wg^T) * (X . Wu^T)); X [M,K], Wg / Wu [N,K] bf16 (gate / up projection in one pass)."""
    _need_cuda(X, Wg, Wu, out)
    if X.dtype != torch.bfloat16 or Wg.dtype != torch.bfloat16 or Wu.dtype != torch.bfloat16:
        raise TypeError("X, Wg, Wu must be bfloat16")
    M, K = X.shape
    N = Wg.shape[0]
    if Wg.shape != Wu.shape or Wg.shape[1] != K or X.stride(1) != 1 or Wg.stride(1) != 1 or Wu.stride(1) != 1:
        raise ValueError("X [M,K], Wg and Wu [N,K] must be K-contiguous with equal shapes")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=X.device)
    n0, n1 = n_range if n_range is not None else (0, N)
    capi.check(capi.lib().axp_sm100_gemm_bf16_swiglu(
        _ptr(X), _ptr(Wg), _ptr(Wu), _ptr(out), M, N, K, X.stride(0), Wg.stride(0), Wu.stride(0), out.stride(0), n0, n1,
        _stream(), _ptr(status_word(X.device))))
    return out


def gemm_fp8_blockscaled_swiglu(X, Wg, Wu, sX, sWg, sWu, out=None, n_range=None):
    """H[:, n0:n1] = bf16(SiLU(X . Wg^T) * (X . Wu^T)) on E4M3 operands: X [M,K] with 1x128 scales sX [M,K/128],
    Wg / Wu [N,K] with 128x128 scales sWg / sWu [ceil(N/128),K/128]."""
    _need_cuda(X, Wg, Wu, sX, sWg, sWu, out)
    for t in (X, Wg, Wu):
        if t.dtype not in (torch.float8_e4m3fn, torch.uint8):
            raise TypeError("X, Wg, Wu must be float8_e4m3fn (or uint8 bytes)")
    M, K = X.shape
    N = Wg.shape[0]
    if Wg.shape != Wu.shape or Wg.shape[1] != K or X.stride(1) != 1 or Wg.stride(1) != 1 or Wu.stride(1) != 1:
        raise ValueError("X [M,K], Wg and Wu [N,K] must be K-contiguous with equal shapes")
    kb, nb = K // 128, (N + 127) // 128
    for s, shape in ((sX, (M, kb)), (sWg, (nb, kb)), (sWu, (nb, kb))):
        if s.dtype != torch.float32 or tuple(s.shape) != shape or not s.is_contiguous():
            raise ValueError(f"scales must be contiguous float32 of shape {shape}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.bfloat16, device=X.device)
    n0, n1 = n_range if n_range is not None else (0, N)
    capi.check(capi.lib().axp_sm100_gemm_fp8_blockscaled_swiglu(
        _ptr(X), _ptr(Wg), _ptr(Wu), _ptr(sX), _ptr(sWg), _ptr(sWu), _ptr(out), M, N, K, X.stride(0), Wg.stride(0), Wu.stride(0),
        out.stride(0), n0, n1, _stream(), _ptr(status_word(X.device))))
    return out


def gemm_fp8_blockscaled_quant(A, B, sA, sB, out=None, scales=None, n_range=None, bias=None, act: int = capi.AXP_ACT_NONE):
    """The block-scaled GEMM with a quantising epilogue: returns (Cq [M,N] float8_e4m3fn, scales [M,N/128] f32), bit for bit
    ``quantize_rows_e4m3(gemm_fp8_blockscaled(...))`` (bias / activation included) without the bf16 C reaching HBM."""
    _need_cuda(A, B, sA, sB, out, scales, bias)
    if not (_is_fp8(A) and _is_fp8(B)):
        raise TypeError("A and B must be float8_e4m3fn (or uint8 bytes)")
    if sA.dtype != torch.float32 or sB.dtype != torch.float32:
        raise TypeError("scales must be float32")
    M, K = A.shape
    N = B.shape[0]
    if B.shape[1] != K or A.stride(1) != 1 or B.stride(1) != 1:
        raise ValueError("A [M,K] and B [N,K] must be K-contiguous")
    if tuple(sA.shape) != (M, K // 128) or tuple(sB.shape) != ((N + 127) // 128, K // 128) or not (sA.is_contiguous() and sB.is_contiguous()):
        raise ValueError("sA [M,K/128] and sB [ceil(N/128),K/128] must be contiguous")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float8_e4m3fn, device=A.device)
    if scales is None:
        scales = torch.empty((M, N // 128), dtype=torch.float32, device=A.device)
    if tuple(out.shape) != (M, N) or out.stride(1) != 1 or not _is_fp8(out):
        raise ValueError("out must be an [M,N] E4M3 (or uint8) matrix with contiguous rows")
    if scales.dtype != torch.float32 or tuple(scales.shape) != (M, N // 128) or not scales.is_contiguous():
        raise ValueError("scales must be contiguous float32 [M, N/128]")
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise ValueError("bias must be a contiguous float32 vector of N elements")
    n0, n1 = n_range if n_range is not None else (0, N)
    capi.check(capi.lib().axp_sm100_gemm_fp8_blockscaled_quant(
        _ptr(A), _ptr(B), _ptr(sA), _ptr(sB), _ptr(bias) if bias is not None else None, act, _ptr(out), _ptr(scales), M, N, K, A.stride(0),
        B.stride(0), out.stride(0), n0, n1, _stream(), _ptr(status_word(A.device))))
    return out, scales


def gemm_fp8_blockscaled_swiglu_quant(X, Wg, Wu, sX, sWg, sWu, out=None, scales=None, n_range=None):
    """The gate / up pass with a quantising epilogue: returns (Hq [M,N] float8_e4m3fn, scales [M,N/128] f32), bit for bit
    ``quantize_rows_e4m3(gemm_fp8_blockscaled_swiglu(...))`` without the bf16 H ever reaching HBM: the A / sA operands of
    the down projection.  N and the column range must be multiples of 128."""
    _need_cuda(X, Wg, Wu, sX, sWg, sWu, out, scales)
    for t in (X, Wg, Wu):
        if t.dtype not in (torch.float8_e4m3fn, torch.uint8):
            raise TypeError("X, Wg, Wu must be float8_e4m3fn (or uint8 bytes)")
    M, K = X.shape
    N = Wg.shape[0]
    if Wg.shape != Wu.shape or Wg.shape[1] != K or X.stride(1) != 1 or Wg.stride(1) != 1 or Wu.stride(1) != 1:
        raise ValueError("X [M,K], Wg and Wu [N,K] must be K-contiguous with equal shapes")
    kb, nb = K // 128, (N + 127) // 128
    for s_, shape in ((sX, (M, kb)), (sWg, (nb, kb)), (sWu, (nb, kb))):
        if s_.dtype != torch.float32 or tuple(s_.shape) != shape or not s_.is_contiguous():
            raise ValueError(f"scales must be contiguous float32 of shape {shape}")
    if out is None:
        out = torch.empty((M, N), dtype=torch.float8_e4m3fn, device=X.device)
    if scales is None:
        scales = torch.empty((M, N // 128), dtype=torch.float32, device=X.device)
    if out.dtype not in (torch.float8_e4m3fn, torch.uint8) or out.stride(1) != 1 or tuple(out.shape) != (M, N):
        raise ValueError("out must be an [M,N] E4M3 (or uint8) matrix with contiguous rows")
    if scales.dtype != torch.float32 or tuple(scales.shape) != (M, N // 128) or not scales.is_contiguous():
        raise ValueError("scales must be contiguous float32 [M, N/128]")
    n0, n1 = n_range if n_range is not None else (0, N)
    capi.check(capi.lib().axp_sm100_gemm_fp8_blockscaled_swiglu_quant(
        _ptr(X), _ptr(Wg), _ptr(Wu), _ptr(sX), _ptr(sWg), _ptr(sWu), _ptr(out), _ptr(scales), M, N, K, X.stride(0), Wg.stride(0),
        Wu.stride(0), out.stride(0), n0, n1, _stream(), _ptr(status_word(X.device))))
    return out, scales


def quantize_rows_e4m3(X, out=None, scales=None):
    """bf16 X [M,K] -> (Q [M,K] float8_e4m3fn, scales [M,K/128] f32): the A / sA operands of the FP8 GEMM."""
    _need_cuda(X, out, scales)
    if X.dtype != torch.bfloat16 or X.dim() != 2 or X.stride(1) != 1:
        raise TypeError("X must be a K-contiguous bfloat16 matrix")
    M, K = X.shape
    if out is None:
        out = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=X.device)
    if scales is None:
        scales = torch.empty((M, K // 128), dtype=torch.float32, device=X.device)
    capi.check(capi.lib().axp_sm100_quantize_rows_e4m3(_ptr(X), _ptr(out), _ptr(scales), M, K, X.stride(0), out.stride(0),
                                                       _stream()))
    return out, scales


def rmsnorm_quantize_rows_e4m3(X, W, eps: float = 1e-5, out=None, scales=None):
    """bf16 X [M,K], weight W [K] -> (Q, scales) of RMSNorm(x) * w in the FP8 GEMM's operand layout; the normalised
    activations are never written."""
    _need_cuda(X, W, out, scales)
    if X.dtype != torch.bfloat16 or X.dim() != 2 or X.stride(1) != 1:
        raise TypeError("X must be a K-contiguous bfloat16 matrix")
    M, K = X.shape
    if W.dtype != torch.bfloat16 or W.numel() != K or not W.is_contiguous():
        raise ValueError("W must be a contiguous bfloat16 vector of K elements")
    if out is None:
        out = torch.empty((M, K), dtype=torch.float8_e4m3fn, device=X.device)
    if scales is None:
        scales = torch.empty((M, K // 128), dtype=torch.float32, device=X.device)
    capi.check(capi.lib().axp_sm100_rmsnorm_quantize_rows_e4m3(_ptr(X), _ptr(W), ctypes.c_float(eps), _ptr(out), _ptr(scales), M, K,
                                                               X.stride(0), out.stride(0), _stream()))
    return out, scales


def mlp_fp8_forward(X, w_norm, Wg, Wu, Wd, sWg, sWu, sWd, eps: float = 1e-5, out=None, workspace=None):
    """One gated MLP block on E4M3 block-scaled weights, three launches and no bf16 intermediate in HBM:
    ``Y = (SiLU(n . Wg^T) * (n . Wu^T)) . Wd^T`` with ``n = RMSNorm(X) * w_norm``.

    X [M,K] bf16; w_norm [K] bf16; Wg, Wu [N,K] and Wd [K,N] E4M3 with 128x128 scales sWg, sWu [N/128,K/128], sWd [K/128,N/128].
    RMSNorm + quantiser -> gate / up GEMM with the quantising epilogue -> down GEMM (bf16 out).  ``workspace`` may hold
    the four intermediates ``(Xq, sX, Hq, sH)`` to avoid allocations.  Returns Y [M,K] bf16."""
    M, K = X.shape
    N = Wg.shape[0]
    if tuple(Wd.shape) != (K, N):
        raise ValueError("Wd must be [K, N] (rows = output features of the block)")
    if workspace is None:
        workspace = (None, None, None, None)
    Xq, sX = rmsnorm_quantize_rows_e4m3(X, w_norm, eps, out=workspace[0], scales=workspace[1])
    Hq, sH = gemm_fp8_blockscaled_swiglu_quant(Xq, Wg, Wu, sX, sWg, sWu, out=workspace[2], scales=workspace[3])
    return gemm_fp8_blockscaled(Hq, Wd, sH, sWd, out=out)


def _attn_dims(Q, K, V):
    B, Hq, S, D = Q.shape
    Bk, Hkv, Sk, Dk = K.shape
    if (Bk, Sk, Dk) != (B, S, D) or V.shape != K.shape or Hq % Hkv != 0:
        raise ValueError("Q [B,Hq,S,D] and K,V [B,Hkv,S,D] with Hq a multiple of Hkv required")
    if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()):
        raise ValueError("Q, K, V must be contiguous")
    return B, Hq, Hkv, S, D


def attn_fwd_bf16(Q, K, V, scale: float, causal: bool = True, out=None, lse=None, bh_range=None):
    """Flash-attention forward (bf16): returns (O [B,Hq,S,D] bf16, LSE [B,Hq,S] f32)."""
    _need_cuda(Q, K, V, out, lse)
    if Q.dtype != torch.bfloat16 or K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16:
        raise TypeError("Q, K, V must be bfloat16")
    B, Hq, Hkv, S, D = _attn_dims(Q, K, V)
    if out is None:
        out = torch.empty_like(Q)
    if lse is None:
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=Q.device)
    b0, b1 = bh_range if bh_range is not None else (0, B * Hq)
    capi.check(capi.lib().axp_sm100_attn_fwd_bf16(
        _ptr(Q), _ptr(K), _ptr(V), _ptr(out), _ptr(lse), B, Hq, Hkv, S, D, ctypes.c_float(scale), int(causal),
        b0, b1, _stream(), _ptr(status_word(Q.device))))
    return out, lse


def attn_splitkv_scratch_bytes(heads: int, Sq: int, num_splits: int) -> int:
    return int(capi.lib().axp_sm100_attn_splitkv_scratch_bytes(heads, Sq, num_splits))


def attn_fwd_bf16_splitkv(Q, K, V, scale: float, causal: bool = True, num_splits: int = 1, scratch=None, out=None, lse=None,
                          bh_range=None):
    """Split-KV attention forward: Q [B,Hq,Sq,D], K / V [B,Hkv,Skv,D] bf16 (Sq <= Skv under the causal mask: the
    queries are the last Sq positions).  `scratch` is a caller-owned uint8 device tensor of at least
    ``attn_splitkv_scratch_bytes(heads, Sq, num_splits)`` bytes; when omitted one is taken from torch's allocator
    (the C-ABI itself allocates nothing).  Returns (O [B,Hq,Sq,D] bf16, LSE [B,Hq,Sq] f32)."""
    _need_cuda(Q, K, V, out, lse, scratch)
    if Q.dtype != torch.bfloat16 or K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16:
        raise TypeError("Q, K, V must be bfloat16")
    if Q.dim() != 4 or K.dim() != 4 or K.shape != V.shape or Q.shape[0] != K.shape[0] or Q.shape[3] != K.shape[3]:
        raise ValueError("Q [B,Hq,Sq,D], K / V [B,Hkv,Skv,D]")
    if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()):
        raise ValueError("Q, K, V must be contiguous")
    B, Hq, Sq, D = Q.shape
    Hkv, Skv = K.shape[1], K.shape[2]
    if out is None:
        out = torch.empty_like(Q)
    if lse is None:
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=Q.device)
    b0, b1 = bh_range if bh_range is not None else (0, B * Hq)
    need = attn_splitkv_scratch_bytes(max(b1 - b0, 1), Sq, num_splits) if num_splits >= 1 else 0
    if scratch is None and need > 0:
        scratch = torch.empty(need, dtype=torch.uint8, device=Q.device)
    capi.check(capi.lib().axp_sm100_attn_fwd_bf16_splitkv(
        _ptr(Q), _ptr(K), _ptr(V), _ptr(out), _ptr(lse), B, Hq, Hkv, Sq, Skv, D, ctypes.c_float(scale), int(causal),
        num_splits, _ptr(scratch) if scratch is not None else None, scratch.numel() if scratch is not None else 0,
        b0, b1, _stream(), _ptr(status_word(Q.device))))
    return out, lse


def attn_fwd_fp8_splitkv(Q, K, V, q_descale, k_descale, v_descale, scale: float, causal: bool = True, num_splits: int = 1,
                         scratch=None, out=None, lse=None, bh_range=None):
    """Split-KV attention forward on an E4M3 KV cache: Q [B,Hq,Sq,D], K / V [B,Hkv,Skv,D] float8_e4m3fn (or uint8 bytes),
    descales float32 [B*Hq] / [B*Hkv]; otherwise like ``attn_fwd_bf16_splitkv``.  Returns (O bf16, LSE f32)."""
    _need_cuda(Q, K, V, q_descale, k_descale, v_descale, out, lse, scratch)
    if not (_is_fp8(Q) and _is_fp8(K) and _is_fp8(V)):
        raise TypeError("Q, K, V must be float8_e4m3fn (or uint8 bytes)")
    if Q.dim() != 4 or K.dim() != 4 or K.shape != V.shape or Q.shape[0] != K.shape[0] or Q.shape[3] != K.shape[3]:
        raise ValueError("Q [B,Hq,Sq,D], K / V [B,Hkv,Skv,D]")
    if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()):
        raise ValueError("Q, K, V must be contiguous")
    B, Hq, Sq, D = Q.shape
    Hkv, Skv = K.shape[1], K.shape[2]
    for d, n in ((q_descale, B * Hq), (k_descale, B * Hkv), (v_descale, B * Hkv)):
        if d.dtype != torch.float32 or d.numel() != n or not d.is_contiguous():
            raise ValueError("descales must be contiguous float32 of B*Hq / B*Hkv elements")
    if out is None:
        out = torch.empty((B, Hq, Sq, D), dtype=torch.bfloat16, device=Q.device)
    if lse is None:
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=Q.device)
    b0, b1 = bh_range if bh_range is not None else (0, B * Hq)
    need = attn_splitkv_scratch_bytes(max(b1 - b0, 1), Sq, num_splits) if num_splits >= 1 else 0
    if scratch is None and need > 0:
        scratch = torch.empty(need, dtype=torch.uint8, device=Q.device)
    capi.check(capi.lib().axp_sm100_attn_fwd_fp8_splitkv(
        _ptr(Q), _ptr(K), _ptr(V), _ptr(q_descale), _ptr(k_descale), _ptr(v_descale), _ptr(out), _ptr(lse), B, Hq, Hkv, Sq, Skv, D,
        ctypes.c_float(scale), int(causal), num_splits, _ptr(scratch) if scratch is not None else None,
        scratch.numel() if scratch is not None else 0, b0, b1, _stream(), _ptr(status_word(Q.device))))
    return out, lse


def attn_partial_bytes(heads: int, Sq: int) -> int:
    return int(capi.lib().axp_sm100_attn_partial_bytes(heads, Sq))


def attn_fwd_bf16_kvshard(Q, K, V, scale: float, causal: bool, kv_pos0: int, skv_total: int, partial=None):
    """Forward pass over a KV shard: Q [B,Hq,Sq,D], local K / V [B,Hkv,Skv_local,D] whose first key is global position
    ``kv_pos0`` of ``skv_total``.  Returns the partial result (uint8 tensor of ``attn_partial_bytes(B*Hq, Sq)`` bytes:
    fp32 accumulators, then (m, l) per row) for ``attn_combine_partials``."""
    _need_cuda(Q, K, V, partial)
    if Q.dtype != torch.bfloat16 or K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16:
        raise TypeError("Q, K, V must be bfloat16")
    if Q.dim() != 4 or K.dim() != 4 or K.shape != V.shape or Q.shape[0] != K.shape[0] or Q.shape[3] != K.shape[3]:
        raise ValueError("Q [B,Hq,Sq,D], K / V [B,Hkv,Skv_local,D]")
    if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()):
        raise ValueError("Q, K, V must be contiguous")
    B, Hq, Sq, D = Q.shape
    Hkv, Skv = K.shape[1], K.shape[2]
    need = attn_partial_bytes(B * Hq, Sq)
    if partial is None:
        partial = torch.empty(need, dtype=torch.uint8, device=Q.device)
    capi.check(capi.lib().axp_sm100_attn_fwd_bf16_kvshard(
        _ptr(Q), _ptr(K), _ptr(V), _ptr(partial), partial.numel(), B, Hq, Hkv, Sq, Skv, kv_pos0, skv_total, D,
        ctypes.c_float(scale), int(causal), 0, B * Hq, _stream(), _ptr(status_word(Q.device))))
    return partial


def attn_fwd_fp8_kvshard(Q, K, V, q_descale, k_descale, v_descale, scale: float, causal: bool, kv_pos0: int, skv_total: int,
                         partial=None):
    """``attn_fwd_bf16_kvshard`` on E4M3 operands (float8_e4m3fn or uint8 bytes) with per-head descales float32 [B*Hq] /
    [B*Hkv]: the partial result of the local keys, for ``attn_combine_partials``."""
    _need_cuda(Q, K, V, q_descale, k_descale, v_descale, partial)
    if not (_is_fp8(Q) and _is_fp8(K) and _is_fp8(V)):
        raise TypeError("Q, K, V must be float8_e4m3fn (or uint8 bytes)")
    if Q.dim() != 4 or K.dim() != 4 or K.shape != V.shape or Q.shape[0] != K.shape[0] or Q.shape[3] != K.shape[3]:
        raise ValueError("Q [B,Hq,Sq,D], K / V [B,Hkv,Skv_local,D]")
    if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()):
        raise ValueError("Q, K, V must be contiguous")
    B, Hq, Sq, D = Q.shape
    Hkv, Skv = K.shape[1], K.shape[2]
    for d, n in ((q_descale, B * Hq), (k_descale, B * Hkv), (v_descale, B * Hkv)):
        if d.dtype != torch.float32 or d.numel() != n or not d.is_contiguous():
            raise ValueError("descales must be contiguous float32 of B*Hq / B*Hkv elements")
    need = attn_partial_bytes(B * Hq, Sq)
    if partial is None:
        partial = torch.empty(need, dtype=torch.uint8, device=Q.device)
    capi.check(capi.lib().axp_sm100_attn_fwd_fp8_kvshard(
        _ptr(Q), _ptr(K), _ptr(V), _ptr(q_descale), _ptr(k_descale), _ptr(v_descale), _ptr(partial), partial.numel(), B, Hq, Hkv, Sq, Skv,
        kv_pos0, skv_total, D, ctypes.c_float(scale), int(causal), 0, B * Hq, _stream(), _ptr(status_word(Q.device))))
    return partial


def attn_combine_partials(partials, shape, out=None, lse=None):
    """Merges partial results (``partials``: uint8 [shares, bytes], one row per share) into O ``shape`` = [B,Hq,Sq,D]
    bf16 and LSE [B,Hq,Sq]."""
    _need_cuda(partials, out, lse)
    if partials.dtype != torch.uint8 or partials.dim() != 2 or partials.stride(1) != 1:
        raise ValueError("partials must be a uint8 [shares, bytes] tensor with contiguous rows")
    B, Hq, Sq, D = shape
    if out is None:
        out = torch.empty(shape, dtype=torch.bfloat16, device=partials.device)
    if lse is None:
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=partials.device)
    capi.check(capi.lib().axp_sm100_attn_combine_partials(_ptr(partials), partials.shape[0], partials.stride(0), _ptr(out), _ptr(lse),
                                                          B * Hq * Sq, _stream()))
    return out, lse


def attn_fwd_bf16_splitkv_static(Q, K, V, scale: float, causal: bool = True, num_splits: int = 1, out=None, lse=None,
                                 bh_range=None):
    """``attn_fwd_bf16_splitkv`` with the library's built-in 16 MiB scratch array: the call allocates nothing when
    ``out`` and ``lse`` are given.  Calls on one device must not overlap in time."""
    _need_cuda(Q, K, V, out, lse)
    if Q.dtype != torch.bfloat16 or K.dtype != torch.bfloat16 or V.dtype != torch.bfloat16:
        raise TypeError("Q, K, V must be bfloat16")
    if Q.dim() != 4 or K.dim() != 4 or K.shape != V.shape or Q.shape[0] != K.shape[0] or Q.shape[3] != K.shape[3]:
        raise ValueError("Q [B,Hq,Sq,D], K / V [B,Hkv,Skv,D]")
    if not (Q.is_contiguous() and K.is_contiguous() and V.is_contiguous()):
        raise ValueError("Q, K, V must be contiguous")
    B, Hq, Sq, D = Q.shape
    Hkv, Skv = K.shape[1], K.shape[2]
    if out is None:
        out = torch.empty_like(Q)
    if lse is None:
        lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=Q.device)
    b0, b1 = bh_range if bh_range is not None else (0, B * Hq)
    capi.check(capi.lib().axp_sm100_attn_fwd_bf16_splitkv_static(
        _ptr(Q), _ptr(K), _ptr(V), _ptr(out), _ptr(lse), B, Hq, Hkv, Sq, Skv, D, ctypes.c_float(scale), int(causal),
        num_splits, b0, b1, _stream(), _ptr(status_word(Q.device))))
    return out, lse


def attn_fwd_fp8(Q, K, V, q_descale, k_descale, v_descale, scale: float, causal: bool = True, out=None, lse=None,
                 bh_range=None):
    """FP8 flash-attention forward with GQA: returns (O bf16, LSE f32)."""
    _need_cuda(Q, K, V, q_descale, k_descale, v_descale, out, lse)
    if not (_is_fp8(Q) and _is_fp8(K) and _is_fp8(V)):
        raise TypeError("Q, K, V must be float8_e4m3fn (or uint8 bytes)")
    B, Hq, Hkv, S, D = _attn_dims(Q, K, V)
    for d, n in ((q_descale, B * Hq), (k_descale, B * Hkv), (v_descale, B * Hkv)):
        if d.dtype != torch.float32 or d.numel() != n or not d.is_contiguous():
            raise ValueError("descales must be contiguous float32 of B*Hq / B*Hkv elements")
    if out is None:
        out = torch.empty((B, Hq, S, D), dtype=torch.bfloat16, device=Q.device)
    if lse is None:
        lse = torch.empty((B, Hq, S), dtype=torch.float32, device=Q.device)
    b0, b1 = bh_range if bh_range is not None else (0, B * Hq)
    capi.check(capi.lib().axp_sm100_attn_fwd_fp8(
        _ptr(Q), _ptr(K), _ptr(V), _ptr(q_descale), _ptr(k_descale), _ptr(v_descale), _ptr(out), _ptr(lse),
        B, Hq, Hkv, S, D, ctypes.c_float(scale), int(causal), b0, b1, _stream(), _ptr(status_word(Q.device))))
    return out, lse


def causal_mask_tile(q_base: int, k_base: int, tile_m: int, tile_n: int, device=None):
    """Device-computed causal mask bits (int64 words, bit r*tile_n+c) and the whole-tile skip flag."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    words = (tile_m * tile_n + 63) // 64
    mask = torch.zeros(words, dtype=torch.int64, device=device)
    skip = torch.zeros(1, dtype=torch.int32, device=device)
    capi.check(capi.lib().axp_sm100_causal_mask_tile(q_base, k_base, tile_m, tile_n, _ptr(mask), _ptr(skip), _stream()))
    return mask, skip


def selftest_bounded_wait(limit_cycles: int = 2_000_000, device=None) -> int:
    """Runs the wait-that-runs-out self-test; returns the status word it produced."""
    device = device or torch.device("cuda", torch.cuda.current_device())
    st = torch.zeros(1, dtype=torch.int32, device=device)
    capi.check(capi.lib().axp_sm100_selftest_bounded_wait(limit_cycles, _stream(), _ptr(st)))
    torch.cuda.synchronize(device)
    return int(st.item()) & 0xFFFFFFFF
