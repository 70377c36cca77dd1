"""ctypes binding of the CPU host oracle (``oracle/host_oracle.cpp``).

TEST INFRASTRUCTURE ONLY: the tests, the smoke check and the benchmark's
CPU-baseline leg load this module; the product package never does.  Arrays are
numpy; bf16 tensors travel as ``uint16`` bit patterns and E4M3 tensors as
``uint8`` bytes.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libhost_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the oracle with the Makefile beside this file; returns the .so path."""
    src = os.path.join(_HERE, "host_oracle.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"] + (["-B"] if force else []))
    return _LIB_PATH


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        try:
            _lib = ctypes.CDLL(_LIB_PATH)
        except OSError:
            build(force=True)
            _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


_i64 = ctypes.c_int64


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def set_num_threads(n: int) -> None:
    """OpenMP threads of the following calls (a launcher may have exported OMP_NUM_THREADS=1)."""
    lib().oracle_set_num_threads(ctypes.c_int(int(n)))


def e4m3_decode(b: np.ndarray) -> np.ndarray:
    b = np.ascontiguousarray(b, dtype=np.uint8)
    out = np.empty(b.shape, dtype=np.float32)
    lib().oracle_e4m3_decode(_p(b), _p(out), _i64(b.size))
    return out


def e4m3_encode_sat(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint8)
    lib().oracle_e4m3_encode_sat(_p(x), _p(out), _i64(x.size))
    return out


def bf16_decode(h: np.ndarray) -> np.ndarray:
    h = np.ascontiguousarray(h, dtype=np.uint16)
    out = np.empty(h.shape, dtype=np.float32)
    lib().oracle_bf16_decode(_p(h), _p(out), _i64(h.size))
    return out


def bf16_encode(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().oracle_bf16_encode(_p(x), _p(out), _i64(x.size))
    return out


def gemm_fp8_blockscaled(A, B, sA, sB, m_range=None, n_range=None, out=None) -> np.ndarray:
    """A [M,K] u8, B [N,K] u8, sA [M,K/128] f32, sB [ceil(N/128),K/128] f32 -> C [M,N] bf16 bits.

    Only rows ``m_range`` and columns ``n_range`` are written (the rest of a fresh
    output is zero)."""
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    sA = np.ascontiguousarray(sA, dtype=np.float32)
    sB = np.ascontiguousarray(sB, dtype=np.float32)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K and K % 128 == 0
    assert sA.shape == (M, K // 128) and sB.shape == ((N + 127) // 128, K // 128)
    C = out if out is not None else np.zeros((M, N), dtype=np.uint16)
    m0, m1 = m_range or (0, M)
    n0, n1 = n_range or (0, N)
    lib().oracle_gemm_fp8_blockscaled(_p(A), _p(B), _p(sA), _p(sB), _p(C), _i64(M), _i64(N), _i64(K),
                                      _i64(K), _i64(K), _i64(N), _i64(m0), _i64(m1), _i64(n0), _i64(n1))
    return C


def gemm_bf16(A, B, m_range=None, n_range=None, out=None) -> np.ndarray:
    """A [M,K], B [N,K] bf16 bits -> C [M,N] bf16 bits (fp32 accumulate)."""
    A = np.ascontiguousarray(A, dtype=np.uint16)
    B = np.ascontiguousarray(B, dtype=np.uint16)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K
    C = out if out is not None else np.zeros((M, N), dtype=np.uint16)
    m0, m1 = m_range or (0, M)
    n0, n1 = n_range or (0, N)
    lib().oracle_gemm_bf16(_p(A), _p(B), _p(C), _i64(M), _i64(N), _i64(K), _i64(K), _i64(K), _i64(N),
                           _i64(m0), _i64(m1), _i64(n0), _i64(n1))
    return C


def gemm_bf16_bias_act(A, B, bias, act: int) -> np.ndarray:
    """bf16(act(A.B^T + bias)) with act 0 = identity, 1 = SiLU; A [M,K], B [N,K] bf16 bits, bias f32 [N]."""
    A = np.ascontiguousarray(A, dtype=np.uint16)
    B = np.ascontiguousarray(B, dtype=np.uint16)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    M, K = A.shape
    N = B.shape[0]
    C = np.zeros((M, N), dtype=np.uint16)
    lib().oracle_gemm_bf16_bias_act(_p(A), _p(B), _p(bias), _p(C), _i64(M), _i64(N), _i64(K), _i64(K), _i64(K), _i64(N),
                                    ctypes.c_int(act))
    return C


def gemm_fp8_blockscaled_bias_act(A, B, sA, sB, bias, act: int) -> np.ndarray:
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    sA = np.ascontiguousarray(sA, dtype=np.float32)
    sB = np.ascontiguousarray(sB, dtype=np.float32)
    bias = np.ascontiguousarray(bias, dtype=np.float32)
    M, K = A.shape
    N = B.shape[0]
    C = np.zeros((M, N), dtype=np.uint16)
    lib().oracle_gemm_fp8_blockscaled_bias_act(_p(A), _p(B), _p(sA), _p(sB), _p(bias), _p(C), _i64(M), _i64(N), _i64(K),
                                               _i64(K), _i64(K), _i64(N), ctypes.c_int(act))
    return C


def gemm_bf16_lincomb(A, B, Cin, alpha: float, beta: float) -> np.ndarray:
    """bf16(alpha * (A.B^T) + beta * Cin); A [M,K], B [N,K], Cin [M,N] bf16 bits."""
    A = np.ascontiguousarray(A, dtype=np.uint16)
    B = np.ascontiguousarray(B, dtype=np.uint16)
    Cin = np.ascontiguousarray(Cin, dtype=np.uint16)
    M, K = A.shape
    N = B.shape[0]
    D = np.zeros((M, N), dtype=np.uint16)
    lib().oracle_gemm_bf16_lincomb(_p(A), _p(B), _p(Cin), _p(D), ctypes.c_float(alpha), ctypes.c_float(beta), _i64(M), _i64(N), _i64(K),
                                   _i64(K), _i64(K), _i64(N), _i64(N))
    return D


def gemm_fp8_blockscaled_lincomb(A, B, sA, sB, Cin, alpha: float, beta: float) -> np.ndarray:
    A = np.ascontiguousarray(A, dtype=np.uint8)
    B = np.ascontiguousarray(B, dtype=np.uint8)
    sA = np.ascontiguousarray(sA, dtype=np.float32)
    sB = np.ascontiguousarray(sB, dtype=np.float32)
    Cin = np.ascontiguousarray(Cin, dtype=np.uint16)
    M, K = A.shape
    N = B.shape[0]
    D = np.zeros((M, N), dtype=np.uint16)
    lib().oracle_gemm_fp8_blockscaled_lincomb(_p(A), _p(B), _p(sA), _p(sB), _p(Cin), _p(D), ctypes.c_float(alpha), ctypes.c_float(beta),
                                              _i64(M), _i64(N), _i64(K), _i64(K), _i64(K), _i64(N), _i64(N))
    return D


def gemm_bf16_swiglu(X, Wg, Wu) -> np.ndarray:
    """bf16(SiLU(X.Wg^T) * (X.Wu^T)); X [M,K], Wg / Wu [N,K] bf16 bits."""
    X = np.ascontiguousarray(X, dtype=np.uint16)
    Wg = np.ascontiguousarray(Wg, dtype=np.uint16)
    Wu = np.ascontiguousarray(Wu, dtype=np.uint16)
    M, K = X.shape
    N = Wg.shape[0]
    H = np.zeros((M, N), dtype=np.uint16)
    lib().oracle_gemm_bf16_swiglu(_p(X), _p(Wg), _p(Wu), _p(H), _i64(M), _i64(N), _i64(K), _i64(K), _i64(K), _i64(N))
    return H


def gemm_fp8_blockscaled_swiglu(X, Wg, Wu, sX, sWg, sWu) -> np.ndarray:
    """bf16(SiLU(X.Wg^T) * (X.Wu^T)) on E4M3 bytes with 1x128 (sX) and 128x128 (sWg, sWu) scales."""
    X = np.ascontiguousarray(X, dtype=np.uint8)
    Wg = np.ascontiguousarray(Wg, dtype=np.uint8)
    Wu = np.ascontiguousarray(Wu, dtype=np.uint8)
    sX = np.ascontiguousarray(sX, dtype=np.float32)
    sWg = np.ascontiguousarray(sWg, dtype=np.float32)
    sWu = np.ascontiguousarray(sWu, dtype=np.float32)
    M, K = X.shape
    N = Wg.shape[0]
    H = np.zeros((M, N), dtype=np.uint16)
    lib().oracle_gemm_fp8_blockscaled_swiglu(_p(X), _p(Wg), _p(Wu), _p(sX), _p(sWg), _p(sWu), _p(H), _i64(M), _i64(N), _i64(K),
                                             _i64(K), _i64(K), _i64(N))
    return H


def rmsnorm_quantize_rows_e4m3(X, W, eps: float):
    """X [M,K] bf16 bits, W [K] bf16 bits -> (Q [M,K] uint8 E4M3 of RMSNorm(x) * w, scales [M,K/128] f32)."""
    X = np.ascontiguousarray(X, dtype=np.uint16)
    W = np.ascontiguousarray(W, dtype=np.uint16).reshape(-1)
    M, K = X.shape
    assert W.size == K and K % 128 == 0
    Q = np.zeros((M, K), dtype=np.uint8)
    S = np.zeros((M, K // 128), dtype=np.float32)
    lib().oracle_rmsnorm_quantize_rows_e4m3(_p(X), _p(W), ctypes.c_float(eps), _p(Q), _p(S), _i64(M), _i64(K), _i64(K), _i64(K))
    return Q, S


def quantize_rows_e4m3(X):
    """bf16 bits X [M,K] -> (E4M3 bytes [M,K], scales f32 [M,K/128])."""
    X = np.ascontiguousarray(X, dtype=np.uint16)
    M, K = X.shape
    Q = np.zeros((M, K), dtype=np.uint8)
    S = np.zeros((M, K // 128), dtype=np.float32)
    lib().oracle_quantize_rows_e4m3(_p(X), _p(Q), _p(S), _i64(M), _i64(K), _i64(K), _i64(K))
    return Q, S


def causal_mask_tile(q_base: int, k_base: int, tile_m: int, tile_n: int):
    """Returns (mask words uint64[ceil(tile_m*tile_n/64)], skip flag)."""
    words = (tile_m * tile_n + 63) // 64
    mask = np.zeros(words, dtype=np.uint64)
    skip = ctypes.c_int(0)
    lib().oracle_causal_mask_tile(_i64(q_base), _i64(k_base), ctypes.c_int(tile_m), ctypes.c_int(tile_n),
                                  _p(mask), ctypes.byref(skip))
    return mask, int(skip.value)


def _attn_shapes(Q, K, V):
    Bq, Hq, S, D = Q.shape
    Bk, Hkv, Sk, Dk = K.shape
    assert (Bk, Sk, Dk) == (Bq, S, D) and V.shape == K.shape and Hq % Hkv == 0
    return Bq, Hq, Hkv, S, D


def attn_fwd_bf16(Q, K, V, scale: float, causal: bool, bh_range=None, q_range=None, out=None):
    """Q [B,Hq,S,D], K/V [B,Hkv,S,D] bf16 bits -> (O bf16 bits, LSE f32 [B,Hq,S])."""
    Q = np.ascontiguousarray(Q, dtype=np.uint16)
    K = np.ascontiguousarray(K, dtype=np.uint16)
    V = np.ascontiguousarray(V, dtype=np.uint16)
    B, Hq, Hkv, S, D = _attn_shapes(Q, K, V)
    O, LSE = out if out is not None else (np.zeros(Q.shape, np.uint16), np.zeros((B, Hq, S), np.float32))
    bh0, bh1 = bh_range or (0, B * Hq)
    q0, q1 = q_range or (0, S)
    lib().oracle_attn_fwd_bf16(_p(Q), _p(K), _p(V), _p(O), _p(LSE), _i64(B), _i64(Hq), _i64(Hkv), _i64(S), _i64(D),
                               ctypes.c_float(scale), ctypes.c_int(int(causal)),
                               _i64(bh0), _i64(bh1), _i64(q0), _i64(q1))
    return O, LSE


def attn_fwd_bf16_qkv(Q, K, V, scale: float, causal: bool):
    """Q [B,Hq,Sq,D], K/V [B,Hkv,Skv,D] bf16 bits with Sq <= Skv under the causal mask (the queries are the last Sq
    positions) -> (O bf16 bits [B,Hq,Sq,D], LSE f32 [B,Hq,Sq])."""
    Q = np.ascontiguousarray(Q, dtype=np.uint16)
    K = np.ascontiguousarray(K, dtype=np.uint16)
    V = np.ascontiguousarray(V, dtype=np.uint16)
    B, Hq, Sq, D = Q.shape
    _, Hkv, Skv, _ = K.shape
    assert K.shape == V.shape and K.shape[0] == B and K.shape[3] == D and Hq % Hkv == 0
    O, LSE = np.zeros(Q.shape, np.uint16), np.zeros((B, Hq, Sq), np.float32)
    lib().oracle_attn_fwd_bf16_qkv(_p(Q), _p(K), _p(V), _p(O), _p(LSE), _i64(B), _i64(Hq), _i64(Hkv), _i64(Sq), _i64(Skv),
                                   _i64(D), ctypes.c_float(scale), ctypes.c_int(int(causal)))
    return O, LSE


def attn_fwd_bf16_tile_recipe(Q, K, V, scale: float, causal: bool, tile_m: int = 128, tile_n: int = 128,
                              bh_range=None, q_range=None):
    Q = np.ascontiguousarray(Q, dtype=np.uint16)
    K = np.ascontiguousarray(K, dtype=np.uint16)
    V = np.ascontiguousarray(V, dtype=np.uint16)
    B, Hq, Hkv, S, D = _attn_shapes(Q, K, V)
    O, LSE = np.zeros(Q.shape, np.uint16), np.zeros((B, Hq, S), np.float32)
    bh0, bh1 = bh_range or (0, B * Hq)
    q0, q1 = q_range or (0, S)
    lib().oracle_attn_fwd_bf16_tile_recipe(_p(Q), _p(K), _p(V), _p(O), _p(LSE), _i64(B), _i64(Hq), _i64(Hkv),
                                           _i64(S), _i64(D), ctypes.c_float(scale), ctypes.c_int(int(causal)),
                                           ctypes.c_int(tile_m), ctypes.c_int(tile_n),
                                           _i64(bh0), _i64(bh1), _i64(q0), _i64(q1))
    return O, LSE


def attn_fwd_fp8(Q, K, V, dq, dk, dv, scale: float, causal: bool, tile_n: int = 128,
                 bh_range=None, q_range=None, out=None, rescale_threshold: float = 8.0):
    """Q [B,Hq,S,D], K/V [B,Hkv,S,D] E4M3 bytes; dq [B*Hq], dk/dv [B*Hkv] f32 descales.

    ``rescale_threshold`` (log2 units): 8 = P taken against a reference maximum that is advanced lazily (the rule the
    sm100 kernel follows); 0 = the standard online softmax with a per-tile running maximum (P <= 1), which knows
    nothing of the kernel's schedule."""
    Q = np.ascontiguousarray(Q, dtype=np.uint8)
    K = np.ascontiguousarray(K, dtype=np.uint8)
    V = np.ascontiguousarray(V, dtype=np.uint8)
    B, Hq, Hkv, S, D = _attn_shapes(Q, K, V)
    dq = np.ascontiguousarray(dq, dtype=np.float32).reshape(-1)
    dk = np.ascontiguousarray(dk, dtype=np.float32).reshape(-1)
    dv = np.ascontiguousarray(dv, dtype=np.float32).reshape(-1)
    assert dq.size == B * Hq and dk.size == B * Hkv and dv.size == B * Hkv
    O, LSE = out if out is not None else (np.zeros(Q.shape, np.uint16), np.zeros((B, Hq, S), np.float32))
    bh0, bh1 = bh_range or (0, B * Hq)
    q0, q1 = q_range or (0, S)
    lib().oracle_attn_fwd_fp8_ex(_p(Q), _p(K), _p(V), _p(dq), _p(dk), _p(dv), _p(O), _p(LSE),
                                 _i64(B), _i64(Hq), _i64(Hkv), _i64(S), _i64(D), ctypes.c_float(scale),
                                 ctypes.c_int(int(causal)), ctypes.c_int(tile_n), ctypes.c_float(rescale_threshold),
                                 _i64(bh0), _i64(bh1), _i64(q0), _i64(q1))
    return O, LSE


def shard_range(units: int, gran: int, world: int, rank: int):
    b, e = _i64(0), _i64(0)
    lib().oracle_shard_range(_i64(units), _i64(gran), ctypes.c_int(world), ctypes.c_int(rank),
                             ctypes.byref(b), ctypes.byref(e))
    return int(b.value), int(e.value)
