"""GPU parity of the activation quantisation producer (bf16 -> E4M3 + 1x128 scales): bit-exact against the
host oracle (every step is one IEEE fp32 operation), and its output fed to the FP8 GEMM."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("M,K", [(1, 128), (7, 384), (256, 1024), (1000, 640), (4096, 4096)])
def test_quantize_is_bit_exact(pkg, oracle, dev, M, K):
    g = torch.Generator().manual_seed(M * 7 + K)
    X = (torch.randn(M, K, generator=g) * torch.exp(torch.randn(M, 1, generator=g) * 2)).bfloat16()
    X[0, :128] = 0                                        # an all-zero block: scale 1, codes 0
    if M > 2:
        X[2, 5] = 3.0e38                                  # huge outlier in one block
    Q, S = pkg.ops.quantize_rows_e4m3(X.to(dev))
    Qw, Sw = oracle.quantize_rows_e4m3(X.view(torch.uint16).numpy())
    assert np.array_equal(Q.view(torch.uint8).cpu().numpy(), Qw)
    assert np.array_equal(S.cpu().numpy().view(np.uint32), Sw.view(np.uint32))
    assert float(S[0, 0]) == 1.0 and not Q.view(torch.uint8)[0, :128].any()


def test_quantize_strided_and_untouched_padding(pkg, oracle, dev):
    M, K = 64, 256
    Xw = torch.randn(M, K + 64).bfloat16().to(dev)
    Qw = torch.full((M, K + 128), 0x55, dtype=torch.uint8, device=dev)
    S = torch.empty((M, K // 128), dtype=torch.float32, device=dev)
    pkg.ops.quantize_rows_e4m3(Xw[:, :K], out=Qw[:, :K].view(torch.float8_e4m3fn), scales=S)
    want_q, want_s = oracle.quantize_rows_e4m3(Xw[:, :K].contiguous().view(torch.uint16).cpu().numpy())
    assert np.array_equal(Qw[:, :K].cpu().numpy(), want_q) and np.array_equal(S.cpu().numpy(), want_s)
    assert (Qw[:, K:] == 0x55).all()


def test_quantize_properties(pkg, dev):
    """Each non-zero block uses the top code (+-448) and dequantises within half an E4M3 step of x."""
    X = torch.randn(512, 2048).bfloat16().to(dev)
    Q, S = pkg.ops.quantize_rows_e4m3(X)
    q = Q.float().view(512, 16, 128)
    assert torch.all(q.abs().amax(-1) == 448.0)
    deq = q * S.view(512, 16, 1)
    x = X.float().view(512, 16, 128)
    step = torch.maximum(deq.abs() * 2.0 ** -3, S.view(512, 16, 1) * 2.0 ** -9)      # spacing of E4M3 at |deq| (subnormal floor)
    assert torch.all((deq - x).abs() <= 0.5 * step * 1.001 + 1e-30)


def test_quantize_then_fp8_gemm_tracks_bf16_gemm(pkg, dev):
    """Producer -> FP8 block-scaled GEMM approximates the bf16 GEMM of the same operands."""
    M, N, K = 512, 768, 1024
    X, W = pkg.synth.bf16_gemm_inputs(M, N, K, seed=3, w_std=0.05)
    X, W = X.to(dev), W.to(dev)
    A, sA = pkg.ops.quantize_rows_e4m3(X)
    # weights: 128x128 block scales, quantised with torch for the test
    Wb = W.float().view(N // 128, 128, K // 128, 128)
    sB = Wb.abs().amax(dim=(1, 3)) / 448.0
    B = (Wb / sB.view(N // 128, 1, K // 128, 1)).reshape(N, K).to(torch.float8_e4m3fn)
    C8 = pkg.ops.gemm_fp8_blockscaled(A, B, sA, sB.contiguous())
    C16 = pkg.ops.gemm_bf16(X, W)
    pkg.ops.check_status(dev)
    rel = (C8.float() - C16.float()).norm() / C16.float().norm()
    assert rel < 5e-2


def test_quantize_tiny_block_with_zeros_has_no_nan(pkg, oracle, dev):
    """A block whose largest magnitude is of denormal size (1 / scale would overflow) and that also holds exact zeros:
    the scale is floored at the smallest normal float, no code is the E4M3 NaN (0x7f / 0xff), and codes and scales
    still equal the oracle's bit for bit."""
    X = torch.zeros(4, 256, dtype=torch.bfloat16)
    X[0, 3] = 1e-38
    X[1, 130] = -3e-39          # a bf16 denormal
    X[2, :128] = 9.2e-41        # the smallest bf16 denormal everywhere in the block
    X[3, 5] = 1.0
    Q, S = pkg.ops.quantize_rows_e4m3(X.to(dev))
    Qw, Sw = oracle.quantize_rows_e4m3(X.view(torch.uint16).numpy())
    q = Q.view(torch.uint8).cpu().numpy()
    assert not np.any((q & 0x7f) == 0x7f)
    assert np.all(np.isfinite(S.cpu().numpy())) and np.all(S.cpu().numpy() > 0)
    assert np.array_equal(q, Qw)
    assert np.array_equal(S.cpu().numpy().view(np.uint32), Sw.view(np.uint32))


def test_quantize_argument_errors(pkg, dev):
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.ops.quantize_rows_e4m3(torch.zeros(4, 200, dtype=torch.bfloat16, device=dev))
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG


@pytest.mark.parametrize("M,K", [(1, 128), (7, 384), (33, 2048), (64, 4096), (16, 8192), (5, 16384), (300, 2176)])
def test_rmsnorm_quantize_is_bit_exact(pkg, oracle, dev, M, K):
    """RMSNorm fused with the quantiser: codes and scales equal the oracle's bit for bit (fixed summation order, IEEE
    sqrt / division), over one to eight register chunks per thread and a ragged last chunk."""
    g = torch.Generator().manual_seed(M * 13 + K)
    X = (torch.randn(M, K, generator=g) * torch.exp(torch.randn(M, 1, generator=g) * 2)).bfloat16()
    W = (1.0 + 0.1 * torch.randn(K, generator=g)).bfloat16()
    X[0, :128] = 0
    Q, S = pkg.ops.rmsnorm_quantize_rows_e4m3(X.to(dev), W.to(dev), eps=1e-5)
    Qw, Sw = oracle.rmsnorm_quantize_rows_e4m3(X.view(torch.uint16).numpy(), W.view(torch.uint16).numpy(), 1e-5)
    assert np.array_equal(S.cpu().numpy().view(np.uint32), Sw.view(np.uint32))
    assert np.array_equal(Q.view(torch.uint8).cpu().numpy(), Qw)


def test_rmsnorm_quantize_tracks_float64_and_argument_errors(pkg, dev):
    M, K = 256, 4096
    X = (torch.randn(M, K) * 3).bfloat16().to(dev)
    W = (1.0 + 0.1 * torch.randn(K)).bfloat16().to(dev)
    Q, S = pkg.ops.rmsnorm_quantize_rows_e4m3(X, W, eps=1e-6)
    x = X.double()
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-6) * W.double()
    deq = (Q.float().view(M, K // 128, 128) * S.view(M, K // 128, 1)).view(M, K).double()
    assert ((deq - y).norm() / y.norm()).item() < 4e-2          # E4M3 has 3 mantissa bits
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.ops.rmsnorm_quantize_rows_e4m3(torch.zeros(2, 16512, dtype=torch.bfloat16, device=dev),
                                           torch.ones(16512, dtype=torch.bfloat16, device=dev))
    assert e.value.code == pkg.capi.AXP_ERR_UNSUPPORTED
    with pytest.raises(ValueError):
        pkg.ops.rmsnorm_quantize_rows_e4m3(X, W[:128])
