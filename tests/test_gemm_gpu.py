"""GPU parity of the sm100 GEMM kernels against the CPU host oracle, through the
C-ABI.  Tolerances: relative Frobenius error <= 1e-2 for FP8 (the stated bar),
and for bf16 GEMM; both paths accumulate in fp32 and round once to bf16, so
element-wise the two may differ by one bf16 ulp where summation order differs."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
TOL = 1e-2


def u8(t):
    return t.view(torch.uint8).cpu().numpy()


def u16(t):
    return t.view(torch.uint16).cpu().numpy()


def rel_fro(got, want):
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


def run_fp8(pkg, dev, A, B, sA, sB, n_range=None, poison=True):
    M, N = A.shape[0], B.shape[0]
    C = torch.full((M, N), float("nan") if poison else 0.0, dtype=torch.bfloat16, device=dev)
    pkg.ops.gemm_fp8_blockscaled(A.to(dev), B.to(dev), sA.to(dev), sB.to(dev), out=C, n_range=n_range)
    pkg.ops.check_status(dev)
    return C


def one_ulp_close(got_bits, want_bits):
    """bf16 bit patterns equal or adjacent (sign-magnitude neighbours)."""
    g = got_bits.astype(np.int32)
    w = want_bits.astype(np.int32)
    return np.abs(g - w) <= 1


@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (128, 256, 128), (200, 384, 256), (1, 8, 128), (129, 520, 1024)])
def test_fp8_blockscaled_matches_oracle(pkg, oracle, dev, M, N, K):
    A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=0)          # cfg0 generator; 512^3 is cfg0 itself
    C = run_fp8(pkg, dev, A, B, sA, sB)
    want = oracle.gemm_fp8_blockscaled(u8(A), u8(B), sA.numpy(), sB.numpy())
    got = u16(C)
    assert not np.isnan(oracle.bf16_decode(got)).any()
    assert rel_fro(oracle.bf16_decode(got), oracle.bf16_decode(want)) <= TOL
    assert one_ulp_close(got, want).mean() > 0.999


def test_fp8_golden_fixture(pkg, oracle, dev, golden):
    g = golden["gemm_small"]
    A = torch.from_numpy(g["A"]).view(torch.float8_e4m3fn)
    B = torch.from_numpy(g["B"]).view(torch.float8_e4m3fn)
    C = run_fp8(pkg, dev, A, B, torch.from_numpy(g["sA"]), torch.from_numpy(g["sB"]))
    assert rel_fro(C.float().cpu().numpy(), g["C_f64"]) <= 3e-3


def test_fp8_column_shards_tile_the_output(pkg, oracle, dev):
    """N-sharding: each rank's [n0,n1) call writes only its columns; the union equals the full call."""
    M, N, K = 256, 1024, 512
    A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=3)
    full = run_fp8(pkg, dev, A, B, sA, sB)
    for world in (2, 3, 4):
        C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        Ad, Bd, sAd, sBd = A.to(dev), B.to(dev), sA.to(dev), sB.to(dev)
        for r in range(world):
            n0, n1 = pkg.shard.gemm_column_range(N, world, r)
            before = C.clone()
            pkg.ops.gemm_fp8_blockscaled(Ad, Bd, sAd, sBd, out=C, n_range=(n0, n1))
            outside = torch.ones(N, dtype=torch.bool, device=dev)
            outside[n0:n1] = False
            assert torch.equal(C[:, outside].view(torch.int16), before[:, outside].view(torch.int16))
        pkg.ops.check_status(dev)
        assert torch.equal(C.view(torch.int16), full.view(torch.int16))


def test_fp8_empty_column_range_is_a_no_op(pkg, dev):
    A, B, sA, sB = pkg.synth.fp8_gemm_inputs(128, 256, 128, seed=1)
    C = torch.zeros((128, 256), dtype=torch.bfloat16, device=dev)
    pkg.ops.gemm_fp8_blockscaled(A.to(dev), B.to(dev), sA.to(dev), sB.to(dev), out=C, n_range=(128, 128))
    pkg.ops.check_status(dev)
    assert not C.any()


def test_fp8_strided_operands(pkg, oracle, dev):
    """lda/ldb/ldc larger than the row length (views into wider buffers)."""
    M, N, K = 256, 256, 256
    A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=5)
    Aw = torch.zeros((M, K + 128), dtype=torch.uint8, device=dev)
    Bw = torch.zeros((N, K + 256), dtype=torch.uint8, device=dev)
    Aw[:, :K] = A.view(torch.uint8).to(dev)
    Bw[:, :K] = B.view(torch.uint8).to(dev)
    Cw = torch.zeros((M, N + 64), dtype=torch.bfloat16, device=dev)
    pkg.ops.gemm_fp8_blockscaled(Aw[:, :K], Bw[:, :K], sA.to(dev), sB.to(dev), out=Cw[:, :N])
    pkg.ops.check_status(dev)
    want = oracle.gemm_fp8_blockscaled(u8(A), u8(B), sA.numpy(), sB.numpy())
    assert rel_fro(Cw[:, :N].float().cpu().numpy(), oracle.bf16_decode(want)) <= TOL
    assert not Cw[:, N:].any()


def test_fp8_scale_linearity(pkg, dev):
    """Doubling sA doubles C exactly (power-of-two scaling commutes with every rounding)."""
    A, B, sA, sB = pkg.synth.fp8_gemm_inputs(256, 512, 512, seed=9)
    C1 = run_fp8(pkg, dev, A, B, sA, sB)
    C2 = run_fp8(pkg, dev, A, B, sA * 2.0, sB)
    assert torch.equal((C1.float() * 2.0).bfloat16().view(torch.int16), C2.view(torch.int16))


@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (128, 256, 64), (200, 264, 136), (8, 8, 8), (384, 1024, 4096)])
def test_bf16_matches_oracle(pkg, oracle, dev, M, N, K):
    X, W = pkg.synth.bf16_gemm_inputs(M, N, K, seed=0)
    Y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    pkg.ops.gemm_bf16(X.to(dev), W.to(dev), out=Y)
    pkg.ops.check_status(dev)
    want = oracle.gemm_bf16(u16(X), u16(W))
    got = u16(Y)
    assert rel_fro(oracle.bf16_decode(got), oracle.bf16_decode(want)) <= TOL
    assert one_ulp_close(got, want).mean() > 0.999


def test_bf16_integer_inputs_are_exact(pkg, oracle, dev):
    g = torch.Generator().manual_seed(2)
    X = torch.randint(-3, 4, (256, 512), generator=g).bfloat16()
    W = torch.randint(-3, 4, (512, 512), generator=g).bfloat16()
    Y = pkg.ops.gemm_bf16(X.to(dev), W.to(dev))
    pkg.ops.check_status(dev)
    assert np.array_equal(u16(Y), oracle.gemm_bf16(u16(X), u16(W)))       # sums are exact integers < 2^8 steps


def test_fp8_full_size_sampled_rows_and_properties(pkg, oracle, dev):
    """8192^3 (the benchmark shape): 64 random rows + tile-boundary rows against the oracle, all columns."""
    M = N = K = 8192
    A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=0, device=dev)
    C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
    pkg.ops.gemm_fp8_blockscaled(A, B, sA, sB, out=C)
    pkg.ops.check_status(dev)
    assert not torch.isnan(C).any()
    rng = np.random.default_rng(0)
    rows = np.unique(np.concatenate([rng.integers(0, M, 64), [0, 127, 128, 255, 256, 4095, 4096, M - 129, M - 128, M - 1]]))
    ridx = torch.from_numpy(rows).to(dev)
    A_s, sA_s = u8(A[ridx]), sA[ridx].cpu().numpy()
    want = oracle.gemm_fp8_blockscaled(A_s, u8(B), sA_s, sB.cpu().numpy())
    got = u16(C[ridx])
    assert rel_fro(oracle.bf16_decode(got), oracle.bf16_decode(want)) <= TOL
    assert one_ulp_close(got, want).mean() > 0.999


def test_bf16_mlp_shapes_sampled_rows(pkg, oracle, dev):
    """Llama-3-8B MLP GEMMs at 16384 tokens (gate/up and down): sampled rows against the oracle."""
    rng = np.random.default_rng(1)
    for (M, N, K) in ((16384, 14336, 4096), (16384, 4096, 14336)):
        X, W = pkg.synth.bf16_gemm_inputs(M, N, K, seed=0, device=dev)
        Y = pkg.ops.gemm_bf16(X, W)
        pkg.ops.check_status(dev)
        rows = np.unique(np.concatenate([rng.integers(0, M, 24), [0, 127, 128, M - 1]]))
        ridx = torch.from_numpy(rows).to(dev)
        want = oracle.gemm_bf16(u16(X[ridx]), u16(W))
        got = u16(Y[ridx])
        assert rel_fro(oracle.bf16_decode(got), oracle.bf16_decode(want)) <= TOL
        del X, W, Y


def test_bounded_wait_returns_status_instead_of_hanging(pkg, dev):
    """A wait on a barrier that nothing arrives on runs out and reports; the context stays usable."""
    st = pkg.ops.selftest_bounded_wait(1_000_000, dev)
    assert st & 0x80000000 and st & 0xFF
    x = torch.ones(4, device=dev)
    assert float(x.sum()) == 4.0


@pytest.mark.parametrize("cta_group,epi_wg", [(1, 2), (1, 4), (2, 2), (2, 4)])
@pytest.mark.parametrize("fp8", [True, False])
def test_kernel_variants_agree_with_oracle(pkg, oracle, dev, cta_group, epi_wg, fp8):
    """Every (CTAs per MMA, epilogue warpgroups) variant of the kernels gives the oracle's result,
    including ragged shapes that leave partial row / column tiles and a shard range."""
    pkg.capi.set_option("gemm.cta_group", cta_group)
    pkg.capi.set_option("gemm.epilogue_warpgroups", epi_wg)
    try:
        for (M, N, K, n_range) in ((512, 768, 1024, None), (200, 392, 256, None), (640, 1024, 512, (256, 768))):
            if fp8:
                A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=11)
                C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
                pkg.ops.gemm_fp8_blockscaled(A.to(dev), B.to(dev), sA.to(dev), sB.to(dev), out=C, n_range=n_range)
                want = oracle.gemm_fp8_blockscaled(u8(A), u8(B), sA.numpy(), sB.numpy())
            else:
                A, B = pkg.synth.bf16_gemm_inputs(M, N, K, seed=11)
                C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
                pkg.ops.gemm_bf16(A.to(dev), B.to(dev), out=C, n_range=n_range)
                want = oracle.gemm_bf16(u16(A), u16(B))
            pkg.ops.check_status(dev)
            n0, n1 = n_range or (0, N)
            got = u16(C)
            assert rel_fro(oracle.bf16_decode(got[:, n0:n1]), oracle.bf16_decode(want[:, n0:n1])) <= TOL
            assert one_ulp_close(got[:, n0:n1], want[:, n0:n1]).mean() > 0.999
            if n_range:
                assert torch.isnan(C[:, :n0]).all() and torch.isnan(C[:, n1:]).all()
    finally:
        pkg.capi.set_option("gemm.cta_group", 0)
        pkg.capi.set_option("gemm.epilogue_warpgroups", 0)


@pytest.mark.parametrize("fp8", [False, True])
@pytest.mark.parametrize("act", [0, 1])
def test_fused_bias_activation_epilogue(pkg, oracle, dev, fp8, act):
    """C = bf16(act(acc + bias[n])) with act identity / SiLU (the reference's BiasActivationVec epilogue),
    on ragged shapes and on a column shard."""
    g = torch.Generator().manual_seed(21)
    for (M, N, K, n_range) in ((256, 512, 512, None), (200, 392, 256, None), (384, 1024, 256, (256, 768))):
        bias = (torch.randn(N, generator=g) * 2.0).float()
        C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        if fp8:
            A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=13)
            sA = sA * 0.125                                 # keeps acc + bias in the range where SiLU bends
            pkg.ops.gemm_fp8_blockscaled(A.to(dev), B.to(dev), sA.to(dev), sB.to(dev), out=C, n_range=n_range,
                                         bias=bias.to(dev), act=act)
            want = oracle.gemm_fp8_blockscaled_bias_act(u8(A), u8(B), sA.numpy(), sB.numpy(), bias.numpy(), act)
        else:
            A, B = pkg.synth.bf16_gemm_inputs(M, N, K, seed=13, w_std=0.1)
            pkg.ops.gemm_bf16(A.to(dev), B.to(dev), out=C, n_range=n_range, bias=bias.to(dev), act=act)
            want = oracle.gemm_bf16_bias_act(u16(A), u16(B), bias.numpy(), act)
        pkg.ops.check_status(dev)
        n0, n1 = n_range or (0, N)
        got = u16(C)
        assert rel_fro(oracle.bf16_decode(got[:, n0:n1]), oracle.bf16_decode(want[:, n0:n1])) <= TOL
        assert np.abs(oracle.bf16_decode(got[:, n0:n1]) - oracle.bf16_decode(want[:, n0:n1])).max() <= 2e-2 * max(
            1.0, float(np.abs(oracle.bf16_decode(want)).max()))
        if n_range:
            assert torch.isnan(C[:, :n0]).all() and torch.isnan(C[:, n1:]).all()


def test_fused_epilogue_argument_errors(pkg, dev):
    A, B = pkg.synth.bf16_gemm_inputs(128, 256, 64, seed=1)
    with pytest.raises(ValueError):
        pkg.ops.gemm_bf16(A.to(dev), B.to(dev), bias=torch.zeros(255, device=dev))
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.ops.gemm_bf16(A.to(dev), B.to(dev), bias=torch.zeros(256, device=dev), act=7)
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG


@pytest.mark.parametrize("cta_group", [0, 1, 2])
def test_swiglu_gate_up_projection(pkg, oracle, dev, cta_group):
    """H = bf16(SiLU(X.Wg^T) * (X.Wu^T)) in one pass (gate and up accumulators side by side in tensor memory),
    on full tiles, ragged shapes and a column shard, for the single-CTA and the CTA-pair kernels."""
    pkg.capi.set_option("gemm.cta_group", cta_group)
    try:
        for (M, N, K, n_range) in ((256, 256, 512, None), (200, 392, 256, None), (384, 1024, 320, (128, 648)),
                                   (1, 8, 64, None), (130, 136, 1024, None)):
            X, Wg = pkg.synth.bf16_gemm_inputs(M, N, K, seed=31, w_std=0.08)
            _, Wu = pkg.synth.bf16_gemm_inputs(M, N, K, seed=32, w_std=0.08)
            H = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
            pkg.ops.gemm_bf16_swiglu(X.to(dev), Wg.to(dev), Wu.to(dev), out=H, n_range=n_range)
            pkg.ops.check_status(dev)
            want = oracle.bf16_decode(oracle.gemm_bf16_swiglu(u16(X), u16(Wg), u16(Wu)))
            n0, n1 = n_range or (0, N)
            got = oracle.bf16_decode(u16(H))
            assert rel_fro(got[:, n0:n1], want[:, n0:n1]) <= TOL
            assert np.abs(got[:, n0:n1] - want[:, n0:n1]).max() <= 2e-2 * max(1.0, float(np.abs(want).max()))
            if n_range:
                assert torch.isnan(H[:, :n0]).all() and torch.isnan(H[:, n1:]).all()
    finally:
        pkg.capi.set_option("gemm.cta_group", 0)


def test_swiglu_equals_two_gemms_and_elementwise(pkg, oracle, dev):
    """Property at MLP size: the fused pass agrees with SiLU(G) * U computed from two plain GEMM launches
    (those round G and U to bf16 first, hence the tolerance), and sampled rows agree with the oracle."""
    M, N, K = 1024, 2048, 1024
    X, Wg = pkg.synth.bf16_gemm_inputs(M, N, K, seed=41, w_std=0.05)
    _, Wu = pkg.synth.bf16_gemm_inputs(M, N, K, seed=42, w_std=0.05)
    Xd, Wgd, Wud = X.to(dev), Wg.to(dev), Wu.to(dev)
    H = pkg.ops.gemm_bf16_swiglu(Xd, Wgd, Wud)
    G = pkg.ops.gemm_bf16(Xd, Wgd).float()
    U = pkg.ops.gemm_bf16(Xd, Wud).float()
    pkg.ops.check_status(dev)
    ref = (G * torch.sigmoid(G) * U).cpu().numpy()
    assert rel_fro(H.float().cpu().numpy(), ref) <= TOL
    rows = [0, 127, 128, 777, 1023]
    want = oracle.bf16_decode(oracle.gemm_bf16_swiglu(u16(X)[rows], u16(Wg), u16(Wu)))
    assert rel_fro(H[rows].float().cpu().numpy(), want) <= 2e-3


def test_swiglu_argument_errors(pkg, dev):
    X, Wg = pkg.synth.bf16_gemm_inputs(128, 256, 64, seed=1)
    with pytest.raises(ValueError):
        pkg.ops.gemm_bf16_swiglu(X.to(dev), Wg.to(dev), Wg[:128].to(dev))
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.ops.gemm_bf16_swiglu(X.to(dev), Wg.to(dev), Wg.to(dev), n_range=(4, 256))
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG


def test_fp8_swiglu_gate_up_projection(pkg, oracle, dev):
    """The gate / up pass on E4M3 block-scaled operands (two scale streams, gate and up accumulators promoted side by
    side): full tiles, ragged shapes, a column shard, several K blocks."""
    for (M, N, K, n_range) in ((256, 256, 512, None), (200, 392, 256, None), (384, 1024, 384, (128, 648)),
                               (1, 8, 128, None), (130, 136, 1024, None)):
        X, Wg, sX, sWg = pkg.synth.fp8_gemm_inputs(M, N, K, seed=51)
        _, Wu, _, sWu = pkg.synth.fp8_gemm_inputs(M, N, K, seed=52)
        sX = sX * 0.0625
        H = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        pkg.ops.gemm_fp8_blockscaled_swiglu(X.to(dev), Wg.to(dev), Wu.to(dev), sX.to(dev), sWg.to(dev), sWu.to(dev), out=H, n_range=n_range)
        pkg.ops.check_status(dev)
        want = oracle.bf16_decode(oracle.gemm_fp8_blockscaled_swiglu(u8(X), u8(Wg), u8(Wu), sX.numpy(), sWg.numpy(), sWu.numpy()))
        n0, n1 = n_range or (0, N)
        got = oracle.bf16_decode(u16(H))
        assert rel_fro(got[:, n0:n1], want[:, n0:n1]) <= TOL
        assert np.abs(got[:, n0:n1] - want[:, n0:n1]).max() <= 2e-2 * max(1.0, float(np.abs(want).max()))
        if n_range:
            assert torch.isnan(H[:, :n0]).all() and torch.isnan(H[:, n1:]).all()


def test_fp8_swiglu_cta_pair_option_reproduces_the_default(pkg, dev):
    """The CTA-pair form of the E4M3 gate / up pass (option gemm.cta_group = 2; single CTAs are the default) gives the same
    bits, on full tiles, a ragged shape and a column shard."""
    for (M, N, K, n_range) in ((512, 512, 512, None), (200, 392, 256, None), (384, 1024, 384, (128, 648))):
        X, Wg, sX, sWg = pkg.synth.fp8_gemm_inputs(M, N, K, seed=71)
        _, Wu, _, sWu = pkg.synth.fp8_gemm_inputs(M, N, K, seed=72)
        d = [t.to(dev) for t in (X, Wg, Wu, sX * 0.0625, sWg, sWu)]
        H1 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        pkg.ops.gemm_fp8_blockscaled_swiglu(*d, out=H1, n_range=n_range)
        pkg.capi.set_option("gemm.cta_group", 2)
        try:
            H2 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
            pkg.ops.gemm_fp8_blockscaled_swiglu(*d, out=H2, n_range=n_range)
        finally:
            pkg.capi.set_option("gemm.cta_group", 0)
        pkg.ops.check_status(dev)
        assert torch.equal(H1.view(torch.int16), H2.view(torch.int16))


@pytest.mark.parametrize("cta_group", [0, 2])
def test_fp8_swiglu_quantising_epilogue_equals_gemm_then_quantiser(pkg, oracle, dev, cta_group):
    """The gate / up pass with the quantising epilogue leaves, bit for bit, what the stand-alone quantiser makes of the bf16
    result of the plain gate / up pass (codes and 1x128 scales), on full tiles, ragged M, several K blocks and a column
    shard; against the CPU oracle chain within the block-scaled GEMM's tolerance after dequantisation."""
    pkg.capi.set_option("gemm.cta_group", cta_group)
    try:
        for (M, N, K, n_range) in ((256, 256, 512, None), (200, 384, 256, None), (384, 1024, 384, (128, 640)), (1, 128, 128, None),
                                   (130, 640, 1024, None)):
            X, Wg, sX, sWg = pkg.synth.fp8_gemm_inputs(M, N, K, seed=81)
            _, Wu, _, sWu = pkg.synth.fp8_gemm_inputs(M, N, K, seed=82)
            d = [t.to(dev) for t in (X, Wg, Wu, sX * 0.0625, sWg, sWu)]
            H = pkg.ops.gemm_fp8_blockscaled_swiglu(*d)
            Qw, Sw = pkg.ops.quantize_rows_e4m3(H)
            Q = torch.full((M, N), 0x7f, dtype=torch.uint8, device=dev)
            S = torch.full((M, N // 128), float("nan"), dtype=torch.float32, device=dev)
            pkg.ops.gemm_fp8_blockscaled_swiglu_quant(*d, out=Q, scales=S, n_range=n_range)
            pkg.ops.check_status(dev)
            n0, n1 = n_range or (0, N)
            assert torch.equal(Q[:, n0:n1], Qw.view(torch.uint8)[:, n0:n1])
            assert torch.equal(S[:, n0 // 128:n1 // 128].view(torch.int32), Sw[:, n0 // 128:n1 // 128].view(torch.int32))
            if n_range:        # nothing outside the shard is touched
                assert (Q[:, :n0] == 0x7f).all() and (Q[:, n1:] == 0x7f).all()
                assert torch.isnan(S[:, :n0 // 128]).all() and torch.isnan(S[:, n1 // 128:]).all()
            # the oracle chain: block-scaled gate / up, then the quantiser (the GPU GEMM is not bit-exact, so dequantised values are compared)
            Hw = oracle.gemm_fp8_blockscaled_swiglu(u8(X), u8(Wg), u8(Wu), (sX * 0.0625).numpy(), sWg.numpy(), sWu.numpy())
            want = oracle.bf16_decode(Hw)[:, n0:n1]
            got = oracle.e4m3_decode(Q.cpu().numpy())[:, n0:n1] * np.repeat(S.cpu().numpy()[:, n0 // 128:n1 // 128], 128, axis=1)
            assert rel_fro(got, want) <= 4e-2          # E4M3 rounding of the outputs (2^-4 relative) on top of the GEMM's tolerance
    finally:
        pkg.capi.set_option("gemm.cta_group", 0)


def test_fp8_swiglu_quantising_epilogue_argument_errors(pkg, dev):
    X, Wg, sX, sWg = pkg.synth.fp8_gemm_inputs(128, 256, 128, seed=1)
    d = [t.to(dev) for t in (X, Wg, Wg, sX, sWg, sWg)]
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.ops.gemm_fp8_blockscaled_swiglu_quant(*d, n_range=(0, 64))                     # not whole 128-column blocks
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG
    X2, W2, sX2, sW2 = pkg.synth.fp8_gemm_inputs(128, 192, 128, seed=1)                  # N not a multiple of 128
    with pytest.raises((pkg.capi.AxpError, ValueError)):
        pkg.ops.gemm_fp8_blockscaled_swiglu_quant(*[t.to(dev) for t in (X2, W2, W2, sX2, sW2, sW2)])


@pytest.mark.parametrize("cta_group", [0, 1])
def test_fp8_gemm_quantising_epilogue_equals_gemm_then_quantiser(pkg, oracle, dev, cta_group):
    """The block-scaled GEMM with the quantising epilogue leaves, bit for bit, what the stand-alone quantiser makes of the bf16
    result (codes and 1x128 scales): plain and with bias + SiLU, ragged M, several K blocks, a column shard."""
    pkg.capi.set_option("gemm.cta_group", cta_group)
    try:
        for (M, N, K, n_range, fused) in ((256, 256, 512, None, False), (200, 384, 256, None, True), (384, 1024, 384, (256, 768), False),
                                          (1, 128, 128, None, False), (130, 640, 1024, (128, 640), True)):
            A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=95)
            d = [t.to(dev) for t in (A, B, sA, sB)]
            bias = (torch.randn(N, generator=torch.Generator().manual_seed(3)) * 4.0).to(dev) if fused else None
            act = pkg.capi.AXP_ACT_SILU if fused else pkg.capi.AXP_ACT_NONE
            C = pkg.ops.gemm_fp8_blockscaled(*d, bias=bias, act=act)
            Qw, Sw = pkg.ops.quantize_rows_e4m3(C)
            Q = torch.full((M, N), 0x7f, dtype=torch.uint8, device=dev)
            S = torch.full((M, N // 128), float("nan"), dtype=torch.float32, device=dev)
            pkg.ops.gemm_fp8_blockscaled_quant(*d, out=Q, scales=S, n_range=n_range, bias=bias, act=act)
            pkg.ops.check_status(dev)
            n0, n1 = n_range or (0, N)
            assert torch.equal(Q[:, n0:n1], Qw.view(torch.uint8)[:, n0:n1])
            assert torch.equal(S[:, n0 // 128:n1 // 128].view(torch.int32), Sw[:, n0 // 128:n1 // 128].view(torch.int32))
            if n_range:
                assert (Q[:, :n0] == 0x7f).all() and (Q[:, n1:] == 0x7f).all()
                assert torch.isnan(S[:, :n0 // 128]).all() and torch.isnan(S[:, n1 // 128:]).all()
    finally:
        pkg.capi.set_option("gemm.cta_group", 0)
    with pytest.raises(pkg.capi.AxpError) as e:
        A, B, sA, sB = (t.to(dev) for t in pkg.synth.fp8_gemm_inputs(128, 256, 128, seed=1))
        pkg.ops.gemm_fp8_blockscaled_quant(A, B, sA, sB, n_range=(0, 192))
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG


def test_fp8_mlp_block_against_the_oracle_chain(pkg, oracle, dev):
    """RMSNorm + quantiser -> E4M3 gate / up with the quantising epilogue -> E4M3 down projection, against the same chain of
    oracle functions.  The first stage is bit-exact; after it the GPU GEMMs differ from the oracle in the last bits, which
    can move single E4M3 codes of H, so the block's output is compared in the Frobenius norm."""
    M, K, N = 200, 512, 1024
    g = torch.Generator().manual_seed(5)
    X = (torch.randn(M, K, generator=g) * 2.0).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(K, generator=g)).to(torch.bfloat16)
    _, Wg, _, sWg = pkg.synth.fp8_gemm_inputs(8, N, K, seed=91)
    _, Wu, _, sWu = pkg.synth.fp8_gemm_inputs(8, N, K, seed=92)
    _, Wd, _, sWd = pkg.synth.fp8_gemm_inputs(8, K, N, seed=93)
    sWg, sWu, sWd = sWg * 0.05, sWu * 0.05, sWd * 0.05
    Y = pkg.ops.mlp_fp8_forward(*(t.to(dev) for t in (X, w, Wg, Wu, Wd, sWg, sWu, sWd)))
    pkg.ops.check_status(dev)
    xq, sx = oracle.rmsnorm_quantize_rows_e4m3(u16(X), u16(w), 1e-5)
    h = oracle.gemm_fp8_blockscaled_swiglu(xq, u8(Wg), u8(Wu), sx, sWg.numpy(), sWu.numpy())
    hq, sh = oracle.quantize_rows_e4m3(h)
    want = oracle.bf16_decode(oracle.gemm_fp8_blockscaled(hq, u8(Wd), sh, sWd.numpy()))
    got = Y.float().cpu().numpy()
    assert np.isfinite(got).all() and got.shape == (M, K)
    assert rel_fro(got, want) <= 2e-2


def test_fp8_swiglu_equals_two_gemms_and_elementwise(pkg, oracle, dev):
    """Property at MLP size: the fused pass agrees with SiLU(G) * U from two plain block-scaled GEMM launches (which
    round G and U to bf16 first, hence the tolerance); sampled rows agree with the oracle; a column-sharded run
    reproduces the unsharded result bit for bit."""
    M, N, K = 1024, 2048, 1024
    X, Wg, sX, sWg = pkg.synth.fp8_gemm_inputs(M, N, K, seed=61)
    _, Wu, _, sWu = pkg.synth.fp8_gemm_inputs(M, N, K, seed=62)
    sX = sX * 0.03125
    d = [t.to(dev) for t in (X, Wg, Wu, sX, sWg, sWu)]
    H = pkg.ops.gemm_fp8_blockscaled_swiglu(*d)
    G = pkg.ops.gemm_fp8_blockscaled(d[0], d[1], d[3], d[4]).float()
    U = pkg.ops.gemm_fp8_blockscaled(d[0], d[2], d[3], d[5]).float()
    pkg.ops.check_status(dev)
    ref = (G * torch.sigmoid(G) * U).cpu().numpy()
    assert rel_fro(H.float().cpu().numpy(), ref) <= TOL
    rows = [0, 127, 128, 777, 1023]
    want = oracle.bf16_decode(oracle.gemm_fp8_blockscaled_swiglu(u8(X)[rows], u8(Wg), u8(Wu), sX.numpy()[rows], sWg.numpy(), sWu.numpy()))
    assert rel_fro(H[rows].float().cpu().numpy(), want) <= 2e-3
    H2 = torch.empty_like(H)
    for n0, n1 in ((0, 768), (768, 2048)):
        pkg.ops.gemm_fp8_blockscaled_swiglu(*d, out=H2, n_range=(n0, n1))
    pkg.ops.check_status(dev)
    assert torch.equal(H2.view(torch.int16), H.view(torch.int16))


def test_fp8_swiglu_argument_errors(pkg, dev):
    X, Wg, sX, sW = pkg.synth.fp8_gemm_inputs(128, 256, 256, seed=1)
    d = [t.to(dev) for t in (X, Wg, Wg, sX, sW, sW)]
    with pytest.raises(ValueError):
        pkg.ops.gemm_fp8_blockscaled_swiglu(d[0], d[1], d[2], d[3], d[4], d[5][:1])
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.ops.gemm_fp8_blockscaled_swiglu(*d, n_range=(64, 256))
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG


@pytest.mark.parametrize("fp8", [False, True])
def test_linear_combination_epilogue(pkg, oracle, dev, fp8):
    """D = bf16(alpha * acc + beta * C_in) (the reference's LinearCombinationVec epilogue): three separate fp32
    operations on both sides, so the comparison is as tight as for the plain GEMM; ragged shapes, a column shard,
    the in-place form, and alpha = 1, beta = 0 equal to the plain kernel bit for bit."""
    g = torch.Generator().manual_seed(33)
    for (M, N, K, n_range, alpha, beta) in ((256, 512, 512, None, 0.75, -1.5), (200, 392, 256, None, 2.0, 0.5),
                                            (384, 1024, 256, (256, 768), -1.0, 1.0)):
        Cin = torch.randn(M, N, generator=g).bfloat16()
        D = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
        if fp8:
            A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=14)
            sA = sA * 0.125
            pkg.ops.gemm_lincomb(A.to(dev), B.to(dev), Cin.to(dev), alpha, beta, sA=sA.to(dev), sB=sB.to(dev), out=D, n_range=n_range)
            want = oracle.gemm_fp8_blockscaled_lincomb(u8(A), u8(B), sA.numpy(), sB.numpy(), u16(Cin), alpha, beta)
        else:
            A, B = pkg.synth.bf16_gemm_inputs(M, N, K, seed=14, w_std=0.1)
            pkg.ops.gemm_lincomb(A.to(dev), B.to(dev), Cin.to(dev), alpha, beta, out=D, n_range=n_range)
            want = oracle.gemm_bf16_lincomb(u16(A), u16(B), u16(Cin), alpha, beta)
        pkg.ops.check_status(dev)
        n0, n1 = n_range or (0, N)
        got = u16(D)
        assert rel_fro(oracle.bf16_decode(got[:, n0:n1]), oracle.bf16_decode(want[:, n0:n1])) <= TOL
        assert np.abs(oracle.bf16_decode(got[:, n0:n1]) - oracle.bf16_decode(want[:, n0:n1])).max() <= 2e-2 * max(
            1.0, float(np.abs(oracle.bf16_decode(want)).max()))
        if n_range:
            assert torch.isnan(D[:, :n0]).all() and torch.isnan(D[:, n1:]).all()
    # in place, and the identity combination
    A, B = pkg.synth.bf16_gemm_inputs(256, 256, 128, seed=2, w_std=0.1)
    Ad, Bd = A.to(dev), B.to(dev)
    plain = pkg.ops.gemm_bf16(Ad, Bd)
    C = torch.randn(256, 256, generator=g).bfloat16().to(dev)
    same = pkg.ops.gemm_lincomb(Ad, Bd, C, 1.0, 0.0)
    assert torch.equal(same, plain)
    two_step = pkg.ops.gemm_lincomb(Ad, Bd, C, 0.5, 2.0)
    pkg.ops.gemm_lincomb(Ad, Bd, C, 0.5, 2.0, out=C)
    pkg.ops.check_status(dev)
    assert torch.equal(C, two_step)
    with pytest.raises(ValueError):
        pkg.ops.gemm_lincomb(Ad, Bd, C[:, :128], 1.0, 1.0)


@pytest.mark.parametrize("M,N,K", [(512, 512, 512), (128, 128, 128), (200, 392, 256), (1, 8, 128), (129, 520, 1024), (1024, 2048, 4096)])
def test_fp8_128x128_two_ctas_per_sm_kernel(pkg, oracle, dev, M, N, K):
    """The 128 x 128-tile FP8 kernel (two CTAs per SM) against the oracle on full, ragged and tiny shapes, with the
    fused epilogues and a column shard; it must agree with the 128 x 256 kernel to the bit (same arithmetic order)."""
    A, B, sA, sB = pkg.synth.fp8_gemm_inputs(M, N, K, seed=M + N + K)
    Ad, Bd, sAd, sBd = A.to(dev), B.to(dev), sA.to(dev), sB.to(dev)
    pkg.capi.set_option("gemm.fp8_tile", 256)
    try:
        ref = pkg.ops.gemm_fp8_blockscaled(Ad, Bd, sAd, sBd)
        pkg.capi.set_option("gemm.fp8_tile", 128)
        got = pkg.ops.gemm_fp8_blockscaled(Ad, Bd, sAd, sBd)
        pkg.ops.check_status(dev)
        assert torch.equal(got, ref)
        if M * N * K <= 512 * 520 * 1024:
            want = oracle.gemm_fp8_blockscaled(u8(A), u8(B), sA.numpy(), sB.numpy())
            assert rel_fro(oracle.bf16_decode(u16(got)), oracle.bf16_decode(want)) <= TOL
        if N >= 512:
            bias = torch.randn(N).float().to(dev)
            C = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
            pkg.ops.gemm_fp8_blockscaled(Ad, Bd, sAd, sBd, out=C, n_range=(128, 384), bias=bias, act=1)
            pkg.capi.set_option("gemm.fp8_tile", 256)
            C2 = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
            pkg.ops.gemm_fp8_blockscaled(Ad, Bd, sAd, sBd, out=C2, n_range=(128, 384), bias=bias, act=1)
            pkg.ops.check_status(dev)
            assert torch.equal(C[:, 128:384], C2[:, 128:384]) and torch.isnan(C[:, :128]).all() and torch.isnan(C[:, 384:]).all()
    finally:
        pkg.capi.set_option("gemm.fp8_tile", 0)
