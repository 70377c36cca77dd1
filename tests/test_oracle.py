"""CPU tests of the host oracle against the committed golden fixtures (no GPU)."""
import numpy as np


def rel_fro(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / np.linalg.norm(b))


def test_e4m3_decode_table(oracle, golden):
    want = golden["codecs"]["e4m3_decode"]
    got = oracle.e4m3_decode(np.arange(256, dtype=np.uint8))
    assert np.array_equal(np.isnan(got), np.isnan(want))
    assert np.array_equal(got[~np.isnan(want)], want[~np.isnan(want)])


def test_e4m3_encode_saturating(oracle, golden):
    g = golden["codecs"]
    assert np.array_equal(oracle.e4m3_encode_sat(g["enc_in"]), g["enc_out"])
    # saturation beyond the fixture's clipped range: +-448, NaN kept
    big = np.array([1e9, -1e9, 449.0, np.inf, -np.inf], dtype=np.float32)
    assert oracle.e4m3_encode_sat(big).tolist() == [0x7E, 0xFE, 0x7E, 0x7E, 0xFE]
    assert oracle.e4m3_encode_sat(np.array([np.nan], np.float32))[0] & 0x7F == 0x7F


def test_bf16_round_to_nearest_even(oracle, golden):
    g = golden["codecs"]
    assert np.array_equal(oracle.bf16_encode(g["bf16_in"]), g["bf16_out"])
    assert np.array_equal(oracle.bf16_decode(g["bf16_out"]), (g["bf16_out"].astype(np.uint32) << 16).view(np.float32))


def test_gemm_fp8_blockscaled_golden(oracle, golden):
    g = golden["gemm_small"]
    C = oracle.bf16_decode(oracle.gemm_fp8_blockscaled(g["A"], g["B"], g["sA"], g["sB"]))
    assert rel_fro(C, g["C_f64"]) < 3e-3          # bf16 output rounding only
    # bf16(fp64 answer) differs from the oracle by at most one bf16 ulp anywhere
    want = oracle.bf16_decode(oracle.bf16_encode(g["C_f64"].astype(np.float32)))
    ulp = np.abs(want) * 2.0 ** -7 + 1e-6
    assert np.all(np.abs(C - want) <= ulp)


def test_gemm_fp8_subrange_matches_full(oracle, golden):
    g = golden["gemm_small"]
    full = oracle.gemm_fp8_blockscaled(g["A"], g["B"], g["sA"], g["sB"])
    part = oracle.gemm_fp8_blockscaled(g["A"], g["B"], g["sA"], g["sB"], m_range=(8, 40), n_range=(128, 160))
    assert np.array_equal(part[8:40, 128:160], full[8:40, 128:160])
    assert not part[:8].any() and not part[:, :128].any()


def test_gemm_bf16_golden(oracle, golden):
    g = golden["gemm_small"]
    Y = oracle.bf16_decode(oracle.gemm_bf16(g["X"], g["W"]))
    assert rel_fro(Y, g["Y_f64"]) < 3e-3


def test_attention_bf16_golden(oracle, golden):
    g = golden["attention_small"]
    for name, causal in (("causal", True), ("full", False)):
        O, LSE = oracle.attn_fwd_bf16(g["Q"], g["K"], g["V"], float(g["scale"]), causal)
        assert np.abs(oracle.bf16_decode(O) - g["O_" + name]).max() < 2e-2
        assert np.abs(LSE - g["LSE_" + name]).max() < 1e-4


def test_attention_tile_recipe_agrees_with_direct_softmax(oracle, golden):
    """The reference's per-tile (m,l) combine / rescale / weight-scale math, taken per row,
    gives the same result as the direct softmax."""
    g = golden["attention_small"]
    O, LSE = oracle.attn_fwd_bf16(g["Q"], g["K"], g["V"], float(g["scale"]), True)
    for tm, tn in ((128, 128), (64, 32), (16, 16)):
        O2, LSE2 = oracle.attn_fwd_bf16_tile_recipe(g["Q"], g["K"], g["V"], float(g["scale"]), True, tm, tn)
        assert np.abs(LSE2 - LSE).max() < 1e-5
        assert np.abs(oracle.bf16_decode(O2) - oracle.bf16_decode(O)).max() < 2e-2
        assert np.abs(oracle.bf16_decode(O2) - g["O_causal"]).max() < 2e-2


def test_attention_fp8_golden(oracle, golden):
    g = golden["attention_small"]
    O, LSE = oracle.attn_fwd_fp8(g["Q8"], g["K8"], g["V8"], g["dq"], g["dk"], g["dv"], float(g["scale"]), True)
    assert rel_fro(oracle.bf16_decode(O), g["O8_causal"]) < 4e-2   # P is quantised to 3 mantissa bits
    assert np.abs(LSE - g["LSE8_causal"]).max() < 1e-3
    # tile size only changes where P is rounded, not the answer
    O2, LSE2 = oracle.attn_fwd_fp8(g["Q8"], g["K8"], g["V8"], g["dq"], g["dk"], g["dv"], float(g["scale"]), True, tile_n=32)
    assert rel_fro(oracle.bf16_decode(O2), oracle.bf16_decode(O).astype(np.float64)) < 2e-2
    assert np.abs(LSE2 - LSE).max() < 1e-4


def test_attention_subrange(oracle, golden):
    g = golden["attention_small"]
    O, LSE = oracle.attn_fwd_bf16(g["Q"], g["K"], g["V"], float(g["scale"]), True)
    O2, LSE2 = oracle.attn_fwd_bf16(g["Q"], g["K"], g["V"], float(g["scale"]), True, bh_range=(1, 3), q_range=(100, 160))
    assert np.array_equal(O2[0, 1:3, 100:], O[0, 1:3, 100:]) and np.array_equal(LSE2[0, 1:3, 100:], LSE[0, 1:3, 100:])
    assert not O2[0, 0].any() and not O2[0, 1, :100].any()


def test_causal_mask_bits_and_skip(oracle):
    for q_base, k_base, tm, tn in ((0, 0, 128, 128), (128, 0, 128, 128), (0, 128, 128, 128), (64, 96, 16, 48), (5, 3, 7, 9)):
        mask, skip = oracle.causal_mask_tile(q_base, k_base, tm, tn)
        r, c = np.divmod(np.arange(tm * tn), tn)
        want = (k_base + c) <= (q_base + r)
        bits = np.unpackbits(mask.view(np.uint8), bitorder="little")[: tm * tn].astype(bool)
        assert np.array_equal(bits, want)
        assert skip == int(k_base > q_base + tm - 1)
        assert (skip == 1) == (not want.any())


def test_shard_ranges_cover_and_align(oracle, pkg):
    for units, gran, world in ((8192, 256, 8), (8192, 256, 3), (14336, 256, 8), (4096, 256, 8), (300, 256, 4), (256, 8, 8), (32, 1, 8)):
        prev = 0
        for r in range(world):
            b, e = oracle.shard_range(units, gran, world, r)
            assert (b, e) == pkg.shard.shard_range(units, gran, world, r)      # bit-exact index work
            assert b == prev and (b % gran == 0 or b == units) and (e % gran == 0 or e == units)
            prev = e
        assert prev == units


def test_fused_epilogue_oracles(oracle, golden):
    g = golden["gemm_small"]
    rng = np.random.default_rng(3)
    bias = rng.standard_normal(g["W"].shape[0]).astype(np.float32)
    y = g["Y_f64"] + bias
    want = {0: y, 1: y / (1.0 + np.exp(-y))}
    for act in (0, 1):
        got = oracle.bf16_decode(oracle.gemm_bf16_bias_act(g["X"], g["W"], bias, act))
        assert rel_fro(got, want[act]) < 3e-3
    bias = (rng.standard_normal(g["B"].shape[0]) * 50).astype(np.float32)
    c = g["C_f64"] + bias
    want = {0: c, 1: c / (1.0 + np.exp(-c))}
    for act in (0, 1):
        got = oracle.bf16_decode(oracle.gemm_fp8_blockscaled_bias_act(g["A"], g["B"], g["sA"], g["sB"], bias, act))
        assert rel_fro(got, want[act]) < 3e-3


def test_quantize_oracle_against_torch(oracle):
    import torch

    g = torch.Generator().manual_seed(11)
    X = (torch.randn(33, 512, generator=g) * 3).bfloat16()
    Q, S = oracle.quantize_rows_e4m3(X.view(torch.uint16).numpy())
    xb = X.float().view(33, 4, 128)
    amax = xb.abs().amax(-1)
    assert np.array_equal(S, (amax / 448.0).numpy())
    want = (xb * (1.0 / (amax / 448.0)).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8)
    assert np.array_equal(Q, want.reshape(33, 512).numpy())


def test_swiglu_oracle(oracle, golden):
    """Gate / up projection: bf16(SiLU(X.Wg^T) * (X.Wu^T)) against float64 on the golden GEMM operands."""
    g = golden["gemm_small"]
    rng = np.random.default_rng(5)
    Wu = oracle.bf16_encode((rng.standard_normal(g["W"].shape) * 0.05).astype(np.float32))
    x = oracle.bf16_decode(g["X"]).astype(np.float64)
    gate = g["Y_f64"]
    up = x @ oracle.bf16_decode(Wu).astype(np.float64).T
    want = gate / (1.0 + np.exp(-gate)) * up
    got = oracle.bf16_decode(oracle.gemm_bf16_swiglu(g["X"], g["W"], Wu))
    assert rel_fro(got, want) < 3e-3
    # gate == 0 gives exactly zero whatever the up product is
    zero = np.zeros_like(g["W"])
    assert not oracle.bf16_decode(oracle.gemm_bf16_swiglu(g["X"], zero, Wu)).any()      # +0 or -0


def test_fp8_swiglu_oracle(oracle):
    """Gate / up projection on E4M3 block-scaled operands against float64 on the dequantised golden operands."""
    rng = np.random.default_rng(9)
    M, N, K = 48, 160, 256
    X = rng.integers(0, 256, (M, K), dtype=np.uint8)
    Wg = rng.integers(0, 256, (N, K), dtype=np.uint8)
    Wu = rng.integers(0, 256, (N, K), dtype=np.uint8)
    for a in (X, Wg, Wu):
        a[(a & 0x7f) == 0x7f] = 0x38          # no NaN encodings
        a[(a & 0x78) >= 0x50] &= 0xb7         # keep magnitudes moderate
    sX = (rng.random((M, K // 128)) + 0.5).astype(np.float32) / 64
    sWg = (rng.random(((N + 127) // 128, K // 128)) + 0.5).astype(np.float32) / 8
    sWu = (rng.random(((N + 127) // 128, K // 128)) + 0.5).astype(np.float32) / 8

    def deq(q, s, rows_per_scale):
        v = oracle.e4m3_decode(q).astype(np.float64).reshape(q.shape[0], K // 128, 128)
        return (v * np.repeat(s.astype(np.float64), rows_per_scale, axis=0)[:q.shape[0], :, None]).reshape(q.shape[0], K)

    x, wg, wu = deq(X, sX, 1), deq(Wg, sWg, 128), deq(Wu, sWu, 128)
    gate, up = x @ wg.T, x @ wu.T
    want = gate / (1.0 + np.exp(-gate)) * up
    got = oracle.bf16_decode(oracle.gemm_fp8_blockscaled_swiglu(X, Wg, Wu, sX, sWg, sWu))
    assert rel_fro(got, want) < 3e-3


def test_attention_separate_lengths_oracle(oracle, golden):
    """Fewer queries than keys: without the mask every row equals the same row of a square problem whose extra
    queries are ignored; under the causal mask the Sq queries are the last Sq positions of the square problem."""
    g = golden["attention_small"]

    def same(a, b):      # the two functions sum in different orders: equal up to one bf16 ulp
        return np.allclose(oracle.bf16_decode(a), oracle.bf16_decode(b), rtol=2.0 ** -7, atol=1e-6)

    Q, K, V, scale = g["Q"], g["K"], g["V"], float(g["scale"])
    S = Q.shape[2]
    Sq = 40
    O_full, L_full = oracle.attn_fwd_bf16(Q, K, V, scale, True)
    O, L = oracle.attn_fwd_bf16_qkv(Q[:, :, S - Sq:], K, V, scale, True)
    assert same(O, O_full[:, :, S - Sq:]) and np.allclose(L, L_full[:, :, S - Sq:], atol=1e-6)
    O_full, L_full = oracle.attn_fwd_bf16(Q, K, V, scale, False)
    O, L = oracle.attn_fwd_bf16_qkv(Q[:, :, :Sq], K, V, scale, False)
    assert same(O, O_full[:, :, :Sq]) and np.allclose(L, L_full[:, :, :Sq], atol=1e-6)
    # equal lengths: the two oracle functions agree
    O, L = oracle.attn_fwd_bf16_qkv(Q, K, V, scale, True)
    O_full, L_full = oracle.attn_fwd_bf16(Q, K, V, scale, True)
    assert same(O, O_full) and np.allclose(L, L_full, atol=1e-6)


def test_lincomb_oracles(oracle, golden):
    """Linear-combination epilogue against float64; alpha = 1, beta = 0 reproduces the plain GEMM bit for bit."""
    g = golden["gemm_small"]
    rng = np.random.default_rng(8)
    Cin = oracle.bf16_encode(rng.standard_normal(g["Y_f64"].shape).astype(np.float32))
    want = 0.75 * g["Y_f64"] - 1.5 * oracle.bf16_decode(Cin).astype(np.float64)
    assert rel_fro(oracle.bf16_decode(oracle.gemm_bf16_lincomb(g["X"], g["W"], Cin, 0.75, -1.5)), want) < 3e-3
    assert np.array_equal(oracle.gemm_bf16_lincomb(g["X"], g["W"], Cin, 1.0, 0.0), oracle.gemm_bf16(g["X"], g["W"]))
    Cin = oracle.bf16_encode((rng.standard_normal(g["C_f64"].shape) * 100).astype(np.float32))
    want = 2.0 * g["C_f64"] + 0.5 * oracle.bf16_decode(Cin).astype(np.float64)
    got = oracle.gemm_fp8_blockscaled_lincomb(g["A"], g["B"], g["sA"], g["sB"], Cin, 2.0, 0.5)
    assert rel_fro(oracle.bf16_decode(got), want) < 3e-3


def test_rmsnorm_quantize_oracle_against_float64(oracle):
    rng = np.random.default_rng(21)
    M, K = 12, 1024
    X = oracle.bf16_encode((rng.standard_normal((M, K)) * 2.5).astype(np.float32))
    W = oracle.bf16_encode((1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32))
    Q, S = oracle.rmsnorm_quantize_rows_e4m3(X, W, 1e-5)
    x = oracle.bf16_decode(X).astype(np.float64)
    y = x / np.sqrt((x * x).mean(-1, keepdims=True) + 1e-5) * oracle.bf16_decode(W).astype(np.float64)
    deq = (oracle.e4m3_decode(Q).reshape(M, K // 128, 128) * S[:, :, None]).reshape(M, K)
    assert rel_fro(deq, y) < 4e-2
    # the block scale is max|y| / 448 of the normalised block
    assert np.allclose(S, np.abs(y).reshape(M, K // 128, 128).max(-1) / 448.0, rtol=1e-5)


def test_fused_operator_goldens(oracle, golden):
    """Oracle against the float64 fixtures of the widened operators (tests/golden/fused_small.npz)."""
    g = golden["fused_small"]
    assert rel_fro(oracle.bf16_decode(oracle.gemm_bf16_swiglu(g["X"], g["Wg"], g["Wu"])), g["H_f64"]) < 3e-3
    got = oracle.gemm_bf16_lincomb(g["X"], g["Wg"], g["Cin"], float(g["alpha"]), float(g["beta"]))
    assert rel_fro(oracle.bf16_decode(got), g["D_f64"]) < 3e-3
    Q, S = oracle.rmsnorm_quantize_rows_e4m3(g["Xn"], g["w"], float(g["eps"]))
    M, K = g["Xn"].shape
    deq = (oracle.e4m3_decode(Q).reshape(M, K // 128, 128) * S[:, :, None]).reshape(M, K)
    assert rel_fro(deq, g["Yn_f64"]) < 4e-2
    assert np.allclose(S, np.abs(g["Yn_f64"]).reshape(M, K // 128, 128).max(-1) / 448.0, rtol=1e-5)
    for name, causal in (("causal", True), ("full", False)):
        O, L = oracle.attn_fwd_bf16_qkv(g["Q"], g["K"], g["V"], float(g["scale"]), causal)
        assert np.abs(oracle.bf16_decode(O) - g["O_" + name]).max() < 1e-2
        assert np.abs(L - g["LSE_" + name]).max() < 1e-4


def test_fp8_attention_oracle_modes_agree_with_the_float64_fixture(oracle, golden):
    """The two P-rounding points of the E4M3 attention oracle (lazy reference maximum, as the sm100 kernel takes it; standard
    per-tile running maximum) are two roundings of the same softmax: both sit at the E4M3 rounding noise of P from the float64
    fixture (P unquantised there), and no further from each other than twice that."""
    g = golden["attention_small"]
    args = (g["Q8"], g["K8"], g["V8"], g["dq"], g["dk"], g["dv"], float(g["scale"]), True)
    lazy = oracle.bf16_decode(oracle.attn_fwd_fp8(*args)[0])
    std, lse_std = oracle.attn_fwd_fp8(*args, rescale_threshold=0.0)
    std = oracle.bf16_decode(std)
    want = g["O8_causal"]
    rel = lambda a, b: float(np.linalg.norm(a - b) / np.linalg.norm(b))
    e_lazy, e_std, e_between = rel(lazy, want), rel(std, want), rel(lazy, std)
    assert e_lazy <= 4e-2 and e_std <= 4e-2
    assert e_between <= 2.0 * max(e_lazy, e_std)
    assert np.abs(lse_std - g["LSE8_causal"]).max() <= 1e-3
