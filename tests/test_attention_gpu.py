"""GPU parity of the sm100 flash-attention kernels against the CPU host oracle,
through the C-ABI.  Tolerances: max-abs <= 2e-2 for bf16 attention, relative
Frobenius error <= 1e-2 for FP8 attention (the stated bars); LSE within 1e-3;
mask bits and skip predicates bit-exact."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def u8(t):
    return t.view(torch.uint8).cpu().numpy()


def u16(t):
    return t.view(torch.uint16).cpu().numpy()


def rel_fro(got, want):
    got, want = got.astype(np.float64), want.astype(np.float64)
    return float(np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30))


@pytest.mark.parametrize("B,Hq,Hkv,S,causal", [
    (1, 1, 1, 128, True), (1, 1, 1, 128, False), (1, 2, 2, 256, True), (2, 4, 2, 512, True),
    (1, 2, 1, 200, True), (1, 2, 1, 328, False), (1, 3, 1, 8, True), (1, 1, 1, 1032, True),
    (2, 4, 2, 16, False), (1, 2, 2, 16, True),      # at most 16 rows: the decode kernel writes O and LSE itself
])
def test_bf16_attention_matches_oracle(pkg, oracle, dev, B, Hq, Hkv, S, causal):
    Q, K, V, scale = pkg.synth.bf16_attention_inputs(B, Hq, S, 128, seed=0, Hkv=Hkv)
    O = torch.full(Q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    L = torch.full((B, Hq, S), float("nan"), dtype=torch.float32, device=dev)
    pkg.ops.attn_fwd_bf16(Q.to(dev), K.to(dev), V.to(dev), scale, causal, out=O, lse=L)
    pkg.ops.check_status(dev)
    Ow, Lw = oracle.attn_fwd_bf16(u16(Q), u16(K), u16(V), scale, causal)
    got = oracle.bf16_decode(u16(O))
    assert not np.isnan(got).any()
    assert np.abs(got - oracle.bf16_decode(Ow)).max() <= 2e-2
    assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3


def test_bf16_attention_golden_fixture(pkg, dev, golden):
    g = golden["attention_small"]
    Q, K, V = (torch.from_numpy(g[n]).view(torch.bfloat16).to(dev) for n in ("Q", "K", "V"))
    for name, causal in (("causal", True), ("full", False)):
        O, L = pkg.ops.attn_fwd_bf16(Q, K, V, float(g["scale"]), causal)
        pkg.ops.check_status(dev)
        assert np.abs(O.float().cpu().numpy() - g["O_" + name]).max() <= 2e-2
        assert np.abs(L.cpu().numpy() - g["LSE_" + name]).max() <= 1e-3


def test_bf16_attention_large_logits_trigger_rescale(pkg, oracle, dev):
    """Scores that keep growing along the sequence force the in-place accumulator rescale."""
    B, H, S, D = 1, 2, 1024, 128
    g = torch.Generator().manual_seed(5)
    Q = torch.randn(B, H, S, D, generator=g)
    K = torch.randn(B, H, S, D, generator=g)
    K = K + (torch.arange(S).view(1, 1, S, 1) / S) * 4.0 * Q.mean(2, keepdim=True).sign()
    Q, K = (Q * 3).bfloat16(), K.bfloat16()
    V = torch.randn(B, H, S, D, generator=g).bfloat16()
    scale = 1.0
    O, L = pkg.ops.attn_fwd_bf16(Q.to(dev), K.to(dev), V.to(dev), scale, False)
    pkg.ops.check_status(dev)
    Ow, Lw = oracle.attn_fwd_bf16(u16(Q), u16(K), u16(V), scale, False)
    want = oracle.bf16_decode(Ow)
    # outputs reach |O| ~ 4 here (near one-hot softmax): allow one bf16 ulp of the value on top of the bar
    assert np.all(np.abs(O.float().cpu().numpy() - want) <= 2e-2 + np.abs(want) * 2.0 ** -7)
    assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3 * max(1.0, float(np.abs(Lw).max()) / 10)


def test_bf16_attention_head_shards_tile_the_output(pkg, dev):
    B, Hq, Hkv, S = 2, 8, 4, 384
    Q, K, V, scale = pkg.synth.bf16_attention_inputs(B, Hq, S, 128, seed=2, Hkv=Hkv)
    Q, K, V = Q.to(dev), K.to(dev), V.to(dev)
    full, lfull = pkg.ops.attn_fwd_bf16(Q, K, V, scale, True)
    for world in (2, 3, 8):
        O = torch.full(Q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
        L = torch.full((B, Hq, S), float("nan"), dtype=torch.float32, device=dev)
        for r in range(world):
            b, e = pkg.shard.attention_head_range(B, Hq, Hkv, world, r)
            pkg.ops.attn_fwd_bf16(Q, K, V, scale, True, out=O, lse=L, bh_range=(b, e))
        pkg.ops.check_status(dev)
        assert torch.equal(O.view(torch.int16), full.view(torch.int16)) and torch.equal(L, lfull)


@pytest.mark.parametrize("B,Hq,Hkv,S,causal", [
    (1, 1, 1, 128, True), (1, 1, 1, 256, False), (2, 8, 2, 512, True), (1, 2, 1, 208, True), (1, 4, 1, 1040, True),
    (1, 2, 1, 16, True), (2, 4, 4, 16, False),      # 16 rows: decode kernel, one KV share
])
def test_fp8_attention_matches_oracle(pkg, oracle, dev, B, Hq, Hkv, S, causal):
    Q, K, V, dq, dk, dv, scale = pkg.synth.fp8_attention_inputs(B, Hq, Hkv, S, 128, seed=0)
    O, L = pkg.ops.attn_fwd_fp8(*(t.to(dev) for t in (Q, K, V, dq, dk, dv)), scale, causal)
    pkg.ops.check_status(dev)
    Ow, Lw = oracle.attn_fwd_fp8(u8(Q), u8(K), u8(V), dq.numpy(), dk.numpy(), dv.numpy(), scale, causal, tile_n=128)
    assert rel_fro(O.float().cpu().numpy(), oracle.bf16_decode(Ow)) <= 1e-2
    assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3


def test_fp8_attention_golden_fixture(pkg, dev, golden):
    g = golden["attention_small"]
    Q, K, V = (torch.from_numpy(g[n]).view(torch.float8_e4m3fn).to(dev) for n in ("Q8", "K8", "V8"))
    dq, dk, dv = (torch.from_numpy(g[n]).to(dev) for n in ("dq", "dk", "dv"))
    O, L = pkg.ops.attn_fwd_fp8(Q, K, V, dq, dk, dv, float(g["scale"]), True)
    pkg.ops.check_status(dev)
    assert rel_fro(O.float().cpu().numpy(), g["O8_causal"]) <= 4e-2     # fixture keeps P unquantised
    assert np.abs(L.cpu().numpy() - g["LSE8_causal"]).max() <= 1e-3


def test_bf16_attention_full_size_sampled_heads(pkg, oracle, dev):
    """cfg3 (B=8,H=32,S=4096,D=128, causal): 3 heads x sampled query rows against the oracle."""
    B, H, S, D = 8, 32, 4096, 128
    Q, K, V, scale = pkg.synth.bf16_attention_inputs(B, H, S, D, seed=0, device=dev)
    O, L = pkg.ops.attn_fwd_bf16(Q, K, V, scale, True)
    pkg.ops.check_status(dev)
    assert not torch.isnan(O).any()
    for bh in (0, 77, B * H - 1):
        b, h = divmod(bh, H)
        q, k, v = (u16(t[b:b + 1, h:h + 1]) for t in (Q, K, V))
        for q0, q1 in ((0, 64), (2040, 2056), (S - 64, S)):
            Ow, Lw = oracle.attn_fwd_bf16(q, k, v, scale, True, q_range=(q0, q1))
            got = O[b, h, q0:q1].float().cpu().numpy()
            assert np.abs(got - oracle.bf16_decode(Ow)[0, 0, q0:q1]).max() <= 2e-2
            assert np.abs(L[b, h, q0:q1].cpu().numpy() - Lw[0, 0, q0:q1]).max() <= 1e-3


def test_fp8_attention_full_size_sampled_heads(pkg, oracle, dev):
    """cfg4 (B=4, 64 q heads / 8 kv heads, S=8192, causal): sampled heads and rows against the oracle."""
    B, Hq, Hkv, S, D = 4, 64, 8, 8192, 128
    Q, K, V, dq, dk, dv, scale = pkg.synth.fp8_attention_inputs(B, Hq, Hkv, S, D, seed=0, device=dev)
    O, L = pkg.ops.attn_fwd_fp8(Q, K, V, dq, dk, dv, scale, True)
    pkg.ops.check_status(dev)
    for bh in (0, 100, B * Hq - 1):
        b, h = divmod(bh, Hq)
        hk = h // (Hq // Hkv)
        q, k, v = u8(Q[b:b + 1, h:h + 1]), u8(K[b:b + 1, hk:hk + 1]), u8(V[b:b + 1, hk:hk + 1])
        a, bb, c = dq[bh:bh + 1].cpu().numpy(), dk[b * Hkv + hk:b * Hkv + hk + 1].cpu().numpy(), dv[b * Hkv + hk:b * Hkv + hk + 1].cpu().numpy()
        for q0, q1 in ((0, 32), (4090, 4106), (S - 32, S)):
            Ow, Lw = oracle.attn_fwd_fp8(q, k, v, a, bb, c, scale, True, q_range=(q0, q1))
            got = O[b, h, q0:q1].float().cpu().numpy()
            assert rel_fro(got, oracle.bf16_decode(Ow)[0, 0, q0:q1]) <= 1e-2
            assert np.abs(L[b, h, q0:q1].cpu().numpy() - Lw[0, 0, q0:q1]).max() <= 1e-3


def _exact_fp8_attention_rows(oracle, q, k, v, dq, dk, dv, scale, q0, q1):
    """float64 causal attention of one head on the dequantised operands, P NOT quantised: rows [q0, q1)."""
    qf = oracle.e4m3_decode(q[0, 0, q0:q1]).astype(np.float64)
    kf = oracle.e4m3_decode(k[0, 0]).astype(np.float64)
    vf = oracle.e4m3_decode(v[0, 0]).astype(np.float64)
    s = qf @ kf.T * (float(scale) * float(dq) * float(dk))
    s = np.where(np.arange(kf.shape[0])[None, :] <= np.arange(q0, q1)[:, None], s, -np.inf)
    p = np.exp(s - s.max(-1, keepdims=True))
    return (p @ vf) / p.sum(-1, keepdims=True) * float(dv)


def test_fp8_attention_against_the_standard_online_softmax(pkg, oracle, dev):
    """The E4M3 recipe rounds P to E4M3 before P.V, so WHERE P is taken (against which reference maximum) decides which
    values are rounded.  By default the kernel advances its reference lazily (a new maximum must exceed it by 2^8), and
    the parity oracle used elsewhere follows that rule.  This test holds the kernel against an oracle that does not know
    the kernel - the standard online softmax (per-tile running maximum, P <= 1) - and against exact float64 attention
    with unquantised P, on cfg4's shape (sampled heads and rows):
      * option attn.rescale = 1 makes the kernel take the standard rule: it must then match the standard oracle within
        the 1e-2 bar (same rounding points, nothing shared with the kernel's schedule);
      * default (lazy): matches the lazy-rule oracle within 1e-2; against the TRUTH both recipes show the E4M3 rounding
        noise of P, a few percent on these peaked softmax rows.  Under the standard rule the largest weight of a tile is
        exactly 1 and therefore exact in E4M3; under the lazy rule it is an arbitrary value in [1, 2^8] and is rounded, so
        the lazy recipe is the noisier one (measured pooled error 0.021 against 0.0125): bounded here at twice the
        standard recipe's."""
    B, Hq, Hkv, S, D = 4, 64, 8, 8192, 128
    Q, K, V, dq, dk, dv, scale = pkg.synth.fp8_attention_inputs(B, Hq, Hkv, S, D, seed=0, device=dev)
    outs = {}
    try:
        for mode, opt in (("lazy", 0), ("standard", 1)):
            pkg.capi.set_option("attn.rescale", opt)
            outs[mode], _ = pkg.ops.attn_fwd_fp8(Q, K, V, dq, dk, dv, scale, True)
            pkg.ops.check_status(dev)
    finally:
        pkg.capi.set_option("attn.rescale", 0)
    worst = {"lazy_kernel_vs_lazy_oracle": 0.0, "std_kernel_vs_std_oracle": 0.0, "lazy_kernel_vs_std_oracle": 0.0}
    sq = {"lazy_kernel": 0.0, "std_kernel": 0.0, "std_oracle": 0.0, "exact": 0.0}      # squared error against exact attention, pooled
    for bh in (3, 130, B * Hq - 2):
        b, h = divmod(bh, Hq)
        hk = h // (Hq // Hkv)
        kv = b * Hkv + hk
        q, k, v = u8(Q[b:b + 1, h:h + 1]), u8(K[b:b + 1, hk:hk + 1]), u8(V[b:b + 1, hk:hk + 1])
        a, bb, c = dq[bh:bh + 1].cpu().numpy(), dk[kv:kv + 1].cpu().numpy(), dv[kv:kv + 1].cpu().numpy()
        for q0, q1 in ((200, 232), (5000, 5032), (S - 32, S)):
            got_lazy = outs["lazy"][b, h, q0:q1].float().cpu().numpy()
            got_std = outs["standard"][b, h, q0:q1].float().cpu().numpy()
            std = oracle.bf16_decode(oracle.attn_fwd_fp8(q, k, v, a, bb, c, scale, True, q_range=(q0, q1), rescale_threshold=0.0)[0])[0, 0, q0:q1]
            lazy = oracle.bf16_decode(oracle.attn_fwd_fp8(q, k, v, a, bb, c, scale, True, q_range=(q0, q1))[0])[0, 0, q0:q1]
            exact = _exact_fp8_attention_rows(oracle, q, k, v, a[0], bb[0], c[0], scale, q0, q1)
            worst["lazy_kernel_vs_lazy_oracle"] = max(worst["lazy_kernel_vs_lazy_oracle"], rel_fro(got_lazy, lazy))
            worst["std_kernel_vs_std_oracle"] = max(worst["std_kernel_vs_std_oracle"], rel_fro(got_std, std))
            worst["lazy_kernel_vs_std_oracle"] = max(worst["lazy_kernel_vs_std_oracle"], rel_fro(got_lazy, std))
            sq["lazy_kernel"] += float(((got_lazy - exact) ** 2).sum())
            sq["std_kernel"] += float(((got_std - exact) ** 2).sum())
            sq["std_oracle"] += float(((std - exact) ** 2).sum())
            sq["exact"] += float((exact ** 2).sum())
    pooled = {k: (sq[k] / sq["exact"]) ** 0.5 for k in ("lazy_kernel", "std_kernel", "std_oracle")}
    print("fp8 attention cfg4 sampled rows: worst rel. Frobenius error", {k: round(v, 5) for k, v in worst.items()},
          "; pooled error against exact attention", {k: round(v, 5) for k, v in pooled.items()})
    assert worst["std_kernel_vs_std_oracle"] <= 1e-2          # the independent check
    assert worst["lazy_kernel_vs_lazy_oracle"] <= 1e-2
    assert pooled["std_kernel"] <= 1.1 * pooled["std_oracle"] + 1e-3
    assert pooled["lazy_kernel"] <= 2.0 * pooled["std_oracle"] + 1e-3


def test_causal_mask_tile_bits_match_oracle(pkg, oracle, dev):
    for q_base, k_base, tm, tn in ((0, 0, 128, 128), (128, 0, 128, 128), (0, 128, 128, 128), (256, 384, 128, 128),
                                   (64, 96, 16, 48), (5, 3, 7, 9), (4096 - 128, 4096 - 128, 128, 128)):
        mask, skip = pkg.ops.causal_mask_tile(q_base, k_base, tm, tn, dev)
        want_mask, want_skip = oracle.causal_mask_tile(q_base, k_base, tm, tn)
        assert np.array_equal(mask.cpu().numpy().view(np.uint64), want_mask)
        assert int(skip.item()) == want_skip


@pytest.mark.parametrize("mode", [1, 2, 3, 4])
def test_attention_exp2_variants(pkg, oracle, dev, mode):
    """Every way of evaluating the exponentials (SFU only, SFU + polynomial for 2, 4 or 3 of every 8 pairs) meets the bar."""
    pkg.capi.set_option("attn.exp_mode", mode)
    try:
        Q, K, V, scale = pkg.synth.bf16_attention_inputs(1, 4, 640, 128, seed=4, Hkv=2)
        O, L = pkg.ops.attn_fwd_bf16(Q.to(dev), K.to(dev), V.to(dev), scale, True)
        pkg.ops.check_status(dev)
        Ow, Lw = oracle.attn_fwd_bf16(u16(Q), u16(K), u16(V), scale, True)
        assert np.abs(O.float().cpu().numpy() - oracle.bf16_decode(Ow)).max() <= 2e-2
        assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3
        Q, K, V, dq, dk, dv, scale = pkg.synth.fp8_attention_inputs(1, 4, 2, 640, 128, seed=4)
        O, L = pkg.ops.attn_fwd_fp8(*(t.to(dev) for t in (Q, K, V, dq, dk, dv)), scale, True)
        pkg.ops.check_status(dev)
        Ow, Lw = oracle.attn_fwd_fp8(u8(Q), u8(K), u8(V), dq.numpy(), dk.numpy(), dv.numpy(), scale, True)
        assert rel_fro(O.float().cpu().numpy(), oracle.bf16_decode(Ow)) <= 1e-2
        assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3
    finally:
        pkg.capi.set_option("attn.exp_mode", 0)


@pytest.mark.parametrize("p_operand,issuers", [(1, 1), (2, 1), (1, 2), (2, 2)])
@pytest.mark.parametrize("S,causal", [(128, True), (640, True), (1152, False), (2048, True)])
def test_fp8_attention_p_operand_routes(pkg, oracle, dev, p_operand, issuers, S, causal):
    """The E4M3 kernel with P handed to the P.V MMA in tensor memory (1) or through shared memory (2):
    both routes meet the bar on one-tile, ragged multi-tile, non-causal and longer causal cases."""
    pkg.capi.set_option("attn.p_operand", p_operand)
    pkg.capi.set_option("attn.issuers", issuers)
    try:
        Q, K, V, dq, dk, dv, scale = pkg.synth.fp8_attention_inputs(1, 4, 2, S, 128, seed=9)
        O, L = pkg.ops.attn_fwd_fp8(*(t.to(dev) for t in (Q, K, V, dq, dk, dv)), scale, causal)
        pkg.ops.check_status(dev)
        Ow, Lw = oracle.attn_fwd_fp8(u8(Q), u8(K), u8(V), dq.numpy(), dk.numpy(), dv.numpy(), scale, causal)
        assert rel_fro(O.float().cpu().numpy(), oracle.bf16_decode(Ow)) <= 1e-2
        assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3
    finally:
        pkg.capi.set_option("attn.p_operand", 0)
        pkg.capi.set_option("attn.issuers", 0)


@pytest.mark.parametrize("kv_tile,issuers", [(64, 1), (64, 2), (128, 1), (128, 2)])
@pytest.mark.parametrize("S,causal,Hq,Hkv", [(64, True, 2, 2), (128, True, 2, 1), (200, True, 4, 2), (640, True, 4, 2),
                                             (1152, False, 2, 2), (2048, True, 2, 1), (328, False, 2, 2)])
def test_bf16_attention_kv_tile_sizes(pkg, oracle, dev, kv_tile, issuers, S, causal, Hq, Hkv):
    """bf16 kernel with 64-key tiles (two S buffers per Q tile) and with 128-key tiles, one MMA-issuing thread or
    one per Q tile: one tile, ragged lengths, a second Q tile that does not exist (S <= 128), GQA, causal and
    non-causal."""
    pkg.capi.set_option("attn.kv_tile", kv_tile)
    pkg.capi.set_option("attn.issuers", issuers)
    try:
        Q, K, V, scale = pkg.synth.bf16_attention_inputs(1, Hq, S, 128, seed=17, Hkv=Hkv)
        O, L = pkg.ops.attn_fwd_bf16(Q.to(dev), K.to(dev), V.to(dev), scale, causal)
        pkg.ops.check_status(dev)
        Ow, Lw = oracle.attn_fwd_bf16(u16(Q), u16(K), u16(V), scale, causal)
        assert np.abs(O.float().cpu().numpy() - oracle.bf16_decode(Ow)).max() <= 2e-2
        assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3
    finally:
        pkg.capi.set_option("attn.kv_tile", 0)
        pkg.capi.set_option("attn.issuers", 0)
