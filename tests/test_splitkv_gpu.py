"""GPU parity of split-KV attention (separate query / key lengths, KV shares combined through scratch memory)
against the CPU host oracle, through the C-ABI.  Tolerances as for the bf16 forward kernel: |O - oracle| <= 2e-2,
|LSE - oracle| <= 1e-3."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def u16(t):
    return t.view(torch.uint16).cpu().numpy()


def make(pkg, B, Hq, Hkv, Sq, Skv, seed):
    Q, _, _, scale = pkg.synth.bf16_attention_inputs(B, Hq, Sq, 128, seed=seed, Hkv=Hkv)
    _, K, V, _ = pkg.synth.bf16_attention_inputs(B, Hq, Skv, 128, seed=seed + 1, Hkv=Hkv)
    return Q, K, V, scale


@pytest.mark.parametrize("splits", [1, 2, 3, 8])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", [
    (2, 8, 2, 1, 1000, True),        # decode: one query per head, ragged key count
    (1, 4, 4, 16, 4096, True),       # speculative / chunked decode
    (1, 2, 1, 300, 304, True),       # more than one Q tile, nearly square
    (1, 2, 2, 256, 2048, False),     # no mask
    (1, 4, 2, 72, 72, True),         # fewer KV tiles than shares: empty shares
    (1, 16, 2, 5, 776, True),        # GQA group of 8 stacked into one 40-row Q tile
    (2, 8, 2, 64, 640, True),        # stacked group fills two Q tiles (4 heads x 64 queries)
    (1, 8, 2, 3, 504, False),        # stacked, no mask
    (1, 16, 2, 4, 1000, True),       # group of 8 heads x 4 queries = 32 rows: above the decode kernel's 16, forward kernel
    (1, 4, 4, 24, 520, True),        # 24 rows per head, no grouping
    (2, 8, 2, 6, 776, False),        # 4 heads x 6 queries = 24 rows, no mask
])
def test_splitkv_matches_oracle(pkg, oracle, dev, splits, B, Hq, Hkv, Sq, Skv, causal):
    Q, K, V, scale = make(pkg, B, Hq, Hkv, Sq, Skv, seed=5)
    O, L = pkg.ops.attn_fwd_bf16_splitkv(Q.to(dev), K.to(dev), V.to(dev), scale, causal, num_splits=splits)
    pkg.ops.check_status(dev)
    Ow, Lw = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, causal)
    assert np.abs(O.float().cpu().numpy() - oracle.bf16_decode(Ow)).max() <= 2e-2
    assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3


def test_splitkv_shares_agree_with_single_pass_and_scratch_is_callers(pkg, dev):
    """Property: any number of shares gives the single-pass result up to the rounding of the combine; the scratch
    buffer is the caller's (poisoned before the call, size from the query function)."""
    Q, K, V, scale = make(pkg, 1, 8, 2, 8, 8192, seed=9)
    Qd, Kd, Vd = Q.to(dev), K.to(dev), V.to(dev)
    O1, L1 = pkg.ops.attn_fwd_bf16_splitkv(Qd, Kd, Vd, scale, True, num_splits=1)
    for splits in (4, 16, 64):
        need = pkg.ops.attn_splitkv_scratch_bytes(8, 8, splits)
        assert need == splits * 8 * 8 * (128 * 4 + 8)
        scratch = torch.full((need,), 0xFF, dtype=torch.uint8, device=dev)        # NaN patterns
        O, L = pkg.ops.attn_fwd_bf16_splitkv(Qd, Kd, Vd, scale, True, num_splits=splits, scratch=scratch)
        pkg.ops.check_status(dev)
        assert (O.float() - O1.float()).abs().max().item() <= 4e-3
        assert (L - L1).abs().max().item() <= 1e-4


def test_splitkv_head_shard_and_argument_errors(pkg, oracle, dev):
    Q, K, V, scale = make(pkg, 1, 4, 2, 4, 512, seed=2)
    Qd, Kd, Vd = Q.to(dev), K.to(dev), V.to(dev)
    O = torch.full_like(Qd, float("nan"))
    pkg.ops.attn_fwd_bf16_splitkv(Qd, Kd, Vd, scale, True, num_splits=2, out=O, bh_range=(1, 3))
    pkg.ops.check_status(dev)
    Ow, _ = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, True)
    assert np.abs(O[:, 1:3].float().cpu().numpy() - oracle.bf16_decode(Ow)[:, 1:3]).max() <= 2e-2
    assert torch.isnan(O[:, 0]).all() and torch.isnan(O[:, 3]).all()
    with pytest.raises(pkg.capi.AxpError) as e:      # scratch too small
        pkg.ops.attn_fwd_bf16_splitkv(Qd, Kd, Vd, scale, True, num_splits=4, scratch=torch.empty(1024, dtype=torch.uint8, device=dev))
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG
    with pytest.raises(pkg.capi.AxpError) as e:      # causal with more queries than keys
        pkg.ops.attn_fwd_bf16_splitkv(Kd[:, :, :64].repeat_interleave(2, 1).contiguous(), Kd[:, :, :32].contiguous(),
                                      Vd[:, :, :32].contiguous(), scale, True)
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG


def u8(t):
    return t.view(torch.uint8).cpu().numpy()


@pytest.mark.parametrize("splits", [1, 2, 5])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", [
    (2, 8, 2, 1, 1008, True),        # decode on an E4M3 KV cache: one query per head, GQA group stacked, ragged key count
    (1, 4, 4, 16, 2048, True),       # speculative / chunked decode, no grouping
    (1, 2, 1, 304, 304, True),       # square, more than one Q tile
    (1, 2, 2, 256, 1024, False),     # no mask, queries = the first rows
    (1, 16, 2, 5, 784, True),        # group of 8 heads stacked into one 40-row Q tile, every row with its head's Q descale
    (1, 8, 2, 64, 640, False),       # stacked group fills two Q tiles
])
def test_fp8_splitkv_matches_oracle(pkg, oracle, dev, splits, B, Hq, Hkv, Sq, Skv, causal):
    """The oracle is the square E4M3 forward pass: under the causal mask the Sq queries are its last Sq positions,
    without the mask any Sq rows (the first ones here).  The KV shares quantise P against their own running maxima,
    hence the same tolerance as the single-pass kernel rather than bit equality."""
    Qs, K, V, dq, dk, dv, scale = pkg.synth.fp8_attention_inputs(B, Hq, Hkv, Skv, 128, seed=21)
    r0 = Skv - Sq if causal else 0
    Q = Qs[:, :, r0:r0 + Sq].contiguous()
    O, L = pkg.ops.attn_fwd_fp8_splitkv(*(t.to(dev) for t in (Q, K, V, dq, dk, dv)), scale, causal, num_splits=splits)
    pkg.ops.check_status(dev)
    Ow, Lw = oracle.attn_fwd_fp8(u8(Qs), u8(K), u8(V), dq.numpy(), dk.numpy(), dv.numpy(), scale, causal, tile_n=128, q_range=(r0, r0 + Sq))
    want = oracle.bf16_decode(Ow)[:, :, r0:r0 + Sq]
    got = O.float().cpu().numpy()
    assert np.abs(L.cpu().numpy() - Lw[:, :, r0:r0 + Sq]).max() <= 1e-3
    if splits == 1:
        # one share rounds P to E4M3 against the same running maxima as the oracle
        assert np.linalg.norm(got - want) <= 1e-2 * np.linalg.norm(want)
        return
    # Several shares round P against their own maxima, so single elements of P round differently than in the oracle.
    # The rounding error of P (2^-4 relative, 3 mantissa bits) passes into O undamped when V is random, for the
    # oracle and for every number of shares alike: O is therefore held against exact (float64) attention on the
    # dequantised operands, and must be as close to it as the oracle's own single-pass result is.
    g = Hq // Hkv
    q = oracle.e4m3_decode(u8(Q)).astype(np.float64) * dq.numpy().reshape(B, Hq, 1, 1)
    k = np.repeat(oracle.e4m3_decode(u8(K)).astype(np.float64) * dk.numpy().reshape(B, Hkv, 1, 1), g, axis=1)
    v = np.repeat(oracle.e4m3_decode(u8(V)).astype(np.float64) * dv.numpy().reshape(B, Hkv, 1, 1), g, axis=1)
    sc = np.einsum("bhqd,bhkd->bhqk", q, k) * scale
    if causal:
        sc = np.where(np.arange(Skv)[None, :] <= (np.arange(Sq)[:, None] + r0), sc, -np.inf)
    pr = np.exp(sc - sc.max(-1, keepdims=True))
    exact = np.einsum("bhqk,bhkd->bhqd", pr / pr.sum(-1, keepdims=True), v)
    err_kernel = np.linalg.norm(got - exact) / np.linalg.norm(exact)
    err_oracle = np.linalg.norm(want - exact) / np.linalg.norm(exact)
    assert err_kernel <= 5e-2 and err_kernel <= 2.0 * err_oracle + 5e-3, (err_kernel, err_oracle)     # both near 2^-4 / sqrt(3)
    assert np.linalg.norm(got - want) <= 6e-2 * np.linalg.norm(want)


def test_fp8_splitkv_equals_single_pass_entry_point_and_rejects_bad_arguments(pkg, dev):
    """One share and Sq = Skv is the plain E4M3 forward pass: bit-identical O and LSE.  Argument errors as for bf16."""
    Q, K, V, dq, dk, dv, scale = (t.to(dev) if torch.is_tensor(t) else t for t in pkg.synth.fp8_attention_inputs(1, 4, 2, 512, 128, seed=3))
    O1, L1 = pkg.ops.attn_fwd_fp8(Q, K, V, dq, dk, dv, scale, True)
    O2, L2 = pkg.ops.attn_fwd_fp8_splitkv(Q, K, V, dq, dk, dv, scale, True, num_splits=1)
    pkg.ops.check_status(dev)
    assert torch.equal(O1.view(torch.int16), O2.view(torch.int16)) and torch.equal(L1, L2)
    with pytest.raises(pkg.capi.AxpError) as e:      # key count not a multiple of 16
        pkg.ops.attn_fwd_fp8_splitkv(Q[:, :, :8].contiguous(), K[:, :, :504].contiguous(), V[:, :, :504].contiguous(), dq, dk, dv, scale, True, num_splits=2)
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG
    with pytest.raises(pkg.capi.AxpError):           # scratch too small
        pkg.ops.attn_fwd_fp8_splitkv(Q, K, V, dq, dk, dv, scale, True, num_splits=4, scratch=torch.empty(256, dtype=torch.uint8, device=dev))


@pytest.mark.parametrize("Sq,Hq,Hkv,causal", [(1, 8, 2, True), (4, 4, 1, True), (16, 2, 2, True), (3, 4, 4, False)])
def test_decode_kernel_rescales_and_agrees_with_forward_kernel(pkg, oracle, dev, Sq, Hq, Hkv, causal):
    """Calls with at most 16 query rows per KV head and several KV shares take the decode kernel (keys on the tensor-memory
    lanes).  Keys grow along the sequence here, so the running reference of every row is raised several times and the
    accumulator rescaled; the result is held against the oracle and against the forward kernel (option attn.decode_kernel)."""
    B, Skv = 2, 1160
    Q, K, V, scale = make(pkg, B, Hq, Hkv, Sq, Skv, seed=11)
    ramp = (1.0 + 9.0 * torch.arange(Skv, dtype=torch.float32) / Skv).view(1, 1, Skv, 1)
    K = (K.float() * ramp).bfloat16()
    Ow, Lw = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, causal)
    res = {}
    try:
        for opt in (1, 2):
            pkg.capi.set_option("attn.decode_kernel", opt)
            O, L = pkg.ops.attn_fwd_bf16_splitkv(Q.to(dev), K.to(dev), V.to(dev), scale, causal, num_splits=3)
            pkg.ops.check_status(dev)
            res[opt] = (O.float().cpu().numpy(), L.cpu().numpy())
            assert np.abs(res[opt][0] - oracle.bf16_decode(Ow)).max() <= 2e-2
            assert np.abs(res[opt][1] - Lw).max() <= 1e-3
    finally:
        pkg.capi.set_option("attn.decode_kernel", 0)
    assert np.abs(res[1][0] - res[2][0]).max() <= 2e-2


def test_fp8_decode_kernel_growing_keys(pkg, oracle, dev):
    """The same on an E4M3 KV cache: P is rounded to E4M3 against the running reference of its row, raised several times."""
    B, Hq, Hkv, Sq, Skv = 1, 8, 2, 2, 1024
    Qs, _, V, dq, dk, dv, scale = pkg.synth.fp8_attention_inputs(B, Hq, Hkv, Skv, 128, seed=31)
    g = torch.Generator().manual_seed(5)
    ramp = (1.0 + 9.0 * torch.arange(Skv, dtype=torch.float32) / Skv).view(1, 1, Skv, 1)
    K = (torch.randn(B, Hkv, Skv, 128, generator=g) * 4.0 * ramp).clamp(-448, 448).to(torch.float8_e4m3fn)
    Q = Qs[:, :, Skv - Sq:].contiguous()
    O, L = pkg.ops.attn_fwd_fp8_splitkv(*(t.to(dev) for t in (Q, K, V, dq, dk, dv)), scale, True, num_splits=4)
    pkg.ops.check_status(dev)
    Ow, Lw = oracle.attn_fwd_fp8(u8(Qs), u8(K), u8(V), dq.numpy(), dk.numpy(), dv.numpy(), scale, True, tile_n=128, q_range=(Skv - Sq, Skv))
    want = oracle.bf16_decode(Ow)[:, :, Skv - Sq:]
    got = O.float().cpu().numpy()
    assert np.abs(L.cpu().numpy() - Lw[:, :, Skv - Sq:]).max() <= 1e-3
    assert np.linalg.norm(got - want) <= 8e-2 * np.linalg.norm(want)      # E4M3 rounding noise of P, see test_fp8_splitkv_matches_oracle


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal,cuts", [
    (1, 4, 2, 200, 1024, True, (0, 384, 768, 1024)),        # three ranks' worth of keys, chunked prefill
    (2, 8, 2, 1, 2048, True, (0, 1024, 2048)),              # decode, stacked GQA heads
    (1, 2, 2, 256, 512, True, (0, 128, 512)),               # square: the first shard is in the past of every late query,
                                                            # the last shard in the future of the early ones
    (1, 4, 1, 72, 640, False, (0, 256, 512, 640)),
    (1, 8, 8, 8, 1536, True, (0, 512, 1032, 1536)),         # eight late queries per head: the last shard is partly in their future
    (1, 4, 2, 3, 904, False, (0, 128, 904)),                # decode kernel on every shard, ragged last shard
])
def test_kv_sharded_partials_combine_to_full_attention(pkg, oracle, dev, B, Hq, Hkv, Sq, Skv, causal, cuts):
    """Sequence-parallel attention emulated on one GPU: the forward pass over each KV shard (global key offset in the
    causal mask) leaves a partial result; combining the shards' results equals attention over all keys."""
    Q, K, V, scale = make(pkg, B, Hq, Hkv, Sq, Skv, seed=12)
    Qd = Q.to(dev)
    parts = []
    for k0, k1 in zip(cuts[:-1], cuts[1:]):
        Kl, Vl = K[:, :, k0:k1].contiguous().to(dev), V[:, :, k0:k1].contiguous().to(dev)
        parts.append(pkg.ops.attn_fwd_bf16_kvshard(Qd, Kl, Vl, scale, causal, k0, Skv))
    O, L = pkg.ops.attn_combine_partials(torch.stack(parts), tuple(Q.shape))
    pkg.ops.check_status(dev)
    Ow, Lw = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, causal)
    assert np.abs(O.float().cpu().numpy() - oracle.bf16_decode(Ow)).max() <= 2e-2
    assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3


@pytest.mark.parametrize("B,Hq,Hkv,S,world,causal", [
    (1, 4, 2, 1024, 2, True),
    (1, 4, 2, 1024, 4, True),
    (2, 4, 4, 640, 3, True),            # unequal shards: 256, 256, 128 positions
    (1, 2, 1, 768, 3, False),
    (1, 8, 2, 256, 4, True),            # more ranks than 128-position blocks: two ranks hold nothing
])
def test_ring_attention_plan_emulated_on_one_gpu(pkg, oracle, dev, B, Hq, Hkv, S, world, causal):
    """Ring attention emulated on one GPU: for every virtual rank the KV-shard passes its plan prescribes (the real
    CUDA entry point with the plan's position arguments; skipped passes as empty partial results), combined, against
    the oracle's attention over the whole sequence, rows of that rank."""
    Q, K, V, scale = make(pkg, B, Hq, Hkv, S, S, seed=17)
    Ow, Lw = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, causal)
    Ow = oracle.bf16_decode(Ow)
    for rank in range(world):
        q0, q1 = pkg.shard.kv_shard_range(S, world, rank)
        if q1 == q0:
            continue
        Ql = Q[:, :, q0:q1].contiguous().to(dev)
        rows = B * Hq * (q1 - q0)
        parts = []
        for k_rank, (k0, k1), kv_pos0, total_arg, run in pkg.shard.ring_shard_plan(S, world, rank, causal):
            if run:
                Kl, Vl = K[:, :, k0:k1].contiguous().to(dev), V[:, :, k0:k1].contiguous().to(dev)
                parts.append(pkg.ops.attn_fwd_bf16_kvshard(Ql, Kl, Vl, scale, causal, kv_pos0, total_arg))
            else:
                parts.append(pkg.shard.empty_partial(rows, 128, dev))
        O, L = pkg.ops.attn_combine_partials(torch.stack(parts), tuple(Ql.shape))
        pkg.ops.check_status(dev)
        assert np.abs(O.float().cpu().numpy() - Ow[:, :, q0:q1]).max() <= 2e-2, (rank, world)
        assert np.abs(L.cpu().numpy() - Lw[:, :, q0:q1]).max() <= 1e-3, (rank, world)


@pytest.mark.parametrize("B,Hq,Hkv,S,world,causal", [
    (1, 4, 2, 1024, 2, True),
    (1, 4, 2, 2048, 4, True),
    (1, 2, 1, 640, 2, False),           # unequal chunks
    (1, 4, 4, 384, 2, True),            # three 128-position blocks over four chunks: one chunk is empty
])
def test_zigzag_ring_passes_emulated_on_one_gpu(pkg, oracle, dev, B, Hq, Hkv, S, world, causal):
    """Zig-zag ring attention emulated on one GPU: for every virtual rank and each of its two position ranges, the passes
    ``ring_passes`` prescribes over all ranks' ranges (real CUDA entry point), combined, against the oracle."""
    Q, K, V, scale = make(pkg, B, Hq, Hkv, S, S, seed=19)
    Ow, Lw = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, causal)
    Ow = oracle.bf16_decode(Ow)
    counts = []
    for rank in range(world):
        mine = pkg.shard.zigzag_ranges(S, world, rank)
        parts = [[] for _ in mine]
        for t in range(world):
            theirs = pkg.shard.zigzag_ranges(S, world, (rank - t) % world)
            for qi, kj, kv_pos0, total_arg, run in pkg.shard.ring_passes(mine, theirs, causal, S):
                if run:
                    (q0, q1), (k0, k1) = mine[qi], theirs[kj]
                    parts[qi].append(pkg.ops.attn_fwd_bf16_kvshard(Q[:, :, q0:q1].contiguous().to(dev), K[:, :, k0:k1].contiguous().to(dev),
                                                                   V[:, :, k0:k1].contiguous().to(dev), scale, causal, kv_pos0, total_arg))
        counts.append(sum(len(p_) for p_ in parts))
        for (q0, q1), ps in zip(mine, parts):
            if q1 == q0:
                continue
            O, L = pkg.ops.attn_combine_partials(torch.stack(ps), (B, Hq, q1 - q0, 128))
            pkg.ops.check_status(dev)
            assert np.abs(O.float().cpu().numpy() - Ow[:, :, q0:q1]).max() <= 2e-2, (rank, q0)
            assert np.abs(L.cpu().numpy() - Lw[:, :, q0:q1]).max() <= 1e-3, (rank, q0)
    if causal and S % (256 * world) == 0:
        assert len(set(counts)) == 1         # equal chunks: every rank runs the same number of passes


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal,cuts", [
    (1, 8, 2, 256, 1024, True, (0, 384, 768, 1024)),        # three shards, late queries
    (2, 8, 2, 1, 2048, True, (0, 1024, 2048)),              # decode on an E4M3 KV cache, stacked GQA heads
    (1, 4, 4, 128, 640, False, (0, 256, 640)),
])
def test_fp8_kv_sharded_partials_combine_to_full_attention(pkg, oracle, dev, B, Hq, Hkv, Sq, Skv, causal, cuts):
    """Sequence-parallel attention on E4M3 operands emulated on one GPU: one KV-shard pass per shard, combined.  The shards
    round P to E4M3 against their own running maxima, so - as for several split-KV shares - the result is held against
    exact float64 attention on the dequantised operands and must be about as close to it as the single-pass oracle is;
    with one shard the pass reproduces the split-KV entry point bit for bit."""
    Qs, K, V, dq, dk, dv, scale = pkg.synth.fp8_attention_inputs(B, Hq, Hkv, Skv, 128, seed=27)
    r0 = Skv - Sq if causal else 0
    Q = Qs[:, :, r0:r0 + Sq].contiguous()
    Qd, dqd, dkd, dvd = Q.to(dev), dq.to(dev), dk.to(dev), dv.to(dev)
    parts = []
    for k0, k1 in zip(cuts[:-1], cuts[1:]):
        parts.append(pkg.ops.attn_fwd_fp8_kvshard(Qd, K[:, :, k0:k1].contiguous().to(dev), V[:, :, k0:k1].contiguous().to(dev), dqd, dkd, dvd,
                                                  scale, causal, k0, Skv))
    O, L = pkg.ops.attn_combine_partials(torch.stack(parts), tuple(Q.shape))
    pkg.ops.check_status(dev)
    Ow, Lw = oracle.attn_fwd_fp8(u8(Qs), u8(K), u8(V), dq.numpy(), dk.numpy(), dv.numpy(), scale, causal, tile_n=128, q_range=(r0, r0 + Sq))
    want = oracle.bf16_decode(Ow)[:, :, r0:r0 + Sq]
    got = O.float().cpu().numpy()
    assert np.abs(L.cpu().numpy() - Lw[:, :, r0:r0 + Sq]).max() <= 1e-3
    g = Hq // Hkv
    q = oracle.e4m3_decode(u8(Q)).astype(np.float64) * dq.numpy().reshape(B, Hq, 1, 1)
    k = np.repeat(oracle.e4m3_decode(u8(K)).astype(np.float64) * dk.numpy().reshape(B, Hkv, 1, 1), g, axis=1)
    v = np.repeat(oracle.e4m3_decode(u8(V)).astype(np.float64) * dv.numpy().reshape(B, Hkv, 1, 1), g, axis=1)
    sc = np.einsum("bhqd,bhkd->bhqk", q, k) * scale
    if causal:
        sc = np.where(np.arange(Skv)[None, :] <= (np.arange(Sq)[:, None] + r0), sc, -np.inf)
    pr = np.exp(sc - sc.max(-1, keepdims=True))
    exact = np.einsum("bhqk,bhkd->bhqd", pr / pr.sum(-1, keepdims=True), v)
    err_kernel = np.linalg.norm(got - exact) / np.linalg.norm(exact)
    err_oracle = np.linalg.norm(want - exact) / np.linalg.norm(exact)
    assert err_kernel <= 5e-2 and err_kernel <= 2.0 * err_oracle + 5e-3, (err_kernel, err_oracle)
    # one shard = the whole key range: the same kernel launch as split-KV with one share leaving a partial result
    whole = pkg.ops.attn_fwd_fp8_kvshard(Qd, K.to(dev), V.to(dev), dqd, dkd, dvd, scale, causal, 0, Skv)
    O1, L1 = pkg.ops.attn_combine_partials(whole.view(1, -1), tuple(Q.shape))
    O2, L2 = pkg.ops.attn_fwd_fp8_splitkv(Qd, K.to(dev), V.to(dev), dqd, dkd, dvd, scale, causal, num_splits=1)
    pkg.ops.check_status(dev)
    assert np.linalg.norm(O1.float().cpu().numpy() - O2.float().cpu().numpy()) <= 1e-2 * np.linalg.norm(O2.float().cpu().numpy())
    assert np.abs(L1.cpu().numpy() - L2.cpu().numpy()).max() <= 1e-3


def test_fp8_kvshard_rejects_bad_arguments(pkg, dev):
    Q, K, V, dq, dk, dv, scale = (t.to(dev) if torch.is_tensor(t) else t for t in pkg.synth.fp8_attention_inputs(1, 4, 2, 256, 128, seed=5))
    small = torch.empty(16, dtype=torch.uint8, device=dev)
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.ops.attn_fwd_fp8_kvshard(Q, K, V, dq, dk, dv, scale, True, 0, 256, partial=small)        # partial buffer too small
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG
    with pytest.raises(pkg.capi.AxpError):
        pkg.ops.attn_fwd_fp8_kvshard(Q, K, V, dq, dk, dv, scale, True, 128, 256)                      # shard reaches past the sequence


def test_fused_operator_goldens_on_gpu(pkg, dev, golden):
    """The widened operators against the committed float64 fixtures (no oracle in the loop)."""
    g = golden["fused_small"]
    t16 = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16).to(dev)
    X, Wg, Wu, Cin = t16(g["X"]), t16(g["Wg"]), t16(g["Wu"]), t16(g["Cin"])
    H = pkg.ops.gemm_bf16_swiglu(X, Wg, Wu).float().cpu().numpy()
    assert np.linalg.norm(H - g["H_f64"]) / np.linalg.norm(g["H_f64"]) < 3e-3
    D = pkg.ops.gemm_lincomb(X, Wg, Cin, float(g["alpha"]), float(g["beta"])).float().cpu().numpy()
    assert np.linalg.norm(D - g["D_f64"]) / np.linalg.norm(g["D_f64"]) < 3e-3
    Qc, S = pkg.ops.rmsnorm_quantize_rows_e4m3(t16(g["Xn"]), t16(g["w"]), float(g["eps"]))
    M, K = g["Xn"].shape
    deq = (Qc.float().view(M, K // 128, 128) * S.view(M, K // 128, 1)).view(M, K).cpu().numpy()
    assert np.linalg.norm(deq - g["Yn_f64"]) / np.linalg.norm(g["Yn_f64"]) < 4e-2
    Q, Kk, V = t16(g["Q"]), t16(g["K"]), t16(g["V"])
    for name, causal in (("causal", True), ("full", False)):
        for splits in (1, 3):
            O, L = pkg.ops.attn_fwd_bf16_splitkv(Q, Kk, V, float(g["scale"]), causal, num_splits=splits)
            assert np.abs(O.float().cpu().numpy() - g["O_" + name]).max() <= 2e-2
            assert np.abs(L.cpu().numpy() - g["LSE_" + name]).max() <= 1e-3
    pkg.ops.check_status(dev)
