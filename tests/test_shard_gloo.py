"""world_size-2 gloo test (CPU) of the multi-GPU host logic: column shards and the
optional all-gather of C when the caller asks for the full output."""
import os
import sys

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, N, M, ret):
    sys.path.insert(0, ROOT)
    import importlib

    shard = importlib.import_module("iro-cuda-ax_b200").shard
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(7)
        full = torch.randn(M, N, generator=g).bfloat16()       # every rank builds the same "answer"
        n0, n1 = shard.gemm_column_range(N, world, rank)
        got = shard.all_gather_columns(full[:, n0:n1].contiguous(), N, world)
        ret[rank] = bool(torch.equal(got, full)) and (n0 % 256 == 0)
    finally:
        dist.destroy_process_group()


def _run(N, M, world=2):
    port = 29600 + (os.getpid() % 200)
    mgr = mp.get_context("spawn").Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, N, M, ret), nprocs=world, join=True)
    assert all(ret[r] for r in range(world)) and len(ret) == world


def test_all_gather_columns_even():
    _run(N=1024, M=40)


def test_all_gather_columns_uneven_blocks():
    _run(N=768, M=24)       # 3 blocks of 256 over 2 ranks: widths 512 and 256


def test_attention_head_ranges_keep_kv_groups_whole(pkg):
    for B, Hq, Hkv, world in ((4, 64, 8, 8), (8, 32, 32, 8), (1, 8, 2, 3)):
        grp = Hq // Hkv
        prev = 0
        for r in range(world):
            b, e = pkg.shard.attention_head_range(B, Hq, Hkv, world, r)
            assert b == prev and b % grp == 0 and e % grp == 0
            prev = e
        assert prev == B * Hq


def _kv_sharded_worker(rank, world, port, q, Skv=320):
    import importlib
    import os
    import sys

    import numpy as np
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module("iro-cuda-ax_b200")
        from oracle import host_oracle as oracle

        B, Hq, Hkv, Sq, D = 1, 4, 2, 24, 128
        Q, _, _, scale = pkg.synth.bf16_attention_inputs(B, Hq, Sq, D, seed=3, Hkv=Hkv)
        _, K, V, _ = pkg.synth.bf16_attention_inputs(B, Hkv, Skv, D, seed=4)
        k0, k1 = pkg.shard.kv_shard_range(Skv, world, rank)

        def u16(t):
            return t.view(torch.uint16).numpy()

        # CPU stand-ins for the two CUDA entry points: partial result = (unnormalised O in fp32, (m * log2 e, l)) of
        # the local keys, in the byte layout of the C-ABI; the combine follows the formula of the header
        def partial_fn(Qt, Kt, Vt, scale, causal, kpos0, total):
            q = oracle.bf16_decode(u16(Qt)).astype(np.float64)
            k = oracle.bf16_decode(u16(Kt)).astype(np.float64)
            v = oracle.bf16_decode(u16(Vt)).astype(np.float64)
            grp = Hq // Hkv
            o = np.zeros((B * Hq * Sq, D), np.float32)
            ml = np.zeros((B * Hq * Sq, 2), np.float32)
            for h in range(Hq):
                s = q[0, h] @ k[0, h // grp].T * scale
                if causal:
                    qi = np.arange(Sq)[:, None] + (total - Sq)
                    kj = np.arange(Kt.shape[2])[None, :] + kpos0
                    s = np.where(kj <= qi, s, -np.inf)
                m = s.max(-1)
                ok = np.isfinite(m)
                p = np.where(ok[:, None], np.exp(s - np.where(ok, m, 0.0)[:, None]), 0.0)
                o[h * Sq:(h + 1) * Sq] = p @ v[0, h // grp]
                ml[h * Sq:(h + 1) * Sq, 0] = np.where(ok, m * 1.4426950408889634, -np.inf)
                ml[h * Sq:(h + 1) * Sq, 1] = p.sum(-1)
            return torch.from_numpy(np.concatenate([o.reshape(-1).view(np.uint8), ml.reshape(-1).view(np.uint8)]))

        def combine_fn(gathered, shape):
            rows = shape[0] * shape[1] * shape[2]
            outs = np.zeros((rows, D)); den = np.zeros(rows); mm = np.full(rows, -np.inf)
            shares = []
            for z in range(gathered.shape[0]):
                raw = gathered[z].numpy()
                o = raw[: rows * D * 4].view(np.float32).reshape(rows, D).astype(np.float64)
                ml = raw[rows * D * 4:].view(np.float32).reshape(rows, 2).astype(np.float64)
                shares.append((o, ml))
                mm = np.maximum(mm, np.where(ml[:, 1] > 0, ml[:, 0], -np.inf))
            for o, ml in shares:
                w = np.where(ml[:, 1] > 0, np.exp2(ml[:, 0] - mm), 0.0)
                outs += w[:, None] * o
                den += w * ml[:, 1]
            return outs / den[:, None], (mm + np.log2(den)) * 0.6931471805599453

        O, L = pkg.shard.attn_kv_sharded(Q, K[:, :, k0:k1].contiguous(), V[:, :, k0:k1].contiguous(), scale, True, Skv, world, rank,
                                         partial_fn=partial_fn, combine_fn=combine_fn)
        Ow, Lw = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, True)
        err = float(np.abs(O.reshape(B, Hq, Sq, D) - oracle.bf16_decode(Ow)).max())
        lerr = float(np.abs(L.reshape(B, Hq, Sq) - Lw).max())
        q.put((rank, (k0, k1), err, lerr))
    finally:
        dist.destroy_process_group()


def test_kv_sharded_attention_exchange_world_size_2():
    """Host logic of sequence-parallel attention on two gloo ranks: shard ranges, the all-gather of the partial
    results in the C-ABI byte layout, and the state combine, with CPU stand-ins for the two CUDA entry points."""
    import torch.multiprocessing as mp

    got = _run_kv_sharded(2, 320)
    assert [g[1] for g in got] == [(0, 256), (256, 320)]         # 128-key blocks: three blocks over two ranks
    for _, _, err, lerr in got:
        assert err <= 1e-2 and lerr <= 1e-4


def _free_port():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_kv_sharded(world, Skv):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_kv_sharded_worker, args=(r, world, port, q, Skv)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
    finally:
        for p in procs:                  # no child outlives the test, whatever happened
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
    return sorted(q.get(timeout=5) for _ in range(world))


def test_kv_sharded_attention_rank_without_keys_still_joins_the_exchange():
    """More ranks than 128-key blocks: the last rank holds no key, launches nothing and contributes an empty partial
    result, so that every rank enters the all-gather and the combined result is still the full attention."""
    got = _run_kv_sharded(3, 256)
    assert [g[1] for g in got] == [(0, 128), (128, 256), (256, 256)]
    for _, _, err, lerr in got:
        assert err <= 1e-2 and lerr <= 1e-4


def _cpu_stand_ins(oracle, B, Hq, Hkv, D):
    """CPU stand-ins for the two CUDA entry points of sharded attention (partial result of a KV shard in the C-ABI byte
    layout; state combine after the formula of the header)."""
    import numpy as np
    import torch

    def u16(t):
        return t.view(torch.uint16).numpy()

    def partial_fn(Qt, Kt, Vt, scale, causal, kpos0, total):
        Sq = Qt.shape[2]
        q = oracle.bf16_decode(u16(Qt)).astype(np.float64)
        k = oracle.bf16_decode(u16(Kt)).astype(np.float64)
        v = oracle.bf16_decode(u16(Vt)).astype(np.float64)
        grp = Hq // Hkv
        o = np.zeros((B * Hq * Sq, D), np.float32)
        ml = np.zeros((B * Hq * Sq, 2), np.float32)
        for h in range(Hq):
            s = q[0, h] @ k[0, h // grp].T * scale
            if causal:
                qi = np.arange(Sq)[:, None] + (total - Sq)
                kj = np.arange(Kt.shape[2])[None, :] + kpos0
                s = np.where(kj <= qi, s, -np.inf)
            m = s.max(-1)
            ok = np.isfinite(m)
            p = np.where(ok[:, None], np.exp(s - np.where(ok, m, 0.0)[:, None]), 0.0)
            o[h * Sq:(h + 1) * Sq] = p @ v[0, h // grp]
            ml[h * Sq:(h + 1) * Sq, 0] = np.where(ok, m * 1.4426950408889634, -np.inf)
            ml[h * Sq:(h + 1) * Sq, 1] = p.sum(-1)
        return torch.from_numpy(np.concatenate([o.reshape(-1).view(np.uint8), ml.reshape(-1).view(np.uint8)]))

    def combine_fn(gathered, shape):
        rows = shape[0] * shape[1] * shape[2]
        outs = np.zeros((rows, D)); den = np.zeros(rows); mm = np.full(rows, -np.inf)
        shares = []
        for z in range(gathered.shape[0]):
            raw = gathered[z].numpy()
            o = raw[: rows * D * 4].view(np.float32).reshape(rows, D).astype(np.float64)
            ml = raw[rows * D * 4:].view(np.float32).reshape(rows, 2).astype(np.float64)
            shares.append((o, ml))
            mm = np.maximum(mm, np.where(ml[:, 1] > 0, ml[:, 0], -np.inf))
        for o, ml in shares:
            w = np.where(ml[:, 1] > 0, np.exp2(ml[:, 0] - mm), 0.0)
            outs += w[:, None] * o
            den += w * ml[:, 1]
        return outs / den[:, None], (mm + np.log2(den)) * 0.6931471805599453

    return u16, partial_fn, combine_fn


def _ring_worker(rank, world, port, q, S, causal, zigzag=False):
    import importlib
    import os
    import sys

    import numpy as np
    import torch
    import torch.distributed as dist

    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        pkg = importlib.import_module("iro-cuda-ax_b200")
        from oracle import host_oracle as oracle

        B, Hq, Hkv, D = 1, 4, 2, 128
        u16, partial_fn, combine_fn = _cpu_stand_ins(oracle, B, Hq, Hkv, D)
        Q, _, _, scale = pkg.synth.bf16_attention_inputs(B, Hq, S, D, seed=5, Hkv=Hkv)
        _, K, V, _ = pkg.synth.bf16_attention_inputs(B, Hkv, S, D, seed=6)
        Ow, Lw = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, causal)
        Ow = oracle.bf16_decode(Ow)
        if zigzag:
            ranges = pkg.shard.zigzag_ranges(S, world, rank)
            cut = lambda T: [T[:, :, a:b].contiguous() for a, b in ranges]
            outs = pkg.shard.attn_ring_zigzag(cut(Q), cut(K), cut(V), scale, causal, S, world, rank, partial_fn=partial_fn, combine_fn=combine_fn)
            passes = sum(1 for t in range(world) for step in pkg.shard.ring_passes(ranges, pkg.shard.zigzag_ranges(S, world, (rank - t) % world), causal, S)
                         if step[4])
        else:
            ranges = [pkg.shard.kv_shard_range(S, world, rank)]
            p0, p1 = ranges[0]
            outs = [pkg.shard.attn_ring(Q[:, :, p0:p1].contiguous(), K[:, :, p0:p1].contiguous(), V[:, :, p0:p1].contiguous(), scale, causal, S,
                                        world, rank, partial_fn=partial_fn, combine_fn=combine_fn)]
            passes = sum(1 for step in pkg.shard.ring_shard_plan(S, world, rank, causal) if step[4])
        err = lerr = 0.0
        for (p0, p1), (O, L) in zip(ranges, outs):
            if p1 > p0:
                err = max(err, float(np.abs(np.asarray(O).reshape(B, Hq, p1 - p0, D) - Ow[:, :, p0:p1]).max()))
                lerr = max(lerr, float(np.abs(np.asarray(L).reshape(B, Hq, p1 - p0) - Lw[:, :, p0:p1]).max()))
        q.put((rank, ranges[0] if not zigzag else tuple(ranges), err, lerr, passes))
    finally:
        dist.destroy_process_group()


def _run_ring(world, S, causal, zigzag=False):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_ring_worker, args=(r, world, port, q, S, causal, zigzag)) for r in range(world)]
    for p in procs:
        p.start()
    try:
        for p in procs:
            p.join(180)
            assert p.exitcode == 0
    finally:
        for p in procs:
            if p.is_alive():
                p.terminate()
                p.join(10)
                if p.is_alive():
                    p.kill()
    return sorted(q.get(timeout=5) for _ in range(world))


def test_ring_attention_world_size_2_causal_and_full():
    """Ring attention on two gloo ranks (queries and keys sharded, K / V shards passed round by point-to-point sends):
    shard plan, causal position arguments, skipped future shards, exchange and combine, with CPU stand-ins for the two
    CUDA entry points."""
    got = _run_ring(2, 320, True)
    assert [g[1] for g in got] == [(0, 256), (256, 320)]
    assert [g[4] for g in got] == [1, 2]                  # under the causal mask rank r runs r + 1 passes
    for _, _, err, lerr, _ in got:
        assert err <= 1e-2 and lerr <= 1e-4
    got = _run_ring(2, 320, False)
    assert [g[4] for g in got] == [2, 2]
    for _, _, err, lerr, _ in got:
        assert err <= 1e-2 and lerr <= 1e-4


def test_ring_attention_three_ranks_one_without_positions():
    """Three ranks, two 128-position blocks: the last rank holds nothing, still forwards the shards it receives and
    returns empty outputs."""
    got = _run_ring(3, 256, True)
    assert [g[1] for g in got] == [(0, 128), (128, 256), (256, 256)]
    assert [g[4] for g in got] == [1, 2, 0]
    for _, _, err, lerr, _ in got:
        assert err <= 1e-2 and lerr <= 1e-4


def test_ring_shard_plan_positions(pkg):
    plan = pkg.shard.ring_shard_plan(640, 3, 1, True)         # rank 1 holds [256, 512)
    assert [(s[0], s[1], s[4]) for s in plan] == [(1, (256, 512), True), (0, (0, 256), True), (2, (512, 640), False)]
    assert all(s[3] == 512 for s in plan)                     # causal: the sequence as far as this rank's last query
    assert [s[2] for s in plan] == [256, 0, 512]
    assert all(s[3] == 640 and s[4] for s in pkg.shard.ring_shard_plan(640, 3, 1, False))


def test_zigzag_ring_attention_balances_the_causal_passes():
    """Zig-zag assignment on two gloo ranks: four chunks, rank r holds chunks r and 3 - r; results equal attention over the
    whole sequence on both chunks of every rank, and under the causal mask both ranks run the same number of passes."""
    got = _run_ring(2, 1024, True, zigzag=True)
    assert [g[1] for g in got] == [((0, 256), (768, 1024)), ((256, 512), (512, 768))]
    assert [g[4] for g in got] == [5, 5]                  # of the 4 x 4 chunk pairs the causal mask keeps 10
    for _, _, err, lerr, _ in got:
        assert err <= 1e-2 and lerr <= 1e-4
    got = _run_ring(2, 640, False, zigzag=True)               # unequal chunks: 256, 128, 128, 128 positions
    assert [g[1] for g in got] == [((0, 256), (512, 640)), ((256, 384), (384, 512))]
    for _, _, err, lerr, _ in got:
        assert err <= 1e-2 and lerr <= 1e-4
