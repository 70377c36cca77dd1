"""How the path shards across the GPUs of one box (one process per GPU).

* GEMM: output columns (N) are split into contiguous ranges whose boundaries are
  multiples of 256 (the CTA tile width, itself a multiple of the 128-wide scale
  block).  Rank r holds B[n0:n1,:] and the matching sB rows and writes
  C[:, n0:n1]; A and sA are replicated.  No collective, unless the caller asks for
  the full C, which is then an all-gather of the column shards.
* Attention: flattened batch x head (bf16) or batch x KV-head group (fp8 GQA) is
  split into contiguous ranges; no collective.
* Long sequences (sequence / context parallelism): ``attn_kv_sharded`` shards the keys (every rank holds all
  queries; one all-gather of partial results), ``attn_ring`` shards queries and keys alike and passes the K / V
  shards round a ring (point-to-point exchange overlapped with the pass over the shard in hand).
"""
from __future__ import annotations


def shard_range(units: int, gran: int, world: int, rank: int) -> tuple[int, int]:
    """Contiguous [begin,end) of `units` items for `rank`, boundaries at multiples of `gran`.

    The first (blocks % world) ranks get one extra block of `gran` items."""
    if world <= 0 or not (0 <= rank < world) or gran <= 0 or units < 0:
        raise ValueError("bad shard arguments")
    blocks = (units + gran - 1) // gran
    base, extra = divmod(blocks, world)
    b0 = rank * base + min(rank, extra)
    b1 = b0 + base + (1 if rank < extra else 0)
    return min(b0 * gran, units), min(b1 * gran, units)


def gemm_column_range(N: int, world: int, rank: int) -> tuple[int, int]:
    return shard_range(N, 256, world, rank)


def attention_head_range(B: int, Hq: int, Hkv: int, world: int, rank: int) -> tuple[int, int]:
    """Range of flattened query heads b*Hq+h; whole KV-head groups stay on one rank."""
    group = Hq // Hkv
    return shard_range(B * Hq, group, world, rank)


def all_gather_columns(c_local, N: int, world: int, group=None, out=None):
    """Full C [M,N] from the ranks' column shards (only when the caller wants the full output).

    Every rank passes its row-major [M, n1-n0] shard.  One all-gather of the shards as they lie (bytes; a shard narrower
    than the widest one is padded first), then one strided placement pass per rank into ``out`` [M,N] (allocated when
    not given)."""
    import torch
    import torch.distributed as dist

    M = c_local.shape[0]
    ranges = [gemm_column_range(N, world, r) for r in range(world)]
    wmax = max(e - b for b, e in ranges)
    if c_local.shape[1] == wmax and c_local.is_contiguous():
        send = c_local
    else:
        send = torch.zeros((M, wmax), dtype=c_local.dtype, device=c_local.device)
        send[:, : c_local.shape[1]] = c_local
    gathered = torch.empty((world * M, wmax), dtype=c_local.dtype, device=c_local.device)      # rank r's shard = rows [r M, (r+1) M)
    # bit patterns travel as bytes: every backend moves uint8, not every one moves bf16
    dist.all_gather_into_tensor(gathered.view(torch.uint8), send.view(torch.uint8), group=group)
    full = out if out is not None else torch.empty((M, N), dtype=c_local.dtype, device=c_local.device)
    for r, (b, e) in enumerate(ranges):
        full[:, b:e].copy_(gathered[r * M : (r + 1) * M, : e - b])
    return full


def kv_shard_range(Skv: int, world: int, rank: int, gran: int = 128) -> tuple[int, int]:
    """Keys [begin,end) of a sequence of `Skv` keys held by `rank` under sequence (context) parallelism."""
    return shard_range(Skv, gran, world, rank)


def attn_kv_sharded(Q, K_local, V_local, scale: float, causal: bool, skv_total: int, world: int, rank: int, group=None,
                    partial_fn=None, combine_fn=None):
    """Attention whose keys are sharded over the ranks (long context): every rank holds all queries
    Q [B,Hq,Sq,D] and the keys ``kv_shard_range(skv_total, world, rank)``.  Each rank runs the forward pass over its
    shard, the partial results (fp32 accumulators and (m, l) per row) are all-gathered - the one exchange step of
    this path, rows * 520 bytes per rank - and every rank combines them into the full O, LSE.

    ``partial_fn`` / ``combine_fn`` default to the CUDA entry points (``ops.attn_fwd_bf16_kvshard``,
    ``ops.attn_combine_partials``); tests of the host logic on CPU ranks pass stand-ins."""
    import torch
    import torch.distributed as dist

    if partial_fn is None or combine_fn is None:
        from . import ops

        partial_fn = partial_fn or ops.attn_fwd_bf16_kvshard
        combine_fn = combine_fn or ops.attn_combine_partials
    k0, k1 = kv_shard_range(skv_total, world, rank)
    if K_local.shape[2] != k1 - k0:
        raise ValueError(f"rank {rank} must hold keys [{k0},{k1}) of {skv_total}, got {K_local.shape[2]}")
    if k1 > k0:
        part = partial_fn(Q, K_local, V_local, scale, causal, k0, skv_total)
    else:
        # a rank without keys (more ranks than 128-key blocks) launches nothing and still joins the exchange, with an
        # empty partial result: (m, l) = (-inf, 0) for every row, which the combine skips (the accumulators are not read)
        part = empty_partial(Q.shape[0] * Q.shape[1] * Q.shape[2], Q.shape[3], Q.device)
    gathered = torch.empty((world, part.numel()), dtype=torch.uint8, device=part.device)
    dist.all_gather_into_tensor(gathered, part.view(1, -1), group=group)
    return combine_fn(gathered, tuple(Q.shape))


def ring_shard_plan(s_total: int, world: int, rank: int, causal: bool):
    """What rank `rank` does in each of the `world` steps of ``attn_ring``: a list of
    ``(k_rank, (k0, k1), kv_pos0, skv_total_arg, run)`` - the rank whose K / V shard is in hand at that step, its key
    range, and the two position arguments of ``axp_sm100_attn_fwd_bf16_kvshard`` for the local queries [q0, q1)
    against it; ``run`` is False when the pass is skipped (no keys, no queries, or - under the causal mask - a shard
    that lies wholly in the future of every local query).

    Under the causal mask local query i (global position q0 + i) sees global keys <= q0 + i.  The entry point's rule
    is "query i sees keys <= i + (skv_total - Sq)", so the call passes skv_total = q1: the sequence as far as this
    rank's last query."""
    q0, q1 = kv_shard_range(s_total, world, rank)
    plan = []
    for t in range(world):
        k_rank = (rank - t) % world
        k0, k1 = kv_shard_range(s_total, world, k_rank)
        run = k1 > k0 and q1 > q0 and not (causal and k0 >= q1)
        plan.append((k_rank, (k0, k1), k0, q1 if causal else s_total, run))
    return plan


def fp8_partial_fn(q_descale, k_descale, v_descale):
    """``partial_fn`` for ``attn_kv_sharded`` / ``attn_ring`` / ``attn_ring_zigzag`` on E4M3 operands: the KV-shard pass of
    ``axp_sm100_attn_fwd_fp8_kvshard`` with the per-head descales (float32 [B*Hq] / [B*Hkv]) bound."""
    from . import ops

    def partial_fn(Q, K, V, scale, causal, kv_pos0, skv_total):
        return ops.attn_fwd_fp8_kvshard(Q, K, V, q_descale, k_descale, v_descale, scale, causal, kv_pos0, skv_total)

    return partial_fn


def zigzag_ranges(s_total: int, world: int, rank: int) -> list[tuple[int, int]]:
    """The two position ranges rank `rank` holds under the zig-zag assignment: the sequence is cut into 2 * world chunks
    (boundaries at multiples of 128) and rank r takes chunks r and 2 * world - 1 - r, an early and a late one, so that
    under the causal mask every rank sees about the same number of (query, key) pairs."""
    return [shard_range(s_total, 128, 2 * world, rank), shard_range(s_total, 128, 2 * world, 2 * world - 1 - rank)]


def ring_passes(q_ranges, k_ranges, causal: bool, s_total: int):
    """The KV-shard passes of one ring step: for every local query range and every key range of the shard in hand,
    ``(qi, kj, kv_pos0, skv_total_arg, run)`` with the position arguments of ``axp_sm100_attn_fwd_bf16_kvshard`` (see
    ``ring_shard_plan``).  Ranges are aligned and disjoint, so a key range lies wholly before a query range, is the
    same range (the diagonal), or lies wholly after it - and is then skipped under the causal mask."""
    out = []
    for qi, (q0, q1) in enumerate(q_ranges):
        for kj, (k0, k1) in enumerate(k_ranges):
            run = k1 > k0 and q1 > q0 and not (causal and k0 >= q1)
            out.append((qi, kj, k0, q1 if causal else s_total, run))
    return out


def _ring(Qs, Ks, Vs, ranges_of, scale, causal, s_total, world, rank, group, partial_fn, combine_fn):
    """Ring attention over lists of position ranges per rank (one range: contiguous shards; two: zig-zag).  Qs / Ks / Vs are
    lists of contiguous tensors, one per range of this rank."""
    import torch
    import torch.distributed as dist

    if partial_fn is None or combine_fn is None:
        from . import ops

        partial_fn = partial_fn or ops.attn_fwd_bf16_kvshard
        combine_fn = combine_fn or ops.attn_combine_partials
    mine = ranges_of(rank)
    for t_, (p0, p1) in zip(zip(Qs, Ks, Vs), mine):
        if t_[0].shape[2] != p1 - p0 or t_[1].shape[2] != p1 - p0 or t_[2].shape != t_[1].shape:
            raise ValueError(f"rank {rank} must hold positions [{p0},{p1}) of {s_total}: Q {tuple(t_[0].shape)}, K {tuple(t_[1].shape)}")
    B, Hq, _, D = Qs[0].shape
    Hkv = Ks[0].shape[1]
    dev = Qs[0].device
    nxt, prv = (rank + 1) % world, (rank - 1) % world
    parts = [[] for _ in mine]             # per local query range: the partial results of the passes that ran
    k_cur, v_cur = list(Ks), list(Vs)
    for t in range(world):
        k_rank = (rank - t) % world
        reqs, k_nxt, v_nxt = [], None, None
        if t + 1 < world:
            k_nxt = [torch.empty((B, Hkv, n1 - n0, D), dtype=Ks[0].dtype, device=dev) for n0, n1 in ranges_of((rank - t - 1) % world)]
            v_nxt = [torch.empty_like(x) for x in k_nxt]
            ops_ = []
            # bit patterns travel as bytes (every backend moves uint8); empty shards are not sent
            for x in k_cur + v_cur:
                if x.numel() > 0:
                    ops_.append(dist.P2POp(dist.isend, x.view(torch.uint8), nxt, group))
            for x in k_nxt + v_nxt:
                if x.numel() > 0:
                    ops_.append(dist.P2POp(dist.irecv, x.view(torch.uint8), prv, group))
            if ops_:
                reqs = dist.batch_isend_irecv(ops_)
        for qi, kj, kv_pos0, total_arg, run in ring_passes(mine, ranges_of(k_rank), causal, s_total):
            if run:
                parts[qi].append(partial_fn(Qs[qi], k_cur[kj], v_cur[kj], scale, causal, kv_pos0, total_arg))
        for r in reqs:
            r.wait()
        if k_nxt is not None:
            k_cur, v_cur = k_nxt, v_nxt
    outs = []
    for qi, (p0, p1) in enumerate(mine):
        if p1 == p0:
            outs.append((torch.empty((B, Hq, 0, D), dtype=torch.bfloat16, device=dev), torch.empty((B, Hq, 0), dtype=torch.float32, device=dev)))
            continue
        if not parts[qi]:       # cannot happen with whole sequences (the diagonal pass always runs); kept for odd inputs
            parts[qi].append(empty_partial(B * Hq * (p1 - p0), D, dev))
        outs.append(combine_fn(torch.stack(parts[qi]), (B, Hq, p1 - p0, D)))
    return outs


def attn_ring(Q_local, K_local, V_local, scale: float, causal: bool, s_total: int, world: int, rank: int, group=None,
              partial_fn=None, combine_fn=None):
    """Ring attention: queries, keys and values of a sequence of ``s_total`` positions are all sharded over the ranks
    (rank r holds positions ``kv_shard_range(s_total, world, r)`` of Q [B,Hq,S_r,D] and of K / V [B,Hkv,S_r,D]).
    In step t a rank runs the KV-shard pass of its queries over the shard of rank (r - t) mod world while that shard
    travels on to rank r + 1 and the next one arrives from rank r - 1 (point-to-point, posted before the pass is
    launched, awaited after it); the partial results are merged by the state combine (the reference's
    CombineSoftmaxStateF32, include/axp/level3/recipes/attention/process.hpp:107-164, across ranks).  Returns
    (O [B,Hq,S_r,D] bf16, LSE [B,Hq,S_r]) for the local queries.

    Under the causal mask the passes over shards that lie in the future of the local queries are skipped, so rank r
    does r + 1 passes: the work is not balanced across the ring; ``attn_ring_zigzag`` balances it.

    ``partial_fn`` / ``combine_fn`` default to the CUDA entry points, as in ``attn_kv_sharded``."""
    return _ring([Q_local], [K_local], [V_local], lambda r: [kv_shard_range(s_total, world, r)], scale, causal, s_total, world, rank,
                 group, partial_fn, combine_fn)[0]


def attn_ring_zigzag(Qs, Ks, Vs, scale: float, causal: bool, s_total: int, world: int, rank: int, group=None, partial_fn=None,
                     combine_fn=None):
    """Ring attention with the zig-zag assignment of positions: rank r holds the two ranges ``zigzag_ranges(s_total,
    world, r)`` (an early and a late chunk of the sequence) as two contiguous tensors each of Q, K and V
    (``Qs = (Q_early, Q_late)`` ...).  A ring step runs up to four KV-shard passes (each local query chunk against each
    chunk of the shard in hand; under the causal mask the ones in the future are skipped), so every rank does about the
    same work.  Returns ``[(O_early, LSE_early), (O_late, LSE_late)]``."""
    if len(Qs) != 2 or len(Ks) != 2 or len(Vs) != 2:
        raise ValueError("zig-zag ring attention takes the early and the late chunk: two tensors each of Q, K and V")
    return _ring(list(Qs), list(Ks), list(Vs), lambda r: zigzag_ranges(s_total, world, r), scale, causal, s_total, world, rank, group,
                 partial_fn, combine_fn)


def empty_partial(rows: int, D: int, device):
    """Partial result of a KV share with no key, in the byte layout of ``axp_sm100_attn_fwd_bf16_kvshard``:
    ``rows * D`` fp32 accumulators, then ``rows`` pairs (m, l) = (-inf, 0)."""
    import torch

    part = torch.zeros(rows * (D * 4 + 8), dtype=torch.uint8, device=device)
    ml = part[rows * D * 4:].view(torch.float32).view(rows, 2)
    ml[:, 0] = float("-inf")
    return part
