#!/usr/bin/env python
"""Benchmark of the sm100 GEMM / attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

Default workload (the one the headline metric is quoted on): FP8 E4M3 block-scaled
GEMM, M=N=K=8192 per GPU, seeded synthetic inputs.  One "step" is one pass of the
GEMM over one set of operands resident in HBM.  With N > 1 (launched by
torch.distributed.run, one rank per GPU) the output columns are sharded: every
rank owns an 8192-column shard of a global N = 8192*N problem (weak scaling), A
is replicated, there is no data-path collective.

The default run also times, in the same process, the other workloads of the metric as sub-records under "workloads"
(bf16 gate/up and down GEMMs, bf16 causal attention, FP8 GQA attention; with N > 1 the attention problems and one
8192^3 FP8 GEMM are SPLIT over the ranks, and "gather" times the NCCL all-gather of the GEMM's column shards), a loop
of at least two seconds ("sustained") and one library E4M3 GEMM as a reference point ("library_reference").

Other workloads (--workload): gemm_fp8_strong, gemm_bf16_gate_up, gemm_bf16_down, gemm_bf16_swiglu, gemm_fp8_swiglu,
gemm_fp8_swiglu_quant (quantising epilogue) / gemm_fp8_swiglu_then_quant (the same result from two kernels), mlp_fp8 (RMSNorm +
quantiser, gate / up, down: one MLP block in three launches),
attn_bf16, attn_fp8, quantize_fp8, rmsnorm_quantize_fp8, attn_decode_bf16, attn_decode_fp8; attn_ring / attn_ring_zigzag (two or more GPUs:
ring attention over one sequence sharded by position, device timing only).

`--impl reference` times the CPU host oracle (the reference library has no
runnable implementation of this path) on the box's host cores, on a bounded row
sample of the same workload.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "FP8 GEMM & attn-fwd TFLOP/s per B200 (% of dense peak) at 1/2/4/8 GPUs"
NOMINAL_TFLOPS = {"e4m3": 4500.0, "bf16": 2250.0}
NVLINK_PEER_GBS = 770.0      # measured peer copy per direction on this pool (nominal 900)
# workloads the default run adds beside the headline one, as sub-records under "workloads"
EXTRA_WORKLOADS = ("gemm_bf16_gate_up", "gemm_bf16_down", "attn_bf16", "attn_fp8")
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of each workload's kernel, from the Nsight Compute
# captures summarised in profiles/*.md (same shapes as the bench; not measured by this script)
NCU_DRAM_BYTES_PER_LAUNCH = {
    "gemm_fp8": 353258240,            # profiles/gemm_fp8_blockscaled_cfg1.md
    "gemm_bf16_gate_up": 1217100032,  # profiles/gemm_bf16_cfg2.md
    "gemm_bf16_down": None,
    "gemm_bf16_swiglu": 3469975296,   # profiles/gemm_bf16_swiglu_cfg2.md
    "gemm_fp8_swiglu": 1463129440,    # profiles/gemm_fp8_swiglu_cfg2.md
    "attn_bf16": 1060898304,          # profiles/attn_fwd_bf16_cfg3.md
    "attn_fp8": 830753024,            # profiles/attn_fwd_fp8_cfg4.md
    "attn_decode_bf16": 1080453336,   # profiles/attn_decode_splitkv.md (decode kernel; the combine kernel moves < 1 MB)
    "attn_decode_fp8": 541634560,     # profiles/attn_decode_fp8_splitkv.md
    "rmsnorm_quantize_fp8": 376897024,  # profiles/rmsnorm_quantize_rows_e4m3.md
    "quantize_fp8": 379043072,        # profiles/quantize_rows_e4m3.md (part of the 138 MB written was still in L2 at kernel end)
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_burst": d["bf16_tflops"], "bf16_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_burst": 1590.0, "bf16_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------- workloads ----
class Workload:
    """A hot-path workload: device operands (two rotating sets, so that consecutive
    steps never find their inputs in L2), the launch, its flops and its CPU sample."""

    name = ""
    dtype = ""
    flops = 0.0          # algorithmic work per step of THIS rank: flops (tensor-bound workloads) or bytes (HBM-bound ones)
    bound = "tensor"
    scaling = "weak"     # "weak": every rank runs the named shape; "strong": the named shape is split over the ranks
    job_flops = None     # strong scaling: the work of the whole job per step (the named shape)

    def __init__(self, pkg, dev, rank, world):
        self.pkg, self.dev, self.rank, self.world = pkg, dev, rank, world

    def total_work(self):
        """Work of all ranks per step."""
        return self.job_flops if self.scaling == "strong" else self.flops * self.world

    def step(self, i):  # device-resident pass
        raise NotImplementedError

    def e2e_spec(self):  # (launch(dev_inputs, dev_outputs), example device inputs, example device outputs)
        raise NotImplementedError


class GemmFp8(Workload):
    name = "cfg1: FP8 E4M3 block-scaled GEMM M=N=K=8192 per GPU (1x128 A scales, 128x128 B scales, bf16 out)"
    dtype = "e4m3"
    M = N = K = 8192
    replicated_inputs = (0, 2)     # A and sA are the same on every rank (e2e: uploaded once, broadcast over NVLink)

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        self.flops = 2.0 * self.M * self.N * self.K
        self.bytes_min = self.M * self.K + self.N * self.K + 2 * self.M * self.N + 4 * (self.M + self.N // 128) * (self.K // 128)
        self.sets = []
        for s in range(sets):
            # A / sA replicated (same seed on every rank); B / sB: this rank's column shard of the global problem
            A, _, sA, _ = pkg.synth.fp8_gemm_inputs(self.M, 128, self.K, seed=s, device=dev)
            _, B, _, sB = pkg.synth.fp8_gemm_inputs(128, self.N, self.K, seed=1000 + 97 * s + rank, device=dev)
            C = torch.empty((self.M, self.N), dtype=torch.bfloat16, device=dev)
            self.sets.append((A, B, sA, sB, C))
        self.host = None

    def step(self, i):
        A, B, sA, sB, C = self.sets[i % len(self.sets)]
        self.pkg.ops.gemm_fp8_blockscaled(A, B, sA, sB, out=C)

    def e2e_spec(self):
        import torch

        A, B, sA, sB, C = self.sets[0]
        dev_in = [A.view(torch.uint8), B.view(torch.uint8), sA, sB]
        return (lambda i, o: self.pkg.ops.gemm_fp8_blockscaled(i[0], i[1], i[2], i[3], out=o[0])), dev_in, [C]

    def cpu_sample(self, oracle, rows):
        """Oracle on `rows` rows of the workload (all N columns, full K); returns flops done."""
        import numpy as np
        import torch

        A, B, sA, sB, _ = self.sets[0]
        a = A[:rows].view(torch.uint8).cpu().numpy()
        b = B.view(torch.uint8).cpu().numpy()
        sa, sb = sA[:rows].cpu().numpy(), sB.cpu().numpy()
        out = np.zeros((rows, self.N), dtype=np.uint16)
        return (lambda: oracle.gemm_fp8_blockscaled(a, b, sa, sb, out=out)), 2.0 * rows * self.N * self.K


class GemmFp8Strong(Workload):
    """cfg1 as the benchmark configuration words it for N GPUs: ONE 8192^3 problem whose output columns are split over the ranks
    (boundaries at multiples of 256); A and sA replicated, no collective unless the full C is asked for."""
    dtype = "e4m3"
    scaling = "strong"
    M = N = K = 8192

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        self.n0, self.n1 = pkg.shard.gemm_column_range(self.N, world, rank)
        w = self.n1 - self.n0
        self.name = f"cfg1 strong: ONE FP8 E4M3 block-scaled GEMM M=N=K=8192 split by output columns over {world} GPUs ({w} columns on this rank)"
        self.job_flops = 2.0 * self.M * self.N * self.K
        self.flops = 2.0 * self.M * w * self.K
        self.bytes_min = self.M * self.K + w * self.K + 2 * self.M * w
        self.sets = []
        for s in range(sets):
            A, B, sA, sB = pkg.synth.fp8_gemm_inputs(self.M, self.N, self.K, seed=s, device=dev)      # same seed on every rank
            Bl, sBl = B[self.n0:self.n1].contiguous(), sB[self.n0 // 128:(self.n1 + 127) // 128].contiguous()
            del B, sB
            self.sets.append((A, Bl, sA, sBl, torch.empty((self.M, w), dtype=torch.bfloat16, device=dev)))

    def step(self, i):
        A, B, sA, sB, C = self.sets[i % len(self.sets)]
        self.pkg.ops.gemm_fp8_blockscaled(A, B, sA, sB, out=C)        # the shard is a GEMM of its own: B rows = its columns

    def e2e_spec(self):
        import torch

        A, B, sA, sB, C = self.sets[0]
        dev_in = [A.view(torch.uint8), B.view(torch.uint8), sA, sB]
        return (lambda i, o: self.pkg.ops.gemm_fp8_blockscaled(i[0], i[1], i[2], i[3], out=o[0])), dev_in, [C]

    replicated_inputs = (0, 2)


class GemmBf16(Workload):
    dtype = "bf16"

    def __init__(self, pkg, dev, rank, world, M, N, K, label, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        self.M, self.N, self.K = M, N, K
        self.name = f"cfg2 {label}: BF16 GEMM M={M} N={N} K={K} per GPU (Llama-3-8B MLP, 16384 tokens)"
        self.flops = 2.0 * M * N * K
        self.bytes_min = 2 * (M * K + N * K + M * N)
        self.sets = []
        for s in range(sets):
            X, _ = pkg.synth.bf16_gemm_inputs(M, 8, K, seed=s, device=dev)
            _, W = pkg.synth.bf16_gemm_inputs(8, N, K, seed=1000 + 97 * s + rank, device=dev)
            self.sets.append((X, W, torch.empty((M, N), dtype=torch.bfloat16, device=dev)))

    def step(self, i):
        X, W, Y = self.sets[i % len(self.sets)]
        self.pkg.ops.gemm_bf16(X, W, out=Y)

    def e2e_spec(self):
        X, W, Y = self.sets[0]
        return (lambda i, o: self.pkg.ops.gemm_bf16(i[0], i[1], out=o[0])), [X, W], [Y]

    def cpu_sample(self, oracle, rows):
        import numpy as np
        import torch

        X, W, _ = self.sets[0]
        x = X[:rows].view(torch.uint16).cpu().numpy()
        w = W.view(torch.uint16).cpu().numpy()
        out = np.zeros((rows, self.N), dtype=np.uint16)
        return (lambda: oracle.gemm_bf16(x, w, out=out)), 2.0 * rows * self.N * self.K


class GemmBf16SwiGLU(Workload):
    """Llama-3-8B MLP gate and up projections in one pass: H = SiLU(X.Wg^T) * (X.Wu^T); the two [M, N] products
    stay in tensor memory, only H is written."""
    dtype = "bf16"
    M, N, K = 16384, 14336, 4096

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        M, N, K = self.M, self.N, self.K
        self.name = f"cfg2 gate+up fused: BF16 GEMM pair + SiLU*mul, M={M} N={N} K={K} per GPU (flops 2*M*2N*K)"
        self.flops = 2.0 * M * 2 * N * K
        self.bytes_min = 2 * (M * K + 2 * N * K + M * N)
        self.sets = []
        for s in range(sets):
            X, _ = pkg.synth.bf16_gemm_inputs(M, 8, K, seed=s, device=dev)
            _, Wg = pkg.synth.bf16_gemm_inputs(8, N, K, seed=1000 + 97 * s + rank, device=dev)
            _, Wu = pkg.synth.bf16_gemm_inputs(8, N, K, seed=2000 + 97 * s + rank, device=dev)
            self.sets.append((X, Wg, Wu, torch.empty((M, N), dtype=torch.bfloat16, device=dev)))

    def step(self, i):
        X, Wg, Wu, H = self.sets[i % len(self.sets)]
        self.pkg.ops.gemm_bf16_swiglu(X, Wg, Wu, out=H)

    def e2e_spec(self):
        X, Wg, Wu, H = self.sets[0]
        return (lambda i, o: self.pkg.ops.gemm_bf16_swiglu(i[0], i[1], i[2], out=o[0])), [X, Wg, Wu], [H]

    def cpu_sample(self, oracle, rows):
        import torch

        X, Wg, Wu, _ = self.sets[0]
        rows = max(1, rows // 2)
        x = X[:rows].view(torch.uint16).cpu().numpy()
        wg, wu = Wg.view(torch.uint16).cpu().numpy(), Wu.view(torch.uint16).cpu().numpy()
        return (lambda: oracle.gemm_bf16_swiglu(x, wg, wu)), 2.0 * rows * 2 * self.N * self.K


class GemmFp8SwiGLU(Workload):
    """The same gate / up pass on E4M3 block-scaled operands (1x128 activation scales, 128x128 weight scales)."""
    dtype = "e4m3"
    M, N, K = 16384, 14336, 4096

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        M, N, K = self.M, self.N, self.K
        self.name = f"cfg2 gate+up fused, FP8: block-scaled E4M3 GEMM pair + SiLU*mul, M={M} N={N} K={K} per GPU (flops 2*M*2N*K)"
        self.flops = 2.0 * M * 2 * N * K
        self.bytes_min = M * K + 2 * N * K + 2 * M * N
        self.sets = []
        for s in range(sets):
            X, Wg, sX, sWg = pkg.synth.fp8_gemm_inputs(M, N, K, seed=3000 + 97 * s + rank, device=dev)
            _, Wu, _, sWu = pkg.synth.fp8_gemm_inputs(8, N, K, seed=4000 + 97 * s + rank, device=dev)
            self.sets.append((X, Wg, Wu, sX * 0.03125, sWg, sWu, torch.empty((M, N), dtype=torch.bfloat16, device=dev)))

    def step(self, i):
        s = self.sets[i % len(self.sets)]
        self.pkg.ops.gemm_fp8_blockscaled_swiglu(*s[:6], out=s[6])

    def e2e_spec(self):
        s = self.sets[0]
        return (lambda i, o: self.pkg.ops.gemm_fp8_blockscaled_swiglu(*i, out=o[0])), list(s[:6]), [s[6]]

    def cpu_sample(self, oracle, rows):
        import torch

        X, Wg, Wu, sX, sWg, sWu, _ = self.sets[0]
        rows = max(1, rows // 2)
        x, wg, wu = X[:rows].view(torch.uint8).cpu().numpy(), Wg.view(torch.uint8).cpu().numpy(), Wu.view(torch.uint8).cpu().numpy()
        sx, sg, su = sX[:rows].cpu().numpy(), sWg.cpu().numpy(), sWu.cpu().numpy()
        return (lambda: oracle.gemm_fp8_blockscaled_swiglu(x, wg, wu, sx, sg, su)), 2.0 * rows * 2 * self.N * self.K


class GemmFp8SwiGLUQuant(GemmFp8SwiGLU):
    """The FP8 gate / up pass with the quantising epilogue: H leaves as E4M3 + 1x128 scales (the down projection's A operand),
    `--two-kernels` semantics for comparison: the plain pass followed by the stand-alone quantiser (option below)."""

    def __init__(self, pkg, dev, rank, world, fused=True, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world, sets)
        self.fused = fused
        M, N = self.M, self.N
        self.name = (f"cfg2 gate+up fused, FP8, E4M3 + 1x128 scales out ({'quantising epilogue' if fused else 'two kernels: bf16 H, then the quantiser'}), "
                     f"M={M} N={N} K={self.K} per GPU (flops 2*M*2N*K)")
        self.launches_per_step = 1 if fused else 2
        self.q = [(torch.empty((M, N), dtype=torch.float8_e4m3fn, device=dev), torch.empty((M, N // 128), dtype=torch.float32, device=dev))
                  for _ in range(sets)]

    def step(self, i):
        s, (Q, S) = self.sets[i % len(self.sets)], self.q[i % len(self.q)]
        if self.fused:
            self.pkg.ops.gemm_fp8_blockscaled_swiglu_quant(*s[:6], out=Q, scales=S)
        else:
            self.pkg.ops.gemm_fp8_blockscaled_swiglu(*s[:6], out=s[6])
            self.pkg.ops.quantize_rows_e4m3(s[6], out=Q, scales=S)

    def e2e_spec(self):
        s, (Q, S) = self.sets[0], self.q[0]
        return (lambda i, o: self.pkg.ops.gemm_fp8_blockscaled_swiglu_quant(*i, out=o[0], scales=o[1])), list(s[:6]), [Q, S]


class MlpFp8(Workload):
    """One Llama-3-8B MLP block at 16384 tokens on E4M3 block-scaled weights: RMSNorm + quantiser, gate / up GEMM with the
    quantising epilogue, down GEMM - three launches, no bf16 intermediate in HBM.  Flops: the three projections."""
    dtype = "e4m3"
    M, K, N = 16384, 4096, 14336
    launches_per_step = 3
    no_host_arms = "a chain of three launches on device-resident weights: device timing only"

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        M, K, N = self.M, self.K, self.N
        self.name = f"FP8 MLP block: RMSNorm+quantise -> gate/up (SwiGLU, quantising epilogue) -> down, M={M} hidden={K} intermediate={N} per GPU"
        self.flops = 3 * 2.0 * M * N * K
        self.bytes_min = 2 * M * K * 2 + 3 * N * K
        _, Wg, _, sWg = pkg.synth.fp8_gemm_inputs(8, N, K, seed=5000 + rank, device=dev)
        _, Wu, _, sWu = pkg.synth.fp8_gemm_inputs(8, N, K, seed=5100 + rank, device=dev)
        _, Wd, _, sWd = pkg.synth.fp8_gemm_inputs(8, K, N, seed=5200 + rank, device=dev)
        self.w = (Wg, Wu, Wd, sWg * 0.05, sWu * 0.05, sWd * 0.05)
        g = torch.Generator(device=dev).manual_seed(77 + rank)
        self.wn = (1.0 + 0.1 * torch.randn(K, generator=g, device=dev)).to(torch.bfloat16)
        self.sets = []
        for s in range(sets):
            X = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
            ws = (torch.empty((M, K), dtype=torch.float8_e4m3fn, device=dev), torch.empty((M, K // 128), dtype=torch.float32, device=dev),
                  torch.empty((M, N), dtype=torch.float8_e4m3fn, device=dev), torch.empty((M, N // 128), dtype=torch.float32, device=dev))
            self.sets.append((X, ws, torch.empty((M, K), dtype=torch.bfloat16, device=dev)))

    def step(self, i):
        X, ws, Y = self.sets[i % len(self.sets)]
        Wg, Wu, Wd, sWg, sWu, sWd = self.w
        self.pkg.ops.mlp_fp8_forward(X, self.wn, Wg, Wu, Wd, sWg, sWu, sWd, out=Y, workspace=ws)


class AttnBf16(Workload):
    name = "cfg3: flash-attention fwd bf16 causal B=8 H=32 S=4096 D=128 per GPU (causal flops 2*B*H*S^2*D)"
    dtype = "bf16"
    B, H, S, D = 8, 32, 4096, 128

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        # N GPUs: the 256 (batch, head) units of the ONE named problem are split into contiguous ranges, no collective
        self.bh = pkg.shard.attention_head_range(self.B, self.H, self.H, world, rank)
        heads = self.bh[1] - self.bh[0]
        self.job_flops = 0.5 * 4.0 * self.B * self.H * self.S * self.S * self.D
        self.flops = self.job_flops * heads / (self.B * self.H)
        self.bytes_min = (4 * 2 * self.S * self.D + 4 * self.S) * heads
        if world > 1:
            self.scaling = "strong"
            self.name += f" -- split by batch x head over {world} GPUs ({heads} heads on this rank)"
        self.sets = []
        for s in range(sets):
            Q, K, V, self.scale = pkg.synth.bf16_attention_inputs(self.B, self.H, self.S, self.D, seed=s, device=dev)
            self.sets.append((Q, K, V, torch.empty_like(Q), torch.empty((self.B, self.H, self.S), dtype=torch.float32, device=dev)))

    def step(self, i):
        Q, K, V, O, L = self.sets[i % len(self.sets)]
        self.pkg.ops.attn_fwd_bf16(Q, K, V, self.scale, True, out=O, lse=L, bh_range=self.bh)

    def e2e_spec(self):
        Q, K, V, O, L = self.sets[0]
        return (lambda i, o: self.pkg.ops.attn_fwd_bf16(i[0], i[1], i[2], self.scale, True, out=o[0], lse=o[1])), \
            [Q, K, V], [O, L]

    def cpu_sample(self, oracle, rows):
        import torch

        Q, K, V, _, _ = self.sets[0]
        heads = max(1, min(self.B * self.H, rows // 64))     # `rows` scales the sample: whole heads
        b = (heads + self.H - 1) // self.H
        q, k, v = (t[:b].view(torch.uint16).cpu().numpy() for t in (Q, K, V))
        return (lambda: oracle.attn_fwd_bf16(q, k, v, self.scale, True, bh_range=(0, heads))), \
            0.5 * 4.0 * heads * self.S * self.S * self.D


class AttnFp8(Workload):
    name = "cfg4: FP8 attention fwd GQA causal B=4 Hq=64 Hkv=8 S=8192 D=128 per GPU (causal flops)"
    dtype = "e4m3"
    B, Hq, Hkv, S, D = 4, 64, 8, 8192, 128

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        # N GPUs: the 32 (batch, KV-head group) units of the ONE named problem are split, whole groups per rank
        self.bh = pkg.shard.attention_head_range(self.B, self.Hq, self.Hkv, world, rank)
        heads = self.bh[1] - self.bh[0]
        self.job_flops = 0.5 * 4.0 * self.B * self.Hq * self.S * self.S * self.D
        self.flops = self.job_flops * heads / (self.B * self.Hq)
        self.bytes_min = self.S * self.D * (3 * heads + 2 * heads * self.Hkv // self.Hq)
        if world > 1:
            self.scaling = "strong"
            self.name += f" -- split by batch x KV-head group over {world} GPUs ({heads} query heads on this rank)"
        self.sets = []
        for s in range(sets):
            Q, K, V, dq, dk, dv, self.scale = pkg.synth.fp8_attention_inputs(self.B, self.Hq, self.Hkv, self.S, self.D,
                                                                             seed=s, device=dev)
            O = torch.empty((self.B, self.Hq, self.S, self.D), dtype=torch.bfloat16, device=dev)
            L = torch.empty((self.B, self.Hq, self.S), dtype=torch.float32, device=dev)
            self.sets.append((Q, K, V, dq, dk, dv, O, L))

    def step(self, i):
        Q, K, V, dq, dk, dv, O, L = self.sets[i % len(self.sets)]
        self.pkg.ops.attn_fwd_fp8(Q, K, V, dq, dk, dv, self.scale, True, out=O, lse=L, bh_range=self.bh)

    def e2e_spec(self):
        import torch

        Q, K, V, dq, dk, dv, O, L = self.sets[0]
        dev_in = [Q.view(torch.uint8), K.view(torch.uint8), V.view(torch.uint8), dq, dk, dv]
        return (lambda i, o: self.pkg.ops.attn_fwd_fp8(i[0], i[1], i[2], i[3], i[4], i[5], self.scale, True,
                                                       out=o[0], lse=o[1])), dev_in, [O, L]

    def cpu_sample(self, oracle, rows):
        import torch

        Q, K, V, dq, dk, dv, _, _ = self.sets[0]
        heads = max(1, min(self.Hq, rows // 256))
        q, k, v = (t[:1].view(torch.uint8).cpu().numpy() for t in (Q, K, V))
        a, b, c = dq[: self.Hq].cpu().numpy(), dk[: self.Hkv].cpu().numpy(), dv[: self.Hkv].cpu().numpy()
        return (lambda: oracle.attn_fwd_fp8(q, k, v, a, b, c, self.scale, True, bh_range=(0, heads))), \
            0.5 * 4.0 * heads * self.S * self.S * self.D


class QuantFp8(Workload):
    """HBM-bound producer of the FP8 GEMM's A operand: bf16 [M,K] -> E4M3 [M,K] + fp32 scales [M,K/128]."""
    name = "quantize: bf16 activations [16384, 8192] -> E4M3 + 1x128 fp32 scales per GPU (producer of cfg1's A operand)"
    metric = "FP8 activation quantisation (bf16 -> E4M3 + 1x128 scales) GB/s per B200"
    dtype = "bf16"
    bound = "hbm"
    M, K = 16384, 8192

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        self.bytes_min = self.M * self.K * 3 + 4 * self.M * (self.K // 128)   # 2 B read + 1 B written per element + scales
        self.flops = float(self.bytes_min)                                      # "work" of this workload is bytes
        self.sets = []
        for s in range(sets):
            X, _ = pkg.synth.bf16_gemm_inputs(self.M, 8, self.K, seed=7 * s + rank, device=dev)
            self.sets.append((X, torch.empty((self.M, self.K), dtype=torch.float8_e4m3fn, device=dev),
                              torch.empty((self.M, self.K // 128), dtype=torch.float32, device=dev)))

    def step(self, i):
        X, Q, S = self.sets[i % len(self.sets)]
        self.pkg.ops.quantize_rows_e4m3(X, out=Q, scales=S)

    def e2e_spec(self):
        import torch

        X, Q, S = self.sets[0]
        return (lambda i, o: self.pkg.ops.quantize_rows_e4m3(i[0], out=o[0].view(torch.float8_e4m3fn), scales=o[1])), \
            [X], [Q.view(torch.uint8), S]

    def cpu_sample(self, oracle, rows):
        import torch

        X, _, _ = self.sets[0]
        rows = max(64, min(self.M, rows * 8))
        x = X[:rows].view(torch.uint16).cpu().numpy()
        return (lambda: oracle.quantize_rows_e4m3(x)), float(rows * self.K * 3 + 4 * rows * (self.K // 128))


class RmsNormQuantFp8(QuantFp8):
    """HBM-bound fused producer: RMSNorm(x) * w -> E4M3 + 1x128 scales, the normalised activations never written."""
    name = "rmsnorm+quantize: bf16 activations [16384, 8192] -> RMSNorm * w -> E4M3 + 1x128 fp32 scales per GPU"
    metric = "RMSNorm + FP8 activation quantisation GB/s per B200 (algorithmic bytes: 2 read + 1 written per element)"

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world, sets)
        self.w = (1.0 + 0.1 * torch.randn(self.K, device=dev)).bfloat16()

    def step(self, i):
        X, Q, S = self.sets[i % len(self.sets)]
        self.pkg.ops.rmsnorm_quantize_rows_e4m3(X, self.w, 1e-5, out=Q, scales=S)

    def e2e_spec(self):
        import torch

        X, Q, S = self.sets[0]
        return (lambda i, o: self.pkg.ops.rmsnorm_quantize_rows_e4m3(i[0], self.w, 1e-5, out=o[0].view(torch.float8_e4m3fn), scales=o[1])), \
            [X], [Q.view(torch.uint8), S]

    def cpu_sample(self, oracle, rows):
        import torch

        X, _, _ = self.sets[0]
        rows = max(64, min(self.M, rows * 8))
        x = X[:rows].view(torch.uint16).cpu().numpy()
        w = self.w.view(torch.uint16).cpu().numpy()
        return (lambda: oracle.rmsnorm_quantize_rows_e4m3(x, w, 1e-5)), float(rows * self.K * 3 + 4 * rows * (self.K // 128))


class AttnDecodeBf16(Workload):
    """HBM-bound decode step: one new query per head against a long KV cache, keys split into shares that run as
    independent CTAs and are combined through scratch memory (split-KV)."""
    name = "decode: bf16 attention, 1 query per head, B=16 Hq=32 Hkv=8 Skv=16384 D=128 per GPU, split-KV x8 (KV cache read once)"
    metric = "decode attention: KV-cache GB/s per B200 (algorithmic bytes = K and V read once)"
    dtype = "bf16"
    bound = "hbm"
    launches_per_step = 2      # the pass over the KV shares and the combine kernel
    B, Hq, Hkv, Sq, Skv, D, SPLITS = 16, 32, 8, 1, 16384, 128, 8

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        self.bytes_min = 2 * 2 * self.B * self.Hkv * self.Skv * self.D + 2 * 2 * self.B * self.Hq * self.Sq * self.D
        self.flops = float(self.bytes_min)
        self.scratch = torch.empty(pkg.ops.attn_splitkv_scratch_bytes(self.B * self.Hq, self.Sq, self.SPLITS), dtype=torch.uint8, device=dev)
        self.sets = []
        for s in range(sets):
            Q, _, _, self.scale = pkg.synth.bf16_attention_inputs(self.B, self.Hq, self.Sq, self.D, seed=100 * rank + s, Hkv=self.Hkv, device=dev)
            _, K, V, _ = pkg.synth.bf16_attention_inputs(self.B, self.Hkv, self.Skv, self.D, seed=100 * rank + s + 50, device=dev)
            self.sets.append((Q, K, V, torch.empty_like(Q), torch.empty((self.B, self.Hq, self.Sq), dtype=torch.float32, device=dev)))

    def step(self, i):
        Q, K, V, O, L = self.sets[i % len(self.sets)]
        self.pkg.ops.attn_fwd_bf16_splitkv(Q, K, V, self.scale, True, num_splits=self.SPLITS, scratch=self.scratch, out=O, lse=L)

    def e2e_spec(self):
        # the KV cache lives on the device; a decode step moves the new queries in and the outputs back
        Q, K, V, O, L = self.sets[0]
        return (lambda i, o: self.pkg.ops.attn_fwd_bf16_splitkv(i[0], K, V, self.scale, True, num_splits=self.SPLITS,
                                                                scratch=self.scratch, out=o[0], lse=o[1])), [Q], [O, L]

    def cpu_sample(self, oracle, rows):
        import torch

        Q, K, V, _, _ = self.sets[0]
        b = 1
        q, k, v = (t[:b].view(torch.uint16).cpu().numpy() for t in (Q, K, V))
        return (lambda: oracle.attn_fwd_bf16_qkv(q, k, v, self.scale, True)), float(self.bytes_min) * b / self.B


class AttnDecodeFp8(Workload):
    """The same decode step on an E4M3 KV cache (half the bytes per key); the query heads of a GQA group share one
    pass over their K / V."""
    name = "decode: E4M3 attention, 1 query per head, B=16 Hq=32 Hkv=8 Skv=16384 D=128 per GPU, split-KV x2 (KV cache read once)"
    metric = "decode attention: KV-cache GB/s per B200 (algorithmic bytes = K and V read once)"
    dtype = "e4m3"
    bound = "hbm"
    launches_per_step = 2      # the pass over the KV shares and the combine kernel
    B, Hq, Hkv, Sq, Skv, D, SPLITS = 16, 32, 8, 1, 16384, 128, 2

    def __init__(self, pkg, dev, rank, world, sets=2):
        import torch

        super().__init__(pkg, dev, rank, world)
        self.bytes_min = 2 * self.B * self.Hkv * self.Skv * self.D + (1 + 2) * self.B * self.Hq * self.Sq * self.D
        self.flops = float(self.bytes_min)
        self.scratch = torch.empty(pkg.ops.attn_splitkv_scratch_bytes(self.B * self.Hq, self.Sq, self.SPLITS), dtype=torch.uint8, device=dev)
        self.sets = []
        for s in range(sets):
            Q, _, _, dq, _, _, self.scale = pkg.synth.fp8_attention_inputs(self.B, self.Hq, self.Hkv, self.Sq, self.D, seed=100 * rank + s, device=dev)
            _, K, V, _, dk, dv, _ = pkg.synth.fp8_attention_inputs(self.B, self.Hkv, self.Hkv, self.Skv, self.D, seed=100 * rank + s + 50, device=dev)
            self.sets.append((Q, K, V, dq, dk, dv, torch.empty((self.B, self.Hq, self.Sq, self.D), dtype=torch.bfloat16, device=dev),
                              torch.empty((self.B, self.Hq, self.Sq), dtype=torch.float32, device=dev)))

    def step(self, i):
        Q, K, V, dq, dk, dv, O, L = self.sets[i % len(self.sets)]
        self.pkg.ops.attn_fwd_fp8_splitkv(Q, K, V, dq, dk, dv, self.scale, True, num_splits=self.SPLITS, scratch=self.scratch, out=O, lse=L)

    def e2e_spec(self):
        Q, K, V, dq, dk, dv, O, L = self.sets[0]
        return (lambda i, o: self.pkg.ops.attn_fwd_fp8_splitkv(i[0], K, V, dq, dk, dv, self.scale, True, num_splits=self.SPLITS,
                                                               scratch=self.scratch, out=o[0], lse=o[1])), [Q], [O, L]

    def cpu_sample(self, oracle, rows):
        import numpy as np
        import torch

        Q, K, V, dq, dk, dv, _, _ = self.sets[0]
        # the host oracle takes equal query and key lengths: the decode query is its last position
        k, v = K[:1].view(torch.uint8).cpu().numpy(), V[:1].view(torch.uint8).cpu().numpy()
        q = np.zeros((1, self.Hq, self.Skv, self.D), dtype=np.uint8)
        q[:, :, -1:] = Q[:1].view(torch.uint8).cpu().numpy()
        a, b, c = dq[:self.Hq].cpu().numpy(), dk[:self.Hkv].cpu().numpy(), dv[:self.Hkv].cpu().numpy()
        return (lambda: oracle.attn_fwd_fp8(q, k, v, a, b, c, self.scale, True, q_range=(self.Skv - 1, self.Skv))), float(self.bytes_min) / self.B


class AttnRing(Workload):
    """Ring attention over the GPUs of the box (opt-in: --workload attn_ring with --gpus >= 2): ONE causal sequence of
    8192 positions per GPU, queries and keys sharded by position, K / V shards passed round by NCCL point-to-point sends
    while the pass over the shard in hand runs.  Under the causal mask rank r runs r + 1 of the N passes, so the last
    rank sets the time: the figure shows what the unbalanced ring delivers, not a balanced one."""
    dtype = "bf16"
    scaling = "strong"
    no_host_arms = "the shards live on the GPUs of a sequence-parallel job: no host-buffer arm and no CPU sample for this workload"
    sharding_note = ("one sequence sharded by position (queries, keys and values alike); per call every rank sends its K / V shard once round the "
                     "ring (NCCL point-to-point) and merges one partial result per shard; causal: rank r runs r + 1 of the N passes")
    B, Hq, Hkv, D, S_PER_GPU = 1, 32, 8, 128, 8192

    def __init__(self, pkg, dev, rank, world, sets=2):
        super().__init__(pkg, dev, rank, world)
        self.S = self.S_PER_GPU * world
        self.name = (f"ring attention: bf16 causal, B=1 Hq=32 Hkv=8 D=128, ONE sequence of {self.S} positions sharded by position over "
                     f"{world} GPUs (8192 per GPU), K/V shards passed round a ring")
        p0, p1 = pkg.shard.kv_shard_range(self.S, world, rank)
        self.job_flops = 0.5 * 4.0 * self.B * self.Hq * float(self.S) * self.S * self.D
        passes = sum(1 for st in pkg.shard.ring_shard_plan(self.S, world, rank, True) if st[4])
        self.flops = self.job_flops / world      # the job's work per GPU: the ring is not balanced, rank r does (r + 1/2) / (N^2 / 2) of it
        self.bytes_min = 0
        self.launches_per_step = passes + 1
        self.kv_bytes_per_step = 2 * self.B * self.Hkv * self.S_PER_GPU * self.D * 2 * (world - 1)         # sent by this rank per call
        self.sets = []
        for s in range(sets):
            # every rank draws its own shard (the values do not matter for the timing; parity is the tests' business)
            Q, _, _, self.scale = pkg.synth.bf16_attention_inputs(self.B, self.Hq, p1 - p0, self.D, seed=100 * s + rank, Hkv=self.Hkv, device=dev)
            _, K, V, _ = pkg.synth.bf16_attention_inputs(self.B, self.Hkv, p1 - p0, self.D, seed=100 * s + rank + 50, device=dev)
            self.sets.append((Q, K, V))

    def step(self, i):
        Q, K, V = self.sets[i % len(self.sets)]
        self.out = self.pkg.shard.attn_ring(Q, K, V, self.scale, True, self.S, self.world, self.rank)


class AttnRingZigzag(AttnRing):
    """The same sequence with the zig-zag assignment of positions (rank r holds chunks r and 2N - 1 - r of 2N): every
    rank runs about the same number of passes under the causal mask."""

    def __init__(self, pkg, dev, rank, world, sets=2):
        Workload.__init__(self, pkg, dev, rank, world)
        self.S = self.S_PER_GPU * world
        self.name = (f"ring attention, zig-zag positions: bf16 causal, B=1 Hq=32 Hkv=8 D=128, ONE sequence of {self.S} positions over "
                     f"{world} GPUs (two chunks of 4096 per GPU), K/V shards passed round a ring")
        self.sharding_note = AttnRing.sharding_note.replace("causal: rank r runs r + 1 of the N passes",
                                                            "zig-zag chunks r and 2N - 1 - r per rank: the causal passes are balanced")
        self.ranges = pkg.shard.zigzag_ranges(self.S, world, rank)
        self.job_flops = 0.5 * 4.0 * self.B * self.Hq * float(self.S) * self.S * self.D
        self.flops = self.job_flops / world
        self.bytes_min = 0
        passes = sum(1 for t in range(world)
                     for st in pkg.shard.ring_passes(self.ranges, pkg.shard.zigzag_ranges(self.S, world, (rank - t) % world), True, self.S) if st[4])
        self.launches_per_step = passes + 2
        self.kv_bytes_per_step = 2 * self.B * self.Hkv * self.S_PER_GPU * self.D * 2 * (world - 1)
        self.sets = []
        for s in range(sets):
            Qs, Ks, Vs = [], [], []
            for c, (a, b) in enumerate(self.ranges):
                Q, _, _, self.scale = pkg.synth.bf16_attention_inputs(self.B, self.Hq, b - a, self.D, seed=100 * s + 2 * rank + c, Hkv=self.Hkv, device=dev)
                _, K, V, _ = pkg.synth.bf16_attention_inputs(self.B, self.Hkv, b - a, self.D, seed=100 * s + 2 * rank + c + 50, device=dev)
                Qs.append(Q); Ks.append(K); Vs.append(V)
            self.sets.append((Qs, Ks, Vs))

    def step(self, i):
        Qs, Ks, Vs = self.sets[i % len(self.sets)]
        self.out = self.pkg.shard.attn_ring_zigzag(Qs, Ks, Vs, self.scale, True, self.S, self.world, self.rank)


def make_workload(name, pkg, dev, rank, world):
    if name in ("attn_ring", "attn_ring_zigzag"):
        if world < 2:
            raise SystemExit(f"{name} needs --gpus >= 2 (one process per GPU under torchrun)")
        return (AttnRing if name == "attn_ring" else AttnRingZigzag)(pkg, dev, rank, world)
    if name == "gemm_fp8":
        return GemmFp8(pkg, dev, rank, world)
    if name == "gemm_fp8_strong":
        return GemmFp8Strong(pkg, dev, rank, world)
    if name == "gemm_bf16_gate_up":
        return GemmBf16(pkg, dev, rank, world, 16384, 14336, 4096, "gate/up")
    if name == "gemm_bf16_down":
        return GemmBf16(pkg, dev, rank, world, 16384, 4096, 14336, "down")
    if name == "gemm_bf16_swiglu":
        return GemmBf16SwiGLU(pkg, dev, rank, world)
    if name == "gemm_fp8_swiglu":
        return GemmFp8SwiGLU(pkg, dev, rank, world)
    if name == "mlp_fp8":
        return MlpFp8(pkg, dev, rank, world)
    if name in ("gemm_fp8_swiglu_quant", "gemm_fp8_swiglu_then_quant"):
        return GemmFp8SwiGLUQuant(pkg, dev, rank, world, fused=(name == "gemm_fp8_swiglu_quant"))
    if name == "attn_decode_fp8":
        return AttnDecodeFp8(pkg, dev, rank, world)
    if name == "attn_bf16":
        return AttnBf16(pkg, dev, rank, world)
    if name == "attn_fp8":
        return AttnFp8(pkg, dev, rank, world)
    if name == "quantize_fp8":
        return QuantFp8(pkg, dev, rank, world)
    if name == "rmsnorm_quantize_fp8":
        return RmsNormQuantFp8(pkg, dev, rank, world)
    if name == "attn_decode_bf16":
        return AttnDecodeBf16(pkg, dev, rank, world)
    raise SystemExit(f"unknown workload {name}")


# -------------------------------------------------------------------- clocks ----
class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self.stop_flag = index, [], set(), None, False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self.stop_flag:
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.002)

    def result(self):
        s = sorted(self.samples)
        return {"sm_mhz": (s[len(s) // 2] if s else None), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s)}


# --------------------------------------------------------------- CPU baseline ----
def time_cpu(fn, budget_s):
    fn()                                        # warm caches / thread pool
    t0 = time.perf_counter()
    n = 0
    while True:
        fn()
        n += 1
        el = time.perf_counter() - t0
        if el >= budget_s or n >= 50:
            return el / n


def cpu_baseline(wl, budget_s=12.0):
    from oracle import host_oracle

    host_oracle.set_num_threads(host_threads())
    rows = 64
    fn, fl = wl.cpu_sample(host_oracle, rows)
    t = time_cpu(fn, 0.5)
    # scale the sample so that one call lasts about a quarter of the budget
    target_rows = int(rows * max(1.0, (budget_s / 4.0) / max(t, 1e-6)))
    target_rows = max(64, min(getattr(wl, "M", 1 << 20), (target_rows // 64) * 64))
    fn, fl = wl.cpu_sample(host_oracle, target_rows)
    t = time_cpu(fn, budget_s / 2.0)
    hbm = wl.bound == "hbm"
    return {"value": fl / t / (1e9 if hbm else 1e12), "unit": "GB/s" if hbm else "TFLOP/s", "cores": host_oracle.num_threads(),
            "kind": "port",
            "sample": f"host oracle on a {target_rows}-row-equivalent slice of the workload ({fl:.3e} {'bytes' if hbm else 'flop'} per call, {t:.2f} s per call)"}


def config_for(wl, world):
    """The `config` object both arms print (identical keys and wording)."""
    return {"workload": wl.name,
            "sharding": (getattr(wl, "sharding_note", None) or ("single GPU" if world == 1 else
                         "headline workload: every rank runs the named shape on its own output-column shard of a world-times wider problem "
                         "(weak scaling, no data-path collective); attention sub-records split the ONE named problem by heads (strong)")),
            "l2": "two operand sets alternate between steps; each set (>= 130 MB per rank) exceeds the 126 MB L2",
            "timing": "GPU arm: CUDA events on the launch stream, max over ranks; reference arm: host wall clock of the CPU oracle"}


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def run_reference(args, rank):
    """Reference arm: the CPU host oracle with all host threads, bounded sample per step."""
    if rank != 0:
        return
    import torch

    pkg = importlib.import_module("iro-cuda-ax_b200")
    from oracle import host_oracle

    # launchers such as torch.distributed.run export OMP_NUM_THREADS=1: ask for every host core explicitly
    host_oracle.set_num_threads(host_threads())
    dev = torch.device("cpu")
    wl = make_workload(args.workload, pkg, dev, 0, 1) if args.workload != "gemm_fp8" else GemmFp8(pkg, dev, 0, 1, sets=1)
    fn, fl = wl.cpu_sample(host_oracle, 64)
    t = time_cpu(fn, 0.5)
    budget = 150.0 / max(1, args.steps + args.warmup)
    rows = int(64 * max(1.0, budget / max(t, 1e-6)))
    rows = max(64, min(getattr(wl, "M", 1 << 20), (rows // 64) * 64))
    fn, fl = wl.cpu_sample(host_oracle, rows)
    for _ in range(args.warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        fn()
    el = time.perf_counter() - t0
    hbm = wl.bound == "hbm"
    unit = "GB/s" if hbm else "TFLOP/s"
    val = fl * args.steps / el / (1e9 if hbm else 1e12)
    sample = (f"{rows}-row-equivalent slice of the workload per step ({fl:.3e} {'bytes' if hbm else 'flop'}), OpenMP over "
              f"{host_oracle.num_threads()} host threads; the reference library has no runnable implementation of this path, "
              "this arm times the CPU host oracle (a port of the recipe semantics)")
    print(json.dumps({
        "impl": "reference", "metric": getattr(wl, "metric", METRIC), "value": val, "unit": unit, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": el / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": config_for(wl, max(1, args.gpus)),
        "cpu_baseline": {"value": val, "unit": unit, "cores": host_oracle.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


# ------------------------------------------------------------ GPU measurement ----
class Ctx:
    """What the measurement helpers share: device, ranks, the package, peaks."""

    def __init__(self, pkg, dev, rank, local_rank, world, dist, peaks):
        self.pkg, self.dev, self.rank, self.local_rank, self.world, self.dist, self.peaks = pkg, dev, rank, local_rank, world, dist, peaks

    def barrier(self):
        import torch

        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, x):
        import torch

        t = torch.tensor([x], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())


def measure(ctx, wl, steps, warmup):
    """W untimed steps, then K steps between a barrier + synchronize on both sides, CUDA events on the launch stream
    (one per launch as well), clocks sampled during the timed region; time = max over ranks."""
    import torch

    for i in range(warmup):
        wl.step(i)
    ctx.pkg.ops.check_status(ctx.dev)
    ctx.barrier()
    sampler = ClockSampler(ctx.local_rank)
    sampler.start()
    stream = torch.cuda.current_stream()
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
    evs[0].record(stream)
    for i in range(steps):
        wl.step(i)
        evs[i + 1].record(stream)
    ctx.barrier()
    sampler.stop_flag = True
    sampler.join()
    ctx.pkg.ops.check_status(ctx.dev)
    per_launch = sorted(evs[i].elapsed_time(evs[i + 1]) for i in range(steps))
    total_ms = ctx.max_over_ranks(evs[0].elapsed_time(evs[-1]))
    return {"ms_per_step": total_ms / steps, "kernel_ms": sum(per_launch) / len(per_launch), "kernel_ms_min": per_launch[0], "kernel_ms_median": per_launch[len(per_launch) // 2],
            "clocks": sampler.result(), "timed_s": total_ms * 1e-3}


def roofline(ctx, wl, key, m):
    """achieved = this rank's algorithmic work per launch / mean launch time; the tensor peak is the cuBLAS bf16 figure of
    MEASURED_PEAKS.json that matches the length of the timed region: the burst figure under one second, else the sustained one."""
    peaks = ctx.peaks
    hbm = wl.bound == "hbm"
    per = 1e9 if hbm else 1e12
    achieved = wl.flops / (m["kernel_ms"] * 1e-3) / per
    traffic = NCU_DRAM_BYTES_PER_LAUNCH.get(key) if wl.scaling == "weak" or ctx.world == 1 else None
    loud = "" if peaks["source"] == "measured" else "FALLBACK (MEASURED_PEAKS.json is missing): "
    if hbm:
        peak = peaks["hbm_gbs"]
        return {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak, "traffic": traffic,
                "peak_source": f"{loud}{peaks['source']} STREAM-style copy {peak} GB/s", "kernel_ms": m["kernel_ms"],
                "kernel_ms_min": m["kernel_ms_min"], "kernel_ms_median": m["kernel_ms_median"], "hbm_min_bytes": wl.bytes_min}
    burst = m["timed_s"] < 1.0
    bf16_peak = peaks["bf16_burst"] if burst else peaks["bf16_sustained"]
    eight_bit = wl.dtype == "e4m3"
    peak = bf16_peak * (2.0 if eight_bit else 1.0)
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic,
            "peak_kind": "burst" if burst else "sustained",
            "peak_source": (f"{loud}{peaks['source']} cuBLAS bf16 {'burst' if burst else 'sustained'} {bf16_peak} TFLOP/s "
                            f"(timed region {m['timed_s'] * 1e3:.1f} ms {'<' if burst else '>='} 1 s)"
                            + (", x2 for the 8-bit tensor rate: no E4M3 figure is measured there" if eight_bit else "")),
            "frac_of_nominal": achieved / NOMINAL_TFLOPS[wl.dtype], "nominal_peak": NOMINAL_TFLOPS[wl.dtype],
            "kernel_ms": m["kernel_ms"], "kernel_ms_min": m["kernel_ms_min"], "kernel_ms_median": m["kernel_ms_median"], "hbm_min_bytes": wl.bytes_min,
            "hbm_gbs_at_min_bytes": wl.bytes_min / (m["kernel_ms"] * 1e-3) / 1e9}


def sub_record(ctx, wl, key, steps, warmup):
    m = measure(ctx, wl, steps, warmup)
    hbm = wl.bound == "hbm"
    per = 1e9 if hbm else 1e12
    rec = {"workload": wl.name, "value": wl.total_work() / (m["ms_per_step"] * 1e-3) / per, "unit": "GB/s" if hbm else "TFLOP/s",
           "scaling": wl.scaling if ctx.world > 1 else "single GPU", "dtype": wl.dtype, "steps": steps, "ms_per_step": m["ms_per_step"],
           "kernel_ms": m["kernel_ms"], "clocks": m["clocks"], "gpu_launches": steps * getattr(wl, "launches_per_step", 1)}
    if ctx.rank == 0:
        rec["roofline"] = roofline(ctx, wl, key, m)
    return rec, m


def sustained_record(ctx, wl, ms_per_step, seconds=2.0):
    """The same launches back to back for at least `seconds`: what the power cap leaves once the burst is over."""
    steps = max(50, int(seconds * 1e3 / max(ms_per_step, 1e-3)) + 1)
    m = measure(ctx, wl, steps, 0)
    val = wl.total_work() / (m["ms_per_step"] * 1e-3) / 1e12
    per_gpu = wl.flops / (m["kernel_ms"] * 1e-3) / 1e12
    peak = ctx.peaks["bf16_sustained"] * (2.0 if wl.dtype == "e4m3" else 1.0)
    return {"value": val, "unit": "TFLOP/s", "steps": steps, "seconds": m["timed_s"], "ms_per_step": m["ms_per_step"], "clocks": m["clocks"],
            "frac_of_sustained_peak": per_gpu / peak, "sustained_peak": peak, "frac_of_nominal": per_gpu / NOMINAL_TFLOPS[wl.dtype],
            "note": "time x median SM MHz lets a reader normalise between runs; no clock setting is touched"}


def library_reference(ctx, steps=20):
    """One library E4M3 GEMM (torch._scaled_mm = cuBLASLt, per-tensor scales, 8192^3, bf16 out) timed in this process as a stated
    reference point for what the tensor pipe of this box delivers in E4M3.  Never on the product path."""
    import torch

    try:
        M = N = K = 8192
        a = torch.randn((M, K), device=ctx.dev).to(torch.float8_e4m3fn)
        b = torch.randn((N, K), device=ctx.dev).to(torch.float8_e4m3fn)
        one = torch.ones((), device=ctx.dev, dtype=torch.float32)
        fn = lambda: torch._scaled_mm(a, b.t(), scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1) / steps
        return {"what": "torch._scaled_mm (cuBLASLt) E4M3 x E4M3 -> bf16, per-tensor scales, M=N=K=8192 (no block scales: not the same recipe)",
                "value": 2.0 * M * N * K / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms, "steps": steps}
    except Exception as e:  # the library call is a reference point only
        return {"unavailable": f"{type(e).__name__}: {e}"[:200]}


def e2e_record(ctx, wl, n_steps):
    """The same metric through the host-buffer entry: pinned host operands in, host result out, every step.  With several
    ranks, operands that are replicated on every rank (`wl.replicated_inputs`) are uploaded by rank 0 only and reach the others by
    an NCCL broadcast over NVLink."""
    import torch

    hostpipe = importlib.import_module("iro-cuda-ax_b200.hostpipe")
    launch, dev_in, dev_out = wl.e2e_spec()
    rep = set(getattr(wl, "replicated_inputs", ())) if ctx.world > 1 else set()
    host_in = [None if (i in rep and ctx.rank != 0) else t.cpu().pin_memory() for i, t in enumerate(dev_in)]
    host_out = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in dev_out]
    h2d = sum(t.numel() * t.element_size() for t in host_in if t is not None)
    d2h = sum(t.numel() * t.element_size() for t in host_out)
    bcast = sum(dev_in[i].numel() * dev_in[i].element_size() for i in rep)
    pipe = hostpipe.HostPipeline(launch, dev_in, dev_out, broadcast=(sorted(rep), ctx.dist) if rep else None)
    for _ in range(3):
        pipe.submit(host_in, host_out)
    pipe.drain()
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(pipe.s_in)
    for _ in range(n_steps):
        pipe.submit(host_in, host_out)
    pipe.record_done(e1)
    pipe.drain()
    ctx.barrier()
    ctx.pkg.ops.check_status(ctx.dev)
    ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / n_steps
    hbm = wl.bound == "hbm"
    tot = torch.tensor([float(h2d), float(d2h)], dtype=torch.float64, device=ctx.dev)
    if ctx.world > 1:
        ctx.dist.all_reduce(tot)
    return {"value": wl.total_work() / (ms * 1e-3) / (1e9 if hbm else 1e12), "unit": "GB/s" if hbm else "TFLOP/s",
            "h2d_bytes_per_step": int(tot[0].item()), "d2h_bytes_per_step": int(tot[1].item()), "ms_per_step": ms, "steps": n_steps,
            "host_link_gbs": (tot[0].item() + tot[1].item()) / (ms * 1e-3) / 1e9,
            "nvlink_broadcast_bytes_per_step": bcast,
            "path": "hostpipe.HostPipeline: pinned host operands -> H2D -> C-ABI kernel -> D2H of the result, every step; three streams, "
                    "two buffer slots; byte counts are summed over all ranks"
                    + ("; replicated operands are uploaded once (rank 0) and broadcast over NVLink (NCCL)" if rep else "")}


def gather_record(ctx, wl, steps):
    """N-sharded GEMM with the full C requested: NCCL all-gather of the column shards + strided placement, timed alone."""
    import torch

    C = wl.sets[0][4]
    full = torch.empty((wl.M, wl.N), dtype=torch.bfloat16, device=ctx.dev)
    for _ in range(3):
        ctx.pkg.shard.all_gather_columns(C, wl.N, ctx.world, out=full)
    ctx.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        ctx.pkg.shard.all_gather_columns(C, wl.N, ctx.world, out=full)
    e1.record()
    ctx.barrier()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1)) / steps
    recv = 2.0 * wl.M * wl.N * (ctx.world - 1) / ctx.world
    return {"ms": ms, "bytes_received_per_gpu": int(recv), "gbs_per_gpu": recv / (ms * 1e-3) / 1e9,
            "frac_of_nvlink_peer_copy": recv / (ms * 1e-3) / 1e9 / NVLINK_PEER_GBS, "nvlink_reference_gbs": NVLINK_PEER_GBS,
            "what": "shard.all_gather_columns: one NCCL all-gather of the row-major [M, w] bf16 shards + one strided placement pass per rank"}


# ----------------------------------------------------------------------- main ----
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="gemm_fp8",
                    choices=["gemm_fp8", "gemm_fp8_strong", "gemm_bf16_gate_up", "gemm_bf16_down", "gemm_bf16_swiglu", "gemm_fp8_swiglu", "gemm_fp8_swiglu_quant", "gemm_fp8_swiglu_then_quant", "mlp_fp8", "attn_bf16", "attn_fp8", "quantize_fp8", "rmsnorm_quantize_fp8", "attn_decode_bf16", "attn_decode_fp8", "attn_ring", "attn_ring_zigzag"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extra", action="store_true", help="headline workload only: no sub-records, no sustained loop, no library reference")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    pkg = importlib.import_module("iro-cuda-ax_b200")
    pkg.capi.lib()                                 # fail loudly if the CUDA library is missing
    ctx = Ctx(pkg, dev, rank, local_rank, world, dist, load_peaks())
    wl = make_workload(args.workload, pkg, dev, rank, world)
    hbm = wl.bound == "hbm"
    unit = "GB/s" if hbm else "TFLOP/s"
    per = 1e9 if hbm else 1e12

    # ---- headline workload: device-resident timing --------------------------------
    m = measure(ctx, wl, args.steps, args.warmup)
    value = wl.total_work() / (m["ms_per_step"] * 1e-3) / per
    line = {
        "metric": getattr(wl, "metric", METRIC), "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": m["ms_per_step"], "higher_is_better": True,
        "scaling": wl.scaling if world > 1 else "weak", "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
        "config": config_for(wl, world), "clocks": m["clocks"], "e2e": None,
        "gpu_launches": args.steps * getattr(wl, "launches_per_step", 1),
    }
    if rank == 0:
        line["roofline"] = roofline(ctx, wl, args.workload, m)
    extras = args.workload == "gemm_fp8" and not args.no_extra

    # ---- end to end: host buffers in, host result out, every step ------------------
    if getattr(wl, "no_host_arms", None):
        line["e2e_note"] = wl.no_host_arms
        if hasattr(wl, "kv_bytes_per_step"):
            line["ring"] = {"kv_bytes_sent_per_gpu_per_call": wl.kv_bytes_per_step, "passes_on_this_rank": wl.launches_per_step - 1}
    elif not args.no_e2e:
        line["e2e"] = e2e_record(ctx, wl, max(4, min(args.steps, 24)))

    # ---- the other workloads of the metric, same process (sub-records) -------------
    if extras:
        del wl
        torch.cuda.empty_cache()
        steps = max(5, min(args.steps, 20))
        subs = {}
        names = list(EXTRA_WORKLOADS) + (["gemm_fp8_strong"] if world > 1 else [])
        for name in names:
            w = make_workload(name, pkg, dev, rank, world)
            torch.cuda.synchronize()
            time.sleep(1.5)      # idle gap: the 20-step burst figure of one workload should not inherit the power state the previous one left
            subs[name], _ = sub_record(ctx, w, name, steps, 3)
            if name == "gemm_fp8_strong":
                g = gather_record(ctx, w, steps)
                g["gemm_ms"] = subs[name]["ms_per_step"]
                g["gemm_plus_gather_ms"] = subs[name]["ms_per_step"] + g["ms"]
                line["gather"] = g
            del w
            torch.cuda.empty_cache()
        line["workloads"] = subs
        if rank == 0:
            line["library_reference"] = library_reference(ctx)
        # last on the GPU, so that the burst figures above are not taken on a part the long loop has just driven into its power cap
        wl = make_workload(args.workload, pkg, dev, rank, world)
        line["sustained"] = sustained_record(ctx, wl, m["ms_per_step"])
    if rank == 0:
        if world == 1 and not args.no_cpu_baseline and not getattr(wl, "no_host_arms", None):
            line["cpu_baseline"] = cpu_baseline(wl)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
