"""The allocation-free split-KV entry point (scratch memory in a file-scope device array of the library) against
the entry point that takes caller-owned scratch: same kernels, same inputs, two calls in a row.  Named to be
collected last; it also passes on its own."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_scratch_entry_matches_caller_scratch_entry_twice(pkg, oracle, dev):
    B, Hq, Hkv, Sq, Skv, splits = 2, 8, 2, 4, 3000, 5
    Q, _, _, scale = pkg.synth.bf16_attention_inputs(B, Hq, Sq, 128, seed=31, Hkv=Hkv, device=dev)
    _, K, V, _ = pkg.synth.bf16_attention_inputs(B, Hkv, Skv, 128, seed=32, device=dev)
    want_O, want_L = pkg.ops.attn_fwd_bf16_splitkv(Q, K, V, scale, True, num_splits=splits)
    O = torch.empty_like(Q)
    L = torch.empty((B, Hq, Sq), dtype=torch.float32, device=dev)
    pkg.ops.status_word(dev)                       # the status word exists before the measured calls
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(dev)
    for call in range(2):
        O.fill_(float("nan"))
        L.fill_(float("nan"))
        pkg.ops.attn_fwd_bf16_splitkv_static(Q, K, V, scale, True, num_splits=splits, out=O, lse=L)
        torch.cuda.synchronize()
        pkg.ops.check_status(dev)
        assert torch.equal(O, want_O), f"call {call}: outputs differ from the caller-scratch entry point"
        assert torch.equal(L, want_L), f"call {call}: LSE differs from the caller-scratch entry point"
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before               # nothing was allocated on the device by the two calls
    # and against the CPU oracle directly, so that this file stands on its own
    import numpy as np

    u16 = lambda t: t.cpu().view(torch.uint16).numpy()
    Ow, Lw = oracle.attn_fwd_bf16_qkv(u16(Q), u16(K), u16(V), scale, True)
    assert np.abs(O.float().cpu().numpy() - oracle.bf16_decode(Ow)).max() <= 2e-2      # the bf16 attention bar
    assert np.abs(L.cpu().numpy() - Lw).max() <= 1e-3


def test_static_scratch_entry_rejects_what_does_not_fit(pkg, dev):
    cap = int(pkg.capi.lib().axp_sm100_attn_splitkv_static_scratch_bytes())
    assert cap == 16 << 20
    B, Hq, Hkv, Sq, Skv = 1, 64, 8, 128, 256
    splits = cap // (Hq * Sq * (128 * 4 + 8)) + 1              # one share too many for 16 MiB
    Q, _, _, scale = pkg.synth.bf16_attention_inputs(B, Hq, Sq, 128, seed=1, Hkv=Hkv, device=dev)
    _, K, V, _ = pkg.synth.bf16_attention_inputs(B, Hkv, Skv, 128, seed=2, device=dev)
    with pytest.raises(pkg.capi.AxpError) as e:
        pkg.ops.attn_fwd_bf16_splitkv_static(Q, K, V, scale, False, num_splits=splits)
    assert e.value.code == pkg.capi.AXP_ERR_BAD_ARG
    O, _ = pkg.ops.attn_fwd_bf16_splitkv_static(Q, K, V, scale, False, num_splits=splits - 1)     # the largest that fits
    want, _ = pkg.ops.attn_fwd_bf16_splitkv(Q, K, V, scale, False, num_splits=splits - 1)
    pkg.ops.check_status(dev)
    assert torch.equal(O, want)
