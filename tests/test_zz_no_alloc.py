"""Decode attention without any allocation (``nvk_decode_attention_paged_static``).

Some users of the decode kernel cannot give it a workspace: a wrapper that keeps the reference's
``launch_decode_attention_paged`` signature has no allocator to ask, and a serving process that has
pledged all free HBM to its KV cache (or that bans ``cudaMalloc`` after start-up) has nothing left to
hand over.  For them the library keeps the split-K scratch in a fixed 32 MiB device array.  This file
checks, through the C ABI, that the allocation-free entry point returns what the workspace-taking one
returns -- the same bits, since both run the same kernels with the same split -- twice in a row (the second
call finds the first call's leftovers in the shared array), that the result is also right (against the CPU
oracle, within the tolerance of every bf16 attention test), and that problems too large for the array are
refused.  It is named so that pytest collects it last.
"""
import numpy as np
import pytest

import oracle
from util import assert_attention_close, nvk, to_dev, to_np, workloads

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def _both(w, num_kv_heads):
    bf = torch.bfloat16
    q = to_dev(w["q"], bf)
    kc, vc = to_dev(w["k_cache"], bf), to_dev(w["v_cache"], bf)
    ctx, bt = to_dev(w["context_lens"]), to_dev(w["block_tables"])
    nbytes = nvk().decode_attention_workspace_bytes(q.shape[0], q.shape[1], num_kv_heads, 128, bt.shape[1], 256)
    assert nbytes > 0, "the case must actually use split-K scratch"
    ws = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    expected = torch.full_like(q, float("nan"))
    nvk().launch_decode_attention_paged(q, kc, vc, ctx, bt, num_kv_heads, 128, 256, w["scale"], expected, ws)
    got = torch.full_like(q, float("nan"))
    nvk().launch_decode_attention_paged_static(q, kc, vc, ctx, bt, num_kv_heads, 128, 256, w["scale"], got)
    torch.cuda.synchronize()
    return got, expected


def test_static_scratch_entry_point_matches_workspace_entry_point_twice():
    wl = workloads()
    first = wl.make_decode_workload(6, 32, 8, 128, 256, 1, 3500, seed=71, pad_blocks_to=16)
    second = wl.make_decode_workload(3, 16, 8, 128, 256, 200, 4000, seed=72, pad_blocks_to=20)
    for w, hkv in ((first, 8), (second, 8)):
        got, expected = _both(w, hkv)
        assert not torch.isnan(got.float()).any()
        assert torch.equal(got, expected)
    ref = oracle.decode_attention_paged(second["q"], second["k_cache"], second["v_cache"], second["context_lens"],
                                        second["block_tables"], 8, 128, 256, second["scale"])
    assert_attention_close(to_np(got), ref)


def test_static_scratch_entry_point_rejects_problems_beyond_its_array():
    bf = torch.bfloat16
    batch, heads, max_blocks = 2048, 32, 64
    assert nvk().decode_attention_workspace_bytes(batch, heads, 8, 128, max_blocks, 256) > (32 << 20)
    q = torch.zeros(batch, heads, 128, dtype=bf, device="cuda")
    kc = torch.zeros(1, 256, 8, 128, dtype=bf, device="cuda")
    ctx = torch.zeros(batch, dtype=torch.int32, device="cuda")
    bt = torch.zeros(batch, max_blocks, dtype=torch.int32, device="cuda")
    out = torch.full_like(q, 7.0)
    with pytest.raises(ValueError, match="built-in"):
        nvk().launch_decode_attention_paged_static(q, kc, kc, ctx, bt, 8, 128, 256, 0.1, out)
    torch.cuda.synchronize()
    assert float(out.min()) == 7.0   # nothing was launched
