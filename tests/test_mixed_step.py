"""A continuous-batching step with prefill rows AND decode rows as one launch (``nvk_attention_mixed_step``): the
prefill rows against the oracle's paged / dense prefill, the decode rows against the oracle's paged decode, and both
bit for bit against the two single-purpose entry points (same kernels' arithmetic, same split policy), for several
divisions of the SMs between the two kinds of work and for int64 index tensors."""
import numpy as np
import pytest

import oracle
from util import assert_attention_close, nvk, to_dev, to_np, workloads

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")

HQ, HKV, D, BS = 8, 2, 128, 256


def _case(paged, seed):
    wl = workloads()
    rng = np.random.default_rng(seed)
    # prefill part
    q_lens, prefix = ([300, 70, 129], [256, 0, 512]) if paged else ([200, 65, 130], [0, 0, 0])
    p = wl.make_prefill_workload(q_lens, prefix, HQ, HKV, D, BS, seed=seed, paged=paged)
    # decode part: its own sequences, in the same cache when the prefill part is paged
    ctx = rng.integers(1, 3000, size=9).astype(np.int32)
    ctx[3] = 0                                                        # an inactive row of a padded batch
    d = wl.make_decode_workload(len(ctx), HQ, HKV, D, BS, 0, 0, seed=seed + 1, context_lens=ctx, pad_blocks_to=14)
    if paged:   # one pool: decode blocks first, prefill blocks shifted behind them
        shift = d["k_cache"].shape[0]
        k_cache = np.concatenate([d["k_cache"], p["k_cache"]])
        v_cache = np.concatenate([d["v_cache"], p["v_cache"]])
        p_tables = (p["block_tables"] + shift).astype(np.int32)
    else:
        k_cache, v_cache, p_tables = d["k_cache"], d["v_cache"], None
    return p, d, k_cache, v_cache, p_tables


@pytest.mark.parametrize("paged", [True, False])
@pytest.mark.parametrize("prefill_blocks", [0, 1, 40, 1000])
def test_mixed_step_matches_oracle_and_the_two_single_purpose_calls(paged, prefill_blocks):
    bf = torch.bfloat16
    p, d, k_cache, v_cache, p_tables = _case(paged, seed=50 + prefill_blocks % 7)
    lib = nvk()
    kc, vc = to_dev(k_cache, bf), to_dev(v_cache, bf)
    pq, dq = to_dev(p["q"], bf), to_dev(d["q"], bf)
    cu_q, cu_k = to_dev(p["cu_q"]), to_dev(p["cu_k"])
    pt = to_dev(p_tables) if paged else None
    pk = None if paged else to_dev(p["k"], bf)
    pv = None if paged else to_dev(p["v"], bf)
    ctx, dt = to_dev(d["context_lens"]), to_dev(d["block_tables"])
    ws = torch.empty(max(16, lib.decode_attention_workspace_bytes(dq.shape[0], HQ, HKV, D, dt.shape[1], BS)), dtype=torch.uint8, device="cuda")
    p_out, d_out = torch.full_like(pq, float("nan")), torch.full_like(dq, float("nan"))
    lib.attention_mixed_step(pq, cu_q, pk, pv, cu_k, pt, p_out, dq, ctx, dt, d_out, kc, vc, HKV, D, BS, p["scale"], ws, prefill_blocks)
    torch.cuda.synchronize()
    assert lib.prefill_status() == 0
    assert not torch.isnan(p_out.float()).any() and not torch.isnan(d_out.float()).any()
    # the oracle
    if paged:
        want_p = oracle.prefill_attention_paged(p["q"], k_cache, v_cache, p["cu_q"], p["cu_k"], p_tables, HKV, D, BS, p["scale"])
    else:
        want_p = oracle.prefill_attention_dense(p["q"], p["k"], p["v"], p["cu_q"], p["cu_k"], HKV, D, p["scale"])
    want_d = oracle.decode_attention_paged(d["q"], k_cache, v_cache, d["context_lens"], d["block_tables"], HKV, D, BS, d["scale"])
    assert_attention_close(to_np(p_out), want_p)
    assert_attention_close(to_np(d_out), want_d)
    assert not to_np(d_out)[3].any()                                   # the inactive row is zeros
    # the single-purpose entry points
    p_ref, d_ref = torch.empty_like(pq), torch.empty_like(dq)
    if paged:
        lib.launch_prefill_attention_paged(pq, cu_q, kc, vc, cu_k, pt, HKV, D, BS, p["scale"], p_ref)
    else:
        lib.launch_prefill_attention_dense(pq, cu_q, pk, pv, cu_k, HKV, D, p["scale"], p_ref)
    lib.launch_decode_attention_paged(dq, kc, vc, ctx, dt, HKV, D, BS, d["scale"], d_ref, ws)
    torch.cuda.synchronize()
    assert torch.equal(p_out, p_ref)
    assert torch.equal(d_out, d_ref)


def test_mixed_step_repeats_with_int64_indices_and_from_a_graph():
    bf = torch.bfloat16
    p, d, k_cache, v_cache, p_tables = _case(True, seed=61)
    lib = nvk()
    L = torch.int64
    kc, vc = to_dev(k_cache, bf), to_dev(v_cache, bf)
    pq, dq = to_dev(p["q"], bf), to_dev(d["q"], bf)
    cu_q, cu_k, pt = to_dev(p["cu_q"]).to(L), to_dev(p["cu_k"]), to_dev(p_tables).to(L)
    ctx, dt = to_dev(d["context_lens"]).to(L), to_dev(d["block_tables"])
    ws = torch.empty(max(16, lib.decode_attention_workspace_bytes(dq.shape[0], HQ, HKV, D, dt.shape[1], BS)), dtype=torch.uint8, device="cuda")
    outs = []

    def step(p_out, d_out):
        lib.attention_mixed_step(pq, cu_q, None, None, cu_k, pt, p_out, dq, ctx, dt, d_out, kc, vc, HKV, D, BS, p["scale"], ws, 30)

    for _ in range(3):                                                 # the ticket counters re-arm between launches
        o = (torch.full_like(pq, float("nan")), torch.full_like(dq, float("nan")))
        step(*o)
        outs.append(o)
    torch.cuda.synchronize()
    gp, gd = torch.empty_like(pq), torch.empty_like(dq)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step(gp, gd)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step(gp, gd)
    for _ in range(2):
        gp.fill_(float("nan"))
        gd.fill_(float("nan"))
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(gp, outs[0][0]) and torch.equal(gd, outs[0][1])
    for o in outs[1:]:
        assert torch.equal(o[0], outs[0][0]) and torch.equal(o[1], outs[0][1])
    assert lib.prefill_status() == 0


def test_mixed_step_refuses_what_it_cannot_run():
    lib = nvk()
    f32 = torch.float32
    q = torch.zeros(4, 2, 128, device="cuda", dtype=f32)
    kc = torch.zeros(1, 256, 2, 128, device="cuda", dtype=f32)
    cu = torch.tensor([0, 4], device="cuda", dtype=torch.int32)
    ws = torch.zeros(1 << 20, device="cuda", dtype=torch.uint8)
    with pytest.raises(ValueError):                                    # fp32 takes the general paths: two calls
        lib.attention_mixed_step(q, cu, q, q, cu, None, q.clone(), q[:1], torch.ones(1, device="cuda", dtype=torch.int32),
                                 torch.zeros(1, 1, device="cuda", dtype=torch.int32), q[:1].clone(), kc, kc, 2, 128, 256, 0.1, ws, 0)
