"""Parity at the benchmark's FULL sizes.  Every output row of both configurations is compared with the reference's own
fp32 kernels (``oracle/_ref``: its attention.cu compiled unmodified, run on the GPU on fp32 copies of the same rounded
inputs -- the "fp32 path" the tolerance is defined against), and with the CPU oracle on a sample where that library is
absent.  Beside that, properties that need no second implementation: scatter / gather round trips, partition of unity
(constant V in, the same constant out), invariance under a physical permutation of the cache blocks, split against
unsplit decode, chunked against single-shot prefill.  Shapes are the decode and prefill benchmark configurations (batch
256 with contexts U[1024,8192]; 16 sequences of U[512,4096] new tokens, half with a paged prefix) at 32/8 heads,
head_dim 128, block_size 256, bf16."""
import ctypes
import os
import importlib

import numpy as np
import pytest

import oracle
from util import MAX_ABS_TOL, MEAN_ABS_TOL, nvk, to_np

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu

HQ, HKV, D, BS = 32, 8, 128, 256


def _reference_kernels():
    """The reference's own CUDA kernels behind oracle/ref_shim.cpp, or None where they were not built.  Test-side only:
    the product never loads this library."""
    path = os.path.join(os.path.dirname(os.path.abspath(oracle.__file__)), "_ref", "libnvk_ref.so")
    if not os.path.exists(path):
        return None
    lib = ctypes.CDLL(path)
    lib.nvkref_last_error.restype = ctypes.c_char_p
    return lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _close(a, b):
    err = (a.float() - b.float()).abs()
    assert float(err.max()) <= MAX_ABS_TOL and float(err.mean()) <= MEAN_ABS_TOL, (float(err.max()), float(err.mean()))


@pytest.fixture(scope="module")
def decode_full():
    import torch
    entry.load_package()
    wl = importlib.import_module("benchmarks.workloads")
    dev = torch.device("cuda:0")
    rng = np.random.default_rng(77)
    ctx = rng.integers(1024, 8193, size=256).astype(np.int32)
    tables, pool = wl.build_block_tables(rng, ctx, BS)
    gen = torch.Generator(device=dev)
    gen.manual_seed(77)
    bf = torch.bfloat16
    kc = torch.empty((pool, BS, HKV, D), device=dev, dtype=bf).normal_(generator=gen)
    vc = torch.empty((pool, BS, HKV, D), device=dev, dtype=bf).normal_(generator=gen)
    q = torch.randn((256, HQ, D), generator=gen, device=dev).to(bf)
    lib = nvk()
    ws = torch.empty(max(16, lib.decode_attention_workspace_bytes(256, HQ, HKV, D, tables.shape[1], BS)), dtype=torch.uint8, device=dev)
    w = {"ctx_np": ctx, "tables_np": tables, "pool": pool, "k": kc, "v": vc, "q": q, "ws": ws,
         "ctx": torch.from_numpy(ctx).to(dev), "tables": torch.from_numpy(tables).to(dev), "scale": 1.0 / np.sqrt(D)}
    out = torch.empty_like(q)
    lib.launch_decode_attention_paged(q, kc, vc, w["ctx"], w["tables"], HKV, D, BS, w["scale"], out, ws)
    torch.cuda.synchronize()
    w["out"] = out
    yield w
    del w


def test_store_round_trip_at_prefill_size():
    import torch
    dev = torch.device("cuda:0")
    tokens, pool = 36864, 36864 // BS + 64
    gen = torch.Generator(device=dev)
    gen.manual_seed(5)
    key = torch.randn((tokens, HKV, D), generator=gen, device=dev).to(torch.bfloat16)
    val = torch.randn((tokens, HKV, D), generator=gen, device=dev).to(torch.bfloat16)
    kc = torch.zeros((pool, BS, HKV, D), device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    slots_np = np.random.default_rng(5).permutation(pool * BS)[:tokens].astype(np.int32)
    slots_np[::97] = -1
    slots = torch.from_numpy(slots_np).to(dev)
    nvk().store_kvcache(key, val, kc, vc, slots)
    torch.cuda.synchronize()
    live = torch.from_numpy(np.nonzero(slots_np >= 0)[0]).to(dev)
    rows = slots[live].long()
    assert torch.equal(kc.view(-1, HKV, D)[rows], key[live]) and torch.equal(vc.view(-1, HKV, D)[rows], val[live])
    # nothing else was touched: the bytes of the whole cache sum to the bytes of the rows that were stored
    assert int(kc.view(torch.int16).long().sum()) == int(key[live].view(torch.int16).long().sum())
    assert int(vc.view(torch.int16).long().sum()) == int(val[live].view(torch.int16).long().sum())


def test_decode_sample_of_rows_matches_oracle(decode_full):
    import torch
    w = decode_full
    pick = [0, 17, 101, 255]
    # only the sampled sequences' blocks travel to the host: a compact cache with remapped tables
    tables = w["tables_np"][pick]
    used = np.unique(np.concatenate([tables[i, :(w["ctx_np"][s] + BS - 1) // BS] for i, s in enumerate(pick)]))
    remap = np.zeros(w["pool"], np.int32)
    remap[used] = np.arange(used.size, dtype=np.int32)
    sel = torch.from_numpy(used.astype(np.int64)).to(w["q"].device)
    kc, vc = to_np(w["k"][sel]), to_np(w["v"][sel])
    ref = oracle.decode_attention_paged(to_np(w["q"][pick]), kc, vc, w["ctx_np"][pick], remap[tables], HKV, D, BS, w["scale"])
    err = np.abs(to_np(w["out"][pick]) - ref)
    assert err.max() <= MAX_ABS_TOL and err.mean() <= MEAN_ABS_TOL


def test_decode_every_row_matches_the_reference_fp32_kernel(decode_full):
    import torch
    ref = _reference_kernels()
    if ref is None:
        pytest.skip("oracle/_ref not built here; the sampled oracle comparison above stands in")
    w = decode_full
    q32, k32, v32 = w["q"].float(), w["k"].float(), w["v"].float()
    out32 = torch.empty_like(q32)
    rc = ref.nvkref_decode_attention_paged(_ptr(q32), _ptr(k32), _ptr(v32), _ptr(w["ctx"]), _ptr(w["tables"]), ctypes.c_int64(256),
                                           ctypes.c_int64(w["tables"].shape[1]), ctypes.c_int64(w["pool"]), HQ, HKV, D, BS,
                                           ctypes.c_float(w["scale"]), _ptr(out32), 2, None)
    assert rc == 0, ref.nvkref_last_error()
    torch.cuda.synchronize()
    del k32, v32
    _close(w["out"], out32)                      # all 256 x 32 rows
    # and the int8-cache and unsplit paths are tied to the same rows by the tests below


def test_decode_constant_values_come_out_unchanged(decode_full):
    import torch
    w = decode_full
    const = torch.linspace(-2, 2, D, device=w["q"].device).to(torch.bfloat16)
    vconst = const.expand(w["pool"], BS, HKV, D).contiguous()
    out = torch.empty_like(w["q"])
    nvk().launch_decode_attention_paged(w["q"], w["k"], vconst, w["ctx"], w["tables"], HKV, D, BS, w["scale"], out, w["ws"])
    torch.cuda.synchronize()
    # softmax weights sum to one: every output row is the constant row (up to the 16-bit rounding of the weights)
    assert float((out.float() - const.float()).abs().max()) <= 2e-2


def test_decode_is_invariant_under_a_physical_permutation_of_the_blocks(decode_full):
    import torch
    w = decode_full
    dev = w["q"].device
    perm = torch.from_numpy(np.random.default_rng(3).permutation(w["pool"])).to(dev)      # new position of block i
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(w["pool"], device=dev)
    k2, v2 = w["k"][inv].contiguous(), w["v"][inv].contiguous()                             # block i now lives at perm[i]
    t2 = perm[w["tables"].long()].to(torch.int32)
    # table entries past a sequence's blocks are padding zeros: keep them valid ids (they are never read)
    out = torch.empty_like(w["q"])
    nvk().launch_decode_attention_paged(w["q"], k2, v2, w["ctx"], t2, HKV, D, BS, w["scale"], out, w["ws"])
    torch.cuda.synchronize()
    assert torch.equal(out, w["out"])          # same arithmetic in the same order: bit-identical


def test_decode_split_and_unsplit_agree(decode_full):
    import torch
    w = decode_full
    out = torch.empty_like(w["q"])
    nvk().launch_decode_attention_paged(w["q"], w["k"], w["v"], w["ctx"], w["tables"], HKV, D, BS, w["scale"], out, None)
    torch.cuda.synchronize()
    _close(out, w["out"])


def test_int8_cache_agrees_with_the_16_bit_cache_at_full_size(decode_full):
    import torch
    w = decode_full
    lib = nvk()
    rows = w["pool"] * BS
    dev = w["q"].device
    kc8 = torch.empty((rows, HKV, D), dtype=torch.int8, device=dev); vc8 = torch.empty_like(kc8)
    ks = torch.empty((rows, HKV), dtype=torch.float16, device=dev); vs = torch.empty_like(ks)
    lib.store_kvcache_int8(w["k"].view(rows, HKV, D), w["v"].view(rows, HKV, D), kc8, vc8, ks, vs,
                           torch.arange(rows, dtype=torch.int32, device=dev))
    # quantise / dequantise round trip: every element within half a quantisation step of its head vector, plus what the
    # fp16 rounding of the stored scale adds (at most 127 steps x 2^-11 of a step)
    deq = kc8[:4096].float() * ks[:4096].float()[..., None]
    step = ks[:4096].float()[..., None]
    assert bool(((deq - w["k"].view(rows, HKV, D)[:4096].float()).abs() <= (0.5 + 127.0 / 2048.0) * step + 1e-6).all())
    out = torch.empty_like(w["q"])
    lib.launch_decode_attention_paged_int8(w["q"], kc8, vc8, ks, vs, w["ctx"], w["tables"], HKV, D, BS, w["scale"], out, w["ws"])
    torch.cuda.synchronize()
    _close(out, w["out"])


@pytest.fixture(scope="module")
def prefill_full():
    import torch
    entry.load_package()
    kb = importlib.import_module("benchmarks.kernel_bench")
    dev = torch.device("cuda:0")
    w = kb.make_prefill_inputs(torch, dev, 2025)
    lib = nvk()
    lib.store_kvcache(w["k_new"], w["v_new"], w["k_cache"], w["v_cache"], w["slot_mapping"])
    lib.launch_prefill_attention_paged(w["q"], w["cu_q"], w["k_cache"], w["v_cache"], w["cu_k"], w["block_tables"], HKV, D, BS,
                                       w["scale"], w["out"])
    torch.cuda.synchronize()
    yield w
    del w


def test_prefill_shortest_sequence_matches_oracle(prefill_full):
    w = prefill_full
    cu_q, cu_k = w["cu_q"].cpu().numpy(), w["cu_k"].cpu().numpy()
    s = int(np.argmin(np.diff(cu_k)))
    q = to_np(w["q"][cu_q[s]:cu_q[s + 1]])
    ref = oracle.prefill_attention_paged(q, to_np(w["k_cache"]), to_np(w["v_cache"]), np.array([0, q.shape[0]], np.int32),
                                         np.array([0, cu_k[s + 1] - cu_k[s]], np.int32), w["block_tables"][s:s + 1].cpu().numpy(),
                                         HKV, D, BS, w["scale"])
    err = np.abs(to_np(w["out"][cu_q[s]:cu_q[s + 1]]) - ref)
    assert err.max() <= MAX_ABS_TOL and err.mean() <= MEAN_ABS_TOL


def test_prefill_every_row_matches_the_reference_fp32_kernel(prefill_full):
    import torch
    ref = _reference_kernels()
    if ref is None:
        pytest.skip("oracle/_ref not built here; the shortest-sequence oracle comparison above stands in")
    w = prefill_full
    q32, k32, v32 = w["q"].float(), w["k_cache"].float(), w["v_cache"].float()
    out32 = torch.empty_like(q32)
    seqs = w["cu_q"].numel() - 1
    rc = ref.nvkref_prefill_attention_paged(_ptr(q32), _ptr(k32), _ptr(v32), _ptr(w["cu_q"]), _ptr(w["cu_k"]), _ptr(w["block_tables"]),
                                            ctypes.c_int64(seqs), ctypes.c_int64(q32.shape[0]), ctypes.c_int64(w["block_tables"].shape[1]),
                                            ctypes.c_int64(w["pool"]), HQ, HKV, D, BS, ctypes.c_float(w["scale"]), _ptr(out32), 2, None)
    assert rc == 0, ref.nvkref_last_error()
    torch.cuda.synchronize()
    del k32, v32
    _close(w["out"], out32)                      # every query row of all 16 sequences, all 32 heads


def test_prefill_constant_values_come_out_unchanged(prefill_full):
    import torch
    w = prefill_full
    const = torch.linspace(-1, 1, D, device=w["q"].device).to(torch.bfloat16)
    vconst = const.expand_as(w["v_cache"]).contiguous()
    out = torch.empty_like(w["q"])
    nvk().launch_prefill_attention_paged(w["q"], w["cu_q"], w["k_cache"], vconst, w["cu_k"], w["block_tables"], HKV, D, BS, w["scale"], out)
    torch.cuda.synchronize()
    assert float((out.float() - const.float()).abs().max()) <= 2e-2


def test_prefill_in_two_chunks_equals_single_shot(prefill_full):
    """The second half of every sequence's new tokens, attended as a later chunk (everything before it read as a paged
    prefix), must reproduce the single-shot rows (the reference checks the same on small shapes,
    tests/test_model_runner.cpp:287-362)."""
    import torch
    w = prefill_full
    dev = w["q"].device
    cu_q, cu_k = w["cu_q"].cpu().numpy().astype(np.int64), w["cu_k"].cpu().numpy().astype(np.int64)
    q_lens = np.diff(cu_q)
    first = q_lens // 2
    rows = np.concatenate([np.arange(cu_q[s] + first[s], cu_q[s + 1]) for s in range(len(q_lens))])
    cu_q2 = np.zeros(len(q_lens) + 1, np.int32)
    cu_q2[1:] = np.cumsum(q_lens - first)
    idx = torch.from_numpy(rows).to(dev)
    q2 = w["q"][idx].contiguous()
    out2 = torch.empty_like(q2)
    nvk().launch_prefill_attention_paged(q2, torch.from_numpy(cu_q2).to(dev), w["k_cache"], w["v_cache"], w["cu_k"], w["block_tables"],
                                         HKV, D, BS, w["scale"], out2)
    torch.cuda.synchronize()
    _close(out2, w["out"][idx])


def test_prefill_launches_on_two_streams_do_not_disturb_each_other(prefill_full):
    """The persistent prefill kernel takes its work items from per-launch ticket counters; launches that overlap on the
    GPU (two streams) must each see a private counter.  Forty interleaved launches, every output compared."""
    import torch
    w = prefill_full
    lib = nvk()
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    outs = [torch.empty_like(w["out"]) for _ in range(4)]
    torch.cuda.synchronize()
    for rep in range(10):
        for k, stream in enumerate((s1, s2, s1, s2)):
            with torch.cuda.stream(stream):
                lib.launch_prefill_attention_paged(w["q"], w["cu_q"], w["k_cache"], w["v_cache"], w["cu_k"], w["block_tables"], HKV, D, BS,
                                                   w["scale"], outs[k])
    torch.cuda.synchronize()
    for o in outs:
        assert torch.equal(o, w["out"])
