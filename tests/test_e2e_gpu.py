"""End-to-end decoder harness on a GPU: the decode path (fused prologue + cache store + paged decode attention)
must continue a sequence exactly as a single prefill over the longer sequence does (the reference checks the same
property for chunked against single-shot prefill, tests/test_model_runner.cpp:287-362), and the benchmark loop
must run with and without the captured decode graph."""
import importlib

import numpy as np
import pytest

import __graft_entry__ as entry

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    import torch
    nvk = entry.load_package()
    nvk.lib()
    get = lambda n: importlib.import_module("benchmarks." + n)  # noqa: E731
    return torch, nvk, get("e2e_model"), get("e2e_schedule"), get("e2e_bench")


def tiny(em, layers=2):
    return em.DecoderConfig(layers=layers, hidden=256, num_heads=4, num_kv_heads=2, head_dim=128, ffn=512, vocab=1000,
                            max_model_len=1024, max_num_seqs=8, max_num_batched_tokens=2048)


@pytest.mark.parametrize("kv_dtype,tol,linears", [("bf16", 0.03, "cublas"), ("int8", 0.06, "cublas"), ("fp8", 0.12, "cublas"), ("bf16", 0.03, "fused")])
def test_decode_continues_a_sequence_like_a_longer_prefill(mods, kv_dtype, tol, linears):
    torch, nvk, em, es, _ = mods
    dev = torch.device("cuda:0")
    cfg = tiny(em)
    rng = np.random.default_rng(5)
    lens = [37, 300, 256]                       # inside a block, across a block boundary, exactly at one
    extra = 3                                   # tokens continued by decode steps
    full = [rng.integers(0, cfg.vocab, size=n + extra) for n in lens]
    model = em.Decoder(nvk, torch, dev, cfg, num_blocks=16, seed=1, kv_dtype=kv_dtype, linears=linears)
    model.ensure_workspace(len(lens), 4)

    hidden = {}

    def run_prefill(m, prompts, key):
        s = es.Schedule(prompts, [1] * len(prompts), cfg.block_size, 16, 4)
        a = s.prefill_arrays(list(range(len(prompts))))
        up = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)  # noqa: E731
        cu, tables = up(a["cu_seqlens_q"]), up(a["block_tables"])

        attend = m.attend_prefill(cu, cu, tables)
        hidden[key] = m.forward(up(a["tokens"]), up(a["positions"]), up(a["slot_mapping"]), attend).float().cpu().numpy()
        return s, a

    # reference: one prefill over the whole sequences
    run_prefill(model, full, "full")
    cu_full = np.concatenate([[0], np.cumsum([len(f) for f in full])])
    # candidate: prefill the prompts, then decode the remaining tokens one at a time on the same cache
    model.kv_cache.zero_()
    s, _ = run_prefill(model, [f[:n] for f, n in zip(full, lens)], "prompt")
    s.output_lens[:] = extra + 1
    meta = np.zeros((len(lens), 3 + 4), dtype=np.int32)
    for step in range(extra):
        assert s.decode_arrays(meta) == len(lens)
        m = torch.from_numpy(meta).to(dev)
        tokens = torch.tensor([int(f[n + step]) for f, n in zip(full, lens)], device=dev)
        positions, slots, ctx, tables = (m[:, 0].contiguous(), m[:, 1].contiguous(), m[:, 2].contiguous(), m[:, 3:].contiguous())

        attend = model.attend_decode(ctx, tables)
        h = model.forward(tokens, positions, slots, attend).float().cpu().numpy()
        for i, n in enumerate(lens):
            want = hidden["full"][cu_full[i] + n + step]
            err = np.abs(h[i] - want).max()
            assert err <= tol * max(1.0, np.abs(want).max()), (i, step, err, np.abs(want).max())


@pytest.mark.parametrize("use_graph,kv_dtype,linears", [(True, "bf16", "cublas"), (False, "bf16", "cublas"), (True, "int8", "cublas"),
                                                        (True, "bf16", "fused")])
def test_benchmark_loop_runs(mods, use_graph, kv_dtype, linears):
    torch, nvk, em, _, eb = mods
    line = eb.run_e2e(nvk, torch, None, 0, 1, torch.device("cuda:0"), tiny(em, layers=2), num_seqs=6, len_lo=5, len_hi=300,
                      seed=2, use_graph=use_graph, kv_dtype=kv_dtype, linears=linears)
    assert line["output_tokens"] > 0 and line["value"] > 0
    assert not line["gemm_status"]
    assert line["config"]["decode_steps"] == line["steps"] - line["config"]["prefill_batches"]
    assert line["gpu_launches"] > 0
