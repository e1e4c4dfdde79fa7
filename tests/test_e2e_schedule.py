"""Host-side scheduling of the end-to-end benchmark (pure numpy): the arrays handed to the attention path follow
the reference's prepare_prefill / prepare_decode formulas (src/engine/model_runner.cpp:482-632)."""
import importlib

import numpy as np
import pytest

import __graft_entry__ as entry


@pytest.fixture(scope="module")
def sch():
    entry.load_package()
    return importlib.import_module("benchmarks.e2e_schedule")


def test_requests_are_seeded_and_in_range(sch):
    p1, o1 = sch.make_requests(8, 1000, 5, 40, seed=3)
    p2, o2 = sch.make_requests(8, 1000, 5, 40, seed=3)
    assert all(np.array_equal(a, b) for a, b in zip(p1, p2)) and np.array_equal(o1, o2)
    assert all(5 <= len(p) <= 40 and p.min() >= 0 and p.max() < 1000 for p in p1)
    assert o1.min() >= 5 and o1.max() <= 40


def test_prefill_batches_respect_limits(sch):
    lens = [300, 300, 300, 50, 900, 10]
    b = sch.plan_prefill_batches(lens, max_num_seqs=3, max_num_batched_tokens=1000)
    assert b == [[0, 1, 2], [3, 4, 5]]
    assert sch.plan_prefill_batches(lens, 2, 10000) == [[0, 1], [2, 3], [4, 5]]
    with pytest.raises(ValueError):
        sch.plan_prefill_batches([2000], 4, 1000)


def test_prefill_arrays_follow_the_reference_formulas(sch):
    bs = 16
    prompts = [np.arange(20), np.arange(5), np.arange(33)]
    s = sch.Schedule(prompts, [4, 4, 4], bs, num_blocks=32, table_width=4)
    a = s.prefill_arrays([0, 1, 2])
    assert a["cu_seqlens_q"].tolist() == [0, 20, 25, 58] and a["cu_seqlens_k"].tolist() == [0, 20, 25, 58]
    assert a["positions"][:20].tolist() == list(range(20)) and a["positions"][20:25].tolist() == list(range(5))
    assert a["last_rows"].tolist() == [19, 24, 57] and a["max_seqlen"] == 33
    assert a["block_tables"].shape == (3, 3)            # widest sequence: 33 tokens = 3 blocks
    for k, (lo, n) in enumerate([(0, 20), (20, 5), (25, 33)]):
        pos = np.arange(n)
        want = a["block_tables"][k][pos // bs].astype(np.int64) * bs + pos % bs
        assert np.array_equal(a["slot_mapping"][lo:lo + n], want)
    used = np.concatenate([a["block_tables"][0, :2], a["block_tables"][1, :1], a["block_tables"][2, :3]])
    assert len(set(used.tolist())) == 6                 # no block handed out twice


def test_decode_arrays_advance_grow_and_retire(sch):
    bs = 4
    prompts = [np.arange(3), np.arange(4), np.arange(6)]
    outs = np.array([3, 2, 1])                          # sequence 2 is finished by its prefill token
    s = sch.Schedule(prompts, outs, bs, num_blocks=16, table_width=3)
    s.prefill_arrays([0, 1, 2])
    assert s.total_decode_steps() == 2
    m = np.zeros((3, 3 + 3), dtype=np.int32)
    assert s.decode_arrays(m) == 2
    # sequence 0: feeds the token at position 3 (still inside block 0); sequence 1: position 4 opens a second block
    assert m[0, 0] == 3 and m[0, 2] == 4 and m[0, 1] == s.tables[0, 0] * bs + 3
    assert m[1, 0] == 4 and m[1, 2] == 5 and m[1, 1] == s.tables[1, 1] * bs + 0 and s.num_blocks_of[1] == 2
    assert m[2, 1] == -1 and m[2, 2] == 0               # inactive row: no store, empty context
    assert np.array_equal(m[:, 3:], s.tables)
    assert s.decode_arrays(m) == 1                      # sequence 1 has produced its 2 tokens
    assert m[1, 1] == -1 and m[1, 2] == 0 and m[0, 0] == 4 and m[0, 1] == s.tables[0, 1] * bs
    assert s.decode_arrays(m) == 0 and (m[:, 1] == -1).all()
    assert int(s.generated.sum()) == int(outs.sum())    # every sequence produced exactly output_len tokens


def test_blocks_needed_covers_the_run(sch):
    prompts, outs = sch.make_requests(16, 100, 5, 60, seed=1)
    lens = np.array([len(p) for p in prompts])
    need = sch.blocks_needed(lens, outs, 8)
    s = sch.Schedule(prompts, outs, 8, num_blocks=need, table_width=(120 + 7) // 8)
    s.prefill_arrays(list(range(16)))
    m = np.zeros((16, 3 + s.table_width), dtype=np.int32)
    for _ in range(s.total_decode_steps()):
        s.decode_arrays(m)
    assert s.active().sum() == 0 and len(s.pool.free) >= 0
    # the last generated token is never fed back, so its slot is never needed
    assert int(s.num_blocks_of.sum()) <= need
