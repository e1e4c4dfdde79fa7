"""Host side of the end-to-end decoder benchmark: requests, paged block allocation and per-step metadata.

Pure numpy, no GPU.  It restates, for the benchmark only, what the reference's scheduler and model runner
hand to the attention path every step:

* requests as in the reference's throughput benchmark (bench.cpp:59-80): random token ids, prompt and
  output lengths uniform in [lo, hi], ``ignore_eos`` (a sequence ends after exactly ``output_len`` tokens);
* prefill-first scheduling under ``max_num_seqs`` / ``max_num_batched_tokens`` (src/engine/scheduler.cpp:31-106);
* 256-token blocks handed out from a free list (src/engine/block_manager.cpp), one more block when a sequence
  crosses a block boundary;
* the arrays of ``prepare_prefill`` / ``prepare_decode`` (src/engine/model_runner.cpp:482-632):
  ``slot = block_id * block_size + offset``, ``context_lens`` including the token being generated,
  ``positions``, ``cu_seqlens`` and zero-padded ``block_tables``.

Decode rows are fixed: sequence ``i`` owns row ``i`` of every decode step for the whole run, and a finished (or
not yet started) sequence leaves an inactive row (``context_len`` 0, ``slot`` -1), so one captured decode graph of
``num_seqs`` rows serves every step.
"""
from __future__ import annotations

import numpy as np


def make_requests(num_seqs=256, vocab=151936, len_lo=100, len_hi=1024, seed=0):
    """Prompt token ids and output lengths of the benchmark's requests."""
    rng = np.random.default_rng(seed)
    prompt_lens = rng.integers(len_lo, len_hi + 1, size=num_seqs)
    output_lens = rng.integers(len_lo, len_hi + 1, size=num_seqs)
    prompts = [rng.integers(0, vocab, size=int(n), dtype=np.int64) for n in prompt_lens]
    return prompts, output_lens.astype(np.int64)


class BlockPool:
    """Free list of cache blocks; ids are handed out in a seeded random order (fragmented tables)."""

    def __init__(self, num_blocks, seed=1):
        self.num_blocks = int(num_blocks)
        self.free = list(np.random.default_rng(seed).permutation(self.num_blocks)[::-1])

    def take(self):
        if not self.free:
            raise RuntimeError("out of KV cache blocks")
        return int(self.free.pop())

    def give(self, ids):
        self.free.extend(int(i) for i in ids)


def blocks_needed(prompt_lens, output_lens, block_size):
    """Blocks that hold every sequence at its final length (the benchmark never preempts)."""
    total = np.asarray(prompt_lens) + np.asarray(output_lens)
    return int(np.sum((total + block_size - 1) // block_size))


def plan_prefill_batches(prompt_lens, max_num_seqs, max_num_batched_tokens):
    """Greedy first-come packing of whole prompts, as the reference's scheduler does while requests wait."""
    batches, cur, tokens = [], [], 0
    for i, n in enumerate(prompt_lens):
        n = int(n)
        if n > max_num_batched_tokens:
            raise ValueError("prompt longer than max_num_batched_tokens")
        if cur and (tokens + n > max_num_batched_tokens or len(cur) >= max_num_seqs):
            batches.append(cur)
            cur, tokens = [], 0
        cur.append(i)
        tokens += n
    if cur:
        batches.append(cur)
    return batches


class Schedule:
    """Block tables and step metadata for a fixed set of sequences."""

    def __init__(self, prompts, output_lens, block_size, num_blocks, table_width, pool_seed=1):
        self.prompts = prompts
        self.prompt_lens = np.array([len(p) for p in prompts], dtype=np.int64)
        self.output_lens = np.asarray(output_lens, dtype=np.int64)
        self.block_size = int(block_size)
        self.table_width = int(table_width)
        self.pool = BlockPool(num_blocks, pool_seed)
        n = len(prompts)
        self.tables = np.zeros((n, self.table_width), dtype=np.int32)
        self.num_blocks_of = np.zeros(n, dtype=np.int64)
        # tokens whose K/V are (or are about to be) in the cache; 0 until the sequence is prefilled
        self.cached = np.zeros(n, dtype=np.int64)
        self.generated = np.zeros(n, dtype=np.int64)

    def _grow(self, i, length):
        need = (int(length) + self.block_size - 1) // self.block_size
        if need > self.table_width:
            raise ValueError("sequence longer than the block table")
        while self.num_blocks_of[i] < need:
            self.tables[i, self.num_blocks_of[i]] = self.pool.take()
            self.num_blocks_of[i] += 1

    def prefill_arrays(self, seq_ids):
        """Arrays of one prefill step over whole prompts (no prefix hits: random prompts never share blocks)."""
        bs = self.block_size
        lens = self.prompt_lens[seq_ids]
        cu = np.zeros(len(seq_ids) + 1, dtype=np.int32)
        cu[1:] = np.cumsum(lens)
        tokens = np.concatenate([self.prompts[i] for i in seq_ids]).astype(np.int64)
        positions = np.concatenate([np.arange(n, dtype=np.int32) for n in lens])
        slots = np.empty(int(cu[-1]), dtype=np.int32)
        for k, i in enumerate(seq_ids):
            self._grow(i, lens[k])
            pos = np.arange(lens[k])
            slots[cu[k]:cu[k + 1]] = self.tables[i, pos // bs].astype(np.int64) * bs + pos % bs
            self.cached[i] = lens[k]
            self.generated[i] = 1            # the prefill step samples the first output token
        width = int(self.num_blocks_of[seq_ids].max())
        return {"tokens": tokens, "positions": positions, "slot_mapping": slots, "cu_seqlens_q": cu,
                "cu_seqlens_k": cu.copy(), "block_tables": np.ascontiguousarray(self.tables[seq_ids, :width]),
                "last_rows": (cu[1:] - 1).astype(np.int64), "max_seqlen": int(lens.max())}

    def active(self):
        return (self.cached > 0) & (self.generated < self.output_lens)

    def decode_arrays(self, out):
        """Fills ``out`` (int32 [num_seqs, 3 + table_width]: position, slot, context_len, block table) for the
        next decode step and advances the sequences.  Returns the number of active rows."""
        act = self.active()
        idx = np.nonzero(act)[0]
        out[:, 0] = 0
        out[:, 1] = -1
        out[:, 2] = 0
        if idx.size == 0:
            return 0
        bs = self.block_size
        pos = self.cached[idx]                      # position of the token fed this step
        crossing = idx[(pos % bs == 0) | (self.num_blocks_of[idx] * bs <= pos)]
        for i in crossing:
            self._grow(i, self.cached[i] + 1)
        out[idx, 0] = pos
        out[idx, 1] = self.tables[idx, pos // bs].astype(np.int64) * bs + pos % bs
        out[idx, 2] = pos + 1                       # context includes the token being generated
        out[:, 3:] = self.tables
        self.cached[idx] += 1
        self.generated[idx] += 1
        return int(idx.size)

    def total_decode_steps(self):
        return int(self.output_lens.max() - 1)
