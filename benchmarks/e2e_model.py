"""End-to-end Qwen3-style decoder used ONLY to measure output tokens per second around the attention path.

What is the product here and what is plumbing: every attention-side operation -- the decode prologue
(split + q/k RMSNorm + RoPE + cache store), paged decode attention, paged varlen prefill attention -- goes through
the C ABI of ``libnvk.so``.  Everything else a decoder needs (embedding, the four linears per layer as plain cuBLAS
GEMMs through ``torch.matmul``, residual RMSNorm, SiLU-gate, greedy sampling, the NCCL all-reduce after o_proj and
down_proj) is torch plumbing with random-init weights; it mirrors the shapes and the tensor-parallel sharding of the
reference (QKV / gate-up column-parallel by head, o_proj / down_proj row-parallel followed by an all-reduce:
src/layers/linear.cpp:306-366; vocabulary-parallel head with a gather for greedy sampling) so that the attention
calls see exactly the per-rank shapes of a real run: ``Hq/t`` query heads, ``Hkv/t`` KV heads, a private cache.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass
class DecoderConfig:
    layers: int = 36
    hidden: int = 4096
    num_heads: int = 32
    num_kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 12288
    vocab: int = 151936
    eps: float = 1e-6
    rope_theta: float = 1e6
    block_size: int = 256
    max_model_len: int = 4096
    max_num_seqs: int = 512
    max_num_batched_tokens: int = 16384


def rope_table(torch, dev, max_positions, head_dim, theta):
    """fp32 [max_positions, head_dim] = [cos | sin], inv_freq = theta^(-2i/D) (src/layers/rotary_embedding.cpp:35-47)."""
    inv = 1.0 / torch.pow(torch.tensor(float(theta), device=dev),
                          torch.arange(0, head_dim, 2, device=dev, dtype=torch.float32) / head_dim)
    ang = torch.arange(max_positions, device=dev, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cat([torch.cos(ang), torch.sin(ang)], dim=1).contiguous()


class Decoder:
    """One tensor-parallel rank of the decoder."""

    def __init__(self, nvk, torch, dev, cfg: DecoderConfig, rank=0, world=1, dist=None, num_blocks=0, seed=0, kv_dtype="bf16", peer_comm=None,
                 linears="cublas"):
        if cfg.num_kv_heads % world or cfg.ffn % world or cfg.vocab % world:
            raise ValueError("heads, ffn and vocab must divide by the tensor-parallel size")
        self.nvk, self.torch, self.dev, self.cfg = nvk, torch, dev, cfg
        self.rank, self.world, self.dist = rank, world, dist
        # optional tp_comm.PeerAllReduce: messages that fit its buffers take the peer-memory kernel, larger ones NCCL
        self.peer_comm = peer_comm if world > 1 else None
        # "fused": at decode sizes the QKV projection runs with the prologue in its epilogue and the row-parallel linears push their
        # partial sums into the all-reduce from theirs (this library's GEMMs); "cublas": plain torch.matmul followed by the kernels
        if linears not in ("cublas", "fused"):
            raise ValueError("linears must be cublas or fused")
        self.fused_linears = linears == "fused"
        self.fused_rows_max = 512
        self.hq, self.hkv = cfg.num_heads // world, cfg.num_kv_heads // world
        self.ffn, self.vocab = cfg.ffn // world, cfg.vocab // world
        bf = torch.bfloat16
        d, hid = cfg.head_dim, cfg.hidden
        gen = torch.Generator(device=dev)

        def weight(tag, rows, cols, row_lo, row_hi, col_lo=0, col_hi=None, std=0.02):
            # every rank draws the same full matrix from the same seed and keeps its shard
            gen.manual_seed(seed * 1000003 + tag)
            full = torch.randn((rows, cols), generator=gen, device=dev, dtype=torch.float32).mul_(std).to(bf)
            return full[row_lo:row_hi, col_lo:(cols if col_hi is None else col_hi)].contiguous()

        r = rank
        self.embed = weight(1, cfg.vocab, hid, 0, cfg.vocab)
        self.lm_head = weight(2, cfg.vocab, hid, r * self.vocab, (r + 1) * self.vocab)
        self.final_norm = torch.ones(hid, device=dev, dtype=bf)
        self.layers = []
        for l in range(cfg.layers):
            t = 100 + 10 * l
            wq = weight(t, cfg.num_heads * d, hid, r * self.hq * d, (r + 1) * self.hq * d)
            wk = weight(t + 1, cfg.num_kv_heads * d, hid, r * self.hkv * d, (r + 1) * self.hkv * d)
            wv = weight(t + 2, cfg.num_kv_heads * d, hid, r * self.hkv * d, (r + 1) * self.hkv * d)
            gate = weight(t + 4, cfg.ffn, hid, r * self.ffn, (r + 1) * self.ffn)
            up = weight(t + 5, cfg.ffn, hid, r * self.ffn, (r + 1) * self.ffn)
            self.layers.append({
                "w_qkv": torch.cat([wq, wk, wv], dim=0).contiguous(),
                "w_o": weight(t + 3, hid, cfg.num_heads * d, 0, hid, r * self.hq * d, (r + 1) * self.hq * d),
                "w_gate_up": torch.cat([gate, up], dim=0).contiguous(),
                "w_down": weight(t + 6, hid, cfg.ffn, 0, hid, r * self.ffn, (r + 1) * self.ffn),
                "norm_in": torch.ones(hid, device=dev, dtype=bf), "norm_post": torch.ones(hid, device=dev, dtype=bf),
                "q_norm": torch.ones(d, device=dev, dtype=bf), "k_norm": torch.ones(d, device=dev, dtype=bf),
            })
            del wq, wk, wv, gate, up
        self.cos_sin = rope_table(torch, dev, cfg.max_model_len, d, cfg.rope_theta)
        self.scale = 1.0 / math.sqrt(d)
        # [2, layers, blocks, block_size, Hkv/t, D] as in allocate_kv_cache (src/engine/model_runner.cpp:355-472)
        self.num_blocks = int(num_blocks)
        if kv_dtype not in ("bf16", "int8", "fp8"):
            raise ValueError("kv_dtype must be bf16, int8 or fp8")
        self.int8 = kv_dtype in ("int8", "fp8")     # an 8-bit cache with per-(token, head) scales: the unfused route
        self.fp8 = kv_dtype == "fp8"                # e4m3 bytes instead of int8 (no counterpart in the reference)
        self.kv_cache = torch.zeros((2, cfg.layers, self.num_blocks, cfg.block_size, self.hkv, d), device=dev,
                                    dtype=(torch.uint8 if self.fp8 else torch.int8) if self.int8 else bf)
        # int8 cache: one fp16 scale per (cache row, KV head), the reference's format (include/kernels/kvcache.h:14-24)
        self.kv_scale = (torch.zeros((2, cfg.layers, self.num_blocks, cfg.block_size, self.hkv), device=dev, dtype=torch.float16)
                         if self.int8 else None)
        self.workspace = None

    # ---- pieces ---------------------------------------------------------------------------------------------
    def rmsnorm(self, x, w):
        return self.torch.nn.functional.rms_norm(x, (x.shape[-1],), w, self.cfg.eps)

    def all_reduce(self, x):
        if self.world > 1:
            self.dist.all_reduce(x)
        return x

    def row_parallel_add_norm(self, a, w, h, norm_w):
        """``h + (a @ w.T summed over the tensor-parallel ranks)`` and its RMSNorm with ``norm_w`` (o_proj / down_proj,
        src/layers/linear.cpp:306-320, followed by the residual add and the next layer norm).  Messages that fit the peer
        buffers take one fused launch (nvk_tp_allreduce_add_rmsnorm); the GEMM writes straight into the addend buffer."""
        n, cols = a.shape[0], w.shape[0]
        comm = self.peer_comm
        if (comm is not None and n * cols <= comm.max_elems and n % self.world == 0 and cols % 8 == 0 and cols <= 8192
                and h.is_contiguous()):
            if (self.fused_linears and n <= self.fused_rows_max and cols % 128 == 0 and a.is_contiguous()
                    and hasattr(comm, "row_linear_all_reduce_add_rmsnorm")):
                return comm.row_linear_all_reduce_add_rmsnorm(a, w, h, norm_w, self.cfg.eps)
            addend, _ = comm.buffers(n, cols)
            self.torch.matmul(a, w.t(), out=addend)
            return comm.all_reduce_add_rmsnorm(h, norm_w, self.cfg.eps, n, cols)
        h = h + self.all_reduce(a @ w.t())
        return h, self.rmsnorm(h, norm_w)

    def ensure_workspace(self, batch, table_width):
        need = self.nvk.decode_attention_workspace_bytes(batch, self.hq, self.hkv, self.cfg.head_dim, table_width,
                                                         self.cfg.block_size)
        if self.workspace is None or self.workspace.numel() < need:
            self.workspace = self.torch.empty(max(need, 1), device=self.dev, dtype=self.torch.uint8)

    def forward(self, tokens, positions, slot_mapping, attend):
        """Hidden states after the last layer.  ``attend(layer_index, q, k, v, out)`` runs attention for one layer
        (``k`` / ``v`` are the step's normalised and rotated keys / values when the cache is int8, else None)."""
        torch, nvk, cfg = self.torch, self.nvk, self.cfg
        h = self.embed[tokens]
        n = h.shape[0]
        q = torch.empty((n, self.hq, cfg.head_dim), device=self.dev, dtype=h.dtype)
        attn = torch.empty_like(q)
        k_step = v_step = rows = None
        if self.int8:
            # As in the reference, an int8 cache takes the unfused route (src/models/transformer.cpp:126-129): the prologue
            # writes the step's K / V into a dense scratch (slot = row), the quantising store then files them in the cache.
            k_step = torch.empty((n, self.hkv, cfg.head_dim), device=self.dev, dtype=h.dtype)
            v_step = torch.empty_like(k_step)
            rows = torch.arange(n, device=self.dev, dtype=torch.int32)
        x = self.rmsnorm(h, self.layers[0]["norm_in"])
        for l, w in enumerate(self.layers):
            if self.fused_linears and not self.int8 and n <= self.fused_rows_max and cfg.head_dim == 128:
                nvk.qkv_linear_norm_rope_store(x if x.is_contiguous() else x.contiguous(), w["w_qkv"], positions, w["q_norm"],
                                               w["k_norm"], cfg.eps, self.cos_sin, slot_mapping, self.kv_cache[0, l],
                                               self.kv_cache[1, l], self.hq, self.hkv, cfg.head_dim, q)
                qkv = None
            else:
                qkv = x @ w["w_qkv"].t()
            if qkv is None:
                pass
            elif self.int8:
                nvk.fused_split_norm_rope_store(qkv, positions, w["q_norm"], w["k_norm"], cfg.eps, self.cos_sin, rows,
                                                k_step, v_step, self.hq, self.hkv, cfg.head_dim, q)
                (nvk.store_kvcache_fp8 if self.fp8 else nvk.store_kvcache_int8)(
                    k_step, v_step, self.kv_cache[0, l], self.kv_cache[1, l], self.kv_scale[0, l], self.kv_scale[1, l], slot_mapping)
            else:
                nvk.fused_split_norm_rope_store(qkv, positions, w["q_norm"], w["k_norm"], cfg.eps, self.cos_sin, slot_mapping,
                                                self.kv_cache[0, l], self.kv_cache[1, l], self.hq, self.hkv, cfg.head_dim, q)
            attend(l, q, k_step, v_step, attn)
            h, x = self.row_parallel_add_norm(attn.view(n, -1), w["w_o"], h, w["norm_post"])
            gu = x @ w["w_gate_up"].t()
            act = torch.nn.functional.silu(gu[:, :self.ffn]) * gu[:, self.ffn:]
            next_norm = self.layers[l + 1]["norm_in"] if l + 1 < len(self.layers) else self.final_norm
            h, x = self.row_parallel_add_norm(act, w["w_down"], h, next_norm)
        return h

    def attend_prefill(self, cu_q, cu_k, tables):
        nvk, cfg = self.nvk, self.cfg

        def attend(l, q, k, v, out):
            if self.int8:   # no prefix hits in this benchmark: the dense keys / values of the step are the whole context
                nvk.launch_prefill_attention_dense(q, cu_q, k, v, cu_k, self.hkv, cfg.head_dim, self.scale, out)
            else:
                nvk.launch_prefill_attention_paged(q, cu_q, self.kv_cache[0, l], self.kv_cache[1, l], cu_k, tables, self.hkv,
                                                   cfg.head_dim, cfg.block_size, self.scale, out)
        return attend

    def attend_decode(self, ctx, tables):
        nvk, cfg = self.nvk, self.cfg

        def attend(l, q, k, v, out):
            if self.int8:
                (nvk.launch_decode_attention_paged_fp8 if self.fp8 else nvk.launch_decode_attention_paged_int8)(
                    q, self.kv_cache[0, l], self.kv_cache[1, l], self.kv_scale[0, l], self.kv_scale[1, l], ctx, tables, self.hkv,
                    cfg.head_dim, cfg.block_size, self.scale, out, self.workspace)
            else:
                nvk.launch_decode_attention_paged(q, self.kv_cache[0, l], self.kv_cache[1, l], ctx, tables, self.hkv,
                                                  cfg.head_dim, cfg.block_size, self.scale, out, self.workspace)
        return attend

    def sample(self, h_rows):
        """Greedy sampling over the vocabulary shards: local max and arg-max, then one gather."""
        torch = self.torch
        logits = (self.rmsnorm(h_rows, self.final_norm) @ self.lm_head.t()).float()
        val, idx = logits.max(dim=-1)
        if self.world == 1:
            return idx
        pair = torch.stack([val, (idx + self.rank * self.vocab).float()], dim=-1).contiguous()   # ids < 2^24: exact
        gathered = torch.empty((self.world,) + pair.shape, device=self.dev, dtype=pair.dtype)
        self.dist.all_gather_into_tensor(gathered, pair)
        best = gathered[..., 0].argmax(dim=0)
        return gathered[..., 1].gather(0, best[None, :])[0].long()

    # ---- steps ----------------------------------------------------------------------------------------------
    def prefill_step(self, arrays):
        """One prefill step over whole prompts; returns the first sampled token of every sequence."""
        torch, nvk, cfg, dev = self.torch, self.nvk, self.cfg, self.dev
        up = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory().to(dev, non_blocking=True)  # noqa: E731
        tokens, positions, slots = up(arrays["tokens"]), up(arrays["positions"]), up(arrays["slot_mapping"])
        cu_q, cu_k, tables = up(arrays["cu_seqlens_q"]), up(arrays["cu_seqlens_k"]), up(arrays["block_tables"])

        h = self.forward(tokens, positions, slots, self.attend_prefill(cu_q, cu_k, tables))
        return self.sample(h[up(arrays["last_rows"])])

    def decode_forward(self, tokens, meta):
        """One decode step on static buffers (capturable): ``meta`` int32 [B, 3 + W] = position, slot, context_len, table."""
        nvk, cfg = self.nvk, self.cfg
        positions, slots, ctx = meta[:, 0].contiguous(), meta[:, 1].contiguous(), meta[:, 2].contiguous()
        tables = meta[:, 3:].contiguous()

        return self.sample(self.forward(tokens, positions, slots, self.attend_decode(ctx, tables)))
