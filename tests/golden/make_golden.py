"""Generates the golden fixtures of tests/golden/ by running the REFERENCE's own CUDA kernels.

Run on a machine with a GPU after ``make -C oracle ref`` has built ``oracle/_ref/libnvk_ref.so`` (the
reference's unmodified attention.cu / kvcache.cu / split_qkv.cu compiled for sm_100a behind
``oracle/ref_shim.cpp``):

    python tests/golden/make_golden.py [output_dir]

Inputs are regenerated from seeds by ``benchmarks/workloads.py`` (the ``CASES`` table below is the
single source of truth, imported by the tests), so a fixture stores only the reference's outputs plus a
checksum of the inputs it was produced from.  Every case is small: the whole directory is a few hundred KB.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

F16, BF16, F32, I32 = 0, 1, 2, 3

# name -> (kind, dtype, generator keyword arguments)
CASES = {
    "decode_f32_qwen06_shape": ("decode", "f32", dict(batch=4, num_heads=16, num_kv_heads=8, head_dim=128, block_size=256,
                                                      ctx_lo=1, ctx_hi=600, seed=501, value_scale=0.5, prescale_q=True,
                                                      rounded=False)),
    "decode_bf16_gqa4": ("decode", "bf16", dict(batch=5, num_heads=32, num_kv_heads=8, head_dim=128, block_size=256,
                                                ctx_lo=1, ctx_hi=900, seed=502)),
    "prefill_dense_f32": ("prefill", "f32", dict(q_lens=[5, 33, 1], prefix_lens=[0, 0, 7], num_heads=4, num_kv_heads=2,
                                                 head_dim=64, block_size=16, seed=503, rounded=False, paged=False)),
    "prefill_paged_bf16_prefix": ("prefill", "bf16", dict(q_lens=[130, 40, 65], prefix_lens=[256, 0, 128], num_heads=2,
                                                          num_kv_heads=1, head_dim=128, block_size=128, seed=504)),
    "store_bf16": ("store", "bf16", dict(tokens=37, row_elems=2 * 128, cache_rows=128, seed=505)),
    "prologue_bf16": ("prologue", "bf16", dict(rows=19, num_q_heads=8, num_kv_heads=2, head_dim=128, cache_rows=256,
                                               max_positions=300, seed=506)),
    # int8 KV cache: every row of a bf16 cache goes through the reference's quantising store, then its int8 decode
    "int8_kv_bf16": ("int8", "bf16", dict(batch=4, num_heads=8, num_kv_heads=2, head_dim=128, block_size=16,
                                          ctx_lo=1, ctx_hi=90, seed=507)),
}


def workloads():
    import __graft_entry__ as entry
    import importlib
    entry.load_package()
    return importlib.import_module("benchmarks.workloads")


def make_inputs(name):
    """Seeded inputs of a case as numpy arrays (float32 holding values representable in the case's dtype)."""
    kind, dtype, kw = CASES[name]
    wl = workloads()
    if kind in ("decode", "int8"):
        return wl.make_decode_workload(**kw)
    if kind == "prefill":
        return wl.make_prefill_workload(**kw)
    if kind == "store":
        rng = np.random.default_rng(kw["seed"])
        key = wl.round_bf16(rng.standard_normal((kw["tokens"], kw["row_elems"])).astype(np.float32))
        value = wl.round_bf16(rng.standard_normal((kw["tokens"], kw["row_elems"])).astype(np.float32))
        slots = rng.permutation(kw["cache_rows"])[:kw["tokens"]].astype(np.int32)
        slots[::5] = -1
        slots[3] = kw["cache_rows"] + 9
        zeros = np.zeros((kw["cache_rows"], kw["row_elems"]), dtype=np.float32)
        return {"key": key, "value": value, "slot_mapping": slots, "k_cache": zeros, "v_cache": zeros.copy()}
    if kind == "prologue":
        w = wl.make_prologue_workload(kw["rows"], kw["num_q_heads"], kw["num_kv_heads"], kw["head_dim"], kw["cache_rows"],
                                      kw["max_positions"], kw["seed"])
        w["slot_mapping"][2] = -1
        w["positions"][4] = kw["max_positions"] + 3
        return w
    raise KeyError(kind)


def input_checksum(inputs) -> str:
    h = hashlib.sha256()
    for k in sorted(inputs):
        v = inputs[k]
        if isinstance(v, np.ndarray):
            h.update(k.encode())
            h.update(np.ascontiguousarray(v).tobytes())
    return h.hexdigest()[:16]


def load_fixture(name):
    """Fixture arrays as float32 (bf16 bit patterns are widened exactly)."""
    data = np.load(os.path.join(HERE, name + ".npz"))
    out = {}
    for k in data.files:
        a = data[k]
        if a.dtype == np.uint16:
            a = (a.astype(np.uint32) << 16).view(np.float32)
        out[k] = a
    return out


def cos_sin_table(max_positions, head_dim, base):
    inv = (1.0 / np.power(np.float32(base), np.arange(0, head_dim, 2, dtype=np.float32) / np.float32(head_dim))).astype(np.float32)
    ang = (np.arange(max_positions, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    return np.concatenate([np.cos(ang), np.sin(ang)], axis=1).astype(np.float32)


def main(out_dir):
    import torch
    ref = ctypes.CDLL(os.path.join(ROOT, "oracle", "_ref", "libnvk_ref.so"))
    ref.nvkref_last_error.restype = ctypes.c_char_p
    dev = torch.device("cuda:0")
    tdt = {"f32": (torch.float32, F32), "bf16": (torch.bfloat16, BF16)}
    P = lambda t: ctypes.c_void_p(t.data_ptr())  # noqa: E731

    def bits(t):   # float32 outputs as they are; bf16 outputs as their 16-bit patterns (see load_fixture)
        return t.cpu().numpy() if t.dtype == torch.float32 else t.cpu().view(torch.int16).numpy().view(np.uint16)

    def check(rc):
        if rc:
            raise RuntimeError(ref.nvkref_last_error().decode())

    os.makedirs(out_dir, exist_ok=True)
    keep = []   # device tensors must outlive the asynchronous launches that read them

    def D(a, dt=None):  # noqa: F811
        t = torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        t = t.to(dt) if dt is not None else t
        keep.append(t)
        return t

    for name, (kind, dtype, kw) in CASES.items():
        w = make_inputs(name)
        tt, code = tdt[dtype]
        out = {"checksum": np.array(input_checksum(w))}
        if kind == "decode":
            q, kc, vc = D(w["q"], tt), D(w["k_cache"], tt), D(w["v_cache"], tt)
            check(ref.nvkref_store_kvcache(P(D(w["k_new"], tt)), P(D(w["v_new"], tt)), P(kc), P(vc), P(D(w["slot_mapping"])), I32,
                                           ctypes.c_int64(kw["batch"]), ctypes.c_int64(kw["num_kv_heads"] * kw["head_dim"]),
                                           ctypes.c_int64(kc.shape[0] * kw["block_size"]), code, None))
            o = torch.empty_like(q)
            ctx, bt = D(w["context_lens"]), D(w["block_tables"])
            check(ref.nvkref_decode_attention_paged(P(q), P(kc), P(vc), P(ctx), P(bt), ctypes.c_int64(kw["batch"]),
                                                    ctypes.c_int64(bt.shape[1]), ctypes.c_int64(kc.shape[0]), kw["num_heads"],
                                                    kw["num_kv_heads"], kw["head_dim"], kw["block_size"],
                                                    ctypes.c_float(w["scale"]), P(o), code, None))
            out["out"] = bits(o)
        elif kind == "int8":
            hkv, d, bs = kw["num_kv_heads"], kw["head_dim"], kw["block_size"]
            blocks = w["k_cache"].shape[0]
            rows = blocks * bs
            key, value = D(w["k_cache"].reshape(rows, hkv, d), tt), D(w["v_cache"].reshape(rows, hkv, d), tt)
            kc = torch.zeros((blocks, bs, hkv, d), dtype=torch.int8, device=dev)
            vc = torch.zeros_like(kc)
            ks = torch.zeros((blocks, bs, hkv), dtype=torch.float16, device=dev)
            vs = torch.zeros_like(ks)
            slots = torch.arange(rows, dtype=torch.int32, device=dev)
            keep.extend([kc, vc, ks, vs, slots])
            check(ref.nvkref_store_kvcache_int8(P(key), P(value), P(kc), P(vc), P(ks), P(vs), P(slots), ctypes.c_int64(rows), hkv, d,
                                                ctypes.c_int64(blocks), bs, code, None))
            q = D(w["q"], tt)
            o = torch.empty_like(q)
            ctx, bt = D(w["context_lens"]), D(w["block_tables"])
            check(ref.nvkref_decode_attention_paged_int8(P(q), P(kc), P(vc), P(ks), P(vs), P(ctx), P(bt), ctypes.c_int64(kw["batch"]),
                                                         ctypes.c_int64(bt.shape[1]), ctypes.c_int64(blocks), kw["num_heads"], hkv, d, bs,
                                                         ctypes.c_float(w["scale"]), P(o), code, None))
            out["k_cache"] = kc.cpu().numpy().reshape(rows, hkv, d)
            out["v_cache"] = vc.cpu().numpy().reshape(rows, hkv, d)
            out["k_scale"] = ks.float().cpu().numpy().reshape(rows, hkv)      # fp16 values, widened exactly
            out["v_scale"] = vs.float().cpu().numpy().reshape(rows, hkv)
            out["out"] = bits(o)
        elif kind == "prefill":
            q = D(w["q"], tt)
            o = torch.empty_like(q)
            cq, ck = D(w["cu_q"]), D(w["cu_k"])
            if kw.get("paged", True):
                kc, vc, bt = D(w["k_cache"], tt), D(w["v_cache"], tt), D(w["block_tables"])
                check(ref.nvkref_prefill_attention_paged(P(q), P(kc), P(vc), P(cq), P(ck), P(bt), ctypes.c_int64(len(kw["q_lens"])),
                                                         ctypes.c_int64(q.shape[0]), ctypes.c_int64(bt.shape[1]),
                                                         ctypes.c_int64(kc.shape[0]), kw["num_heads"], kw["num_kv_heads"],
                                                         kw["head_dim"], kw["block_size"], ctypes.c_float(w["scale"]), P(o), code, None))
            else:
                k, v = D(w["k"], tt), D(w["v"], tt)
                check(ref.nvkref_prefill_attention_dense(P(q), P(k), P(v), P(cq), P(ck), ctypes.c_int64(len(kw["q_lens"])),
                                                         ctypes.c_int64(q.shape[0]), ctypes.c_int64(k.shape[0]), kw["num_heads"],
                                                         kw["num_kv_heads"], kw["head_dim"], ctypes.c_float(w["scale"]), P(o), code, None))
            out["out"] = bits(o)
        elif kind == "store":
            kc, vc = D(w["k_cache"], tt), D(w["v_cache"], tt)
            check(ref.nvkref_store_kvcache(P(D(w["key"], tt)), P(D(w["value"], tt)), P(kc), P(vc), P(D(w["slot_mapping"])), I32,
                                           ctypes.c_int64(kw["tokens"]), ctypes.c_int64(kw["row_elems"]),
                                           ctypes.c_int64(kw["cache_rows"]), code, None))
            out["k_cache"] = bits(kc)
            out["v_cache"] = bits(vc)
        elif kind == "prologue":
            hq, hkv, d = kw["num_q_heads"], kw["num_kv_heads"], kw["head_dim"]
            table = cos_sin_table(kw["max_positions"], d, w["rope_base"])
            kc = torch.zeros(kw["cache_rows"], hkv, d, dtype=tt, device=dev)
            vc = torch.zeros_like(kc)
            qo = torch.empty(kw["rows"], hq, d, dtype=tt, device=dev)
            check(ref.nvkref_fused_split_norm_rope_store(
                P(D(w["qkv"], tt)), P(D(w["positions"])), P(D(w["q_norm_weight"], tt)), P(D(w["k_norm_weight"], tt)),
                ctypes.c_float(w["eps"]), P(D(table)), ctypes.c_int64(kw["max_positions"]), P(D(w["slot_mapping"])), P(kc), P(vc),
                ctypes.c_int64(kw["cache_rows"]), ctypes.c_int64(kw["rows"]), hq, hkv, d, P(qo), code, None))
            out["q_out"] = bits(qo)
            out["k_cache"] = bits(kc)
            out["v_cache"] = bits(vc)
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, name + ".npz"), **out)
        print("wrote", name, {k: getattr(v, "shape", None) for k, v in out.items()})


if __name__ == "__main__":
    # python tests/golden/make_golden.py [output_dir] [case ...]: with case names, only those fixtures are (re)written
    if len(sys.argv) > 2:
        CASES = {k: v for k, v in CASES.items() if k in sys.argv[2:]}
    main(sys.argv[1] if len(sys.argv) > 1 else HERE)
