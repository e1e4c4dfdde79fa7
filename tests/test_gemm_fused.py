"""The linears on either side of attention as this library's tcgen05 GEMMs with fused epilogues.

* ``nvk_linear`` against a torch fp32 matmul of the same 16-bit inputs rounded once (tolerance: accumulation order only).
* ``nvk_qkv_linear_norm_rope_store`` against the unfused sequence it replaces -- torch matmul rounded to the 16-bit type,
  then the CPU oracle's fused_split_norm_rope_store -- V rows bit-exact where the two GEMMs round alike, q / K within one
  unit of the 16-bit type of the oracle applied to the kernel's own product.
* ``nvk_tp_row_linear_allreduce_add_rmsnorm`` for 2, 4, 8 ranks on one GPU against torch: per-rank partial products rounded
  to the 16-bit type, summed in fp32 in rank order, rounded once, residual added, fp32 RMSNorm.
"""
import importlib

import numpy as np
import pytest

import oracle
from util import nvk, to_dev, to_np, workloads

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,out_features,in_features", [(256, 512, 4096), (37, 128, 64), (300, 384, 1000), (1, 256, 72), (129, 1024, 12288)])
def test_linear_matches_torch(dtype, rows, out_features, in_features):
    gen = torch.Generator(device="cuda").manual_seed(rows + in_features)
    x = torch.randn((rows, in_features), generator=gen, device="cuda").to(dtype)
    w = (torch.randn((out_features, in_features), generator=gen, device="cuda") / in_features ** 0.5).to(dtype)
    out = torch.full((rows, out_features), float("nan"), device="cuda", dtype=dtype)
    nvk().linear(x, w, out)
    torch.cuda.synchronize()
    assert nvk().gemm_status() == 0
    want = x.float() @ w.float().t()
    err = (out.float() - want).abs()
    ulp = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    assert bool((err <= want.abs().clamp_min(0.05) * 2 * ulp + 1e-3).all()), float(err.max())


@pytest.mark.parametrize("num_q_heads,num_kv_heads,rows,hidden", [(32, 8, 256, 4096), (4, 1, 37, 512), (6, 2, 130, 1024)])
def test_qkv_linear_with_prologue_matches_gemm_then_oracle_prologue(num_q_heads, num_kv_heads, rows, hidden):
    bf, d, max_pos = torch.bfloat16, 128, 300
    heads = num_q_heads + 2 * num_kv_heads
    gen = torch.Generator(device="cuda").manual_seed(heads)
    x = torch.randn((rows, hidden), generator=gen, device="cuda").to(bf)
    w = (torch.randn((heads * d, hidden), generator=gen, device="cuda") / hidden ** 0.5).to(bf)
    wl = workloads()
    pw = wl.make_prologue_workload(rows, num_q_heads, num_kv_heads, d, max(512, rows + 64), max_pos, seed=3)
    pw["slot_mapping"][3] = -1
    pw["positions"][5] = max_pos + 7
    table = oracle.build_cos_sin_cache(max_pos, d, pw["rope_base"])
    cache_rows = max(512, rows + 64)
    kc = torch.zeros(cache_rows, num_kv_heads, d, dtype=bf, device="cuda")
    vc = torch.zeros_like(kc)
    q_out = torch.full((rows, num_q_heads, d), float("nan"), dtype=bf, device="cuda")
    nvk().qkv_linear_norm_rope_store(x, w, to_dev(pw["positions"]), to_dev(pw["q_norm_weight"], bf), to_dev(pw["k_norm_weight"], bf),
                                     pw["eps"], to_dev(table), to_dev(pw["slot_mapping"]), kc, vc, num_q_heads, num_kv_heads, d, q_out)
    # the product as this library's GEMM rounds it (checked against torch above), then the oracle's prologue
    qkv = torch.empty((rows, heads * d), dtype=bf, device="cuda")
    nvk().linear(x, w, qkv)
    torch.cuda.synchronize()
    assert nvk().gemm_status() == 0
    kc_ref = np.zeros((cache_rows, num_kv_heads, d), np.float32)
    vc_ref = np.zeros_like(kc_ref)
    q_ref = oracle.fused_split_norm_rope_store(to_np(qkv), pw["positions"], pw["q_norm_weight"], pw["k_norm_weight"], pw["eps"], table,
                                               pw["slot_mapping"], kc_ref, vc_ref, num_q_heads, num_kv_heads, d)
    assert np.array_equal(to_np(vc), vc_ref)                      # V: the rounded product, copied
    for got, ref in ((to_np(q_out), q_ref), (to_np(kc), kc_ref)):
        tol = np.maximum(np.abs(ref), 1e-3) * 2.0 ** -7
        assert (np.abs(got - ref) <= tol).all()
        assert (got == ref).mean() > 0.98
    # and the identity-slot / no-norm forms
    k2 = torch.zeros(rows, num_kv_heads, d, dtype=bf, device="cuda")
    v2 = torch.zeros_like(k2)
    q2 = torch.empty_like(q_out)
    nvk().qkv_linear_norm_rope_store(x, w, to_dev(pw["positions"]), None, None, pw["eps"], to_dev(table), None, k2, v2, num_q_heads,
                                     num_kv_heads, d, q2)
    k3, v3, q3 = torch.zeros_like(k2), torch.zeros_like(v2), torch.empty_like(q2)
    nvk().fused_split_norm_rope_store(qkv, to_dev(pw["positions"]), None, None, pw["eps"], to_dev(table), None, k3, v3, num_q_heads,
                                      num_kv_heads, d, q3)
    torch.cuda.synchronize()
    assert torch.equal(v2, v3)
    for a, b in ((q2, q3), (k2, k3)):
        assert bool(((a.float() - b.float()).abs() <= b.float().abs().clamp_min(1e-3) * 2.0 ** -7).all())


@pytest.mark.parametrize("world", [2, 4, 8])
def test_row_parallel_linear_with_allreduce_epilogue_matches_torch(world):
    tc = importlib.import_module("benchmarks.tp_comm")
    dtype, rows, cols, k_local = torch.bfloat16, 8 * world, 1024, 256
    comm = tc.InProcessAllReduce(nvk(), torch, torch.device("cuda"), world, rows * cols, dtype)
    gen = torch.Generator(device="cuda").manual_seed(world)
    norm_w = (1.0 + 0.1 * torch.randn(cols, generator=gen, device="cuda")).to(dtype)
    residuals = [torch.randn((rows, cols), generator=gen, device="cuda").to(dtype)] * world
    residuals = [r.clone() for r in residuals]
    for it in range(3):                                       # repeated: the epoch advances, staging slots are reused
        xs = [torch.randn((rows, k_local), generator=gen, device="cuda").to(dtype) for _ in range(world)]
        ws = [(torch.randn((cols, k_local), generator=gen, device="cuda") / (world * k_local) ** 0.5).to(dtype) for _ in range(world)]
        comm.row_linear_launch(xs, ws, residuals, norm_w, 1e-6)
        torch.cuda.synchronize()
        assert nvk().gemm_status() == 0
        # what the unfused sequence computes, with this library's own GEMM for the partial products
        acc = torch.zeros((rows, cols), device="cuda", dtype=torch.float32)
        for x, w in zip(xs, ws):
            part = torch.empty((rows, cols), device="cuda", dtype=dtype)
            nvk().linear(x, w, part)
            acc += part.float()
        torch.cuda.synchronize()
        want_h = residuals[0] + acc.to(dtype)
        hf = want_h.float()
        want_x = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * norm_w.float()
        for r in range(world):
            h = comm.result[r].view(rows, cols)
            x_norm = comm.normed[r].view(rows, cols)
            assert torch.equal(h, want_h), (it, r)
            assert torch.equal(x_norm, comm.normed[0].view(rows, cols))
            assert bool(((x_norm.float() - want_x).abs() <= want_x.abs().clamp_min(1e-2) * 2.0 ** -7).all())
            assert comm.status(r) == 0
        residuals = [comm.result[r].view(rows, cols).clone() for r in range(world)]
    # a plain fused all-reduce on the same buffers afterwards: the two kinds of calls may alternate
    for a in comm.addend:
        a.copy_(torch.randn(a.shape, generator=gen, device="cuda"))
    comm.launch(rows, cols, residuals=residuals, weight=norm_w)
    torch.cuda.synchronize()
    acc = torch.zeros(rows * cols, device="cuda", dtype=torch.float32)
    for a in comm.addend:
        acc += a.float()
    assert torch.equal(comm.result[0].view(rows, cols), residuals[0] + acc.to(dtype).view(rows, cols))


def test_gemm_entry_points_refuse_what_they_cannot_run():
    x = torch.zeros(4, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        nvk().linear(x, torch.zeros(100, 64, device="cuda", dtype=torch.bfloat16), torch.zeros(4, 100, device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ValueError):
        nvk().linear(x.float(), torch.zeros(128, 64, device="cuda"), torch.zeros(4, 128, device="cuda"))
    assert nvk().gemm_status() == 0
