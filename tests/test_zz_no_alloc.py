"""Decode attention through ``rf_attn_decode_static`` -- the entry point for callers that may not
allocate device memory (a control loop that cannot take cudaMalloc's device-wide sync, a host
runtime that already owns every byte of the GPU).  Its split-KV scratch is a fixed buffer inside
the library, so this test hands it nothing but inputs and outputs, calls the exported C symbol
directly, and checks the result against the ordinary entry point (caller-provided scratch) on two
consecutive calls that reuse the same built-in buffer.

Collected last on purpose: a run that stops at the first failure has then already exercised
every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _paged_case(seed, B, Hq, Hkv, hd, kv_lens, dt):
    g = torch.Generator(device="cuda").manual_seed(seed)
    maxp = max((l + 15) // 16 for l in kv_lens) + 1
    total = B * maxp + 2
    perm = torch.randperm(total, generator=torch.Generator().manual_seed(seed))[: B * maxp].to(torch.int32).view(B, maxp)
    k_pool = torch.zeros(total, Hkv, 16, hd, device="cuda", dtype=dt)
    v_pool = torch.zeros_like(k_pool)
    for s, L in enumerate(kv_lens):
        npg = (L + 15) // 16
        pages = perm[s, :npg].long().cuda()
        kk = torch.randn(npg, Hkv, 16, hd, device="cuda", generator=g).to(dt)
        vv = torch.randn(npg, Hkv, 16, hd, device="cuda", generator=g).to(dt)
        k_pool[pages], v_pool[pages] = kk, vv
    q = torch.randn(B, Hq * hd, device="cuda", generator=g).to(dt)
    return q, k_pool, v_pool, perm.cuda().contiguous(), torch.tensor(kv_lens, dtype=torch.int32, device="cuda")


def _args(N, q, out, k_pool, v_pool, pt, kv_len, Hq, Hkv, hd, max_kv, status):
    from rhinoforge_b200.ops.kernels import dtype_code
    a = N.RfAttn()
    a.q, a.ldq, a.out, a.ldo = q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0)
    a.q_rows_total = q.shape[0]
    a.num_seqs, a.Hq, a.Hkv, a.hd = q.shape[0], Hq, Hkv, hd
    a.k_pool, a.v_pool, a.pool_pages = k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0]
    a.page_table, a.pt_stride = pt.data_ptr(), pt.stride(0)
    a.kv_len, a.max_kv_len = kv_len.data_ptr(), max_kv
    a.status, a.dtype = status.data_ptr(), dtype_code(q.dtype)
    return a


def test_static_scratch_decode_matches_regular_entry_point_twice():
    from rhinoforge_b200 import _native as N
    from rhinoforge_b200.ops import kernels as K
    lib = N.lib()
    fn = lib.rf_attn_decode_static            # the exported C symbol itself
    fn.restype = C.c_int
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    Hq, Hkv, hd, dt = 16, 4, 128, torch.float16
    # two different problems back to back: the second call finds the first call's partials in the buffer
    for seed, kv_lens in ((11, [700, 33, 1024, 257]), (12, [90, 1500, 640])):
        B = len(kv_lens)
        q, k_pool, v_pool, pt, kv_len = _paged_case(seed, B, Hq, Hkv, hd, kv_lens, dt)
        ref = torch.zeros_like(q)
        ws = K.attn_decode_scratch(B, Hq, hd, "cuda")
        K.attention_decode(q, ref, Hq=Hq, Hkv=Hkv, hd=hd, kv_len=kv_len, max_kv_len=max(kv_lens), k_pool=k_pool,
                           v_pool=v_pool, page_table=pt, ws=ws, status=status)
        out = torch.zeros_like(q)
        a = _args(N, q, out, k_pool, v_pool, pt, kv_len, Hq, Hkv, hd, max(kv_lens), status)
        # Free device memory as the driver reports it: unlike PyTorch's allocator statistics this also sees a
        # cudaMalloc made inside the library.  (On the first iteration the kernels are already loaded: the regular
        # entry point above ran the same ones.)
        torch.cuda.synchronize()
        free_before, _ = torch.cuda.mem_get_info()
        torch_before = torch.cuda.memory_allocated()
        rc = fn(C.byref(a), stream)
        assert rc == 0, lib.rf_last_error().decode()
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert free_after >= free_before, (free_before, free_after)
        assert torch.cuda.memory_allocated() == torch_before
        assert status[0].item() == 0, status.tolist()
        torch.testing.assert_close(out.float(), ref.float(), rtol=4e-3, atol=4e-3)
        assert out.abs().sum().item() > 0


def test_static_scratch_decode_refuses_oversized_requests():
    from rhinoforge_b200 import _native as N
    lib = N.lib()
    fn = lib.rf_attn_decode_static
    fn.restype = C.c_int
    status = torch.zeros(8, dtype=torch.int32, device="cuda")
    Hq, Hkv, hd, dt = 64, 1, 256, torch.float16
    kv_lens = [8192] * 8      # few CTAs and a long context: many splits, far beyond the built-in buffer
    B = len(kv_lens)
    q = torch.zeros(B, Hq * hd, device="cuda", dtype=dt)
    out = torch.zeros_like(q)
    k_pool = torch.zeros(4, Hkv, 16, hd, device="cuda", dtype=dt)
    pt = torch.zeros(B, 513, dtype=torch.int32, device="cuda")
    kv_len = torch.tensor(kv_lens, dtype=torch.int32, device="cuda")
    a = _args(N, q, out, k_pool, k_pool, pt, kv_len, Hq, Hkv, hd, 8192, status)
    rc = fn(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc != 0
    msg = lib.rf_last_error().decode()
    assert "built-in buffer" in msg and "rf_attn_decode()" in msg
