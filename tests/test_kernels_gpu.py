"""Numerics of every sm_100a kernel against a plain PyTorch fp32 reference of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = [torch.float16, torch.bfloat16]


def _tol(dt):
    return (2e-2, 2e-2) if dt == torch.bfloat16 else (4e-3, 4e-3)


def _close(a, b, dt, scale=1.0):
    rtol, atol = _tol(dt)
    torch.testing.assert_close(a.float(), b.float(), rtol=rtol, atol=atol * scale)


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)


@pytest.fixture()
def status():
    s = torch.zeros(8, dtype=torch.int32, device="cuda")
    yield s
    torch.cuda.synchronize()
    assert s[0].item() == 0, f"kernel status {s.tolist()}"


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K", [(1, 256, 512), (5, 384, 1024), (16, 4096, 4096), (64, 1000, 4304), (200, 640, 320),
                                   (128, 256, 64), (300, 512, 1024), (1024, 768, 2048), (257, 1152, 1152)])
def test_gemm_plain(dt, M, N, K, status):
    from rhinoforge_b200.ops import kernels as K_
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(dt)
    y = K_.gemm(x, w, status=status)
    ref = x.float() @ w.float().t()
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()))


@pytest.mark.parametrize("swap", [0, 1])
@pytest.mark.parametrize("splits", [1, 3])
def test_gemm_epilogue_bias_residual_scale(swap, splits, status):
    from rhinoforge_b200.ops import kernels as K_
    dt = torch.float16
    M, N, K = 48, 640, 1536
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(dt)
    b = torch.randn(N, device="cuda").to(dt)
    sc = (torch.rand(N, device="cuda") + 0.5).to(dt)
    r = torch.randn(M, N, device="cuda").to(dt)
    rs = torch.rand(M, device="cuda") + 0.5
    y = K_.gemm(x, w, bias=b, scale=sc, residual=r, row_scale=rs, status=status, force_swap=swap,
                force_splits=splits)
    ref = (x.float() @ w.float().t()) * rs[:, None] * sc.float() + b.float() + r.float()
    _close(y, ref, dt, scale=4.0)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,swap,splits", [(3, 1, 1), (40, 1, 2), (40, 0, 1), (300, 0, 1)])
@pytest.mark.parametrize("act", ["silu_mul", "gelu_tanh_mul"])
def test_gemm_dual_glu(dt, M, swap, splits, act, status):
    from rhinoforge_b200.ops import kernels as K_
    N, K = 384, 1024
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(2 * N, K, device="cuda") * 0.05).to(dt)
    y = K_.gemm(x, w, act=act, dual=True, status=status, force_swap=swap, force_splits=splits)
    g = x.float() @ w[:N].float().t()
    u = x.float() @ w[N:].float().t()
    a = torch.nn.functional.silu(g) if act == "silu_mul" else torch.nn.functional.gelu(g, approximate="tanh")
    _close(y, a * u, dt, scale=2.0)


@pytest.mark.parametrize("act", ["gelu_tanh", "gelu_erf", "silu"])
def test_gemm_unary_act(act, status):
    from rhinoforge_b200.ops import kernels as K_
    dt = torch.float16
    x = (torch.randn(70, 512, device="cuda") * 0.5).to(dt)
    w = (torch.randn(256, 512, device="cuda") * 0.05).to(dt)
    y = K_.gemm(x, w, act=act, status=status)
    z = x.float() @ w.float().t()
    ref = {"gelu_tanh": lambda t: torch.nn.functional.gelu(t, approximate="tanh"),
           "gelu_erf": torch.nn.functional.gelu, "silu": torch.nn.functional.silu}[act](z)
    _close(y, ref, dt)


def test_gemm_is_deterministic(status):
    from rhinoforge_b200.ops import kernels as K_
    x = (torch.randn(32, 4096, device="cuda") * 0.5).half()
    w = (torch.randn(1024, 4096, device="cuda") * 0.05).half()
    a = K_.gemm(x, w, status=status, force_splits=4).clone()
    b = K_.gemm(x, w, status=status, force_splits=4)
    assert torch.equal(a, b)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M", [1, 2, 3, 8])
@pytest.mark.parametrize("int8", [False, True])
def test_gemv(dt, M, int8):
    from rhinoforge_b200.ops import kernels as K_
    N, K = 515, 1024
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    r = torch.randn(M, N, device="cuda").to(dt)
    if int8:
        w = torch.randint(-127, 128, (N, K), device="cuda", dtype=torch.int8)
        sc = (torch.rand(N, device="cuda") * 0.01).to(dt)
        y = K_.gemm(x, w, scale=sc, residual=r, use_gemv=True)
        ref = (x.float() @ w.float().t()) * sc.float() + r.float()
    else:
        w = (torch.randn(N, K, device="cuda") * 0.05).to(dt)
        y = K_.gemm(x, w, residual=r, use_gemv=True)
        ref = x.float() @ w.float().t() + r.float()
    _close(y, ref, dt, scale=4.0)


def test_gemv_dual():
    from rhinoforge_b200.ops import kernels as K_
    x = (torch.randn(2, 512, device="cuda") * 0.5).half()
    w = (torch.randn(2 * 300, 512, device="cuda") * 0.05).half()
    y = K_.gemm(x, w, act="silu_mul", dual=True, use_gemv=True)
    g, u = x.float() @ w[:300].float().t(), x.float() @ w[300:].float().t()
    _close(y, torch.nn.functional.silu(g) * u, torch.float16)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("gemma", [False, True])
def test_rmsnorm(dt, gemma):
    from rhinoforge_b200.ops import kernels as K_
    x = torch.randn(37, 1024, device="cuda").to(dt)
    r = torch.randn(37, 1024, device="cuda").to(dt)
    w = (torch.randn(1024, device="cuda") * 0.1 + (0 if gemma else 1)).to(dt)
    ro = torch.empty_like(x)
    y = K_.rmsnorm(x, w, 1e-6, residual=r, residual_out=ro, gemma=gemma)
    h = (x.float() + r.float()).to(dt).float()
    n = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + 1e-6)
    ref = n * (1 + w.float()) if gemma else w.float() * n.to(dt).float()
    _close(y, ref, dt)
    _close(ro, h, dt)


def test_rmsnorm_adarms_and_gated_residual():
    from rhinoforge_b200.ops import kernels as K_
    dt = torch.float16
    B, T, H = 3, 50, 1024
    x = torch.randn(B * T, H, device="cuda").to(dt)
    mod = (torch.randn(B, 3 * H, device="cuda") * 0.3).to(dt)
    y = K_.rmsnorm(x, None, 1e-6, mod=mod, rows_per_mod=T)
    n = x.float() * torch.rsqrt(x.float().pow(2).mean(-1, keepdim=True) + 1e-6)
    sc, sh, gt = mod.float().view(B, 1, 3 * H).chunk(3, -1)
    ref = (n.view(B, T, H) * (1 + sc) + sh).view(B * T, H)
    _close(y, ref, dt)
    x2 = x.clone()
    K_.gated_residual(x2, y, mod, T)
    _close(x2, (x.float().view(B, T, H) + gt * y.float().view(B, T, H)).view(B * T, H), dt)


@pytest.mark.parametrize("dt", DT)
def test_layernorm_l2norm(dt):
    from rhinoforge_b200.ops import kernels as K_
    x = torch.randn(33, 1152, device="cuda").to(dt)
    w, b = torch.randn(1152, device="cuda").to(dt), torch.randn(1152, device="cuda").to(dt)
    y = K_.layernorm(x, w, b, 1e-6)
    _close(y, torch.nn.functional.layer_norm(x.float(), (1152,), w.float(), b.float(), 1e-6), dt)
    z = K_.l2norm(x[:, :128].contiguous(), 1e-6)
    xf = x[:, :128].float()
    _close(z, xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + 1e-6), dt)


def _rope_tables(max_pos, rot, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, rot, 2, device=device).float() / rot))
    ang = torch.arange(max_pos, device=device).float()[:, None] * inv[None]
    return ang.cos().contiguous(), ang.sin().contiguous()


def _rot_half(x):
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], -1)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("hd,rot", [(128, 128), (256, 64), (64, 64)])
def test_qk_norm_rope_kv_insert(dt, hd, rot):
    from rhinoforge_b200.ops import kernels as K_
    Hq, Hkv, T = 6, 2, 21
    seqs = 3
    qkv = torch.randn(T, (Hq + 2 * Hkv) * hd, device="cuda").to(dt)
    orig = qkv.clone()
    qw, kw = (torch.rand(hd, device="cuda") + 0.5).to(dt), (torch.rand(hd, device="cuda") + 0.5).to(dt)
    cos, sin = _rope_tables(512, rot, 1e6, "cuda")
    seq_of_tok = torch.arange(T, device="cuda", dtype=torch.int32) % seqs
    pos = (torch.arange(T, device="cuda", dtype=torch.int32) // seqs + 30).contiguous()
    pages = 16
    k_pool = torch.zeros(pages, Hkv, 16, hd, device="cuda", dtype=dt)
    v_pool = torch.zeros_like(k_pool)
    page_table = torch.arange(seqs * 4, device="cuda", dtype=torch.int32).view(seqs, 4).contiguous()
    K_.qk_norm_rope_kv(qkv, Hq, Hkv, hd, pos=pos, cos=cos, sin=sin, rot_dim=rot, q_norm_w=qw, k_norm_w=kw,
                       k_pool=k_pool, v_pool=v_pool, page_table=page_table, seq_of_tok=seq_of_tok)
    o = orig.float().view(T, Hq + 2 * Hkv, hd)

    def ref(x, w):
        n = (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6)).to(dt).float() * w.float()
        n = n.to(dt).float()
        c = cos[pos.long()][:, None, :].repeat(1, 1, 2)
        s = sin[pos.long()][:, None, :].repeat(1, 1, 2)
        r = n[..., :rot] * c + _rot_half(n[..., :rot]) * s
        return torch.cat([r, n[..., rot:]], -1)

    q_ref, k_ref, v_ref = ref(o[:, :Hq], qw), ref(o[:, Hq:Hq + Hkv], kw), o[:, Hq + Hkv:]
    _close(qkv.view(T, -1, hd)[:, :Hq], q_ref, dt)
    for t in range(T):
        s, p = int(seq_of_tok[t]), int(pos[t])
        page = int(page_table[s, p // 16])
        _close(k_pool[page, :, p % 16], k_ref[t], dt)
        _close(v_pool[page, :, p % 16], v_ref[t], dt)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("hd,rot,Hq,Hkv", [(64, 64, 6, 6), (128, 128, 5, 2), (256, 64, 3, 1), (128, 64, 4, 4)])
@pytest.mark.parametrize("variant", ["plain", "norm", "gemma_rope_first", "mrope_vnorm", "pool"])
def test_qk_norm_rope_kv_prefill_sized(dt, hd, rot, Hq, Hkv, variant):
    """Launches of 512 tokens or more take the 16-byte kernel: the same rows through one 640-token launch and through
    two launches of 320 (below the switch, the scalar kernel) must agree to one rounding step, in every mode."""
    from rhinoforge_b200.ops import kernels as K_
    torch.manual_seed(3)
    T, half = 640, rot // 2
    W = (Hq + 2 * Hkv) * hd
    qkv = (torch.randn(T, W, device="cuda") * 0.7).to(dt)
    axes = 3 if variant == "mrope_vnorm" else 1
    pos = torch.randint(0, 900, (T, axes), device="cuda", dtype=torch.int32)
    ang = torch.arange(1024, device="cuda", dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(half, device="cuda") / half))[None]
    kw = dict(pos=pos, cos=ang.cos().contiguous(), sin=ang.sin().contiguous(), rot_dim=rot)
    if variant in ("norm", "gemma_rope_first", "mrope_vnorm", "pool"):
        kw.update(q_norm_w=(1 + 0.1 * torch.randn(hd, device="cuda")).to(dt), k_norm_w=(1 + 0.1 * torch.randn(hd, device="cuda")).to(dt))
    if variant == "gemma_rope_first":
        kw.update(gemma=True, rope_before_norm=True)
    if variant == "mrope_vnorm":
        kw.update(axis_of_freq=torch.randint(0, 3, (half,), device="cuda", dtype=torch.int8), v_norm=True)
    outs = []
    pt = torch.randperm(T // 16 + 2, device="cuda").to(torch.int32)[None].contiguous()     # one shuffled page table for both runs
    for chunks in (1, 2):
        buf = qkv.clone()
        q_out = torch.zeros(T, Hq * hd, device="cuda", dtype=dt) if variant == "pool" else None
        pools = None
        if variant == "pool":
            pages = T // 16 + 2
            pools = (torch.zeros(pages, Hkv, 16, hd, device="cuda", dtype=dt), torch.zeros(pages, Hkv, 16, hd, device="cuda", dtype=dt))
        n = T // chunks
        for c in range(chunks):
            sl = slice(c * n, (c + 1) * n)
            extra = {}
            if variant == "pool":
                extra = dict(k_pool=pools[0], v_pool=pools[1], page_table=pt, seq_of_tok=torch.zeros(n, device="cuda", dtype=torch.int32),
                             cache_pos=torch.arange(c * n, (c + 1) * n, device="cuda", dtype=torch.int32), q_out=q_out[sl])
            K_.qk_norm_rope_kv(buf[sl], Hq, Hkv, hd, **{**kw, "pos": pos[sl].contiguous()}, **extra)
        torch.cuda.synchronize()
        outs.append((buf, q_out, pools))
    (b1, q1, p1), (b2, q2, p2) = outs

    def same(x, y):            # one rounding step of the 16-bit type at most (the two kernels may contract their FMAs differently)
        tol = (2.0 ** -10 if dt == torch.float16 else 2.0 ** -7) * max(1.0, float(y.float().abs().max()))
        return float((x.float() - y.float()).abs().max()) <= tol
    assert same(b1, b2)
    if variant == "pool":
        assert same(q1, q2) and same(p1[0], p2[0]) and same(p1[1], p2[1])
        assert float(p1[0].abs().max()) > 0 and float(q1.abs().max()) > 0
    else:
        assert not torch.equal(b1, qkv)


def test_mrope_axis_select():
    from rhinoforge_b200.ops import kernels as K_
    dt, hd, T = torch.float16, 128, 9
    qkv = torch.randn(T, 3 * hd, device="cuda").to(dt)
    orig = qkv.clone()
    cos, sin = _rope_tables(256, hd, 1e6, "cuda")
    pos = torch.randint(0, 200, (T, 3), device="cuda", dtype=torch.int32)
    sec = [24, 20, 20]
    axis = torch.zeros(hd // 2, dtype=torch.int8)
    for dim, off in ((1, 1), (2, 2)):
        axis[off:sec[dim] * 3:3] = dim
    K_.qk_norm_rope_kv(qkv, 1, 1, hd, pos=pos, cos=cos, sin=sin, axis_of_freq=axis.cuda(), write_k_inplace=True)
    idx = pos.long()[:, axis.long().cuda()]  # [T, hd/2]
    f = torch.arange(hd // 2, device="cuda")
    c = cos[idx, f].repeat(1, 2)
    s = sin[idx, f].repeat(1, 2)
    for h in range(2):
        x = orig.float().view(T, 3, hd)[:, h]
        _close(qkv.view(T, 3, hd)[:, h], x * c + _rot_half(x) * s, dt)


def _sdpa_ref(q, k, v, mask):
    # q [Hq, Lq, hd], k/v [Hkv, Lk, hd], mask [Lq, Lk] bool
    G = q.shape[0] // k.shape[0]
    k = k.repeat_interleave(G, 0)
    v = v.repeat_interleave(G, 0)
    s = (q.float() @ k.float().transpose(1, 2)) / math.sqrt(q.shape[-1])
    s = s.masked_fill(~mask[None], float("-inf"))
    p = torch.softmax(s, -1)
    p = torch.nan_to_num(p)
    return p @ v.float()


def _paged(Hkv, hd, kv_lens, dt, extra_pages=3):
    seqs = len(kv_lens)
    maxp = max((l + 15) // 16 for l in kv_lens) + 1
    total = seqs * maxp + extra_pages
    perm = torch.randperm(total)[: seqs * maxp].to(torch.int32).view(seqs, maxp)
    k_pool = torch.zeros(total, Hkv, 16, hd, device="cuda", dtype=dt)
    v_pool = torch.zeros_like(k_pool)
    ks, vs = [], []
    for s, L in enumerate(kv_lens):
        k = torch.randn(Hkv, L, hd, device="cuda").to(dt)
        v = torch.randn(Hkv, L, hd, device="cuda").to(dt)
        for t in range(L):
            pg = int(perm[s, t // 16])
            k_pool[pg, :, t % 16] = k[:, t]
            v_pool[pg, :, t % 16] = v[:, t]
        ks.append(k)
        vs.append(v)
    return k_pool, v_pool, perm.cuda().contiguous(), ks, vs


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("hd,Hq,Hkv", [(128, 8, 2), (64, 4, 4), (256, 8, 1)])
def test_attn_prefill_paged_causal(dt, hd, Hq, Hkv, status):
    from rhinoforge_b200.ops import kernels as K_
    q_lens, kv_lens = [70, 33, 128], [70, 97, 128]
    k_pool, v_pool, pt, ks, vs = _paged(Hkv, hd, kv_lens, dt)
    q_start = [0, 70, 103]
    Tq = sum(q_lens)
    q = torch.randn(Tq, Hq * hd, device="cuda").to(dt)
    out = torch.zeros_like(q)
    i32 = lambda l: torch.tensor(l, dtype=torch.int32, device="cuda")
    K_.attention_prefill(q, out, Hq=Hq, Hkv=Hkv, hd=hd, q_start=i32(q_start), q_len=i32(q_lens), kv_len=i32(kv_lens),
                         max_q_len=max(q_lens), k_pool=k_pool, v_pool=v_pool, page_table=pt, causal=True,
                         status=status)
    for s in range(3):
        Lq, Lk = q_lens[s], kv_lens[s]
        qs = q[q_start[s]:q_start[s] + Lq].view(Lq, Hq, hd).transpose(0, 1)
        qi = torch.arange(Lq, device="cuda")[:, None] + (Lk - Lq)
        mask = torch.arange(Lk, device="cuda")[None] <= qi
        ref = _sdpa_ref(qs, ks[s], vs[s], mask).transpose(0, 1).reshape(Lq, Hq * hd)
        _close(out[q_start[s]:q_start[s] + Lq], ref, dt)


@pytest.mark.parametrize("mode", ["bidir", "mask", "segments", "window"])
def test_attn_prefill_contiguous_masks(mode, status):
    from rhinoforge_b200.ops import kernels as K_
    dt, hd, H = torch.float16, 64, 4
    L = 201
    qkv = torch.randn(L, 3 * H * hd, device="cuda").to(dt)
    q, k, v = qkv[:, :H * hd], qkv[:, H * hd:2 * H * hd], qkv[:, 2 * H * hd:]
    out = torch.zeros(L, H * hd, device="cuda", dtype=dt)
    i32 = lambda l: torch.tensor(l, dtype=torch.int32, device="cuda")
    kw = dict(Hq=H, Hkv=H, hd=hd, q_start=i32([0]), q_len=i32([L]), kv_len=i32([L]), max_q_len=L, k=k, v=v,
              kv_start=i32([0]), causal=False, status=status)
    full = torch.ones(L, L, dtype=torch.bool, device="cuda")
    if mode == "bidir":
        mask = full
    elif mode == "mask":
        mask = torch.rand(L, L, device="cuda") > 0.3
        mask[:, 0] = True
        kw["mask"] = mask.contiguous()
    elif mode == "segments":
        seg = (torch.arange(L, device="cuda") // 37).to(torch.int32)
        mask = seg[:, None] == seg[None]
        kw["seg_q"], kw["seg_k"] = seg, seg
    else:
        kw["causal"], kw["window"] = True, 48
        i = torch.arange(L, device="cuda")
        mask = (i[None] <= i[:, None]) & (i[None] > i[:, None] - 48)
    K_.attention_prefill(q, out, **kw)
    tr = lambda t: t.reshape(L, H, hd).transpose(0, 1)
    ref = _sdpa_ref(tr(q), tr(k), tr(v), mask).transpose(0, 1).reshape(L, H * hd)
    _close(out, ref, dt)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("hd,Hq,Hkv", [(128, 32, 8), (128, 8, 1), (64, 4, 2), (256, 8, 1)])
@pytest.mark.parametrize("split", [False, True])
def test_attn_decode_paged(dt, hd, Hq, Hkv, split, status):
    from rhinoforge_b200.ops import kernels as K_
    kv_lens = [1, 17, 300, 1025, 64]
    k_pool, v_pool, pt, ks, vs = _paged(Hkv, hd, kv_lens, dt)
    B = len(kv_lens)
    q = torch.randn(B, Hq * hd, device="cuda").to(dt)
    out = torch.zeros_like(q)
    ws = K_.attn_decode_scratch(B, Hq, hd, "cuda") if split else None
    K_.attention_decode(q, out, Hq=Hq, Hkv=Hkv, hd=hd, kv_len=torch.tensor(kv_lens, dtype=torch.int32, device="cuda"),
                        max_kv_len=max(kv_lens), k_pool=k_pool, v_pool=v_pool, page_table=pt, ws=ws, status=status)
    for s in range(B):
        L = kv_lens[s]
        ref = _sdpa_ref(q[s].view(Hq, 1, hd), ks[s], vs[s], torch.ones(1, L, dtype=torch.bool, device="cuda"))
        _close(out[s], ref.reshape(Hq * hd), dt)


def test_embedding_scatter_eltwise_cast_argmax():
    from rhinoforge_b200.ops import kernels as K_
    dt = torch.float16
    table = torch.randn(1000, 256, device="cuda").to(dt)
    ids = torch.tensor([3, 999, -1, 0, 17], dtype=torch.int32, device="cuda")
    e = K_.embedding(table, ids, scale=2.0)
    ref = table[ids.clamp(min=0).long()].float() * 2.0
    ref[2] = 0
    _close(e, ref, dt)
    dst = torch.zeros(10, 256, device="cuda", dtype=dt)
    K_.scatter_rows(dst, e, torch.tensor([9, 1, -1, 4, 0], dtype=torch.int32, device="cuda"))
    assert torch.equal(dst[9], e[0]) and torch.equal(dst[0], e[4]) and dst[2].abs().sum() == 0
    a, b = torch.randn(77, 256, device="cuda").to(dt), torch.randn(77, 256, device="cuda").to(dt)
    _close(K_.eltwise("silu_mul", a, b), torch.nn.functional.silu(a.float()) * b.float(), dt)
    _close(K_.eltwise("axpy", a, b, alpha=-0.1), a.float() - 0.1 * b.float(), dt)
    _close(K_.eltwise("mul_row", a, b[0].contiguous()), a.float() * b[0].float(), dt)
    u8 = torch.randint(0, 256, (3, 64), dtype=torch.uint8, device="cuda")
    _close(K_.cast_u8(u8, dt, 1 / 127.5, -1.0), u8.float() / 127.5 - 1.0, dt)
    logits = torch.randn(5, 151936, device="cuda").to(dt)
    logits[2, 77] = 100.0
    logits[3, 151935] = 100.0
    ids2, vals = K_.argmax(logits, offset=10, return_vals=True)
    assert torch.equal(ids2.long() - 10, logits.float().argmax(-1))
    _close(vals, logits.float().max(-1).values, dt)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K,swap,splits", [(16, 384, 1024, -1, 0), (64, 1000, 2048, 1, 4), (9, 256, 512, 1, 1),
                                               (300, 640, 1024, 0, 1), (1024, 512, 2048, 0, 1), (130, 256, 4096, 1, 2)])
def test_gemm_w8a16_tensor_core(dt, M, N, K, swap, splits, status):
    """int8 weights widened in the mainloop, (X . Q^T) * scale in the epilogue."""
    from rhinoforge_b200.ops import kernels as K_
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    q = torch.randint(-127, 128, (N, K), device="cuda", dtype=torch.int8)
    sc = (torch.rand(N, device="cuda") * 0.004 + 0.001).to(dt)
    r = torch.randn(M, N, device="cuda").to(dt)
    y = K_.gemm(x, q, scale=sc, residual=r, status=status, force_swap=swap, force_splits=splits)
    ref = (x.float() @ q.float().t()) * sc.float() + r.float()
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()) * (4 if dt == torch.bfloat16 else 1))


@pytest.mark.parametrize("M,swap", [(24, 1), (300, 0)])
def test_gemm_w8a16_dual_glu(M, swap, status):
    from rhinoforge_b200.ops import kernels as K_
    dt, N, K = torch.float16, 384, 1024
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    q = torch.randint(-127, 128, (2 * N, K), device="cuda", dtype=torch.int8)
    sc = (torch.rand(2 * N, device="cuda") * 0.002 + 0.0005).to(dt)
    y = K_.gemm(x, q, scale=sc, act="silu_mul", dual=True, status=status, force_swap=swap)
    z = (x.float() @ q.float().t()) * sc.float()
    _close(y, torch.nn.functional.silu(z[:, :N]) * z[:, N:], dt, scale=2.0)


def test_engine_w8a16_matches_dequantised_oracle():
    """Whole decoder with int8 weights: greedy tokens follow the oracle run on the dequantised weights."""
    from rhinoforge_b200.models.decoder import TorchDecoder, random_state_dict, tiny_config
    from rhinoforge_b200.quant._common import dequantize_linear_per_channel, quantize_linear_per_channel
    from rhinoforge_b200.runtime.engine import DecoderEngine
    cfg = tiny_config(num_layers=2)
    sd = random_state_dict(cfg, seed=0, dtype=torch.float16, norm_jitter=0.05)
    deq = {}
    for k, v in sd.items():
        if v.dim() == 2 and "embed" not in k:
            qq, s = quantize_linear_per_channel(v)
            deq[k] = dequantize_linear_per_channel(qq, s)
        else:
            deq[k] = v
    if "lm_head.weight" not in sd:            # tied embeddings: the head is the quantised embedding matrix
        deq["lm_head.weight"] = dequantize_linear_per_channel(*quantize_linear_per_channel(sd["model.embed_tokens.weight"]))
    oracle = TorchDecoder(cfg, deq, dtype=torch.float32, device="cuda")
    eng = DecoderEngine(cfg, lambda n: sd[n] if n in sd else sd["model.embed_tokens.weight"], dtype=torch.float16,
                        max_batch=2, max_seq_len=96, quant="w8a16")
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab_size, (L,), generator=g) for L in (19, 40)]
    _, logits = eng.prefill(prompts, return_logits=True)
    for b, p in enumerate(prompts):
        oracle.reset()
        ref = oracle.forward(p[None].cuda())[0, -1]
        torch.testing.assert_close(logits[b].float(), ref.float(), rtol=1e-2, atol=1e-2)
    toks = eng.generate(prompts, 6)
    assert toks.shape == (2, 6)
    eng.check_status()
    eng.close()


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K,swap,splits", [(16, 384, 1024, -1, 0), (64, 1000, 2048, 1, 4), (9, 200, 520, 1, 1),
                                               (300, 640, 1024, 0, 1), (1024, 512, 2048, 0, 1), (700, 130, 264, 0, 1)])
def test_gemm_packed_weights(dt, M, N, K, swap, splits, status):
    """Tile-major (bulk-copy) weight layout gives the same result as row-major weights."""
    from rhinoforge_b200.ops import kernels as K_
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(dt)
    b = torch.randn(N, device="cuda").to(dt)
    r = torch.randn(M, N, device="cuda").to(dt)
    wp = K_.pack_weight(w)
    y = K_.gemm(x, wp, packed_shape=(N, K), bias=b, residual=r, status=status, force_swap=swap, force_splits=splits)
    ref = x.float() @ w.float().t() + b.float() + r.float()
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()))


@pytest.mark.parametrize("M,swap", [(24, 1), (300, 0)])
def test_gemm_packed_dual_and_int8(M, swap, status):
    from rhinoforge_b200.ops import kernels as K_
    dt, N, K = torch.float16, 200, 1024                    # N not a multiple of 128: sections are padded separately
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(2 * N, K, device="cuda") * 0.05).to(dt)
    y = K_.gemm(x, K_.pack_weight(w, 2), packed_shape=(2 * N, K), act="silu_mul", dual=True, status=status, force_swap=swap)
    z = x.float() @ w.float().t()
    _close(y, torch.nn.functional.silu(z[:, :N]) * z[:, N:], dt, scale=2.0)
    q = torch.randint(-127, 128, (2 * N, K), device="cuda", dtype=torch.int8)
    sc = (torch.rand(2 * N, device="cuda") * 0.002 + 0.0005).to(dt)
    y = K_.gemm(x, K_.pack_weight(q, 2), packed_shape=(2 * N, K), scale=sc, act="silu_mul", dual=True, status=status,
                force_swap=swap)
    z = (x.float() @ q.float().t()) * sc.float()
    _close(y, torch.nn.functional.silu(z[:, :N]) * z[:, N:], dt, scale=2.0)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K,dual", [(2500, 2048, 520, False), (4100, 1280, 1024, False), (2304, 2560, 512, True),
                                        (20000, 256, 128, False), (1152, 2560, 512, True), (5000, 2048, 520, False),
                                        (4900, 1152, 256, False), (4900, 2048, 4096, False)])
def test_gemm_persistent_kernel(dt, M, N, K, dual, status):
    """Large token counts take the persistent kernel (one CTA per SM walking tiles): 128-row tiles with two
    accumulator buffers (the first, second, fourth and fifth shapes) and 256-row tiles (the others); ragged M
    (a last half-tile partly or wholly past the end), N not a multiple of the tile, several tiles per CTA,
    a ring shorter and longer than K, bias + residual, GLU epilogue."""
    from rhinoforge_b200.ops import kernels as K_
    torch.manual_seed(M)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    rows = 2 * N if dual else N
    w = (torch.randn(rows, K, device="cuda") * 0.05).to(dt)
    wp = K_.pack_weight(w, 2 if dual else 1)
    if dual:
        y = K_.gemm(x, wp, packed_shape=(rows, K), act="silu_mul", dual=True, status=status)
        z = x.float() @ w.float().t()
        ref = torch.nn.functional.silu(z[:, :N]) * z[:, N:]
    else:
        b = torch.randn(N, device="cuda").to(dt)
        r = torch.randn(M, N, device="cuda").to(dt)
        y = K_.gemm(x, wp, packed_shape=(rows, K), bias=b, residual=r, status=status)
        ref = x.float() @ w.float().t() + b.float() + r.float()
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()))
    y2 = K_.gemm(x, wp, packed_shape=(rows, K), act="silu_mul", dual=True, status=status) if dual else \
        K_.gemm(x, wp, packed_shape=(rows, K), bias=b, residual=r, status=status)
    assert torch.equal(y, y2), "two launches of the same GEMM must agree bit for bit"
    if not dual:
        # without a residual the results leave through staging tiles and tiled bulk stores
        y3 = K_.gemm(x, wp, packed_shape=(rows, K), bias=b, status=status)
        _close(y3, x.float() @ w.float().t() + b.float(), dt, scale=max(1.0, ref.abs().max().item()))
        view = torch.zeros(M, N + 8, device="cuda", dtype=dt)           # strided output rows
        K_.gemm(x, wp, packed_shape=(rows, K), out=view[:, :N], status=status)
        _close(view[:, :N], x.float() @ w.float().t(), dt, scale=max(1.0, ref.abs().max().item()))
        assert float(view[:, N:].abs().max()) == 0.0, "columns past N must stay untouched"
        # residual already in the output buffer (out == residual): the add happens in the bulk reduce
        acc = r.clone()
        K_.gemm(x, wp, packed_shape=(rows, K), residual=acc, out=acc, status=status)
        _close(acc, x.float() @ w.float().t() + r.float(), dt, scale=max(1.0, ref.abs().max().item()))


def test_manual_graph_capture_replays_with_refilled_inputs(status):
    """``graph.capture``: one recording run, then replays that refill the static input buffers; a changed shape is refused."""
    from rhinoforge_b200.graph import capture
    from rhinoforge_b200.ops import kernels as K_
    w = (1.0 + 0.1 * torch.randn(256, device="cuda")).half()
    x = torch.randn(40, 256, device="cuda").half()
    out = torch.empty_like(x)

    def fn(inp):
        K_.rmsnorm(inp, w, 1e-6, out=out)
        return out

    g = capture(fn, x)
    assert g.replayable, g.non_replayable_reason
    ref = lambda t: (w.float() * (t.float() * torch.rsqrt(t.float().pow(2).mean(-1, keepdim=True) + 1e-6)))
    torch.cuda.synchronize()
    _close(g.cached_output, ref(x), torch.float16)
    x2 = torch.randn(40, 256, device="cuda").half()
    y = g.replay(x2)
    torch.cuda.synchronize()
    _close(y, ref(x2), torch.float16)
    st = g.stats()
    assert st["replays"] == 1 and st["build_count"] == 1 and st["node_count"] >= 1
    with pytest.raises(RuntimeError, match="shape_bucket"):
        g.replay(torch.randn(41, 256, device="cuda").half())
    g.invalidate()


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("dual", [False, True])
def test_gemm_w8a16_large_m_widens_once_and_matches(dt, dual, status):
    """W8A16 with a prefill-sized token count and caller scratch: the int8 image is widened once and the 16-bit
    (persistent) kernel runs; the result equals ``(x . q^T) * scale`` like the in-loop path without scratch."""
    from rhinoforge_b200.ops import kernels as K_
    torch.manual_seed(3)
    M, N, K = 2304, 2560, 512
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    rows = 2 * N if dual else N
    q = torch.randint(-127, 128, (rows, K), device="cuda", dtype=torch.int8)
    sc = (torch.rand(rows, device="cuda") * 0.002 + 0.0005).to(dt)
    qp = K_.pack_weight(q, 2 if dual else 1)
    scratch = torch.empty(2 * qp.numel(), dtype=torch.uint8, device="cuda")
    kw = dict(packed_shape=(rows, K), scale=sc, status=status)
    if dual:
        kw.update(act="silu_mul", dual=True)
    y = K_.gemm(x, qp, w_scratch=scratch, **kw)
    y0 = K_.gemm(x, qp, **kw)
    z = (x.float() @ q.float().t()) * sc.float()
    ref = torch.nn.functional.silu(z[:, :N]) * z[:, N:] if dual else z
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()))
    _close(y0, ref, dt, scale=max(1.0, ref.abs().max().item()))


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K", [(64, 4096, 512), (64, 4096, 1024), (50, 1024, 192), (8, 2048, 64)])
def test_gemm_short_k_splits_down_to_one_block_per_cta(dt, M, N, K, status):
    """Short-K weight-streaming shapes (tensor-parallel out-projections): the planner may give every CTA of the
    cluster a single k block (or fewer splits than blocks when K is tiny); bias, residual and the rotated K start are
    all in play."""
    from rhinoforge_b200.ops import kernels as K_
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(dt)
    b = torch.randn(N, device="cuda").to(dt)
    r = torch.randn(M, N, device="cuda").to(dt)
    ref = x.float() @ w.float().t() + b.float() + r.float()
    y = K_.gemm(x, K_.pack_weight(w), packed_shape=(N, K), bias=b, residual=r, status=status)
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()))
    y2 = K_.gemm(x, w, bias=b, residual=r, status=status)                  # row-major weights, same planner
    _close(y2, ref, dt, scale=max(1.0, ref.abs().max().item()))
    for s in (1, 8):
        if s * 64 <= max(K, 64) or s == 1:
            y3 = K_.gemm(x, K_.pack_weight(w), packed_shape=(N, K), bias=b, residual=r, status=status, force_splits=s)
            _close(y3, ref, dt, scale=max(1.0, ref.abs().max().item()))


def _close_elementwise(y, ref, dt):
    """Every element within fp16 / bf16 rounding of ITS OWN reference value (plus a small absolute floor), so a
    wrong low-magnitude column cannot hide behind the largest entry of the matrix."""
    rel = 2.0 ** -7 if dt == torch.bfloat16 else 2.0 ** -10
    err = (y.float() - ref.float()).abs()
    bound = rel * ref.float().abs() * 2.0 + (6e-2 if dt == torch.bfloat16 else 6e-3)
    bad = (err > bound).nonzero()
    assert bad.numel() == 0, f"{bad.shape[0]} elements off; first {bad[0].tolist()}: {y[tuple(bad[0])].item()} vs {ref[tuple(bad[0])].item()}"


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K,dual", [(1, 4096, 4096, False), (7, 384, 2048, False), (16, 1000, 1024, False),
                                        (64, 2048, 4096, True), (64, 4096, 12288, False), (33, 1280, 512, True),
                                        (200, 640, 2560, False), (256, 1152, 1024, False), (96, 8192, 1024, True),
                                        (64, 151936, 1024, False)])
def test_gemm_stream_k(dt, M, N, K, dual, status):
    """The persistent stream-K kernel (tile-major weights, at most 256 tokens): shares that start and end inside a
    tile (partials parked in scratch and added by the tile's finisher), several tiles per CTA, ragged N, one token,
    a full 256-token tile, GLU pairs, a vocabulary-sized N; bias, per-channel scale, per-row scale and residual;
    two launches agree bit for bit."""
    from rhinoforge_b200 import _native as N_
    from rhinoforge_b200.ops import kernels as K_
    old_mode = N_.lib().rf_gemm_streamk_mode(2)          # every shape that fits, not only the large-N ones
    try:
        _stream_k_case(dt, M, N, K, dual, status)
    finally:
        N_.lib().rf_gemm_streamk_mode(old_mode)


def _stream_k_case(dt, M, N, K, dual, status):
    from rhinoforge_b200.ops import kernels as K_
    torch.manual_seed(M * 7 + N)
    rows = 2 * N if dual else N
    plan = K_.gemm_plan(M, N, K, dtype=dt, dual=dual, packed=True)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(rows, K, device="cuda") * (1.0 / math.sqrt(K))).to(dt)
    wp = K_.pack_weight(w, 2 if dual else 1)
    z = x.float() @ w.float().t()
    if dual:
        y = K_.gemm(x, wp, packed_shape=(rows, K), act="silu_mul", dual=True, status=status)
        ref = torch.nn.functional.silu(z[:, :N]) * z[:, N:]
        y2 = K_.gemm(x, wp, packed_shape=(rows, K), act="silu_mul", dual=True, status=status)
    else:
        b = torch.randn(N, device="cuda").to(dt)
        sc = (torch.rand(N, device="cuda") + 0.5).to(dt)
        rs = torch.rand(M, device="cuda") + 0.5
        r = torch.randn(M, N, device="cuda").to(dt)
        y = K_.gemm(x, wp, packed_shape=(rows, K), bias=b, scale=sc, row_scale=rs, residual=r, status=status)
        ref = z * rs[:, None] * sc.float() + b.float() + r.float()
        y2 = K_.gemm(x, wp, packed_shape=(rows, K), bias=b, scale=sc, row_scale=rs, residual=r, status=status)
        # in place: the residual already sits in the output buffer
        acc = r.clone()
        K_.gemm(x, wp, packed_shape=(rows, K), residual=acc, out=acc, status=status)
        _close_elementwise(acc, z + r.float(), dt)
    _close_elementwise(y, ref, dt)
    assert torch.equal(y, y2), "two launches of the same GEMM must agree bit for bit"
    assert plan is None or plan["persistent"] in (0, 2)


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K,group,dual", [(1, 1024, 4096, 64, False), (16, 1000, 1024, 32, False), (64, 384, 2048, 128, False),
                                              (64, 2048, 1024, 0, False), (33, 1280, 512, 64, True), (200, 640, 2560, 32, False),
                                              (300, 512, 1024, 64, False), (300, 768, 512, 128, True), (8, 256, 192, 64, False)])
def test_gemm_w4a16(dt, M, N, K, group, dual, status):
    """int4 weights in the tile-major image: nibbles widened and group scales applied by the converter warps of the
    main loop (per-channel scales in the epilogue when group = 0); reference = x @ dequantised weights in fp32."""
    from rhinoforge_b200.ops import kernels as K_
    torch.manual_seed(N + K + group)
    rows = 2 * N if dual else N
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    q = torch.randint(-8, 8, (rows, K), device="cuda", dtype=torch.int8)
    r = torch.randn(M, N, device="cuda").to(dt)
    kw = dict(packed_shape=(rows, K), w_bits=4, w_group=group, status=status)
    if group:
        sc = (torch.rand(rows, K // group, device="cuda") * 0.03 + 0.005).to(dt)
        img = K_.pack_weight_int4(q, sc, group, sections=2 if dual else 1, dtype=dt)
        wd = q.float().view(rows, K // group, group) * sc.float()[..., None]
        wd = wd.view(rows, K)
    else:
        sc = (torch.rand(rows, device="cuda") * 0.03 + 0.005).to(dt)
        img = K_.pack_weight_int4(q, sections=2 if dual else 1)
        kw["scale"] = sc
        wd = q.float() * sc.float()[:, None]
    assert img.numel() == K_.N.lib().rf_pack_w4_bytes(rows, K, 2 if dual else 1, group)
    z = x.float() @ wd.t()
    if dual:
        y = K_.gemm(x, img, act="silu_mul", dual=True, **kw)
        ref = torch.nn.functional.silu(z[:, :N]) * z[:, N:]
    else:
        y = K_.gemm(x, img, residual=r, **kw)
        ref = z + r.float()
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()) * (4 if dt == torch.bfloat16 else 1))


@pytest.mark.parametrize("group,from_packed", [(64, False), (32, True), (0, False)])
def test_engine_w4a16_matches_dequantised_oracle(group, from_packed):
    """Whole decoder with int4 projections (lm_head 16-bit): prefill logits follow the oracle run on the dequantised
    weights, whether the engine quantises 16-bit weights itself or reads a packed 4-bit checkpoint."""
    from rhinoforge_b200.models.decoder import TorchDecoder, random_state_dict, tiny_config
    from rhinoforge_b200.quant.int4_pack import pack_int4
    from rhinoforge_b200.runtime.engine import DecoderEngine
    cfg = tiny_config(num_layers=2)
    sd = random_state_dict(cfg, seed=0, dtype=torch.float16, norm_jitter=0.05)

    def quant(w):
        wf = w.float()
        grp = wf.view(wf.shape[0], -1, group) if group else wf.view(wf.shape[0], 1, -1)
        sc = (grp.abs().amax(-1) / 7.0).clamp_min(1e-8)
        q = torch.round(grp / sc[..., None]).clamp_(-8, 7)
        return q.to(torch.int8).view_as(wf), sc, (q * sc[..., None].half().float()).view_as(wf)

    deq, packed, scales = {}, {}, {}
    for k, v in sd.items():
        if v.dim() == 2 and "embed" not in k and "lm_head" not in k:
            q, sc, d = quant(v)
            deq[k], packed[k], scales[k] = d, pack_int4(q), sc.half()
        else:
            deq[k] = v
    oracle = TorchDecoder(cfg, deq, dtype=torch.float32, device="cuda")

    def get(n):
        if n not in sd:
            return sd["model.embed_tokens.weight"]
        return packed[n] if (from_packed and n in packed) else sd[n]
    get.scale = lambda n: scales.get(n)
    eng = DecoderEngine(cfg, get, dtype=torch.float16, max_batch=2, max_seq_len=96, quant="w4a16", w4_group=group)
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab_size, (L,), generator=g) for L in (19, 40)]
    _, logits = eng.prefill(prompts, return_logits=True)
    for b, p in enumerate(prompts):
        oracle.reset()
        ref = oracle.forward(p[None].cuda())[0, -1]
        torch.testing.assert_close(logits[b].float(), ref.float(), rtol=2e-2, atol=2e-2)
    toks = eng.generate(prompts, 6)
    assert toks.shape == (2, 6)
    eng.check_status()
    eng.close()


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K,dual", [(1, 1024, 2048, False), (48, 520, 1024, False), (64, 768, 512, True), (300, 512, 1024, False)])
def test_gemm_nvfp4(dt, M, N, K, dual, status):
    """NVFP4 weights (e2m1 codes, e4m3 block scale per 16 columns, fp32 tensor scale) through the 4-bit main loop;
    reference = x @ the exact fp32 weight the codes stand for."""
    from rhinoforge_b200.ops import kernels as K_
    from rhinoforge_b200.quant.nvfp4_pack import dequantize_nvfp4, quantize_nvfp4
    torch.manual_seed(N + K)
    rows = 2 * N if dual else N
    w = torch.randn(rows, K, device="cuda") * 0.05
    codes, sc, ts = quantize_nvfp4(w)
    wd = dequantize_nvfp4(codes, sc, ts)
    img = K_.pack_weight_nvfp4(codes, sc, ts, sections=2 if dual else 1, dtype=dt)
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    kw = dict(packed_shape=(rows, K), w_bits=4, w_group=16, w_fp4=True, status=status)
    z = x.float() @ wd.t()
    if dual:
        y = K_.gemm(x, img, act="silu_mul", dual=True, **kw)
        ref = torch.nn.functional.silu(z[:, :N]) * z[:, N:]
    else:
        y = K_.gemm(x, img, **kw)
        ref = z
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()) * (4 if dt == torch.bfloat16 else 1))


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,H,I,splits", [(1, 1024, 2048, 0), (64, 1024, 3072, 0), (16, 512, 1024, 1), (200, 768, 1536, 0),
                                           (33, 1280, 512, 4)])
def test_gemm_folded_rmsnorm(dt, M, H, I, splits, status):
    """RMSNorm without a kernel of its own: the residual GEMM writes per-tile sums of squares of its finished rows, the
    next projection (norm weights multiplied into its columns) scales its rows by their reciprocal RMS.  Reference:
    rmsnorm(hidden) * w @ W2^T on the rows the first GEMM stored."""
    from rhinoforge_b200.ops import kernels as K_
    torch.manual_seed(M + H)
    x = (torch.randn(M, I, device="cuda") * 0.5).to(dt)
    w1 = (torch.randn(H, I, device="cuda") * 0.05).to(dt)
    resid = torch.randn(M, H, device="cuda").to(dt)
    nw = (1.0 + 0.2 * torch.randn(H, device="cuda")).to(dt)
    w2 = (torch.randn(2 * I, H, device="cuda") * 0.05).to(dt)
    bias = (torch.randn(2 * I, device="cuda") * 0.1).to(dt)
    tiles = (H + 127) // 128
    ss = torch.full((tiles, 256), float("nan"), device="cuda")
    hidden = resid.clone()
    K_.gemm(x, K_.pack_weight(w1), packed_shape=(H, I), residual=hidden, out=hidden, ss_out=ss, status=status,
            force_splits=splits)
    ref_h = (x.float() @ w1.float().t() + resid.float())
    _close(hidden, ref_h, dt, scale=max(1.0, ref_h.abs().max().item()))
    want_ss = hidden.float().pow(2).view(M, tiles, -1).sum(-1).t()             # [tiles, M] of the rows as stored
    torch.testing.assert_close(ss[:, :M], want_ss, rtol=1e-4, atol=1e-3)
    w2f = (w2.float() * nw.float()[None]).to(dt)                                # norm weights folded into the columns
    y = K_.gemm(hidden, K_.pack_weight(w2f, 2), packed_shape=(2 * I, H), bias=bias, act="silu_mul", dual=True, ss_in=ss,
                ss_dim=H, ss_eps=1e-6, status=status)
    hn = hidden.float() * torch.rsqrt(hidden.float().pow(2).mean(-1, keepdim=True) + 1e-6) * nw.float()
    z = hn @ w2.float().t() + bias.float()
    ref = torch.nn.functional.silu(z[:, :I]) * z[:, I:]
    _close(y, ref, dt, scale=max(1.0, ref.abs().max().item()) * (4 if dt == torch.bfloat16 else 1))


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K", [(128, 384, 1536), (128, 1536, 384), (41, 1536, 2048), (50, 1024, 4096), (31, 1024, 1024),
                                   (7, 72, 136), (130, 200, 72), (256, 512, 640), (1, 384, 384), (1028, 1152, 384), (600, 384, 1536)])
@pytest.mark.parametrize("packed", [False, True])
def test_gemm_small_latency_kernel(dt, M, N, K, packed, status, monkeypatch):
    """Shapes the latency-bound kernel takes (few rows, small weight): every epilogue option against fp32 PyTorch, and the
    same call with the kernel switched off (the streaming kernel) within rounding."""
    from rhinoforge_b200.ops import kernels as K_
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(N, K, device="cuda") * 0.05).to(dt)
    b = torch.randn(N, device="cuda").to(dt)
    r = torch.randn(M, N, device="cuda").to(dt)
    wk = K_.pack_weight(w) if packed else w
    kw = dict(packed_shape=(N, K)) if packed else {}
    ref = x.float() @ w.float().t()
    _close(K_.gemm(x, wk, **kw), ref, dt, scale=max(1.0, float(ref.abs().max())))
    full = torch.nn.functional.gelu(ref + b.float(), approximate="tanh") + r.float()
    got = K_.gemm(x, wk, bias=b, act="gelu_tanh", residual=r, **kw)
    _close(got, full, dt, scale=max(1.0, float(full.abs().max())))
    # per-column factor before the bias (the gate of a gated residual): r + (x.w^T * s + b)
    sc = (torch.randn(N, device="cuda") * 0.5).to(dt)
    gated = ref * sc.float() + b.float() + r.float()
    _close(K_.gemm(x, wk, scale=sc, bias=b, residual=r, **kw), gated, dt, scale=max(1.0, float(gated.abs().max())))
    # strided output / input views
    buf = torch.zeros(M, N + 16, device="cuda", dtype=dt)
    K_.gemm(x, wk, out=buf[:, 8:8 + N], **kw)
    _close(buf[:, 8:8 + N], ref, dt, scale=max(1.0, float(ref.abs().max())))
    assert float(buf[:, :8].abs().max()) == 0 and float(buf[:, 8 + N:].abs().max()) == 0


def test_gemm_forced_wide_tile_over_odd_block_count(status):
    """A forced 256-wide tile on a tile-major weight with an odd number of 128-row blocks (N = 1152: nine) falls back to
    128-wide tiles instead of copying a tenth block that is not there; token-row split K (pushed partial slices) on
    the same shape at 2 and 4 splits."""
    from rhinoforge_b200.ops import kernels as K_
    M, N, K = 768, 1152, 1152
    x = (torch.randn(M, K, device="cuda") * 0.5).half()
    w = (torch.randn(N, K, device="cuda") * 0.05).half()
    r = torch.randn(M, N, device="cuda").half()
    wp = K_.pack_weight(w)
    ref = x.float() @ w.float().t() + r.float()
    for kw in (dict(force_bn=256), dict(force_bn=256, force_splits=2), dict(force_bn=128, force_splits=4), dict(force_splits=3)):
        got = K_.gemm(x, wp, packed_shape=(N, K), residual=r, status=status, **kw)
        _close(got, ref, torch.float16, scale=max(1.0, float(ref.abs().max())))


@pytest.mark.parametrize("dt", DT)
@pytest.mark.parametrize("M,N,K", [(50, 4096, 1024), (128, 1536, 384), (31, 136, 200)])
@pytest.mark.parametrize("packed", [False, True])
def test_gemm_small_dual_glu(dt, M, N, K, packed, status):
    from rhinoforge_b200.ops import kernels as K_
    x = (torch.randn(M, K, device="cuda") * 0.5).to(dt)
    w = (torch.randn(2 * N, K, device="cuda") * 0.05).to(dt)
    b = (torch.randn(2 * N, device="cuda") * 0.1).to(dt)
    wk = K_.pack_weight(w, sections=2) if packed else w
    kw = dict(packed_shape=(2 * N, K)) if packed else {}
    gte, up = x.float() @ w[:N].float().t() + b[:N].float(), x.float() @ w[N:].float().t() + b[N:].float()
    ref = torch.nn.functional.silu(gte) * up
    got = K_.gemm(x, wk, bias=b, act="silu_mul", dual=True, **kw)
    _close(got, ref, dt, scale=max(1.0, float(ref.abs().max())))
