"""GPU checks of the small fused kernels of the verify step against plain torch fp32 formulas."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    return _lib.lib()


def _st():
    return torch.cuda.current_stream().cuda_stream


@pytest.mark.parametrize("H", [5120, 512, 100, 8 * 4 * 1024 + 8])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm_in_place(lib, H, with_delta):
    g = torch.Generator(device="cuda").manual_seed(H)
    h = torch.randn(16, H, generator=g, device="cuda").to(BF)
    d = torch.randn(16, H, generator=g, device="cuda").to(BF) if with_delta else None
    w = (1 + 0.1 * torch.randn(H, generator=g, device="cuda")).to(BF)
    x = torch.empty_like(h)
    h0 = h.clone()
    st = lib.dflash_add_rmsnorm(h.data_ptr(), None if d is None else d.data_ptr(), w.data_ptr(), h.data_ptr(), x.data_ptr(),
                                16, H, 1e-6, 0, _st())
    assert st == 0
    want_h = (h0.float() + d.float()).to(BF) if with_delta else h0
    assert torch.equal(h, want_h)
    hf = want_h.float()
    want_x = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * w.float()
    assert float((x.float() - want_x).abs().max() / want_x.abs().max()) <= 1e-2


@pytest.mark.parametrize("V", [151936, 18992, 1000, 7, 2048 + 3])
def test_argmax_first_maximum(lib, V):
    g = torch.Generator(device="cuda").manual_seed(V)
    logits = torch.randn(16, V, generator=g, device="cuda").to(BF)
    logits[3, V // 2] = 100.0
    logits[3, V - 1] = 100.0          # tie: the first index wins
    logits[5, 0] = 100.0
    out = torch.empty(16, dtype=torch.int32, device="cuda")
    assert lib.dflash_argmax(logits.data_ptr(), out.data_ptr(), 16, V, 0, _st()) == 0
    lf = logits.float()
    want = torch.stack([(lf[t] == lf[t].max()).nonzero()[0, 0] for t in range(16)]).to(torch.int32)
    assert torch.equal(out, want)
    # an unaligned row start (view into a wider buffer)
    wide = torch.randn(16 * (V + 3) + 8, generator=g, device="cuda").to(BF)
    view = wide[1:1 + 16 * V].view(16, V)
    assert lib.dflash_argmax(view.data_ptr(), out.data_ptr(), 16, V, 0, _st()) == 0
    lf = view.float()
    want = torch.stack([(lf[t] == lf[t].max()).nonzero()[0, 0] for t in range(16)]).to(torch.int32)
    assert torch.equal(out, want)


def test_swiglu_and_embed(lib):
    g = torch.Generator(device="cuda").manual_seed(1)
    gu = torch.randn(16, 2 * 1024, generator=g, device="cuda").to(BF)
    y = torch.empty(16, 1024, dtype=BF, device="cuda")
    assert lib.dflash_swiglu(gu.data_ptr(), y.data_ptr(), 16, 1024, 0, _st()) == 0
    want = torch.nn.functional.silu(gu[:, :1024].float()) * gu[:, 1024:].float()
    assert float((y.float() - want).abs().max() / want.abs().max()) <= 1e-2
    table = torch.randn(300, 64, generator=g, device="cuda").to(BF)
    ids = torch.tensor([0, 299, 5, 7] * 4, dtype=torch.int32, device="cuda")
    h = torch.empty(16, 64, dtype=BF, device="cuda")
    assert lib.dflash_embed(ids.data_ptr(), table.data_ptr(), h.data_ptr(), 16, 64, 300, 0, _st()) == 0
    assert torch.equal(h, table[ids.long()])


# ---- the attention layer's glue against formulas written from the reference's hook (runtime.py:527-555, 611-612) ----
def _rope_half_split(x, pos, rope_dims, base):
    """mlx `nn.RoPE(traditional=False)`: channel i < rope_dims/2 pairs with i + rope_dims/2; angle pos * base^(-2i/rope_dims)."""
    half = rope_dims // 2
    i = torch.arange(half, dtype=torch.float64)
    theta = pos.double()[:, None] * torch.pow(torch.tensor(base, dtype=torch.float64), -2.0 * i / rope_dims)[None]
    cs, sn = torch.cos(theta).float(), torch.sin(theta).float()
    out = x.clone()
    x1, x2 = x[..., :half], x[..., half:rope_dims]
    out[..., :half] = x1 * cs[:, None] - x2 * sn[:, None]
    out[..., half:rope_dims] = x1 * sn[:, None] + x2 * cs[:, None]
    return out


def _attn_prep_case(T, Hq, Hk, D, seed):
    g = torch.Generator().manual_seed(seed)
    ld = 2 * Hq * D + 2 * Hk * D + 8
    proj = torch.randn(T, ld, generator=g).bfloat16()
    qn = (1.0 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    kn = (1.0 + 0.1 * torch.randn(D, generator=g)).bfloat16()
    return proj, qn, kn, ld


@pytest.mark.parametrize("offset,rope_dims,T", [(0, 64, 16), (77, 64, 16), (4096, 64, 16), (5, 128, 7), (300, 0, 3)])
def test_attn_prep_norm_rope_and_append(lib, offset, rope_dims, T):
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    Hq, Hk, D, cap, eps, base = 4, 2, 128, 4200, 1e-6, 1e7
    proj, qn, kn, ld = _attn_prep_case(T, Hq, Hk, D, seed=offset + rope_dims)
    d = "cuda"
    q = torch.zeros(Hq, T, D, dtype=torch.bfloat16, device=d)
    kc = torch.full((Hk, cap, D), 7.0, dtype=torch.bfloat16, device=d)
    vc = torch.full((Hk, cap, D), 7.0, dtype=torch.bfloat16, device=d)
    pj, qn_d, kn_d = proj.to(d), qn.to(d), kn.to(d)
    k_off, v_off = 2 * Hq * D, 2 * Hq * D + Hk * D
    st = lib.dflash_attn_prep(pj.data_ptr(), ld, k_off, v_off, qn_d.data_ptr(), kn_d.data_ptr(), q.data_ptr(), kc.data_ptr(),
                              vc.data_ptr(), cap * D, cap, T, Hq, Hk, D, rope_dims, offset, eps, base, _lib.BF16, _st())
    assert st == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    pf = proj.float()
    pos = torch.arange(offset, offset + T)
    rms = lambda t, w: (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps) * w.float()).bfloat16().float()   # noqa: E731
    qr = pf[:, :2 * Hq * D].reshape(T, Hq, 2 * D)[..., :D]                       # (query | gate) per head
    kr = pf[:, k_off:k_off + Hk * D].reshape(T, Hk, D)
    q_ref, k_ref = rms(qr, qn), rms(kr, kn)
    if rope_dims:
        q_ref, k_ref = _rope_half_split(q_ref, pos, rope_dims, base), _rope_half_split(k_ref, pos, rope_dims, base)
    v_ref = proj[:, v_off:v_off + Hk * D].reshape(T, Hk, D)
    assert float((q.cpu().float().permute(1, 0, 2) - q_ref).abs().max()) <= 2e-2 * float(q_ref.abs().max())
    assert float((kc.cpu().float()[:, offset:offset + T].permute(1, 0, 2) - k_ref).abs().max()) <= 2e-2 * float(k_ref.abs().max())
    assert torch.equal(vc.cpu()[:, offset:offset + T].permute(1, 0, 2), v_ref)
    # nothing else in the caches moved
    untouched = torch.ones(cap, dtype=torch.bool)
    untouched[offset:offset + T] = False
    assert torch.all(kc.cpu()[:, untouched] == 7.0) and torch.all(vc.cpu()[:, untouched] == 7.0)


def test_attn_prep_refuses_rows_beyond_the_cache(lib):
    """Host offset: refused before anything is launched.  Device offset: the rows that fit are stored, the others are
    dropped, the device error word says so, and the allocation behind the cache is untouched (no fault is provoked:
    the store is skipped)."""
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    T, Hq, Hk, D, cap = 16, 4, 2, 128, 64
    proj, qn, kn, ld = _attn_prep_case(T, Hq, Hk, D, seed=9)
    d = "cuda"
    q = torch.zeros(Hq, T, D, dtype=torch.bfloat16, device=d)
    # one allocation: [k cache | guard | v cache | guard]
    buf = torch.full((2, Hk * cap * D + 4096,), 3.0, dtype=torch.bfloat16, device=d)
    kc, vc = buf[0, :Hk * cap * D], buf[1, :Hk * cap * D]
    pj, qn_d, kn_d = proj.to(d), qn.to(d), kn.to(d)
    k_off, v_off = 2 * Hq * D, 2 * Hq * D + Hk * D
    args = (pj.data_ptr(), ld, k_off, v_off, qn_d.data_ptr(), kn_d.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), cap * D, cap,
            T, Hq, Hk, D, 64)
    st = lib.dflash_attn_prep(*args, cap - 8, 1e-6, 1e7, _lib.BF16, _st())
    assert st == -2 and b"capacity" in lib.dflash_last_error_string()
    off = torch.tensor([cap - 8], dtype=torch.int32, device=d)
    st = lib.dflash_attn_prep_dev_offset(*args, off.data_ptr(), 1e-6, 1e7, _lib.BF16, _st())
    assert st == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    code = lib.dflash_device_error(0)
    assert code & 0xFF == 31 and 8 <= (code >> 8) < 16
    assert lib.dflash_device_error(0) == 0                      # reading clears it
    kcv = kc.view(Hk, cap, D).cpu()
    assert torch.all(kcv[:, :cap - 8] == 3.0) and not torch.any(kcv[:, cap - 8:] == 3.0)
    assert torch.all(buf[:, Hk * cap * D:].cpu() == 3.0)       # the guard regions
    # the last head's rows beyond the capacity would have landed in the guard; head 0's in head 1's first rows
    assert torch.all(kcv[1, :8] == 3.0)


def test_attn_post_gate(lib):
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    T, Hq, D = 16, 4, 128
    g = torch.Generator().manual_seed(4)
    ld = 2 * Hq * D + 40
    proj = torch.randn(T, ld, generator=g).bfloat16()
    o = torch.randn(Hq, T, D, generator=g).bfloat16()
    out = torch.zeros(T, Hq * D + 64, dtype=torch.bfloat16, device="cuda")
    pj, od = proj.cuda(), o.cuda()
    st = lib.dflash_attn_post(od.data_ptr(), pj.data_ptr(), ld, out.data_ptr(), out.shape[1], T, Hq, D, _lib.BF16, _st())
    assert st == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    gate = proj.float()[:, :2 * Hq * D].reshape(T, Hq, 2 * D)[..., D:]
    ref = (o.float().permute(1, 0, 2) * torch.sigmoid(gate)).bfloat16().reshape(T, Hq * D)
    got = out.cpu()[:, :Hq * D]
    assert float((got.float() - ref.float()).abs().max()) <= 1e-2 * float(ref.float().abs().max())
    assert not out.cpu()[:, Hq * D:].any()
