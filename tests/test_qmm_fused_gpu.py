"""The matmul's fused epilogues (dflash_verify_qmm_fused) against plain torch formulas.

What is folded in is what the reference leaves to MLX's graph around every quantised linear of a decoder layer
(mlx-lm's `rms_norm`, residual `+`, `swiglu`, as hooked by dflash_mlx/runtime.py:351-452 and :515-613); the formulas
below are written from those definitions, not from the kernels.

Tolerances: matmul outputs max|y - ref| / (max|ref| + 1e-3) <= 1e-2 (bf16); the partial sums of squares 1e-5 relative
(fp32, different summation order only)."""
import ctypes

import pytest
import torch

from oracle import qmm as oq

pytestmark = pytest.mark.gpu
REL = 1e-2


@pytest.fixture(scope="module")
def env():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    lib = _lib.lib()
    ws = torch.zeros(lib.dflash_verify_qmm_workspace_bytes(16, 17408, 34816, 64) + (1 << 20), dtype=torch.uint8, device="cuda")
    return lib, verify_step.QmmEpilogue, ws, _lib


def _fused(env, x, wq, s, b, out, ep, M, K, N):
    lib, _, ws, _lib = env
    st = lib.dflash_verify_qmm_fused(x.data_ptr(), wq.data_ptr(), s.data_ptr(), b.data_ptr(), None, out.data_ptr(), M, K, N,
                                     64, _lib.BF16, ctypes.byref(ep), ws.data_ptr(), ws.numel(),
                                     torch.cuda.current_stream().cuda_stream)
    assert st == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    assert lib.dflash_device_error(0) == 0


def _w_hat(wq, s, b):
    return oq.dequantize(wq, s, b, 64, round_to=torch.bfloat16).float()


@pytest.mark.parametrize("M,K,N", [(16, 5120, 1024), (16, 2048, 640), (7, 1024, 200), (16, 17408, 5120)])
def test_residual_epilogue(env, M, K, N):
    """mode 1: h += x . W^T (stored bf16), scaled = h * next_w, partial sums of h^2 per token."""
    _, Ep, _, _ = env
    x, wq, s, b = oq.make_qmm_case(M, K, N, seed=101 + N, x_std=8.0 / K ** 0.5, w_std=0.05)
    g = torch.Generator().manual_seed(7)
    h0 = torch.randn(M, N, generator=g).to(torch.bfloat16)
    nw = (1.0 + 0.1 * torch.randn(N, generator=g)).to(torch.bfloat16)
    acc = x.float() @ _w_hat(wq, s, b).t()
    h_ref = (h0.float() + acc).to(torch.bfloat16)
    d = "cuda"
    h = h0.to(d).clone()
    scaled = torch.zeros(M, N, dtype=torch.bfloat16, device=d)
    parts = 4 * ((N + 127) // 128)
    ssq = torch.full((parts, 16), -1.0, dtype=torch.float32, device=d)
    nw_d = nw.to(d)
    ep = Ep(mode=1, residual=h.data_ptr(), next_w=nw_d.data_ptr(), scaled=scaled.data_ptr(), out_ssq=ssq.data_ptr())
    _fused(env, x.to(d), wq.to(d), s.to(d), b.to(d), h, ep, M, K, N)
    assert oq.max_rel_err(h.cpu(), h_ref.float()) <= REL
    # what follows is exact given the h the kernel produced
    hk = h.cpu().float()
    assert torch.equal(scaled.cpu(), (hk * nw.float()).to(torch.bfloat16))
    got = ssq.cpu().sum(dim=0)
    want = (hk * hk).sum(dim=1)
    assert torch.allclose(got[:M], want, rtol=1e-5, atol=1e-6)
    assert torch.all(got[M:] == 0)


@pytest.mark.parametrize("M,K,N,parts", [(16, 5120, 2048, 160), (16, 1024, 384, 1), (5, 2048, 130, 37)])
def test_token_factor_epilogue(env, M, K, N, parts):
    """mode 0 with in_ssq: y = (x . W^T) * rsqrt(sum(ssq) / dim + eps)."""
    _, Ep, _, _ = env
    x, wq, s, b = oq.make_qmm_case(M, K, N, seed=55 + N, x_std=1.0, w_std=0.05)
    g = torch.Generator().manual_seed(9)
    ssq = torch.rand(parts, 16, generator=g) * (K / parts)
    eps, dim = 1e-6, float(K)
    inv = torch.rsqrt(ssq.double().sum(dim=0) / dim + eps).float()
    ref = (x.float() @ _w_hat(wq, s, b).t()) * inv[:M, None]
    d = "cuda"
    y = torch.zeros(M, N, dtype=torch.bfloat16, device=d)
    ssq_d = ssq.to(d)
    ep = Ep(mode=0, in_parts=parts, in_dim=dim, eps=eps, in_ssq=ssq_d.data_ptr())
    _fused(env, x.to(d), wq.to(d), s.to(d), b.to(d), y, ep, M, K, N)
    assert oq.max_rel_err(y.cpu(), ref) <= REL


@pytest.mark.parametrize("M,K,I", [(16, 5120, 17408), (16, 1024, 192), (9, 2048, 77)])
def test_swiglu_epilogue(env, M, K, I):
    """mode 2: interleaved (gate, up) rows -> silu(gate) * up, gate and up rounded to bf16 first."""
    _, Ep, _, _ = env
    N = 2 * I
    x, wq, s, b = oq.make_qmm_case(M, K, N, seed=77 + I, x_std=8.0 / K ** 0.5, w_std=0.05)   # rows: gate block | up block
    gu = (x.float() @ _w_hat(wq, s, b).t()).to(torch.bfloat16).float()
    gate, up = gu[:, :I], gu[:, I:]
    ref = torch.nn.functional.silu(gate) * up
    order = torch.arange(N).view(2, I).t().reshape(-1)
    d = "cuda"
    y = torch.zeros(M, I, dtype=torch.bfloat16, device=d)
    ep = Ep(mode=2)
    _fused(env, x.to(d), wq[order].contiguous().to(d), s[order].contiguous().to(d), b[order].contiguous().to(d), y, ep, M, K, N)
    assert oq.max_rel_err(y.cpu(), ref) <= 1.5e-2     # one more bf16 rounding (gate, up) than a plain matmul


def test_norm_split_equals_rmsnorm(env):
    """producer (mode 1) + consumer (mode 0, in_ssq) = residual add -> RMSNorm -> linear, to bf16 accuracy."""
    lib, Ep, _, _ = env
    M, K1, H, N2 = 16, 1024, 2048, 512
    x, w1, s1, b1 = oq.make_qmm_case(M, K1, H, seed=5, x_std=8.0 / K1 ** 0.5, w_std=0.05)
    _, w2, s2, b2 = oq.make_qmm_case(M, H, N2, seed=6, w_std=0.05)
    g = torch.Generator().manual_seed(11)
    h0 = torch.randn(M, H, generator=g).to(torch.bfloat16)
    nw = (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16)
    eps = 1e-6
    h_ref = (h0.float() + x.float() @ _w_hat(w1, s1, b1).t()).to(torch.bfloat16).float()
    xn = (h_ref * torch.rsqrt((h_ref * h_ref).mean(dim=1, keepdim=True) + eps) * nw.float()).to(torch.bfloat16).float()
    ref = xn @ _w_hat(w2, s2, b2).t()
    d = "cuda"
    h = h0.to(d).clone()
    hw = torch.zeros(M, H, dtype=torch.bfloat16, device=d)
    parts = 4 * (H // 128)
    ssq = torch.zeros(parts, 16, dtype=torch.float32, device=d)
    nw_d = nw.to(d)
    _fused(env, x.to(d), w1.to(d), s1.to(d), b1.to(d), h,
           Ep(mode=1, residual=h.data_ptr(), next_w=nw_d.data_ptr(), scaled=hw.data_ptr(), out_ssq=ssq.data_ptr()), M, K1, H)
    y = torch.zeros(M, N2, dtype=torch.bfloat16, device=d)
    _fused(env, hw, w2.to(d), s2.to(d), b2.to(d), y,
           Ep(mode=0, in_parts=parts, in_dim=float(H), eps=eps, in_ssq=ssq.data_ptr()), M, H, N2)
    assert oq.max_rel_err(y.cpu(), ref) <= REL


def test_refusals(env):
    lib, Ep, ws, _lib = env
    t = torch.zeros(16, 1024, dtype=torch.bfloat16, device="cuda")
    assert lib.dflash_verify_qmm_fused_supported(16, 1000, 64, 64, _lib.BF16) == 0
    assert lib.dflash_verify_qmm_fused_supported(16, 1024, 64, 32, _lib.BF16) == 0
    assert lib.dflash_verify_qmm_fused_supported(16, 1024, 64, 64, _lib.BF16) == 1
    ep = Ep(mode=1)   # no residual
    st = lib.dflash_verify_qmm_fused(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 16, 1024, 64,
                                     64, _lib.BF16, ctypes.byref(ep), ws.data_ptr(), ws.numel(), None)
    assert st == -1 and b"residual" in lib.dflash_last_error_string()
    ep = Ep(mode=2)
    st = lib.dflash_verify_qmm_fused(t.data_ptr(), t.data_ptr(), t.data_ptr(), t.data_ptr(), None, t.data_ptr(), 16, 1024, 63,
                                     64, _lib.BF16, ctypes.byref(ep), ws.data_ptr(), ws.numel(), None)
    assert st == -2


def test_next_matmul_hint_changes_nothing(env):
    """dflash_verify_qmm_prefetch_next only makes the next call's kernel pull the announced weights into L2: the
    results of that call are bit for bit those of an unannounced call; a hint naming a shape the tensor-memory kernel
    does not take is ignored; a hint is consumed by one call."""
    lib, _, ws, _lib = env
    M, K, N = 16, 2048, 1536
    x, wq, s, b = oq.make_qmm_case(M, K, N, seed=5, x_std=8.0 / K ** 0.5, w_std=0.05)
    _, wq2, s2, b2 = oq.make_qmm_case(M, 1024, 640, seed=6, x_std=0.2, w_std=0.05)
    d = "cuda"
    xd, wd, sd, bd = x.to(d), wq.to(d), s.to(d), b.to(d)
    w2, s2d, b2d = wq2.to(d), s2.to(d), b2.to(d)
    st = torch.cuda.current_stream().cuda_stream

    def run():
        y = torch.empty(M, N, dtype=torch.bfloat16, device=d)
        rc = lib.dflash_verify_qmm(xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), None, y.data_ptr(), M, K, N, 64,
                                   _lib.BF16, ws.data_ptr(), ws.numel(), st)
        assert rc == 0, lib.dflash_last_error_string()
        torch.cuda.synchronize()
        return y

    plain = run()
    lib.dflash_verify_qmm_prefetch_next(w2.data_ptr(), s2d.data_ptr(), b2d.data_ptr(), 1024, 640)
    hinted = run()
    after = run()                                     # the hint is gone
    lib.dflash_verify_qmm_prefetch_next(w2.data_ptr(), s2d.data_ptr(), b2d.data_ptr(), 1000, 640)   # K % 512 != 0: ignored
    odd = run()
    assert lib.dflash_device_error(0) == 0
    assert torch.equal(plain, hinted) and torch.equal(plain, after) and torch.equal(plain, odd)
    assert oq.max_rel_err(plain.cpu(), x.float() @ _w_hat(wq, s, b).t()) <= REL
