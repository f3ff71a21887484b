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
