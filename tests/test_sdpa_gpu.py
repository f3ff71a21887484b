"""GPU parity of the 16-row verify attention (through the C ABI) against the CPU oracle (dense softmax with
the reference's visibility rule).  Tolerance: max|o - o_ref| / (max|o_ref| + 1e-3) <= 1e-2 (bf16)."""
import pytest
import torch

from oracle import sdpa as osd

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import kernels
    return kernels


def _rel(a, b):
    a, b = a.detach().cpu().float(), b.detach().cpu().float()
    return float((a - b).abs().max() / (b.abs().max() + 1e-3))


@pytest.mark.parametrize("N", [1024, 4096, 8192, 32768])
def test_config3_kv_sweep(K, N):
    """16 query heads, 2 KV heads, head_dim 256, bf16, causal over the last 16 positions."""
    q, k, v, scale = osd.make_sdpa_case(N, seed=0xDF1C)
    ref = osd.sdpa_ref(q, k, v, scale, out_dtype=torch.float32)
    out = K.batched_sdpa_2pass_exact(q.cuda(), k.cuda(), v.cuda(), scale)
    assert out.shape == q.shape and out.dtype == q.dtype
    assert _rel(out, ref) <= REL_TOL


@pytest.mark.parametrize("B,Hq,Hk,D,N,dtype", [
    (1, 24, 4, 256, 4112, torch.bfloat16),     # the dense model's attention: 24 query / 4 KV heads
    (2, 4, 4, 128, 100, torch.bfloat16),       # no GQA, ragged N, batch 2
    (1, 8, 1, 128, 16, torch.float16),         # only the 16 new positions
    (1, 20, 2, 128, 777, torch.float16),       # 10 heads per KV head: two groups of query heads
    (1, 2, 2, 256, 65, torch.bfloat16),
])
def test_shapes(K, B, Hq, Hk, D, N, dtype):
    q, k, v, scale = osd.make_sdpa_case(N, seed=3, B=B, Hq=Hq, Hk=Hk, D=D, dtype=dtype)
    ref = osd.sdpa_ref(q, k, v, scale, out_dtype=torch.float32)
    out = K.batched_sdpa_2pass_exact(q.cuda(), k.cuda(), v.cuda(), scale)
    assert _rel(out, ref) <= REL_TOL


@pytest.mark.parametrize("splits", [1, 2, 5, 16, 64])
def test_split_count_invariance(K, splits):
    q, k, v, scale = osd.make_sdpa_case(2048, seed=9)
    base = K.batched_sdpa_2pass_exact(q.cuda(), k.cuda(), v.cuda(), scale, num_splits=1)
    out = K.batched_sdpa_2pass_exact(q.cuda(), k.cuda(), v.cuda(), scale, num_splits=splits)
    assert _rel(out, base.float()) <= 1e-3 * 8     # bf16 output rounding dominates


def test_masks(K):
    q, k, v, scale = osd.make_sdpa_case(300, seed=11, Hq=4, Hk=2, D=128)
    gen = torch.Generator().manual_seed(5)
    bmask = torch.rand(1, 4, 16, 300, generator=gen) > 0.2
    amask = (0.5 * torch.randn(1, 1, 16, 300, generator=gen)).to(torch.bfloat16)
    amask[..., 7] = float("-inf")
    for m in (bmask, amask):
        ref = osd.sdpa_ref(q, k, v, scale, m, out_dtype=torch.float32)
        out = K.batched_sdpa_2pass_exact(q.cuda(), k.cuda(), v.cuda(), scale, m.cuda())
        assert _rel(out, ref) <= REL_TOL


def test_strided_kv_cache_view(K):
    """Keys/values as a prefix view of a larger preallocated cache (seq stride = D, head stride = capacity*D)."""
    q, k, v, scale = osd.make_sdpa_case(1040, seed=13)
    cap = 2048
    kc = torch.zeros(1, 2, cap, 256, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    kc[:, :, :1040] = k.cuda()
    vc[:, :, :1040] = v.cuda()
    ref = osd.sdpa_ref(q, k, v, scale, out_dtype=torch.float32)
    out = K.batched_sdpa_2pass_exact(q.cuda(), kc[:, :, :1040], vc[:, :, :1040], scale)
    assert _rel(out, ref) <= REL_TOL


def test_declined_inputs_return_none(K):
    q, k, v, scale = osd.make_sdpa_case(64, seed=1, Hq=2, Hk=1, D=128)
    assert K.batched_sdpa_2pass_exact(q[:, :, :8].cuda(), k.cuda(), v.cuda(), scale) is None        # q_len != 16
    assert K.batched_sdpa_2pass_exact(q.float().cuda(), k.float().cuda(), v.float().cuda(), scale) is None
    assert K.batched_sdpa_2pass_exact(q[..., :64].cuda(), k[..., :64].cuda(), v[..., :64].cuda(), scale) is None
    assert K.batched_sdpa_2pass_exact(q[0].cuda(), k.cuda(), v.cuda(), scale) is None
