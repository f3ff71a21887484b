"""CPU checks of the oracle's own pieces (no GPU): bit layout, quantiser, rounding variants, 2-pass attention."""
import torch

from oracle import qmm as oq
from oracle import sdpa as osd


def test_pack_unpack_roundtrip_and_bit_layout():
    gen = torch.Generator().manual_seed(0)
    codes = torch.randint(0, 16, (5, 64), generator=gen)
    w = oq.pack_nibbles(codes)
    assert w.shape == (5, 8) and w.dtype == torch.int32
    assert torch.equal(oq.unpack_nibbles(w), codes)
    # nibble i of word j is element 8j+i at bits 4i..4i+3 (verify_qmm.py:70-75)
    word = int(w[2, 3].item()) & 0xFFFFFFFF
    for i in range(8):
        assert (word >> (4 * i)) & 0xF == int(codes[2, 24 + i])


def test_quantiser_reconstruction_error_is_bounded_by_a_step():
    gen = torch.Generator().manual_seed(1)
    w = torch.randn(32, 256, generator=gen) * 0.02
    wq, s, b = oq.quantize_affine(w, 64, 4, out_dtype=torch.float32)
    deq = oq.dequantize(wq, s, b, 64)
    step = s.abs().repeat_interleave(64, dim=1)
    # the scheme snaps the scale so that the larger-magnitude edge is exact; the other edge may clip by < 1 step
    err = (deq - w).abs() / step
    assert float(err.max()) <= 1.0 + 1e-3 and float(err.mean()) <= 0.3


def test_kernel_rounding_variant_is_within_the_reference_gate():
    """The reference accepts |verify - stock| <= 8e-3 abs and 2e-2 rel for bf16 (test_verify_qmm_parity.py:83-98);
    rounding the dequantised weight to bf16 (what its Metal kernel does) must sit inside that gate."""
    K, N = 5120, 512
    gen = torch.Generator().manual_seed(2)
    sc = 1.0 / K ** 0.5
    x = (torch.randn(16, K, generator=gen) * sc).bfloat16()
    w = (torch.randn(N, K, generator=gen) * sc).bfloat16().float()
    wq, s, b = oq.quantize_affine(w, 64, 4)
    stock = oq.qmm_ref(x, wq, s, b, 64, out_dtype=torch.float32)
    kern = oq.qmm_ref(x, wq, s, b, 64, kernel_rounding=True, out_dtype=torch.float32)
    assert float((stock - kern).abs().max()) <= 8e-3
    assert oq.max_rel_err(kern, stock) <= 2e-2
    exact = oq.qmm_ref(x, wq, s, b, 64, accumulate=torch.float64, out_dtype=torch.float32)
    assert oq.max_rel_err(stock, exact) <= 1e-5


def test_two_pass_attention_matches_dense():
    q, k, v, scale = osd.make_sdpa_case(200, seed=4, Hq=4, Hk=2, D=128)
    dense = osd.sdpa_ref(q, k, v, scale, out_dtype=torch.float32)
    for blocks in (32, 64):
        two = osd.sdpa_2pass_ref(q, k, v, scale, blocks)
        assert float((two.float() - dense).abs().max()) <= 2e-2
    # causal rule: the last query row sees every key, the first one all but the last 15
    q1 = q.clone()
    vis = osd._visible(200, 16)
    assert int(vis[15].sum()) == 200 and int(vis[0].sum()) == 185
