"""GPU behaviour of the verify linear layer, after tests/test_verify_linear_parity.py of the reference:
non-16 row counts are bit-identical to the stock layer, 16 rows are bit-identical to ``verify_matmul``."""
import os

import pytest
import torch
from torch import nn

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mods():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    os.environ["DFLASH_VERIFY_QMM"] = "1"
    from dflash_mlx_b200 import verify_linear, verify_qmm
    lin = nn.Linear(512, 1024, bias=True)
    with torch.no_grad():
        lin.weight.copy_(torch.randn(1024, 512) * 0.1)
    ql = verify_linear.QuantizedLinear.from_linear(lin.cuda(), group_size=64, bits=4)
    return verify_linear, verify_qmm, ql


@pytest.mark.parametrize("M", [1, 8, 32])
def test_parity_non_verify(mods, M):
    vl, vq, ql = mods
    v = vl.VerifyQuantizedLinear.from_quantized(ql)
    x = (torch.randn(M, 512, device="cuda") * 0.5).bfloat16()
    assert torch.equal(ql(x), v(x))


def test_parity_verify_m16(mods):
    vl, vq, ql = mods
    v = vl.VerifyQuantizedLinear.from_quantized(ql)
    x = (torch.randn(2, 8, 512, device="cuda") * 0.5).bfloat16()
    direct = vq.verify_matmul(x, ql.weight, ql.scales, ql.biases, transpose=True, group_size=64, bits=4) + ql.bias
    y = v(x)
    assert y.shape == (2, 8, 1024)
    assert torch.equal(direct, y)
    from oracle import qmm as oq
    ref = oq.qmm_ref(x.cpu(), ql.weight.cpu(), ql.scales.cpu(), ql.biases.cpu(), 64, out_dtype=torch.float32) + ql.bias.cpu().float()
    assert oq.max_rel_err(y, ref) <= 1e-2
