"""GPU parity of the verify matmul (through the C ABI) against the CPU oracle.

Tolerance: max|y - y_ref| / (max|y_ref| + 1e-3) <= 1e-2 (the bf16 bound this build is held to; the
reference's own gate is 2e-2, tests/test_verify_qmm_parity.py:83-98)."""
import os

import pytest
import torch

from oracle import qmm as oq

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2


@pytest.fixture(scope="module")
def vq():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    os.environ["DFLASH_VERIFY_QMM"] = "1"
    from dflash_mlx_b200 import verify_qmm
    return verify_qmm


def _run(vq, M, K, N, G=64, dtype=torch.bfloat16, seed=0xDF1A, bias=False, x_std=1.0, w_std=0.02):
    x, wq, s, b = oq.make_qmm_case(M, K, N, seed=seed, group_size=G, dtype=dtype, x_std=x_std, w_std=w_std)
    bias_t = None
    if bias:
        bias_t = (0.1 * torch.randn(N, generator=torch.Generator().manual_seed(seed + 1))).to(dtype)
    ref = oq.qmm_ref(x, wq, s, b, G, out_dtype=torch.float32)
    if bias_t is not None:
        ref = ref + bias_t.float()
    d = "cuda"
    y = vq.quantized_matmul(x.to(d), wq.to(d), s.to(d), b.to(d), group_size=G, bias=None if bias_t is None else bias_t.to(d))
    torch.cuda.synchronize()
    assert y.shape == (M, N) and y.dtype == dtype
    return oq.max_rel_err(y, ref), y


def test_config1_single_op(vq):
    """x bf16 [16,4096] ~N(0,1); W ~N(0,0.02) int4 g64 -> [16,12288]; seed 0xDF1A."""
    err, y = _run(vq, 16, 4096, 12288)
    assert err <= REL_TOL, err
    # also through the reference-named entry point with a leading batch dim
    x, wq, s, b = oq.make_qmm_case(16, 4096, 12288, seed=0xDF1A)
    y2 = vq.verify_matmul(x.reshape(1, 16, 4096).cuda(), wq.cuda(), s.cuda(), b.cuda(), group_size=64, bits=4)
    assert y2.shape == (1, 16, 12288)
    assert torch.equal(y2.reshape(16, -1), y)


@pytest.mark.parametrize("K,N", [(5120, 17408), (17408, 5120), (5120, 1024), (6144, 5120), (5120, 8192),
                                 (4096, 5120), (2048, 512), (512, 2048)])
def test_model_shapes(vq, K, N):
    err, _ = _run(vq, 16, K, N, x_std=1.0 / (K ** 0.5) * 8, w_std=0.05)
    assert err <= REL_TOL, err


@pytest.mark.parametrize("M", [1, 4, 8, 12, 15])
def test_fewer_rows(vq, M):
    err, _ = _run(vq, M, 1024, 256)
    assert err <= REL_TOL, err


@pytest.mark.parametrize("G", [32, 128])
def test_other_group_sizes(vq, G):
    err, _ = _run(vq, 16, 2048, 320, G=G)
    assert err <= REL_TOL, err


def test_float16(vq):
    err, _ = _run(vq, 16, 2048, 512, dtype=torch.float16, x_std=0.5)
    assert err <= 4e-3, err


@pytest.mark.parametrize("K,N,M", [(128, 8, 16), (2496, 504, 16), (192, 40, 7), (1088, 104, 16)])
def test_general_kernel_ragged_shapes(vq, K, N, M):
    """K not a multiple of 8 groups: the reference's random sweep shapes (K=64*[2,40), N=8*[1,64))."""
    err, _ = _run(vq, M, K, N, x_std=1.0 / (K ** 0.5), w_std=1.0 / (K ** 0.5))
    assert err <= REL_TOL, err


def test_more_than_16_rows_and_bias(vq):
    err, _ = _run(vq, 40, 1024, 192, bias=True)
    assert err <= REL_TOL, err


@pytest.mark.parametrize("blocks", [1, 2, 3, 5, 37, 148, 296])
def test_block_count_does_not_change_the_answer(vq, blocks):
    """Split-count invariance: every partition of the work gives the same numbers to fp32 rounding,
    and the partial-tile tickets leave the workspace clean for the next call."""
    from dflash_mlx_b200 import _lib
    lib = _lib.lib()
    err0, y0 = _run(vq, 16, 4096, 640)
    lib.dflash_verify_qmm_set_max_blocks(blocks)
    try:
        err1, y1 = _run(vq, 16, 4096, 640)
        err2, y2 = _run(vq, 16, 4096, 640)
    finally:
        lib.dflash_verify_qmm_set_max_blocks(0)
    assert err1 <= REL_TOL and err2 <= REL_TOL
    assert torch.equal(y1, y2), "two identical launches must agree bit for bit"
    assert oq.max_rel_err(y1, y0.float()) <= 4e-3
    assert lib.dflash_device_error(0) == 0


@pytest.mark.parametrize("impl,want", [(0, 2), (1, 1)])
def test_both_kernels_on_config1(vq, impl, want):
    """bf16 / group 64: the tcgen05 kernel by default, the mma.sync kernel on request; both within tolerance."""
    from dflash_mlx_b200 import _lib
    lib = _lib.lib()
    lib.dflash_verify_qmm_set_impl(impl)
    try:
        err, y = _run(vq, 16, 4096, 12288)
        assert lib.dflash_verify_qmm_last_impl() == want
        assert err <= REL_TOL, err
        err2, y2 = _run(vq, 16, 4096, 12288)
        assert torch.equal(y, y2)
        for K, N, M in [(5120, 1024, 16), (17408, 5120, 16), (2048, 200, 5), (512, 128, 16), (6144, 5120, 16)]:
            e, _ = _run(vq, M, K, N, x_std=8.0 / K ** 0.5, w_std=0.05)
            assert e <= REL_TOL, (K, N, M, e)
    finally:
        lib.dflash_verify_qmm_set_impl(0)
    assert lib.dflash_device_error(0) == 0


def test_bad_arguments_raise(vq):
    x, wq, s, b = oq.make_qmm_case(16, 512, 64, seed=1)
    with pytest.raises(ValueError):
        vq.quantized_matmul(x, wq, s, b)                       # CPU tensors: there is no CPU path
    with pytest.raises(ValueError):
        vq.quantized_matmul(x.cuda(), wq.cuda(), s.cuda(), b.cuda(), bits=8)
    with pytest.raises(ValueError):
        vq.quantized_matmul(x.cuda().float(), wq.cuda(), s.cuda(), b.cuda())
    with pytest.raises(ValueError):
        vq.quantized_matmul(x.cuda(), wq.cuda()[:, :10], s.cuda(), b.cuda())


def test_kernel_choice_by_shape(vq):
    """Default policy: bf16 / group-64 shapes with K % 512 == 0 run the tcgen05 kernel, other dtypes and group sizes the
    mma.sync kernel, ragged K the general kernel; impl 1 forces the mma.sync kernel.  Both fast kernels are within
    tolerance of the oracle and of each other."""
    from dflash_mlx_b200 import _lib
    lib = _lib.lib()
    K, N = 5120, 12288
    try:
        lib.dflash_verify_qmm_set_impl(0)
        e0, y0 = _run(vq, 16, K, N)
        assert lib.dflash_verify_qmm_last_impl() == 2
        lib.dflash_verify_qmm_set_impl(1)
        e1, y1 = _run(vq, 16, K, N)
        assert lib.dflash_verify_qmm_last_impl() == 1
        assert e0 <= REL_TOL and e1 <= REL_TOL, (e0, e1)
        assert oq.max_rel_err(y0.float(), y1.float()) <= 6e-3
        lib.dflash_verify_qmm_set_impl(0)
        e2, _ = _run(vq, 16, 16384, 1024)             # a long K: row tiles cut over many thread blocks
        assert lib.dflash_verify_qmm_last_impl() == 2 and e2 <= REL_TOL
        _run(vq, 16, 2048, 512, dtype=torch.float16, x_std=0.5)
        assert lib.dflash_verify_qmm_last_impl() == 1
        _run(vq, 16, 2048, 320, G=128)
        assert lib.dflash_verify_qmm_last_impl() == 1
        _run(vq, 16, 1088, 104)
        assert lib.dflash_verify_qmm_last_impl() == 3
    finally:
        lib.dflash_verify_qmm_set_impl(0)
    assert lib.dflash_device_error(0) == 0


@pytest.mark.parametrize("M", [1, 5, 16])
@pytest.mark.parametrize("K,N", [(512, 128), (1024, 200), (2048, 136), (4608, 1000)])
def test_tcgen05_kernel_edges(vq, M, K, N):
    """Fewer than 16 rows (the missing rows of the activation tile are zero-filled by the TMA), N that is not a multiple
    of the 128-row tile, one to nine units of K, with and without a bias; twice, bit for bit."""
    from dflash_mlx_b200 import _lib
    lib = _lib.lib()
    err, y = _run(vq, M, K, N, bias=(N % 3 == 0))
    assert lib.dflash_verify_qmm_last_impl() == 2
    assert err <= REL_TOL, err
    err2, y2 = _run(vq, M, K, N, bias=(N % 3 == 0))
    assert torch.equal(y, y2)
    assert lib.dflash_device_error(0) == 0
