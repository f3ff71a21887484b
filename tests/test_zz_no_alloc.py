"""The allocation-free attention entry point against the ordinary one.

`dflash_verify_sdpa_static` exists for hosts that cannot hand the library a workspace (all device memory
already owned by their pool, or allocator calls forbidden where they sit).  It must give the same bits as
`dflash_verify_sdpa`, call after call, because it runs the same two kernels and only the home of the
split-KV scratch differs.  This file sorts last on purpose: a failing run has already run everything else."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, q, k, v, out, scale, splits=0, mask=None):
    c = ctypes
    fn = lib.dflash_verify_sdpa_static
    fn.restype = c.c_int
    fn.argtypes = [c.c_void_p] * 5 + [c.c_int] * 5 + [c.c_longlong] * 4 + [c.c_float, c.c_int, c.c_int, c.c_void_p]
    B, Hq, _, D = q.shape
    Hk, N = k.shape[1], k.shape[2]
    return fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), None if mask is None else mask.data_ptr(), out.data_ptr(), B, Hq,
              Hk, N, D, k.stride(1), k.stride(2),
              v.stride(1), v.stride(2), float(scale), 0, splits, torch.cuda.current_stream().cuda_stream)


def test_static_scratch_matches_workspace_entry_point_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib, kernels
    from oracle import sdpa as osd
    lib = _lib.lib()
    lib.dflash_verify_sdpa_static_capacity.restype = ctypes.c_size_t
    assert lib.dflash_verify_sdpa_static_capacity() == 32 << 20
    for n_kv, seed in ((4096, 21), (1024, 22)):          # two calls in a row, the second reuses the array
        q, k, v, scale = osd.make_sdpa_case(n_kv, seed=seed)
        q, k, v = q.cuda(), k.cuda(), v.cuda()
        want = kernels.batched_sdpa_2pass_exact(q, k, v, scale)
        got = torch.empty_like(q)
        st = _call_static(lib, q, k, v, got, scale)
        assert st == 0, lib.dflash_last_error_string()
        torch.cuda.synchronize()
        assert torch.equal(got, want)
        ref = osd.sdpa_ref(q.cpu(), k.cpu(), v.cpu(), scale, out_dtype=torch.float32)
        assert float((got.cpu().float() - ref).abs().max() / (ref.abs().max() + 1e-3)) <= 1e-2
    # a shape whose scratch does not fit is refused with a message, nothing is launched
    q, k, v, scale = osd.make_sdpa_case(8192, seed=23, Hq=64, Hk=2)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    st = _call_static(lib, q, k, v, torch.empty_like(q), scale, splits=64)
    assert st == -4 and b"built-in array" in lib.dflash_last_error_string()


def test_static_scratch_other_head_dim_mask_and_single_split():
    """Head dimension 128, an additive mask, and one key range per KV head (no split): each the same bits as the
    workspace entry point."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib, kernels
    from oracle import sdpa as osd
    lib = _lib.lib()
    # D = 128
    q, k, v, scale = osd.make_sdpa_case(2048, seed=31, Hq=8, Hk=2, D=128)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    got = torch.empty_like(q)
    assert _call_static(lib, q, k, v, got, scale) == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    assert torch.equal(got, kernels.batched_sdpa_2pass_exact(q, k, v, scale))
    # boolean mask hiding a third of the keys (converted to the additive form the C ABI takes)
    q, k, v, scale = osd.make_sdpa_case(1536, seed=32)
    q, k, v = q.cuda(), k.cuda(), v.cuda()
    keep = torch.rand(1, 1, 16, 1536, generator=torch.Generator().manual_seed(33)) > 0.33
    keep[..., :16] = True
    want = kernels.batched_sdpa_2pass_exact(q, k, v, scale, mask=keep.cuda())
    add = torch.where(keep, torch.zeros((), dtype=q.dtype), torch.full((), torch.finfo(q.dtype).min, dtype=q.dtype))
    add = add.expand(1, q.shape[1], 16, 1536).contiguous().cuda()
    got = torch.empty_like(q)
    assert _call_static(lib, q, k, v, got, scale, mask=add) == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    assert torch.equal(got, want)
    ref = osd.sdpa_ref(q.cpu(), k.cpu(), v.cpu(), scale, mask=keep, out_dtype=torch.float32)
    assert float((got.cpu().float() - ref).abs().max() / (ref.abs().max() + 1e-3)) <= 1e-2
    # one key range per KV head
    got1 = torch.empty_like(q)
    assert _call_static(lib, q, k, v, got1, scale, splits=1) == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    assert torch.equal(got1, kernels.batched_sdpa_2pass_exact(q, k, v, scale, num_splits=1))
    assert lib.dflash_device_error(0) == 0
