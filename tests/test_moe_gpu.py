"""GPU parity of the mixture-of-experts block (routing, expert-gathered matmuls, weighted SwiGLU) against the CPU
oracle.  Tolerance: output max-rel <= 1e-2 (bf16), routing identical (logits are injected, as for the reference's
implementations)."""
import pytest
import torch

from oracle import moe as om

pytestmark = pytest.mark.gpu
REL_TOL = 1e-2


@pytest.fixture(scope="module")
def mod():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib, moe
    return _lib, moe


def _cuda(d):
    return {k: v.cuda() for k, v in d.items()}


def _run(mod, x, logits, gu, dn, top_k, inter, E, **kw):
    _lib, moe = mod
    T, H = x.shape
    blk = moe.MoEBlock(T, H, inter, E, top_k, "cuda", **kw)
    if kw:                                          # a rank holds only its own experts (+ the shared one if it owns it)
        gu, dn = moe.slice_experts(gu, dn, E, inter, H, kw["e_lo"], kw["e_hi"], kw["with_shared"])
    out = torch.full((T, H), 7.0, dtype=torch.bfloat16, device="cuda")
    blk(x.cuda(), logits.cuda(), _cuda(gu), _cuda(dn), out)
    torch.cuda.synchronize()
    return blk, out.cpu()


def _rel(a, b):
    return float((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6))


@pytest.mark.parametrize("T,H,inter,E,k,seed", [(16, 512, 512, 16, 4, 1), (16, 2048, 512, 64, 8, 2), (5, 1024, 512, 8, 2, 3),
                                                (16, 512, 1024, 12, 3, 4)])
def test_block_matches_oracle(mod, T, H, inter, E, k, seed):
    x, logits, gu, dn = om.make_moe_case(seed, T=T, H=H, inter=inter, E=E)
    want = om.moe_ref(x, logits, gu, dn, k, inter=inter)
    blk, got = _run(mod, x, logits, gu, dn, k, inter, E)
    ids, w, _ = om.route_ref(logits, k)
    assert torch.equal(blk.topk_ids.cpu().long(), ids)
    assert float((blk.topk_w.cpu() - w).abs().max()) <= 2e-3
    n = int(blk.n_active.cpu())
    assert n == len(set(ids.flatten().tolist())) + 1
    assert blk.slot_expert.cpu()[: n - 1].tolist() == sorted(set(ids.flatten().tolist())) and int(blk.slot_expert.cpu()[n - 1]) == E
    assert _rel(got, want) <= REL_TOL
    assert mod[0].lib().dflash_device_error(0) == 0


def test_all_tokens_choose_the_same_experts_and_repeat_is_bitwise_equal(mod):
    x, logits, gu, dn = om.make_moe_case(5, T=16, H=512, inter=512, E=16)
    logits[:, :16] = logits[0:1, :16]             # identical routing for every token: 4 active experts + shared
    want = om.moe_ref(x, logits, gu, dn, 4, inter=512)
    blk, got = _run(mod, x, logits, gu, dn, 4, 512, 16)
    assert int(blk.n_active.cpu()) == 5
    assert _rel(got, want) <= REL_TOL
    out2 = torch.empty_like(got).cuda()
    blk(x.cuda(), logits.cuda(), _cuda(gu), _cuda(dn), out2)
    torch.cuda.synchronize()
    assert torch.equal(out2.cpu(), got)


def test_expert_parallel_parts_sum_to_the_whole(mod):
    x, logits, gu, dn = om.make_moe_case(6, T=16, H=1024, inter=512, E=32)
    whole = om.moe_ref(x, logits, gu, dn, 8, inter=512)
    total = torch.zeros(16, 1024)
    for r in range(4):
        want = om.moe_ref(x, logits, gu, dn, 8, inter=512, e_lo=8 * r, e_hi=8 * r + 8, with_shared=(r == 0))
        _, got = _run(mod, x, logits, gu, dn, 8, 512, 32, e_lo=8 * r, e_hi=8 * r + 8, with_shared=(r == 0))
        assert _rel(got, want) <= REL_TOL
        total += got.float()
    assert _rel(total, whole) <= 2e-2


def test_rank_without_active_experts_writes_zeros(mod):
    x, logits, gu, dn = om.make_moe_case(7, T=16, H=512, inter=512, E=16)
    logits[:, 8:16] = -30.0                        # nobody chooses experts 8..15
    blk, got = _run(mod, x, logits, gu, dn, 4, 512, 16, e_lo=8, e_hi=16, with_shared=False)
    assert int(blk.n_active.cpu()) == 0
    assert float(got.float().abs().max()) == 0.0


def test_graph_capture_with_changing_routing(mod):
    _lib, moe = mod
    x, logits, gu, dn = om.make_moe_case(8, T=16, H=512, inter=512, E=16)
    blk = moe.MoEBlock(16, 512, 512, 16, 4, "cuda")
    xs, ls, g, d = x.cuda(), logits.cuda(), _cuda(gu), _cuda(dn)
    out = torch.empty(16, 512, dtype=torch.bfloat16, device="cuda")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        blk(xs, ls, g, d, out)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            blk(xs, ls, g, d, out)
    torch.cuda.current_stream().wait_stream(side)
    for seed in (9, 10):                           # new routing through the same graph: sizes are read on the device
        x2, l2, _, _ = om.make_moe_case(seed, T=16, H=512, inter=512, E=16)
        xs.copy_(x2)
        ls.copy_(l2)
        graph.replay()
        torch.cuda.synchronize()
        assert _rel(out.cpu(), om.moe_ref(x2, l2, gu, dn, 4, inter=512)) <= REL_TOL
    assert _lib.lib().dflash_device_error(0) == 0


@pytest.mark.parametrize("T,H,inter,E,k,seed", [(16, 512, 512, 16, 4, 21), (16, 2048, 512, 64, 8, 22), (5, 1024, 512, 8, 2, 23)])
def test_mma_sync_gather_kernels_still_match_the_oracle(mod, T, H, inter, E, k, seed):
    """The expert-gathered matmuls run on the tcgen05 kernel by default; dflash_verify_qmm_set_impl(1) selects the
    mma.sync gather kernels (exact integer nibbles, scale applied to the accumulator).  Both meet the oracle; they agree
    with each other within the same tolerance."""
    _lib, _ = mod
    lib = _lib.lib()
    x, logits, gu, dn = om.make_moe_case(seed, T=T, H=H, inter=inter, E=E)
    want = om.moe_ref(x, logits, gu, dn, k, inter=inter)
    _, tc = _run(mod, x, logits, gu, dn, k, inter, E)
    assert lib.dflash_verify_qmm_last_impl() == 2
    try:
        lib.dflash_verify_qmm_set_impl(1)
        _, old = _run(mod, x, logits, gu, dn, k, inter, E)          # its own block: a workspace is not shared between the kernels
        assert lib.dflash_verify_qmm_last_impl() == 1
    finally:
        lib.dflash_verify_qmm_set_impl(0)
    assert lib.dflash_device_error(0) == 0
    assert _rel(tc, want) <= REL_TOL and _rel(old, want) <= REL_TOL and _rel(tc, old) <= REL_TOL
