"""Programmatic dependent launch must not change results: the verify step (eager and as a CUDA graph) and a chain of
matmuls that share one workspace give bit-identical outputs with the launch attribute on and off."""
import pytest
import torch

from oracle import qmm as oq
from tests.test_verify_step import small_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def lib():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib
    handle = _lib.lib()
    before = handle.dflash_get_pdl()
    yield handle
    handle.dflash_set_pdl(before)


def _model():
    from dflash_mlx_b200.verify_step import HybridVerifyModel, weights_to
    cfg, W, caches, ids, ctx = small_case()
    m = HybridVerifyModel(cfg, weights_to(W, "cuda"), "cuda")

    def restore():
        for l in range(len(caches["state"])):
            m.state[0][l].copy_(caches["state"][l])
            m.state[1][l].copy_(caches["state"][l])
            m.conv[0][l].copy_(caches["conv"][l])
            m.conv[1][l].copy_(caches["conv"][l])
        for l in range(len(caches["k"])):
            m.kcache[l].copy_(caches["k"][l])
            m.vcache[l].copy_(caches["v"][l])
        m.cur = 0
        m.offset = ctx
        m._armed = False
    return m, ids.cuda(), restore


def test_switch_round_trips(lib):
    lib.dflash_set_pdl(0)
    assert lib.dflash_get_pdl() == 0
    lib.dflash_set_pdl(1)
    assert lib.dflash_get_pdl() == 1


def test_verify_step_identical_with_and_without(lib):
    m, ids, restore = _model()
    out = {}
    for on in (0, 1, 0, 1):
        lib.dflash_set_pdl(on)
        restore()
        m.arm_rollback()
        logits = m.verify(ids).clone()
        torch.cuda.synchronize()
        res = (logits, m.tokens.clone(), m.state[m.cur ^ 1].clone(), m.tape.clone())
        if on in out:
            for a, b in zip(out[on], res):
                assert torch.equal(a, b)          # the kernels are deterministic run to run
        out[on] = res
    for a, b in zip(out[0], out[1]):
        assert torch.equal(a, b)
    assert lib.dflash_device_error(0) == 0


def test_captured_step_identical(lib):
    m, ids, restore = _model()
    lib.dflash_set_pdl(0)
    restore()
    m.arm_rollback()
    want = m.verify(ids).clone()
    want_tok = m.tokens.clone()
    torch.cuda.synchronize()
    lib.dflash_set_pdl(1)
    restore()
    m.arm_rollback()
    m.capture()
    for _ in range(3):                            # replays start from the same committed caches
        restore()
        m._armed = True
        m.verify_captured(ids)
        torch.cuda.synchronize()
        assert torch.equal(m.tokens, want_tok)
        assert torch.equal(m.logits.view(-1)[: want.numel()].view_as(want), want)
    assert lib.dflash_device_error(0) == 0


def test_matmul_chain_on_one_workspace(lib):
    """y1 = x W1^T, y2 = y1 W2^T, y3 = y2 W3^T back to back on one stream and one workspace: each launch may start
    while the previous one drains, but reads its input and touches the workspace only after the previous one ended."""
    from dflash_mlx_b200.verify_qmm import verify_matmul
    torch.manual_seed(5)
    K = 2048
    x = (torch.randn(16, K) * 0.5).to(torch.bfloat16).cuda()
    Ws = [tuple(t.cuda() for t in oq.random_quantized(K, K, seed=10 + i, group_size=64)) for i in range(3)]
    res = {}
    for on in (0, 1):
        lib.dflash_set_pdl(on)
        outs = []
        for _ in range(4):
            h = x
            for (w, s, b) in Ws:
                h = verify_matmul(h, w, s, b, group_size=64)
            outs.append(h.clone())
        torch.cuda.synchronize()
        for o in outs[1:]:
            assert torch.equal(o, outs[0])
        res[on] = outs[0]
    assert torch.equal(res[0], res[1])
    assert lib.dflash_device_error(0) == 0
