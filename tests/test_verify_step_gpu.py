"""GPU parity of the whole 16-token verify step + rollback against the CPU oracle on a small hybrid model
(3 GatedDeltaNet layers + 1 full-attention layer).  Tolerances: logits max-rel <= 3e-2 (bf16 activations through
four layers), greedy tokens identical wherever the oracle's top-2 margin exceeds that bound, fp32 GDN state
after rollback <= 1e-2 relative (its inputs are bf16 activations), first-layer state <= 2e-3 (a projection output that
lands on the other side of a bf16 rounding boundary moves it by that much; the recurrence itself is held to 1e-4 on
identical inputs in tests/test_gdn_gpu.py)."""
import pytest
import torch

from oracle import gdn as og
from oracle import model as om
from tests.test_verify_step import small_case

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _verify_kernel_numerics():
    """The oracle dequantises like the reference's verify kernels (weights rounded to bf16, verify_qmm.py:75): that is the
    path a 16-token verify pass takes in the reference and what the tensor-core matmul reproduces, so first-layer
    quantities can be held to 1e-4."""
    old, om.KERNEL_ROUNDING = om.KERNEL_ROUNDING, True
    yield
    om.KERNEL_ROUNDING = old


def _rel(a, b):
    a, b = a.detach().cpu().float(), b.detach().cpu().float()
    return float((a - b).abs().max() / (b.abs().max() + 1e-6))


@pytest.fixture(scope="module")
def setup():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200.verify_step import HybridVerifyModel, weights_to
    cfg, W, caches, ids, ctx = small_case()
    m = HybridVerifyModel(cfg, weights_to(W, "cuda"), "cuda")
    for l in range(len(caches["state"])):
        m.state[m.cur][l].copy_(caches["state"][l])
        m.conv[m.cur][l].copy_(caches["conv"][l])
    for l in range(len(caches["k"])):
        m.kcache[l].copy_(caches["k"][l])
        m.vcache[l].copy_(caches["v"][l])
    m.offset = ctx
    return cfg, W, caches, ids, ctx, m


def test_logits_tokens_and_rollback(setup):
    cfg, W, caches, ids, ctx, m = setup
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    ref_logits, ref_toks, ref_new, tapes = om.verify_step_ref(cfg, W, ids, clone(caches), ctx)
    m.arm_rollback()
    logits = m.verify(ids.cuda())
    torch.cuda.synchronize()
    assert m.launches_per_step > 20
    assert _rel(logits, ref_logits) <= 3e-2
    # greedy argmax where the oracle's margin is larger than the error bound
    rl = ref_logits.float()
    top2 = rl.topk(2, dim=-1).values
    sure = (top2[:, 0] - top2[:, 1]) > 3e-2 * rl.abs().max()
    assert int(sure.sum()) >= 1
    assert torch.equal(m.tokens.cpu()[sure], ref_toks[sure])
    # per-layer tape and forward state
    for l, tp in enumerate(tapes):
        # layer 0: identical inputs, but one bf16 ulp of a projection output shows; the fused step applies the input norm as
        # a column scale before and a token factor after the matmul, so its x is rounded at another place (bf16(h * w)
        # instead of bf16(h * inv * w)): 2^-9 relative per element of x instead of bit-equal inputs
        tol = (1e-2 if m.fused else 2e-3) if l == 0 else 2e-2
        assert _rel(m.tape[l], tp["tape"]) <= tol, l
        assert _rel(m.state[m.cur ^ 1][l], ref_new["state"][l]) <= tol, l
    assert _rel(m.tape_qkv[0], tapes[0]["qkv"]) <= 1e-2          # a bf16 matmul output: ulp-level differences
    # rollback to 5 accepted drafts (6 committed positions), host int
    n_acc = 5
    snap_cur = m.cur
    m.rollback(n_acc, drafted_tokens=15)
    torch.cuda.synchronize()
    assert m.cur == snap_cur ^ 1 and m.offset == ctx + n_acc + 1 and not m._armed
    for l, tp in enumerate(tapes):
        want = og.tape_replay_ref(tp["tape"][None], tp["k"][None], tp["g"][None], caches["state"][l][None], steps=n_acc + 1)[0]
        assert _rel(m.state[m.cur][l], want) <= ((1e-2 if m.fused else 2e-3) if l == 0 else 2e-2), l
        conv = og.rebuild_conv_state(caches["conv"][l][None], tp["qkv"][None], n_acc + 1, cfg.conv_kernel)[0]
        if l == 0:
            assert _rel(m.conv[m.cur][l], conv) <= 1e-2


def test_fused_epilogues_against_the_unfused_step(setup):
    """The step whose norms, residual adds and SwiGLU run inside the matmul epilogues against the same step built from
    separate kernels: same greedy tokens wherever the margin is clear, logits within the step's bf16 bound."""
    from dflash_mlx_b200.verify_step import HybridVerifyModel, weights_to
    cfg, W, caches, ids, ctx, m_default = setup
    assert m_default.fused
    outs = []
    for fused in (True, False):
        m = HybridVerifyModel(cfg, weights_to(W, "cuda"), "cuda", fused=fused)
        for l in range(len(caches["state"])):
            m.state[m.cur][l].copy_(caches["state"][l])
            m.conv[m.cur][l].copy_(caches["conv"][l])
        for l in range(len(caches["k"])):
            m.kcache[l].copy_(caches["k"][l])
            m.vcache[l].copy_(caches["v"][l])
        m.offset = ctx
        logits = m.verify(ids.cuda()).float().clone()
        torch.cuda.synchronize()
        outs.append((logits, m.tokens.clone(), m.h.clone(), m.launches_per_step))
        if not fused:      # the unfused step's first layer sees bit-equal inputs: held to the tighter bound
            clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
            _, _, _, tapes = om.verify_step_ref(cfg, W, ids, clone(caches), ctx)
            assert _rel(m.tape[0], tapes[0]["tape"]) <= 2e-3
    (lf, tf, hf, nf), (lu, tu, hu, nu) = outs
    assert nf < nu - 2 * cfg.layers
    assert _rel(lf, lu) <= 3e-2 and _rel(hf, hu) <= 3e-2
    top2 = lu.topk(2, dim=-1).values
    sure = (top2[:, 0] - top2[:, 1]) > 3e-2 * lu.abs().max()
    assert torch.equal(tf[sure], tu[sure])


def test_device_side_accept_length_and_full_accept(setup):
    cfg, W, caches, ids, ctx, m = setup
    # restore the committed buffers, run again, roll back with the accepted length living on the device
    for l in range(len(caches["state"])):
        m.state[m.cur][l].copy_(caches["state"][l])
        m.conv[m.cur][l].copy_(caches["conv"][l])
    m.offset = ctx
    m.arm_rollback()
    m.verify(ids.cuda())
    tape0 = m.tape[0].clone()
    k0, g0 = m.tape_k[0].clone(), m.tape_g[0].clone()
    n_dev = torch.tensor([8], dtype=torch.int32, device="cuda")
    m.rollback(n_dev)
    torch.cuda.synchronize()
    want = og.tape_replay_ref(tape0.cpu()[None], k0.cpu()[None], g0.cpu()[None], caches["state"][0][None], steps=9)[0]
    assert _rel(m.state[m.cur][0], want) <= 1e-4
    # fully accepted block: the forward state is kept, no replay
    for l in range(len(caches["state"])):
        m.state[m.cur][l].copy_(caches["state"][l])
        m.conv[m.cur][l].copy_(caches["conv"][l])
    m.offset = ctx
    m.arm_rollback()
    m.verify(ids.cuda())
    fwd = m.state[m.cur ^ 1].clone()
    m.rollback(15, drafted_tokens=15)
    assert torch.equal(m.state[m.cur], fwd) and m.offset == ctx + 16


def test_moe_step_matches_oracle():
    """The same step with a mixture-of-experts MLP in every layer (16 experts, top-2, shared expert): logits within
    tolerance, and the captured graph (routing sizes read on the device) reproduces the eager result."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200.verify_step import HybridVerifyModel, weights_to
    from dflash_mlx_b200 import _lib
    from tests.test_verify_step import small_moe_case
    cfg, W, caches, ids, ctx = small_moe_case()
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    m = HybridVerifyModel(cfg, weights_to(W, "cuda"), "cuda")

    def restore():
        for l in range(len(caches["state"])):
            m.state[0][l].copy_(caches["state"][l]); m.state[1][l].copy_(caches["state"][l])
            m.conv[0][l].copy_(caches["conv"][l]); m.conv[1][l].copy_(caches["conv"][l])
        for l in range(len(caches["k"])):
            m.kcache[l].copy_(caches["k"][l]); m.vcache[l].copy_(caches["v"][l])
        m.cur, m.offset, m._armed = 0, ctx, False

    restore()
    m.arm_rollback()
    logits = m.verify(ids.cuda()).clone()
    torch.cuda.synchronize()
    # the oracle routes with the router logits the CUDA path produced (injected, so routing is identical)
    injected = [m.router_logits[i].cpu() for i in range(cfg.layers)]
    ref_logits, ref_toks, _, _ = om.verify_step_ref(cfg, W, ids, clone(caches), ctx, router_logits=injected)
    assert _rel(logits, ref_logits) <= 3e-2
    slots = m.moe_active_slots()
    assert len(slots) == cfg.layers and all(2 <= s <= 17 for s in slots)
    restore()
    m.arm_rollback()
    eager = m.verify(ids.cuda()).clone()
    toks = m.tokens.clone()
    restore()
    m._armed = True
    m.capture()
    restore()
    m._armed = True
    m.verify_captured(ids.cuda())
    torch.cuda.synchronize()
    assert torch.equal(m.tokens, toks)
    assert torch.equal(m.logits.view(-1)[: eager.numel()].view_as(eager), eager)
    assert "experts" in m.algorithmic_bytes()
    assert _lib.lib().dflash_device_error(0) == 0


def test_device_side_cycle_matches_host_driven_cycle():
    """verify -> accept -> roll back with the cache position on the device, as ONE replayed graph per cycle, against the
    same cycles driven from the host (eager launches, host integers): identical tokens, accepted lengths, recurrent
    state, conv window, KV cache and position after every cycle, for several cycles and accepted lengths."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200.verify_step import HybridVerifyModel, weights_to
    from dflash_mlx_b200 import _lib
    cfg, W, caches, ids, ctx = small_case()
    Wc = weights_to(W, "cuda")

    def fresh():
        m = HybridVerifyModel(cfg, Wc, "cuda")
        for l in range(len(caches["state"])):
            m.state[0][l].copy_(caches["state"][l]); m.conv[0][l].copy_(caches["conv"][l])
        for l in range(len(caches["k"])):
            m.kcache[l].copy_(caches["k"][l]); m.vcache[l].copy_(caches["v"][l])
        m.cur, m.offset = 0, ctx
        return m

    host, dev = fresh(), fresh()
    dev.enable_device_offset()
    gen = torch.Generator().manual_seed(77)
    T = cfg.block
    accepted = []
    for cyc in range(5):
        # a block whose first `want` drafted tokens agree with the target (built greedily with the host model)
        want = [0, 3, 15, 1, 7][cyc]
        block = torch.randint(0, cfg.vocab, (T,), generator=gen, dtype=torch.int32).cuda()
        snap = (host.cur, host.offset, [host.state[i].clone() for i in range(2)], [host.conv[i].clone() for i in range(2)],
                host.kcache.clone(), host.vcache.clone())
        for j in range(want):
            host.arm_rollback()
            host.verify(block)
            block[j + 1] = host.tokens[j]
            host.cur, host.offset = snap[0], snap[1]
            for i in range(2):
                host.state[i].copy_(snap[2][i]); host.conv[i].copy_(snap[3][i])
            host.kcache.copy_(snap[4]); host.vcache.copy_(snap[5])
        if want < T - 1:                          # make sure the next drafted token is wrong
            host.arm_rollback()
            host.verify(block)
            block[want + 1] = (host.tokens[want] + 1) % cfg.vocab
            host.cur, host.offset = snap[0], snap[1]
            for i in range(2):
                host.state[i].copy_(snap[2][i]); host.conv[i].copy_(snap[3][i])
            host.kcache.copy_(snap[4]); host.vcache.copy_(snap[5])
        # host-driven cycle
        host.arm_rollback()
        host.verify(block)
        n_host = int(host.match_acceptance_length(block[1:], host.tokens))
        toks_host = host.tokens.clone()
        host.rollback(n_host, drafted_tokens=T - 1)
        # device-driven cycle, one graph launch
        n_dev = dev.cycle_captured(block)
        torch.cuda.synchronize()
        assert n_host == want
        assert int(n_dev) == n_host
        assert torch.equal(dev.tokens, toks_host)
        assert dev.cur == host.cur
        assert torch.equal(dev.state[dev.cur], host.state[host.cur])
        assert torch.equal(dev.conv[dev.cur], host.conv[host.cur])
        assert int(dev.offset_dev) == host.offset
        assert torch.equal(dev.kcache[:, :, : host.offset], host.kcache[:, :, : host.offset])
        accepted.append(n_host)
    assert accepted == [0, 3, 15, 1, 7]
    assert dev.sync_offset() == host.offset
    assert len(dev._cycle_graphs) == 2            # one graph per parity of the state buffers, reused afterwards
    assert _lib.lib().dflash_device_error(0) == 0


def test_hidden_state_capture_for_the_draft_model(setup):
    """`capture_layer_ids` semantics of the reference's target forward (key k = residual stream after layer k-1, key 0 =
    embeddings) and the context feature the draft model is fed (concatenation along the feature axis)."""
    cfg, W, caches, ids, ctx, m = setup
    for l in range(len(caches["state"])):
        m.state[m.cur][l].copy_(caches["state"][l])
        m.conv[m.cur][l].copy_(caches["conv"][l])
    for l in range(len(caches["k"])):
        m.kcache[l].copy_(caches["k"][l]); m.vcache[l].copy_(caches["v"][l])
    m.offset = ctx
    m.set_capture_layers({0, 2, cfg.layers})
    m.arm_rollback()
    m.verify(ids.cuda())
    torch.cuda.synchronize()
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    cap = {}
    om.verify_step_ref(cfg, W, ids, clone(caches), ctx, captured=cap)
    assert torch.equal(m.captured[0].cpu(), cap[0])                      # embeddings: a gather, exact
    assert _rel(m.captured[1], cap[2]) <= 3e-2
    assert _rel(m.captured[2], cap[cfg.layers]) <= 3e-2
    feat = m.context_feature([1, cfg.layers - 1])                        # target layer ids -> keys id + 1
    assert feat.shape == (cfg.block, 2 * cfg.hidden)
    assert torch.equal(feat[:, : cfg.hidden], m.captured[1]) and torch.equal(feat[:, cfg.hidden:], m.captured[2])
    m.set_capture_layers(())
    m._armed = False


def _fresh_model(cfg, Wc, caches, ctx):
    from dflash_mlx_b200.verify_step import HybridVerifyModel
    m = HybridVerifyModel(cfg, Wc, "cuda")
    for l in range(len(caches["state"])):
        m.state[0][l].copy_(caches["state"][l]); m.conv[0][l].copy_(caches["conv"][l])
    for l in range(len(caches["k"])):
        m.kcache[l].copy_(caches["k"][l]); m.vcache[l].copy_(caches["v"][l])
    m.cur, m.offset = 0, ctx
    return m


def test_device_cycle_against_the_oracle_cycle():
    """One whole cycle on the device (verify, greedy posterior, acceptance, state replay, conv window, position: the
    accept/commit kernel + the replay kernel) against the same cycle computed by the CPU oracle alone
    (runtime.py:101-108, 878-907; recurrent_rollback_cache.py:148-171)."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200.verify_step import weights_to
    cfg, W, caches, ids, ctx = small_case()
    Wc = weights_to(W, "cuda")
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    T = cfg.block
    for want in (0, 4, 15):
        # drafted tokens that agree with the oracle's greedy tokens on the first `want` positions
        block = ids.clone()
        for _ in range(want + 1):
            _, toks, _, _ = om.verify_step_ref(cfg, W, block, clone(caches), ctx)
            n_now = int(om.match_acceptance_length(block[1:], toks))
            if n_now >= want:
                break
            block[n_now + 1] = toks[n_now]
        ref_logits, ref_toks, ref_new, tapes = om.verify_step_ref(cfg, W, block, clone(caches), ctx)
        n_ref = int(om.match_acceptance_length(block[1:], ref_toks))
        if n_ref > want and want < T - 1:
            block[want + 1] = (ref_toks[want] + 1) % cfg.vocab
            ref_logits, ref_toks, ref_new, tapes = om.verify_step_ref(cfg, W, block, clone(caches), ctx)
            n_ref = int(om.match_acceptance_length(block[1:], ref_toks))
        m = _fresh_model(cfg, Wc, caches, ctx)
        m.enable_device_offset()
        n_dev = m.cycle(block.cuda())
        torch.cuda.synchronize()
        # rows whose greedy choice is clear must agree; then the accepted length can only differ through an unclear row
        rl = ref_logits.float()
        top2 = rl.topk(2, dim=-1).values
        sure = (top2[:, 0] - top2[:, 1]) > 3e-2 * rl.abs().max()
        assert torch.equal(m.tokens.cpu()[sure], ref_toks[sure])
        if bool(sure[: n_ref + 1].all()):
            assert int(n_dev) == n_ref
        n = int(n_dev)
        assert int(m.offset_dev) == ctx + n + 1 and int(m.kvlen_dev) == ctx + n + 1 + T
        for l, tp in enumerate(tapes):
            want_state = og.tape_replay_ref(tp["tape"][None], tp["k"][None], tp["g"][None], caches["state"][l][None], steps=n + 1)[0]
            assert _rel(m.state[m.cur][l], want_state) <= (1e-2 if l == 0 else 2e-2), l
            conv = og.rebuild_conv_state(caches["conv"][l][None], tp["qkv"][None], n + 1, cfg.conv_kernel)[0]
            if l == 0:
                assert _rel(m.conv[m.cur][l], conv) <= 1e-2
        m.check_device_error("test")


@pytest.mark.parametrize("T_short", [1, 5, 12])
def test_blocks_shorter_than_the_configured_one(T_short):
    """The block length is the draft's (runtime.py:1676-1678): 1 .. block tokens go through the same kernels."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200.verify_step import weights_to
    cfg, W, caches, ids, ctx = small_case()
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    short = ids[:T_short].clone()
    ref_logits, ref_toks, ref_new, tapes = om.verify_step_ref(cfg, W, short, clone(caches), ctx)
    m = _fresh_model(cfg, weights_to(W, "cuda"), caches, ctx)
    m.arm_rollback()
    logits = m.verify(short.cuda())
    torch.cuda.synchronize()
    assert logits.shape == (T_short, cfg.vocab)
    assert _rel(logits, ref_logits) <= 3e-2
    rl = ref_logits.float()
    top2 = rl.topk(2, dim=-1).values
    sure = (top2[:, 0] - top2[:, 1]) > 3e-2 * rl.abs().max()
    assert torch.equal(m.tokens.cpu()[:T_short][sure], ref_toks[sure])
    for l, tp in enumerate(tapes):
        assert _rel(m.tape[l][:T_short], tp["tape"]) <= (1e-2 if l == 0 else 2e-2), l
    # the attention layer appended exactly T_short rows at the right positions
    assert _rel(m.kcache[0][:, ctx:ctx + T_short], ref_new["k"][0][:, ctx:ctx + T_short]) <= 2e-2
    # commit 1 + accepted positions of the short block (host path)
    n_acc = min(2, T_short - 1)
    m.rollback(n_acc, drafted_tokens=T_short - 1)
    torch.cuda.synchronize()
    assert m.offset == ctx + n_acc + 1
    want = og.tape_replay_ref(tapes[0]["tape"][None], tapes[0]["k"][None], tapes[0]["g"][None], caches["state"][0][None],
                              steps=n_acc + 1)[0]
    assert _rel(m.state[m.cur][0], want) <= 1e-2
    m.check_device_error("test")


def test_suppressed_tokens_are_never_the_greedy_choice(setup):
    """greedy_tokens_with_mask (runtime.py:90-98): masked logits count as -1e9 in the logits' type."""
    cfg, W, caches, ids, ctx, m = setup
    m.arm_rollback()
    plain = m.verify(ids.cuda()).float().clone()
    toks_plain = m.tokens.clone()
    mask = torch.zeros(cfg.vocab, dtype=torch.bool, device="cuda")
    mask[toks_plain.long()] = True                  # suppress every row's winner
    mask[::7] = True
    m.arm_rollback()
    logits = m.verify(ids.cuda(), suppress_token_mask=mask)
    torch.cuda.synchronize()
    assert torch.equal(logits.float(), plain)       # the logits themselves are untouched
    floor = torch.tensor(-1e9, dtype=torch.bfloat16, device="cuda").float()
    want = torch.where(mask[None, :], floor, logits.float()).argmax(dim=-1).to(torch.int32)
    assert torch.equal(m.tokens, want)
    assert not bool(mask[m.tokens.long()].any())


def test_moe_fused_chain_against_separate_kernels():
    """One GPU, mixture-of-experts layers: the router, the gathered gate|up matmul (post-norm finished from its partial
    sums) and the summed down projection (residual add, next norm's scale and partial sums) as one chain of matmul
    epilogues, against the same step with separate add + RMSNorm kernels.  Both passes route by the first pass's router
    logits (a near-tie in the top-k is a discontinuity of the model, not an arithmetic difference).  3e-2 of the
    largest logit / hidden value, as for the dense chain."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200.verify_step import HybridVerifyModel, weights_to
    from dflash_mlx_b200 import _lib
    from tests.test_verify_step import small_moe_case
    cfg, W, caches, ids, ctx = small_moe_case()
    Wd = weights_to(W, "cuda")

    def load(m):
        for l in range(len(caches["state"])):
            m.state[m.cur][l].copy_(caches["state"][l])
            m.conv[m.cur][l].copy_(caches["conv"][l])
        for l in range(len(caches["k"])):
            m.kcache[l].copy_(caches["k"][l])
            m.vcache[l].copy_(caches["v"][l])
        m.offset = ctx

    mf = HybridVerifyModel(cfg, Wd, "cuda")
    if not mf.fused:
        pytest.skip("the expert block's epilogues do not apply to this shape")
    mu = HybridVerifyModel(cfg, Wd, "cuda", fused=False)
    assert not mu.fused
    load(mf)
    load(mu)
    lf = mf.verify(ids.cuda()).float().clone()
    mu.routing_from = mf.router_logits
    lu = mu.verify(ids.cuda()).float().clone()
    torch.cuda.synchronize()
    assert _lib.lib().dflash_device_error(0) == 0
    assert mf.launches_per_step < mu.launches_per_step
    assert _rel(lf, lu) <= 3e-2 and _rel(mf.h, mu.h) <= 3e-2
    top2 = lu.topk(2, dim=-1).values
    sure = (top2[:, 0] - top2[:, 1]) > 3e-2 * lu.abs().max()
    assert torch.equal(mf.tokens[sure], mu.tokens[sure])
