"""Step-level GPU parity at the benchmark's real layer dimensions, against the CPU oracle (oracle/model.py).

One GatedDeltaNet layer + one full-attention layer of configuration 4 (hidden 5120, SwiGLU 17408, 24 query / 4 KV heads
of 256, context 4096 so that the block sits at positions 4096..4111) and of configuration 5 (hidden 2048, 256 experts
top-8 + a shared expert of intermediate 512, 16 query / 2 KV heads, context 8192) run through HybridVerifyModel; the
vocabulary is cut to 8192 rows to keep the CPU oracle to seconds (the full-width lm_head is covered by the matmul
tests).  Tolerances: logits max-rel <= 3e-2 (bf16 activations through two layers), greedy tokens identical on every row
whose top-2 margin in the oracle exceeds that bound (the number of such rows is printed and asserted), first-layer
tape / state <= 2e-3 (their inputs are bf16 outputs of the input projection: one bf16 ulp of a matmul output moves
them by that much; the recurrence itself is held to 1e-4 on identical inputs in tests/test_gdn_gpu.py).  The oracle
dequantises as the reference's verify kernels do (weights rounded to bf16)."""
import pytest
import torch

from oracle import model as om

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _verify_kernel_numerics():
    """The oracle dequantises like the reference's verify kernels (weights rounded to bf16, verify_qmm.py:75)."""
    old, om.KERNEL_ROUNDING = om.KERNEL_ROUNDING, True
    yield
    om.KERNEL_ROUNDING = old


def _rel(a, b):
    a, b = a.detach().cpu().float(), b.detach().cpu().float()
    return float((a - b).abs().max() / (b.abs().max() + 1e-6))


def _case(cfg, seed, context):
    from dflash_mlx_b200.verify_step import init_weights
    W = init_weights(cfg, seed, "cpu")
    gen = torch.Generator().manual_seed(seed + 1)
    Lg = sum(not cfg.is_attention(i) for i in range(cfg.layers))
    La = cfg.layers - Lg
    caches = {"conv": [torch.randn(3, cfg.conv_dim, generator=gen).bfloat16() for _ in range(Lg)],
              "state": [0.1 * torch.randn(cfg.gdn_v_heads, cfg.gdn_dv, cfg.gdn_dk, generator=gen) for _ in range(Lg)],
              "k": [torch.zeros(cfg.kv_heads, cfg.max_context, cfg.head_dim).bfloat16() for _ in range(La)],
              "v": [torch.zeros(cfg.kv_heads, cfg.max_context, cfg.head_dim).bfloat16() for _ in range(La)]}
    for c in caches["k"] + caches["v"]:
        c[:, :context] = torch.randn(cfg.kv_heads, context, cfg.head_dim, generator=gen).bfloat16()
    ids = torch.randint(0, cfg.vocab, (16,), generator=gen, dtype=torch.int32)
    return W, caches, ids


def _load(m, caches, ctx):
    for l in range(len(caches["state"])):
        m.state[m.cur][l].copy_(caches["state"][l])
        m.conv[m.cur][l].copy_(caches["conv"][l])
    for l in range(len(caches["k"])):
        m.kcache[l].copy_(caches["k"][l])
        m.vcache[l].copy_(caches["v"][l])
    m.offset = ctx


def _check_tokens(m, ref_logits, ref_toks, bound):
    rl = ref_logits.float()
    top2 = rl.topk(2, dim=-1).values
    sure = (top2[:, 0] - top2[:, 1]) > bound * rl.abs().max()
    n = int(sure.sum())
    print(f"greedy tokens compared on {n} of 16 rows")
    assert n >= 8, n
    assert torch.equal(m.tokens.cpu()[sure], ref_toks[sure])
    return n


def test_dense_layers_at_configuration_4_dimensions():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib
    from dflash_mlx_b200.verify_step import HybridConfig, HybridVerifyModel, weights_to
    cfg = HybridConfig(layers=2, attn_every=2, vocab=8192, max_context=4096 + 64)
    assert cfg.hidden == 5120 and cfg.intermediate == 17408 and cfg.q_heads == 24 and cfg.kv_heads == 4
    ctx = 4096
    W, caches, ids = _case(cfg, 41, ctx)
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    ref_logits, ref_toks, ref_new, tapes = om.verify_step_ref(cfg, W, ids, clone(caches), ctx)
    m = HybridVerifyModel(cfg, weights_to(W, "cuda"), "cuda")
    _load(m, caches, ctx)
    m.arm_rollback()
    logits = m.verify(ids.cuda())
    torch.cuda.synchronize()
    assert _rel(logits, ref_logits) <= 3e-2
    _check_tokens(m, ref_logits, ref_toks, 3e-2)
    # the fused step rounds the normed input at another place (bf16(h * w) instead of bf16(h * inv * w)): 1.5e-2 there
    tol0 = 1.5e-2 if m.fused else 2e-3
    assert _rel(m.tape[0], tapes[0]["tape"]) <= tol0
    assert _rel(m.state[m.cur ^ 1][0], ref_new["state"][0]) <= tol0
    # the attention layer's new K rows (q/k norm + RoPE at positions 4096..4111) and V rows in the cache
    assert _rel(m.kcache[0][:, ctx:ctx + 16], ref_new["k"][0][:, ctx:ctx + 16]) <= 2e-2
    assert _rel(m.vcache[0][:, ctx:ctx + 16], ref_new["v"][0][:, ctx:ctx + 16]) <= 2e-2
    assert _lib.lib().dflash_device_error(0) == 0


def test_moe_layers_at_configuration_5_dimensions():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib
    from dflash_mlx_b200.verify_step import HybridConfig, HybridVerifyModel, weights_to
    cfg = HybridConfig.moe_cfg5(layers=2, attn_every=2, vocab=8192)
    assert cfg.hidden == 2048 and cfg.moe_experts == 256 and cfg.moe_top_k == 8 and cfg.max_context == 8192 + 64
    ctx = 8192
    W, caches, ids = _case(cfg, 43, ctx)
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    m = HybridVerifyModel(cfg, weights_to(W, "cuda"), "cuda")
    _load(m, caches, ctx)
    m.arm_rollback()
    logits = m.verify(ids.cuda()).clone()
    torch.cuda.synchronize()
    # the oracle routes with the router logits the CUDA path produced, so that routing is identical by construction
    injected = [m.router_logits[i].cpu() for i in range(cfg.layers)]
    ref_logits, ref_toks, ref_new, tapes = om.verify_step_ref(cfg, W, ids, clone(caches), ctx, router_logits=injected)
    assert _rel(logits, ref_logits) <= 3e-2
    _check_tokens(m, ref_logits, ref_toks, 3e-2)
    # (the fused chain rounds the normed input at another place, as in the dense test above)
    assert _rel(m.tape[0], tapes[0]["tape"]) <= (1.5e-2 if m.fused else 2e-3)
    # and the router itself: the CUDA router logits against the oracle's router matmul on the oracle's activations
    free_logits, _, _, _ = om.verify_step_ref(cfg, W, ids, clone(caches), ctx)
    assert _rel(logits, free_logits) <= 6e-2          # a near-tie in a top-8 choice may swap one expert
    slots = m.moe_active_slots()
    assert all(8 <= s <= 129 for s in slots), slots
    assert _lib.lib().dflash_device_error(0) == 0
