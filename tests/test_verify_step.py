"""CPU checks of the verify-step oracle (oracle/model.py): the speculative-consistency property the reference's
tape design exists for - verifying 16 tokens and rolling back to `a` accepted equals processing only those `a`."""
import torch

from dflash_mlx_b200.verify_step import HybridConfig, init_weights
from oracle import gdn as og
from oracle import model as om

SMALL = dict(layers=4, hidden=512, intermediate=1024, q_heads=4, kv_heads=2, head_dim=128, rope_dims=32,
             gdn_k_heads=2, gdn_v_heads=4, gdn_dk=128, gdn_dv=128, vocab=2048, max_context=320)


def small_case(seed=5, context=64):
    cfg = HybridConfig(**SMALL)
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
    return cfg, W, caches, ids, context


SMALL_MOE = dict(SMALL, intermediate=512, moe_experts=16, moe_top_k=2, moe_inter=512)


def small_moe_case(seed=11, context=64):
    """The small hybrid model with a mixture-of-experts MLP (16 experts, top-2, one shared expert) in every layer."""
    cfg0, W0, caches, ids, ctx = small_case(seed, context)
    cfg = HybridConfig(**SMALL_MOE)
    return cfg, init_weights(cfg, seed, "cpu"), caches, ids, ctx


def test_moe_step_oracle_runs_and_expert_parallel_parts_add_up():
    import copy
    cfg, W, caches, ids, ctx = small_moe_case()
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    logits, toks, _, _ = om.verify_step_ref(cfg, W, ids, clone(caches), ctx)
    assert logits.shape == (16, cfg.vocab) and torch.isfinite(logits.float()).all()
    # one layer's MoE output equals the sum of two expert-parallel halves (the first owns the shared expert)
    from oracle import moe as omoe
    L = W["layers"][0]
    x = torch.randn(16, cfg.hidden, generator=torch.Generator().manual_seed(3)).bfloat16()
    lg = torch.randn(16, cfg.moe_experts + 1, generator=torch.Generator().manual_seed(4)).bfloat16()
    whole = omoe.moe_ref(x, lg, L["experts_gate_up"], L["experts_down"], 2, inter=512)
    a = omoe.moe_ref(x, lg, L["experts_gate_up"], L["experts_down"], 2, inter=512, e_lo=0, e_hi=8, with_shared=True)
    b = omoe.moe_ref(x, lg, L["experts_gate_up"], L["experts_down"], 2, inter=512, e_lo=8, e_hi=16, with_shared=False)
    err = float((whole.float() - a.float() - b.float()).abs().max() / whole.float().abs().max())
    assert err <= 1e-2


def test_rollback_equals_processing_only_the_accepted_tokens():
    cfg, W, caches, ids, ctx = small_case()
    clone = lambda c: {k: [t.clone() for t in v] for k, v in c.items()}  # noqa: E731
    logits, toks, new, tapes = om.verify_step_ref(cfg, W, ids, clone(caches), ctx)
    assert logits.shape == (16, cfg.vocab) and toks.shape == (16,)
    a = 6
    _, _, new_a, _ = om.verify_step_ref(cfg, W, ids[:a], clone(caches), ctx)
    for l, tp in enumerate(tapes):
        rolled = og.tape_replay_ref(tp["tape"][None], tp["k"][None], tp["g"][None], caches["state"][l][None], steps=a)[0]
        torch.testing.assert_close(rolled, new_a["state"][l], rtol=2e-2, atol=2e-3)   # bf16 activations upstream
        conv = og.rebuild_conv_state(caches["conv"][l][None], tp["qkv"][None], a, cfg.conv_kernel)[0]
        torch.testing.assert_close(conv.float(), new_a["conv"][l].float(), rtol=2e-2, atol=2e-2)
    # layer 0 sees identical inputs in both runs: exact
    rolled0 = og.tape_replay_ref(tapes[0]["tape"][None], tapes[0]["k"][None], tapes[0]["g"][None],
                                 caches["state"][0][None], steps=a)[0]
    torch.testing.assert_close(rolled0, new_a["state"][0], rtol=1e-5, atol=1e-6)


def test_acceptance_length():
    d = torch.tensor([3, 4, 5, 9, 7])
    p = torch.tensor([3, 4, 5, 6, 7, 8])
    assert om.match_acceptance_length(d, p) == 3
    assert om.match_acceptance_length(d[:0], p) == 0
    from dflash_mlx_b200.verify_step import HybridVerifyModel
    assert int(HybridVerifyModel.match_acceptance_length(d, p)) == 3
