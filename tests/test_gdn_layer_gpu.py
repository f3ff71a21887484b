"""The one-launch GatedDeltaNet layer (dflash_gdn_layer) against (a) the three calls it replaces - bit for bit where the
arithmetic is the same - and (b) plain torch formulas written from the reference's layer hook
(dflash_mlx/runtime.py:368-445: depthwise causal conv + SiLU, q/k RMSNorm and scaling, `compute_g`, beta, the gated
delta rule, the gated RMSNorm) and its rollback cache (recurrent_rollback_cache.py:116-171).

Tolerances: the state / tape against the formulas 2e-3 relative to the largest value (bf16 inputs, fp32 recurrence; the
recurrence alone is held to 1e-4 in tests/test_gdn_gpu.py); bf16 outputs 1e-2."""
import pytest
import torch

pytestmark = pytest.mark.gpu
BF = torch.bfloat16


def _rel(a, b):
    a, b = a.detach().cpu().float(), b.detach().cpu().float()
    return float((a - b).abs().max() / (b.abs().max() + 1e-6))


def _case(T, Hk, Hv, Dv, Kc, seed):
    g = torch.Generator().manual_seed(seed)
    Dk = 128
    conv_dim = 2 * Hk * Dk + Hv * Dv
    ld = conv_dim + Hv * Dv + 2 * Hv + 24          # a padded row stride
    proj = torch.randn(16, ld, generator=g).to(BF)
    conv_state = torch.randn(Kc - 1, conv_dim, generator=g).to(BF)
    conv_w = (0.5 * torch.randn(conv_dim, Kc, generator=g)).to(BF)
    A_log = torch.log(0.5 + 4.0 * torch.rand(Hv, generator=g)).float()
    dt_bias = (0.5 * torch.randn(Hv, generator=g)).float()
    g_norm = (1.0 + 0.1 * torch.randn(Dv, generator=g)).to(BF)
    state = (0.1 * torch.randn(Hv, Dv, Dk, generator=g)).float()
    return dict(T=T, Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, Kc=Kc, ld=ld, conv_dim=conv_dim, proj=proj, conv_state=conv_state,
                conv_w=conv_w, A_log=A_log, dt_bias=dt_bias, g_norm=g_norm, state=state)


def _torch_formulas(c, eps=1e-6):
    """Independent restatement in torch (fp32 arithmetic, bf16 where the reference's arrays are bf16)."""
    T, Hk, Hv, Dk, Dv, Kc, cd = c["T"], c["Hk"], c["Hv"], c["Dk"], c["Dv"], c["Kc"], c["conv_dim"]
    proj = c["proj"][:T]
    qkv = proj[:, :cd]
    z = proj[:, cd:cd + Hv * Dv].reshape(T, Hv, Dv).float()
    b = proj[:, cd + Hv * Dv: cd + Hv * Dv + Hv].float()
    a = proj[:, cd + Hv * Dv + Hv: cd + Hv * Dv + 2 * Hv].float()
    x = torch.cat([c["conv_state"], qkv], dim=0).float()                     # [Kc-1+T, cd]
    new_conv = torch.cat([c["conv_state"], qkv], dim=0)[T:T + Kc - 1]
    w = c["conv_w"].float()
    conv = sum(x[j:j + T] * w[:, j][None] for j in range(Kc))
    conv = torch.nn.functional.silu(conv.to(BF).float()).to(BF).float()
    q = conv[:, :Hk * Dk].reshape(T, Hk, Dk)
    k = conv[:, Hk * Dk:2 * Hk * Dk].reshape(T, Hk, Dk)
    v = conv[:, 2 * Hk * Dk:].reshape(T, Hv, Dv)
    rms = lambda t: (t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)).to(BF).float()   # noqa: E731
    q = (rms(q) * (Dk ** -0.5) ** 2).to(BF).float()
    k = (rms(k) * Dk ** -0.5).to(BF)
    sp = torch.nn.functional.softplus((a + c["dt_bias"][None]).to(BF).float())
    gate = torch.exp(-torch.exp(c["A_log"])[None] * sp)                       # [T, Hv]
    beta = torch.sigmoid(b).to(BF).float()
    S = c["state"].clone()                                                    # [Hv, Dv, Dk]
    rep = Hv // Hk
    ys, tape = [], []
    for t in range(T):
        kt = k[t].float().repeat_interleave(rep, dim=0)                       # [Hv, Dk]
        qt = q[t].repeat_interleave(rep, dim=0)
        S = S * gate[t][:, None, None]
        kv = torch.einsum("hvk,hk->hv", S, kt)
        delta = (v[t] - kv) * beta[t][:, None]
        S = S + delta[:, :, None] * kt[:, None, :]
        ys.append(torch.einsum("hvk,hk->hv", S, qt))
        tape.append(delta)
    y = torch.stack(ys).to(BF).float()                                        # [T, Hv, Dv]
    n = (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + eps) * c["g_norm"].float()).to(BF).float()
    out = (n * torch.nn.functional.silu(z)).to(BF)
    return dict(out=out.reshape(T, Hv * Dv), state=S, tape=torch.stack(tape), k=k, g=gate, new_conv=new_conv, qkv=qkv)


def _run_record_norm(c):
    """dflash_gdn_prep, then the record pass with the gated RMSNorm in the same launch."""
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    lib = _lib.lib()
    d = "cuda"
    T, Hk, Hv, Dk, Dv, Kc, cd, ld = (c[k] for k in ("T", "Hk", "Hv", "Dk", "Dv", "Kc", "conv_dim", "ld"))
    dev = {k: c[k].to(d) for k in ("proj", "conv_state", "conv_w", "A_log", "dt_bias", "g_norm", "state")}
    z = lambda *s, dt=BF: torch.zeros(*s, dtype=dt, device=d)   # noqa: E731
    o = dict(state=z(Hv, Dv, Dk, dt=torch.float32), tape=z(T, Hv, Dv, dt=torch.float32), k=z(T, Hk, Dk),
             g=z(T, Hv, dt=torch.float32), new_conv=z(Kc - 1, cd), qkv=z(T, cd), out=z(T, Hv * Dv))
    z_off = cd
    b_off = z_off + Hv * Dv
    a_off = b_off + Hv
    st = torch.cuda.current_stream().cuda_stream
    q, v, beta = z(T, Hk, Dk), z(T, Hv, Dv), z(T, Hv, dt=torch.float32)
    rc = lib.dflash_gdn_prep(dev["proj"].data_ptr(), ld, z_off, b_off, a_off, dev["conv_state"].data_ptr(),
                             dev["conv_w"].data_ptr(), None, dev["A_log"].data_ptr(), dev["dt_bias"].data_ptr(), q.data_ptr(),
                             o["k"].data_ptr(), v.data_ptr(), o["g"].data_ptr(), beta.data_ptr(), o["new_conv"].data_ptr(),
                             o["qkv"].data_ptr(), T, Hk, Hv, Dk, Dv, Kc, 1e-6, _lib.BF16, st)
    assert rc == 0, lib.dflash_last_error_string()
    rc = lib.dflash_gdn_forward_tape_norm(q.data_ptr(), o["k"].data_ptr(), v.data_ptr(), o["g"].data_ptr(), beta.data_ptr(),
                                          dev["state"].data_ptr(), o["state"].data_ptr(), o["tape"].data_ptr(),
                                          dev["proj"].data_ptr(), ld, z_off, dev["g_norm"].data_ptr(), o["out"].data_ptr(),
                                          Hv * Dv, 1, T, Hk, Hv, Dk, Dv, 1e-6, _lib.BF16, _lib.F32, st)
    assert rc == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    assert lib.dflash_device_error(0) == 0
    return o


def _run(c, fused):
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    lib = _lib.lib()
    d = "cuda"
    T, Hk, Hv, Dk, Dv, Kc, cd, ld = (c[k] for k in ("T", "Hk", "Hv", "Dk", "Dv", "Kc", "conv_dim", "ld"))
    dev = {k: c[k].to(d) for k in ("proj", "conv_state", "conv_w", "A_log", "dt_bias", "g_norm", "state")}
    z = lambda *s, dt=BF: torch.zeros(*s, dtype=dt, device=d)   # noqa: E731
    o = dict(state=z(Hv, Dv, Dk, dt=torch.float32), tape=z(T, Hv, Dv, dt=torch.float32), k=z(T, Hk, Dk),
             g=z(T, Hv, dt=torch.float32), new_conv=z(Kc - 1, cd), qkv=z(T, cd), out=z(T, Hv * Dv))
    z_off = cd
    b_off = z_off + Hv * Dv
    a_off = b_off + Hv
    st = torch.cuda.current_stream().cuda_stream
    if fused:
        rc = lib.dflash_gdn_layer(dev["proj"].data_ptr(), ld, z_off, b_off, a_off, dev["conv_state"].data_ptr(),
                                  dev["conv_w"].data_ptr(), None, dev["A_log"].data_ptr(), dev["dt_bias"].data_ptr(),
                                  dev["g_norm"].data_ptr(), dev["state"].data_ptr(), o["state"].data_ptr(), o["tape"].data_ptr(),
                                  o["k"].data_ptr(), o["g"].data_ptr(), o["new_conv"].data_ptr(), o["qkv"].data_ptr(),
                                  o["out"].data_ptr(), Hv * Dv, T, Hk, Hv, Dk, Dv, Kc, 1e-6, _lib.BF16, _lib.F32, st)
        assert rc == 0, lib.dflash_last_error_string()
    else:
        q, v, beta, y = z(T, Hk, Dk), z(T, Hv, Dv), z(T, Hv, dt=torch.float32), z(T, Hv, Dv)
        rc = lib.dflash_gdn_prep(dev["proj"].data_ptr(), ld, z_off, b_off, a_off, dev["conv_state"].data_ptr(),
                                 dev["conv_w"].data_ptr(), None, dev["A_log"].data_ptr(), dev["dt_bias"].data_ptr(), q.data_ptr(),
                                 o["k"].data_ptr(), v.data_ptr(), o["g"].data_ptr(), beta.data_ptr(), o["new_conv"].data_ptr(),
                                 o["qkv"].data_ptr(), T, Hk, Hv, Dk, Dv, Kc, 1e-6, _lib.BF16, st)
        assert rc == 0, lib.dflash_last_error_string()
        # (the default record kernel: the one-launch layer shares its step function, so state and tape agree bit for bit)
        rc = lib.dflash_gdn_forward_tape(q.data_ptr(), o["k"].data_ptr(), v.data_ptr(), o["g"].data_ptr(), beta.data_ptr(), None,
                                         dev["state"].data_ptr(), o["state"].data_ptr(), y.data_ptr(), o["tape"].data_ptr(), 1, T,
                                         Hk, Hv, Dk, Dv, 0, _lib.BF16, _lib.F32, st)
        assert rc == 0, lib.dflash_last_error_string()
        rc = lib.dflash_gated_rmsnorm(y.data_ptr(), dev["proj"].data_ptr(), ld, z_off, dev["g_norm"].data_ptr(),
                                      o["out"].data_ptr(), T, Hv, Dv, 1e-6, _lib.BF16, st)
        assert rc == 0, lib.dflash_last_error_string()
    torch.cuda.synchronize()
    assert lib.dflash_device_error(0) == 0
    return o


@pytest.mark.parametrize("T,Hk,Hv,Dv,Kc", [(16, 16, 32, 128, 4), (16, 2, 4, 128, 4), (7, 2, 2, 64, 3), (1, 1, 2, 16, 2),
                                            (16, 4, 8, 96, 8)])
def test_one_launch_layer(T, Hk, Hv, Dv, Kc):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    c = _case(T, Hk, Hv, Dv, Kc, seed=100 + Hv + Dv + T)
    fused, three = _run(c, True), _run(c, False)
    for name in ("state", "tape", "k", "g", "new_conv", "qkv"):
        assert torch.equal(fused[name], three[name]), name
    # k . q per token and the output norm's sum of squares are added in another order: last-bit differences only
    assert _rel(fused["out"], three["out"]) <= 8e-3
    assert float((fused["out"].float() - three["out"].float()).abs().gt(0).float().mean()) <= 0.02
    ref = _torch_formulas(c)
    for o in (fused, three):
        assert torch.equal(o["qkv"].cpu(), ref["qkv"]) and torch.equal(o["new_conv"].cpu(), ref["new_conv"])
        assert _rel(o["k"], ref["k"]) <= 1e-2
        assert _rel(o["g"], ref["g"]) <= 1e-5
        assert _rel(o["tape"], ref["tape"]) <= 2e-3
        assert _rel(o["state"], ref["state"]) <= 2e-3
        assert _rel(o["out"], ref["out"]) <= 1e-2


def test_refusals():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    lib = _lib.lib()
    assert lib.dflash_gdn_layer_supported(16, 16, 32, 128, 128, 4, _lib.BF16, _lib.F32) == 1
    assert lib.dflash_gdn_layer_supported(16, 16, 32, 64, 128, 4, _lib.BF16, _lib.F32) == 0      # Dk
    assert lib.dflash_gdn_layer_supported(16, 16, 32, 128, 256, 4, _lib.BF16, _lib.F32) == 0     # Dv
    assert lib.dflash_gdn_layer_supported(17, 16, 32, 128, 128, 4, _lib.BF16, _lib.F32) == 0     # tokens
    assert lib.dflash_gdn_layer_supported(16, 16, 32, 128, 128, 4, _lib.BF16, _lib.BF16) == 0    # state dtype


@pytest.mark.parametrize("T,Hk,Hv,Dv,Kc", [(16, 16, 32, 128, 4), (16, 2, 4, 128, 4), (7, 2, 2, 64, 3), (1, 1, 2, 16, 2),
                                            (16, 4, 8, 96, 8)])
def test_record_pass_with_the_output_norm_in_the_same_launch(T, Hk, Hv, Dv, Kc):
    """dflash_gdn_forward_tape_norm against dflash_gdn_forward_tape + dflash_gated_rmsnorm: state and tape bit for bit, the
    normed output up to the order in which the norm's sum of squares is added (last-bit differences on a few elements),
    and against the torch formulas with the tolerances of the three-call path."""
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    c = _case(T, Hk, Hv, Dv, Kc, seed=300 + Hv + Dv + T)
    two, three = _run_record_norm(c), _run(c, False)
    for name in ("state", "tape", "k", "g", "new_conv", "qkv"):
        assert torch.equal(two[name], three[name]), name
    assert _rel(two["out"], three["out"]) <= 8e-3
    assert float((two["out"].float() - three["out"].float()).abs().gt(0).float().mean()) <= 0.02
    ref = _torch_formulas(c)
    assert _rel(two["out"], ref["out"]) <= 1e-2 and _rel(two["state"], ref["state"]) <= 2e-3


def test_record_norm_refusals():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib, verify_step
    verify_step._declare()
    lib = _lib.lib()
    assert lib.dflash_gdn_forward_tape_norm_supported(16, 16, 32, 128, 128, _lib.BF16, _lib.F32) == 1
    assert lib.dflash_gdn_forward_tape_norm_supported(16, 16, 32, 128, 256, _lib.BF16, _lib.F32) == 0   # more than 8 blocks per head
    assert lib.dflash_gdn_forward_tape_norm_supported(16, 16, 32, 64, 128, _lib.BF16, _lib.F32) == 0    # Dk
    assert lib.dflash_gdn_forward_tape_norm_supported(17, 16, 32, 128, 128, _lib.BF16, _lib.F32) == 0   # tokens
    assert lib.dflash_gdn_forward_tape_norm_supported(16, 16, 32, 128, 128, _lib.BF16, _lib.BF16) == 0  # state dtype
