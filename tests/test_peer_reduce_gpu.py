"""Fused row-parallel sum + residual add + RMSNorm over peer memory (csrc/peer.cu).

One GPU: the data path with one rank, two ranks emulated by reducers wired to each other inside one process (the
"other" rank's kernel runs first with a short wait limit and gives up, so no launch ever waits for a later one), the
give-up path (a flag that nothing sets -> device error 21, context still usable) and graph replay.
Two GPUs (skipped otherwise): two processes over CUDA IPC, the verify step with the fused kernel against the same
step with NCCL all-reduce."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def env():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from dflash_mlx_b200 import _lib
    from dflash_mlx_b200.parallel import PeerReducer
    return _lib, PeerReducer


def _ref(h, deltas, w, eps):
    acc = torch.zeros_like(h, dtype=torch.float32)
    for d in deltas:
        acc += d.float()
    h2 = (h.float() + acc).to(torch.bfloat16)
    hf = h2.float()
    x = (hf * torch.rsqrt(hf.pow(2).mean(dim=-1, keepdim=True) + eps) * w.float()).to(torch.bfloat16)
    return h2, x


def _rand(T, H, seed):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).cuda()  # noqa: E731
    return mk(T, H), mk(T, H), (1.0 + 0.1 * torch.randn(H, generator=g)).to(torch.bfloat16).cuda()


@pytest.mark.parametrize("protocol", [1, 2])
@pytest.mark.parametrize("T,H", [(16, 5120), (16, 2048), (5, 264)])
def test_single_rank_matches_reference_and_alternates_slots(env, T, H, protocol):
    _lib, PeerReducer = env
    red = PeerReducer(0, 1, T, H, "cuda")
    red.set_protocol(protocol)
    try:
        for call in range(3):                      # sequence numbers 1, 2, 3: both inbox slots get used
            h, d, w = _rand(T, H, 10 + call)
            x = torch.empty_like(h)
            want_h, want_x = _ref(h, [d], w, 1e-6)
            red.reduce_add_rmsnorm(d, h, w, x, 1e-6, _lib.BF16)
            torch.cuda.synchronize()
            assert torch.equal(h, want_h)
            assert float((x.float() - want_x.float()).abs().max()) <= 1e-2 * float(want_x.float().abs().max())
        assert _lib.lib().dflash_device_error(0) == 0
    finally:
        red.set_protocol(0)
        red.close()


@pytest.mark.parametrize("protocol", [1, 2])
def test_two_ranks_on_one_device_and_give_up_path(env, protocol):
    _lib, PeerReducer = env
    T, H = 16, 5120
    r0, r1 = PeerReducer.local_group(2, T, H, "cuda")
    r0.set_protocol(protocol)
    lib = _lib.lib()
    try:
        r0.set_wait_polls(2048)                    # process-wide: a wait that cannot succeed ends in about a millisecond
        h0, d0, w = _rand(T, H, 1)
        h1, d1, _ = _rand(T, H, 2)
        h1.copy_(h0)                               # the residual stream is replicated on the ranks
        x0, x1 = torch.empty_like(h0), torch.empty_like(h0)
        want_h, want_x = _ref(h0, [d0, d1], w, 1e-6)
        h1_before = h1.clone()
        # "rank 1" first: it pushes its rows and flags, finds no rows of rank 0, gives up
        r1.reduce_add_rmsnorm(d1, h1, w, x1, 1e-6, _lib.BF16)
        torch.cuda.synchronize()
        assert lib.dflash_device_error(0) == 21    # recorded, and cleared by the read
        assert torch.equal(h1, h1_before)          # a row that gave up writes nothing
        # "rank 0" now finds rank 1's rows already there
        r0.reduce_add_rmsnorm(d0, h0, w, x0, 1e-6, _lib.BF16)
        torch.cuda.synchronize()
        assert lib.dflash_device_error(0) == 0
        assert torch.equal(h0, want_h)
        assert float((x0.float() - want_x.float()).abs().max()) <= 1e-2 * float(want_x.float().abs().max())
        # the context is still usable after the give-up
        assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0
    finally:
        r0.set_wait_polls(1 << 22)
        r0.set_protocol(0)
        r0.close()


def test_graph_replay_advances_the_sequence(env):
    _lib, PeerReducer = env
    T, H = 16, 5120
    red = PeerReducer(0, 1, T, H, "cuda")
    try:
        h, d, w = _rand(T, H, 3)
        x = torch.empty_like(h)
        h_start = h.clone()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            red.reduce_add_rmsnorm(d, h, w, x, 1e-6, _lib.BF16)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                red.reduce_add_rmsnorm(d, h, w, x, 1e-6, _lib.BF16)
        torch.cuda.current_stream().wait_stream(side)
        want = h_start.clone()
        want_h, _ = _ref(want, [d], w, 1e-6)       # the eager call above
        for _ in range(3):                         # each replay adds d once more
            g.replay()
            want_h, want_x = _ref(want_h, [d], w, 1e-6)
        torch.cuda.synchronize()
        assert torch.equal(h, want_h)
        assert _lib.lib().dflash_device_error(0) == 0
    finally:
        red.close()


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_fused_step_matches_nccl_step():
    env2 = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29613", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29613", os.path.join(ROOT, "tests", "peer_step_worker.py")]
    res = subprocess.run(cmd, cwd=ROOT, env=env2, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "PEER_STEP_OK" in res.stdout


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpus_expert_all_to_all_matches_step_without_dispatch():
    env2 = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29617", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
           "127.0.0.1", "--master-port", "29617", os.path.join(ROOT, "tests", "peer_step_worker.py"), "moe"]
    res = subprocess.run(cmd, cwd=ROOT, env=env2, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    assert "MOE_EXCHANGE_OK" in res.stdout
