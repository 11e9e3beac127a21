"""Expert-parallel path: exchange plan (pure host logic) and a two-rank run over gloo on CPU with
the stages served by the oracle; the same worker runs on GPUs with NCCL (marked gpu, needs >= 2)."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(n, mode, port, scheme="a2a"):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", "ep_worker.py"), mode,
           scheme]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=600)


def test_plan_exchange_is_consistent():
    from ek_b200.ep import plan_exchange
    g = torch.Generator().manual_seed(1)
    world, E = 4, 16
    counts_all = torch.randint(0, 5, (world, E), generator=g, dtype=torch.int32)
    plans = [plan_exchange(counts_all, r, world) for r in range(world)]
    for r in range(world):
        send, recv, cs = plans[r]
        assert sum(send) == int(counts_all[r].sum())
        for d in range(world):
            assert send[d] == plans[d][1][r]                # what r sends to d is what d expects from r
        assert cs.shape == (world, E // world)
        assert [int(x) for x in cs.sum(1)] == recv
    with pytest.raises(ValueError):
        plan_exchange(counts_all[:, :15], 0, world)


@pytest.mark.parametrize("world,scheme", [(2, "a2a"), (4, "a2a"), (2, "gather"), (4, "gather")])
def test_expert_parallel_over_gloo_matches_single_process_oracle(world, scheme):
    r = _launch(world, "cpu", 29600 + world + (10 if scheme == "gather" else 0), scheme)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("OK") == world


def test_replicated_experts_follow_the_owner_table_over_gloo():
    """Two experts are held by two ranks each; the per-pass owner table moves them between their
    holders and the layer output stays the single-process oracle's."""
    r = _launch(2, "cpu", 29640, "gather_replica")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("OK") == 2


def test_stack_of_layers_over_gloo():
    """Three layers with weights of their own, each fed the previous one's output, every layer
    checked against the single-process oracle on the input it really got."""
    r = _launch(2, "cpu", 29645, "gather_stack")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("OK") == 2 and r.stdout.count("good") == 2 * 2 * 3


def test_choose_owners_is_the_same_on_every_rank_and_rotates():
    from ek_b200.ep import choose_owners
    holders = [[0], [0, 1], [1], [1, 0]]
    a, b = choose_owners(holders, 0), choose_owners(holders, 1)
    assert a.tolist() != b.tolist() and a[0] == 0 and a[2] == 1
    assert all(int(a[e]) in holders[e] and int(b[e]) in holders[e] for e in range(4))
    cold = choose_owners(holders, 0, counts=torch.tensor([5, 1, 5, 9]))
    assert int(cold[1]) == 0                 # below the mean load: stays at home


@pytest.mark.gpu
@pytest.mark.parametrize("scheme", ["a2a", "gather", "peer", "gather_replica", "peer_replica"])
def test_expert_parallel_over_nccl_matches_oracle(scheme):
    """"peer": dispatch and combine by the library's own kernels over peer memory (NCCL only sets
    the process group up and exchanges the IPC handles)."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    r = _launch(2, "gpu", 29650 + {"a2a": 0, "gather": 1, "peer": 2, "gather_replica": 3, "peer_replica": 4}[scheme], scheme)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("OK") == 2


@pytest.mark.gpu
@pytest.mark.parametrize("scheme", ["peer_stack", "gather_stack"])
def test_stack_of_layers_over_nccl_matches_oracle(scheme):
    """The shape of the full-model configuration in small: a stack of expert-parallel layers with
    weights of their own on 2 GPUs, the output of a layer feeding the next, every layer checked."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    r = _launch(2, "gpu", 29660 + (scheme == "gather_stack"), scheme)
    print("\n".join(ln for ln in r.stdout.splitlines() if " layer " in ln))      # the measured margins, for -rP
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("OK") == 2 and r.stdout.count("good") == 2 * 2 * 3


@pytest.mark.gpu
def test_peer_scheme_reports_a_missing_rank_as_timeout():
    """A rank that does not show up for a pass: the other rank's bounded device-side waits run out,
    the host reads EK_TIMEOUT and the backend keeps working.  No fault, no hang: the missing rank
    left between passes."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29655", os.path.join(ROOT, "tests", "ep_worker.py"), "gpu", "peer_timeout"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert r.stdout.count("OK") == 2 and "status 17" in r.stdout
