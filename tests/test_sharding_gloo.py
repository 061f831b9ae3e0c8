"""Batch sharding and the gradient all-reduce, on CPU ranks over gloo (world size 2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from npa_b200.sharding import allreduce_gradients, shard_batch, shard_range


def test_shard_range_partitions_every_batch():
    for B in (0, 1, 4, 7, 64, 256):
        for W in (1, 2, 3, 4, 8):
            spans = [shard_range(B, r, W) for r in range(W)]
            assert spans[0][0] == 0 and spans[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _model(seed=0):
    torch.manual_seed(seed)
    return torch.nn.Sequential(torch.nn.Linear(6, 16), torch.nn.ReLU(), torch.nn.Linear(16, 3, bias=False))


def _worker(rank, world, port, B, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        z = torch.randn(B, 10, 6, generator=g)           # per-system "perception" of 10 particles
        y = torch.randn(B, 10, 3, generator=g)
        model = _model()
        lo, hi = shard_range(B, rank, world)
        loss = ((model(shard_batch(z, rank, world)) - shard_batch(y, rank, world)) ** 2).mean()
        loss.backward()
        sent = allreduce_gradients(model.parameters(), weight=(hi - lo) / B)
        ret[rank] = (sent, [p.grad.clone() for p in model.parameters()])
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B", [4, 5])
def test_sharded_gradients_equal_single_process(B):
    world, port = 2, _free_port()
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, port, B, ret), nprocs=world, join=True)
    g = torch.Generator().manual_seed(5)
    z = torch.randn(B, 10, 6, generator=g)
    y = torch.randn(B, 10, 3, generator=g)
    model = _model()
    ((model(z) - y) ** 2).mean().backward()
    ref = [p.grad for p in model.parameters()]
    n_floats = sum(p.numel() for p in model.parameters())
    for r in range(world):
        sent, grads = ret[r]
        assert sent == n_floats            # one flat buffer holding every parameter
        for a, b in zip(grads, ref):
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-7)


def test_allreduce_is_a_no_op_without_a_group():
    model = _model()
    model(torch.randn(3, 6)).sum().backward()
    before = [p.grad.clone() for p in model.parameters()]
    assert allreduce_gradients(model.parameters()) == 0
    assert all(torch.equal(a, p.grad) for a, p in zip(before, model.parameters()))


def test_cpu_binding_is_a_no_op_without_nvml():
    """Without a GPU driver the helper reports None and leaves the affinity of the process alone."""
    import os
    from npa_b200.sharding import bind_to_gpu_cpus
    before = os.sched_getaffinity(0)
    assert bind_to_gpu_cpus(0) is None
    assert os.sched_getaffinity(0) == before
