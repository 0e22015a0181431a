"""Two CPU ranks over gloo exercise the multi-process host logic the benchmark uses on GPUs:
launcher environment parsing, the common start line, max-over-ranks timing and the whole-job rate."""

import os
import socket

import pytest
import torch
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, results):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    sys.path.insert(0, str(root / "robotics-the-speedup-paradox_b200"))
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from rk_b200 import replicas

    info = replicas.rank_info()
    device = torch.device("cpu")
    replicas.init(info, device)
    replicas.barrier(info, device)
    # rank r pretends its timed region took 10 + 5 r ms and its end-to-end region 20 - 3 r ms
    slow = replicas.max_over_ranks([10.0 + 5.0 * rank, 20.0 - 3.0 * rank], info, device)
    begin, end = replicas.shard_range(7, info)
    rate = replicas.whole_job_rate(1000.0, info, slow[0])
    results[rank] = (info.rank, info.world, slow, (begin, end), rate)
    replicas.barrier(info, device)
    replicas.finish()


@pytest.mark.timeout(120)
def test_two_gloo_ranks_agree_on_slowest_time_and_job_rate():
    world = 2
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_rank_main, args=(world, port, results), nprocs=world, join=True)
    assert sorted(results.keys()) == [0, 1]
    for rank in range(world):
        r, w, slow, shard, rate = results[rank]
        assert (r, w) == (rank, world)
        assert slow == [15.0, 20.0]  # element-wise maxima: rank 1's first value, rank 0's second
        assert rate == pytest.approx(1000.0 * 2 / 15e-3)
    # the two shards tile [0, 7) without overlap, the first rank taking the extra unit
    assert results[0][3] == (0, 4) and results[1][3] == (4, 7)


def _column_parallel_main(rank, world, port, results):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    sys.path.insert(0, str(root / "robotics-the-speedup-paradox_b200"))
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from rk_b200 import replicas

    info = replicas.rank_info()
    device = torch.device("cpu")
    replicas.init(info, device)
    torch.manual_seed(0)  # same full layer and input on every rank
    full = torch.nn.Linear(64, 48, bias=True).requires_grad_(False)
    x = torch.randn(3, 5, 64)
    layer = replicas.ColumnParallelLinear(full, info)
    out = layer(x)
    results[rank] = (tuple(out.shape), bool(torch.equal(out, full(x))), layer.slab,
                     bool(torch.equal(layer.local.weight, full.weight[rank * 24:(rank + 1) * 24])))
    replicas.barrier(info, device)
    replicas.finish()


@pytest.mark.timeout(120)
def test_column_parallel_slabs_gather_to_the_full_output_on_two_gloo_ranks():
    world = 2
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_column_parallel_main, args=(world, port, results), nprocs=world, join=True)
    for rank in range(world):
        shape, same, slab, owns_rows = results[rank]
        assert shape == (3, 5, 48) and slab == 24
        assert owns_rows  # rank r holds weight rows [24 r, 24 r + 24)
        assert same  # a slab of a linear is bit-identical to the same columns of the full linear


class _PerTensorQuantLinear(torch.nn.Module):
    """CPU stand-in for a per-tensor-scaled quantized linear (codes = round(w / scale), one scale for
    the whole weight), exposing the slicing hook the quantized modules are sharded through."""

    def __init__(self, codes, scale):
        super().__init__()
        self.codes, self.scale = codes, scale
        self.out_features, self.in_features = codes.shape

    @classmethod
    def from_linear(cls, linear):
        scale = linear.weight.abs().max() / 127.0
        return cls(torch.round(linear.weight / scale), scale)

    def shard_output_rows(self, begin, end):
        return _PerTensorQuantLinear(self.codes[begin:end].clone(), self.scale)

    def forward(self, x):
        return (x @ self.codes.T) * self.scale


def _column_parallel_quantized_main(rank, world, port, results):
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parents[1]
    sys.path.insert(0, str(root / "robotics-the-speedup-paradox_b200"))
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from rk_b200 import replicas

    info = replicas.rank_info()
    device = torch.device("cpu")
    replicas.init(info, device)
    torch.manual_seed(0)
    full = torch.nn.Linear(64, 48, bias=False).requires_grad_(False)
    with torch.no_grad():
        full.weight[40] *= 9.0  # the largest weight sits in the last slab: slab-wise scales would differ
    x = torch.randn(7, 64)
    one_gpu = _PerTensorQuantLinear.from_linear(full)
    layer = replicas.ColumnParallelLinear(full, info, _PerTensorQuantLinear.from_linear)
    out, want = layer(x), one_gpu(x)
    rel = float((out - want).norm() / want.norm())
    # what the sharded mode must NOT do: quantize every slab by itself
    slab = torch.nn.Linear(64, 24, bias=False).requires_grad_(False)
    with torch.no_grad():
        slab.weight.copy_(full.weight[rank * 24:(rank + 1) * 24])
    own_scale = float(_PerTensorQuantLinear.from_linear(slab).scale)
    results[rank] = (rel, float(layer.local.scale) == float(one_gpu.scale), own_scale == float(one_gpu.scale))
    replicas.barrier(info, device)
    replicas.finish()


@pytest.mark.timeout(120)
def test_column_parallel_quantized_slabs_share_the_one_gpu_scale():
    """Quantize once, shard the codes: the gathered output equals the one-GPU output exactly
    (relative Frobenius difference 0), because every slab keeps the whole weight's scale."""
    world = 2
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_column_parallel_quantized_main, args=(world, port, results), nprocs=world, join=True)
    assert results[0][0] == 0.0 and results[1][0] == 0.0
    assert results[0][1] and results[1][1]          # both slabs carry the shared scale
    assert not results[0][2] and results[1][2]      # a slab quantized alone would not (rank 0 lacks the largest weight)


def test_single_process_defaults_and_validation():
    import sys
    from pathlib import Path

    sys.path.insert(0, str(Path(__file__).resolve().parents[1] / "robotics-the-speedup-paradox_b200"))
    from rk_b200 import replicas

    info = replicas.rank_info({})
    assert (info.rank, info.world, info.local_rank) == (0, 1, 0)
    assert replicas.max_over_ranks([3.0, 1.0], info, torch.device("cpu")) == [3.0, 1.0]
    assert replicas.shard_range(5, info) == (0, 5)
    with pytest.raises(ValueError):
        replicas.rank_info({"RANK": "2", "WORLD_SIZE": "2"})
    with pytest.raises(ValueError):
        replicas.whole_job_rate(1.0, info, 0.0)
