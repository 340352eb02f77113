"""Host logic of the multi-GPU path on CPU: batch slicing, and a world-size-2 gloo run in which each
rank computes its own shard (with the CPU oracle standing in for the device) and the gathered
result equals the single-process result bit for bit -- there is no collective on the data path."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def load_shard():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry

    pkg = entry.load_package()
    import importlib

    return importlib.import_module(pkg.__name__ + ".shard")


def test_batch_slices_cover_everything_once():
    sh = load_shard()
    for batch in (0, 1, 7, 8, 64):
        for world in (1, 2, 3, 8):
            sl = sh.batch_slices(batch, world)
            assert len(sl) == world and sl[0][0] == 0 and sl[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(sl, sl[1:]))
            sizes = [b - a for a, b in sl]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        sh.batch_slices(4, 0)


def test_flops_convention():
    sh = load_shard()
    assert sh.flops(8, 1024, 12, 64) == pytest.approx(38.65e9, rel=1e-3)
    assert sh.flops(8, 1024, 12, 64, backward=False) == pytest.approx(12.88e9, rel=1e-3)


def _worker(rank, world, port, tmp):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, ROOT)
    from oracle import oracle

    sh = load_shard()
    B, T, H, D = 4, 24, 2, 8
    rng = np.random.default_rng(5)
    x = rng.standard_normal((B, T, 3 * H * D), dtype=np.float32)
    g = rng.standard_normal((B, T, H * D), dtype=np.float32)
    xs, gs = sh.shard(x, rank, world), sh.shard(g, rank, world)
    out = torch.from_numpy(oracle.forward(np.ascontiguousarray(xs), H))
    dx = torch.from_numpy(oracle.backward(np.ascontiguousarray(xs), np.ascontiguousarray(gs), H))
    # the only communication: gathering results and the max-over-ranks of a timing
    outs = [torch.empty_like(out) for _ in range(world)]
    dxs = [torch.empty_like(dx) for _ in range(world)]
    dist.all_gather(outs, out)
    dist.all_gather(dxs, dx)
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        full_out = oracle.forward(x, H)
        full_dx = oracle.backward(x, g, H)
        ok = (np.array_equal(torch.cat(outs).numpy(), full_out) and np.array_equal(torch.cat(dxs).numpy(), full_dx)
              and t.item() == float(world))
        with open(os.path.join(tmp, "ok"), "w") as f:
            f.write("1" if ok else "0")
    dist.destroy_process_group()


def test_two_rank_gloo_shards_reassemble(tmp_path, oracle):
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert open(tmp_path / "ok").read() == "1"


def test_bench_cpu_binding_is_harmless_without_nvml():
    """bench.py binds a rank to the cores NVML lists for its GPU; without a GPU (or NVML) it must return
    None and leave the process's affinity alone."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("bench_for_test", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    before = os.sched_getaffinity(0)
    got = bench.bind_to_gpu_cpus(0)
    after = os.sched_getaffinity(0)
    if torch.cuda.is_available():
        assert got is None or (isinstance(got, int) and got == len(after) and after <= before)
        os.sched_setaffinity(0, before)
    else:
        assert got is None and after == before
