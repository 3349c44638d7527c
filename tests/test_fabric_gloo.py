"""Multi-rank bookkeeping of vibetensor_b200.fabric on CPU: world_size 2 and 3 over gloo.

The kernels need a GPU, so the ranks here get a torch-CPU stand-in for the local ops
(`local_ops=`); what is under test is everything around them: placement construction from
per-rank row counts, offsets, the choice between "local only" and "partial + all-reduce",
the identity for empty shards, the global divisor of a sharded mean, error paths, and that a
rank raising an exception between steps does not hang its peers."""
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


class CpuStandIn:
    """torch-CPU stand-in with the signatures fabric.py uses from vibetensor_b200.ops."""

    @staticmethod
    def binary(name, a, b):
        return {"add": torch.add, "mul": torch.mul}[name](a, b)

    @staticmethod
    def reduce(name, x, dims, keepdim=False, partial=False, first_shard=True):
        dims = list(dims) if dims else list(range(x.dim()))
        acc = x.float() if (partial and x.dtype in (torch.bfloat16, torch.float16)) else x
        if name == "sum":
            return acc.sum(dim=dims, keepdim=keepdim)
        if name == "mean":
            return acc.mean(dim=dims, keepdim=keepdim)
        # the library's scan: NaN never wins a comparison; a NaN at position 0 of the reduced
        # slice wins outright -- unless the shard is not the first one (first_shard=False)
        ident = float("-inf") if name == "max" else float("inf")
        f = torch.amax if name == "max" else torch.amin
        if not acc.dtype.is_floating_point:
            return f(acc, dim=dims, keepdim=keepdim)
        out = f(torch.nan_to_num(acc, nan=ident, posinf=float("inf"), neginf=float("-inf")), dim=dims, keepdim=keepdim)
        if first_shard:
            first = acc[tuple(slice(0, 1) if d in dims else slice(None) for d in range(acc.dim()))]
            first = first if keepdim else first.reshape(out.shape)
            out = torch.where(torch.isnan(first), first, out)
        return out

    @staticmethod
    def scale_cast(partial, scale, out_dtype):
        return (partial * scale).to(out_dtype)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, fn_name, errq):
    try:
        sys.path.insert(0, ROOT)
        os.environ["MASTER_ADDR"] = "127.0.0.1"
        os.environ["MASTER_PORT"] = str(port)
        dist.init_process_group("gloo", rank=rank, world_size=world,
                                timeout=__import__("datetime").timedelta(seconds=60))
        globals()[fn_name](rank, world)
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def _run(fn_name, world):
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, fn_name, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            errs.append((-1, "rank still alive after 120 s"))
    assert not errs, "\n".join(f"rank {r}:\n{t}" for r, t in errs)
    assert all(p.exitcode == 0 for p in procs)


def _global(world, tail, seed=4, uneven=True):
    rng = np.random.default_rng(seed)
    rows = [5 + (2 * r if uneven else 0) for r in range(world)]
    x = rng.standard_normal((sum(rows),) + tail, dtype=np.float32)
    offs = np.concatenate([[0], np.cumsum(rows)])
    return x, rows, offs


def case_reductions(rank, world):
    from vibetensor_b200 import fabric
    mesh = fabric.FabricMesh.from_world()
    x, rows, offs = _global(world, (6,))
    shard = torch.from_numpy(x[offs[rank]:offs[rank + 1]].copy())
    ft = fabric.FabricTensor.sharded_1d_row(mesh, shard)
    assert ft.global_shape == x.shape
    assert ft.placement.shard_offsets == tuple(int(o) for o in offs[:-1])
    ops = CpuStandIn
    np.testing.assert_allclose(fabric.sum(ft, local_ops=ops).item(), x.sum(dtype=np.float64), rtol=1e-5)
    np.testing.assert_allclose(fabric.amax(ft, local_ops=ops).item(), x.max())
    np.testing.assert_allclose(fabric.amin(ft, local_ops=ops).item(), x.min())
    m = fabric.mean(ft, dim=0, local_ops=ops)
    np.testing.assert_allclose(m.numpy(), x.mean(0), rtol=1e-5, atol=1e-6)   # divisor = GLOBAL rows
    assert fabric.sum(ft, dim=0, keepdim=True, local_ops=ops).shape == (1, 6)
    # a reduction that does not cross the sharded dim stays sharded, no communication
    loc = fabric.sum(ft, dim=1, local_ops=ops)
    assert isinstance(loc, fabric.FabricTensor) and loc.global_shape == (x.shape[0],)
    np.testing.assert_allclose(loc.shard.numpy(), x[offs[rank]:offs[rank + 1]].sum(1), rtol=1e-5, atol=1e-6)
    # elementwise: same placement -> local
    s = fabric.add(ft, ft, local_ops=ops)
    assert torch.equal(s.shard, shard + shard) and s.placement == ft.placement
    # bf16 shards: partials are fp32, mean is cast back
    fb = fabric.FabricTensor.sharded_1d_row(mesh, shard.bfloat16())
    mb = fabric.mean(fb, dim=0, local_ops=ops)
    assert mb.dtype == torch.bfloat16
    want = torch.from_numpy(x).bfloat16().float().mean(0)
    np.testing.assert_allclose(mb.float().numpy(), want.numpy(), rtol=1e-2, atol=1e-2)


def case_nan_rule_across_shards(rank, world):
    """max / min: a NaN wins only at GLOBAL position 0.  A NaN in the first row of a later shard
    is ignored, exactly as on one GPU; a NaN in the very first row decides the result on every
    rank; and an empty leading shard hands the rule to the next rank."""
    from vibetensor_b200 import fabric
    mesh = fabric.FabricMesh.from_world()
    ops = CpuStandIn
    x, rows, offs = _global(world, (4,), seed=6)
    x[offs[1], 2] = np.nan          # first row of shard 1, column 2: must be ignored
    x[0, 1] = np.nan                # global row 0, column 1: wins
    ft = fabric.FabricTensor.sharded_1d_row(mesh, torch.from_numpy(x[offs[rank]:offs[rank + 1]].copy()))
    got = fabric.amax(ft, dim=0, local_ops=ops).numpy()
    want = np.nanmax(x, axis=0)
    want[1] = np.nan
    np.testing.assert_array_equal(got, want)
    got = fabric.amin(ft, dim=0, local_ops=ops).numpy()
    want = np.nanmin(x, axis=0)
    want[1] = np.nan
    np.testing.assert_array_equal(got, want)
    # full reduce: global element 0 is not NaN here, so the NaNs elsewhere are ignored
    assert fabric.amax(ft, local_ops=ops).item() == np.nanmax(x)
    # rank 0 empty: rank 1 owns global row 0
    y = x[offs[1]:]
    lo = 0 if rank == 0 else offs[rank] - offs[1]
    hi = 0 if rank == 0 else offs[rank + 1] - offs[1]
    fy = fabric.FabricTensor.sharded_1d_row(mesh, torch.from_numpy(y[lo:hi].copy()))
    got = fabric.amax(fy, dim=0, local_ops=ops).numpy()
    want = np.nanmax(y, axis=0)
    want[2] = np.nan                # y[0, 2] is the NaN planted above: now at global position 0
    np.testing.assert_array_equal(got, want)


def case_empty_shard_and_errors(rank, world):
    from vibetensor_b200 import fabric
    mesh = fabric.FabricMesh.from_world()
    rng = np.random.default_rng(9)
    rows = 0 if rank == world - 1 else 4
    shard = torch.from_numpy(rng.standard_normal((rows, 3), dtype=np.float32))
    ft = fabric.FabricTensor.sharded_1d_row(mesh, shard)
    gathered = [None] * world
    dist.all_gather_object(gathered, shard.numpy())
    full = np.concatenate(gathered)
    ops = CpuStandIn
    np.testing.assert_allclose(fabric.sum(ft, local_ops=ops).item(), full.sum(dtype=np.float64), rtol=1e-5)
    np.testing.assert_allclose(fabric.amax(ft, local_ops=ops).item(), full.max())
    np.testing.assert_allclose(fabric.mean(ft, dim=0, local_ops=ops).numpy(), full.mean(0), rtol=1e-5, atol=1e-6)
    # mismatched placements are rejected on every rank
    other = fabric.FabricTensor.replicated(mesh, torch.zeros(3))
    with pytest.raises(fabric.FabricError, match="share mesh and placement"):
        fabric.add(ft, other, local_ops=ops)
    with pytest.raises(ValueError, match="dim out of range"):
        fabric.sum(ft, dim=5, local_ops=ops)
    with pytest.raises(fabric.FabricError, match="unsupported reduction"):
        fabric.reduce("prod", ft, local_ops=ops)
    # the product backend refuses CPU tensors: there is no CPU compute path to fall into
    with pytest.raises(ValueError, match="no CPU path"):
        fabric.sum(ft)


def case_tail_mismatch(rank, world):
    from vibetensor_b200 import fabric
    mesh = fabric.FabricMesh.from_world()
    shard = torch.zeros((2, 3 + rank))
    with pytest.raises(fabric.FabricError, match="tail dims"):
        fabric.FabricTensor.sharded_1d_row(mesh, shard)


def case_rank_failure_between_steps(rank, world):
    """A rank that raises between steps leaves no collective half-entered: the others finish
    the step they are in and learn of the failure through the store before the next one."""
    from vibetensor_b200 import fabric
    mesh = fabric.FabricMesh.from_world()
    store = dist.distributed_c10d._get_default_store()
    ft = fabric.FabricTensor.sharded_1d_row(mesh, torch.ones((4, 2)))
    assert fabric.sum(ft, local_ops=CpuStandIn).item() == 8.0 * world
    failed = False
    try:
        if rank == world - 1:
            raise RuntimeError("injected host-side failure")
    except RuntimeError:
        failed = True
    store.set(f"status/{rank}", "failed" if failed else "ok")
    states = [store.get(f"status/{r}").decode() for r in range(world)]   # blocks until all posted
    assert states[world - 1] == "failed"
    # every rank sees the failure and skips the next collective instead of hanging in it
    if "failed" in states:
        return


@pytest.mark.parametrize("world", [2, 3])
def test_sharded_reductions_and_elementwise(world):
    _run("case_reductions", world)


@pytest.mark.parametrize("world", [2, 3])
def test_nan_wins_only_at_global_position_zero(world):
    _run("case_nan_rule_across_shards", world)


def test_empty_shard_and_error_paths():
    _run("case_empty_shard_and_errors", 2)


def test_tail_mismatch_is_reported_on_every_rank():
    _run("case_tail_mismatch", 2)


def test_rank_failure_between_steps_does_not_hang_peers():
    _run("case_rank_failure_between_steps", 2)


def test_placement_invariants():
    sys.path.insert(0, ROOT)
    from vibetensor_b200 import fabric
    mesh = fabric.FabricMesh((0, 1, 2))
    with pytest.raises(fabric.FabricError, match="same length"):
        fabric.FabricPlacement("sharded_1d_row", mesh, (9, 2), (0, 3))
    with pytest.raises(fabric.FabricError, match="shard_offsets\\[0\\] == 0"):
        fabric.FabricPlacement("sharded_1d_row", mesh, (9, 2), (1, 3, 6))
    with pytest.raises(fabric.FabricError, match="non-decreasing"):
        fabric.FabricPlacement("sharded_1d_row", mesh, (9, 2), (0, 6, 3))
    with pytest.raises(fabric.FabricError, match="all zeros"):
        fabric.FabricPlacement("replicated", mesh, (9, 2), (0, 1, 0))
    with pytest.raises(fabric.FabricError, match="Invalid FabricPlacement.kind"):
        fabric.FabricPlacement("diagonal", mesh, (9, 2), (0, 0, 0))
    pl = fabric.FabricPlacement("sharded_1d_row", mesh, (9, 2), (0, 3, 6))
    assert [pl.rows_of(r) for r in range(3)] == [3, 3, 3]
    assert fabric.split_rows(10, 4) == [(0, 3), (3, 3), (6, 2), (8, 2)]
