"""Sharded reductions and elementwise over NCCL on 2 GPUs (skipped with fewer): each rank
runs the real kernels on its shard; results are checked against the CPU oracle applied to
the concatenated global tensor.  NVLS is switched off for these short-lived groups."""
import os
import socket
import sys
import traceback

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _gather_shards(dist, shard, rows, world):
    """Every rank's shard (row counts differ, so padded to the longest and trimmed)."""
    pad = torch.zeros((max(rows),) + tuple(shard.shape[1:]), device=shard.device, dtype=shard.dtype)
    pad[: shard.shape[0]] = shard
    out = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(out, pad)
    return [o[: rows[r]] for r, o in enumerate(out)]


def _worker(rank, world, port, errq):
    try:
        sys.path.insert(0, ROOT)
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import datetime
        import torch.distributed as dist
        import oracle
        from vibetensor_b200 import fabric
        torch.cuda.set_device(rank)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                                timeout=datetime.timedelta(seconds=120))
        port_ = oracle.port()
        rng = np.random.default_rng(4)
        rows = [3000 + 500 * r for r in range(world)]
        offs = np.concatenate([[0], np.cumsum(rows)])
        x = rng.standard_normal((sum(rows), 96), dtype=np.float32)
        mesh = fabric.FabricMesh.from_world()
        shard = torch.from_numpy(x[offs[rank]:offs[rank + 1]].copy()).cuda()
        ft = fabric.FabricTensor.sharded_1d_row(mesh, shard)
        assert ft.global_shape == x.shape
        scale = np.abs(x).sum(dtype=np.float64)
        assert abs(fabric.sum(ft).item() - x.sum(dtype=np.float64)) <= 1e-5 * scale
        assert fabric.amax(ft).item() == port_.reduce("max", x, oracle.F32)
        assert fabric.amin(ft).item() == port_.reduce("min", x, oracle.F32)
        m = fabric.mean(ft, dim=0).cpu().numpy()
        np.testing.assert_allclose(m, port_.reduce("mean", x, oracle.F32, dim=0), rtol=1e-5, atol=1e-6)
        # bf16 mean(dim=0): fp32 partials across ranks, one rounding at the end
        xb = oracle.f32_to_bf16_bits(x).reshape(x.shape)
        sb = torch.from_numpy(xb[offs[rank]:offs[rank + 1]].view(np.int16).copy()).view(torch.bfloat16).cuda()
        mb = fabric.mean(fabric.FabricTensor.sharded_1d_row(mesh, sb), dim=0)
        assert mb.dtype == torch.bfloat16
        want = oracle.to_f32(port_.reduce("mean", xb, oracle.BF16, dim=0), oracle.BF16)
        want_bf16_mean = want
        np.testing.assert_allclose(mb.float().cpu().numpy(), want, rtol=1e-2, atol=1e-2)
        # local ops keep the placement
        s2 = fabric.mul(ft, ft)
        assert torch.equal(s2.shard, shard * shard)
        loc = fabric.sum(ft, dim=1)
        np.testing.assert_allclose(loc.shard.cpu().numpy(), x[offs[rank]:offs[rank + 1]].sum(1), rtol=1e-5, atol=1e-5)
        # prepared reductions: the fused form (one launch: reduce + exchange over peer memory +
        # scale + cast) against the partial + all-reduce form and the oracle; repeated runs walk
        # both halves of the exchange buffer; every rank must end with the same bits
        def same_everywhere(t):
            flat = t.reshape(-1).float().contiguous()
            allv = [torch.empty_like(flat) for _ in range(world)]
            dist.all_gather(allv, flat)
            assert all(torch.equal(a.view(torch.int32), allv[0].view(torch.int32)) for a in allv)

        p2p = torch.cuda.can_device_access_peer(rank, (rank + 1) % world)
        for name, dim in (("sum", None), ("max", None), ("min", None), ("mean", 0), ("sum", 0), ("max", 0)):
            fused = fabric.prepare_reduce(name, ft, dim)
            plain = fabric.prepare_reduce(name, ft, dim, fused=False)
            assert plain.fused is None
            if p2p:
                assert fused.fused is not None, f"{name} dim={dim}: expected the fused exchange"
            for rep in range(5):
                shard.mul_(1.0009765625)          # the same update on every rank: data changes, placement stays
                a, b = fused.run().clone(), plain.run().clone()
                same_everywhere(a)
                if name in ("max", "min"):
                    assert torch.equal(a, b), (name, dim, rep)
                else:
                    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
            full = np.concatenate([s.cpu().numpy() for s in _gather_shards(dist, shard, rows, world)])
            got = fused.run().cpu().numpy()
            if name in ("max", "min"):
                np.testing.assert_array_equal(got, port_.reduce(name, full, oracle.F32, dim=dim))
            else:
                # against the fp64 truth, within 1e-5 of max(|truth|, sqrt(sum of squares)): the
                # reference's own sequential fp32 loop is further from the truth than that on
                # slices this long, so it cannot be the yardstick for a differently ordered sum
                f64 = full.astype(np.float64)
                truth = f64.sum(axis=dim)
                scale = np.maximum(np.abs(truth), np.sqrt((f64 * f64).sum(axis=dim)))
                if name == "mean":
                    n = full.shape[0] if dim is not None else full.size
                    truth, scale = truth / n, scale / n
                assert np.all(np.abs(got.astype(np.float64) - truth) <= 1e-5 * scale), (name, dim)
            if fused.fused is not None:
                fused.comm.check()
        # bf16 mean through the fused form: fp32 partials cross the link, one rounding at the end
        fb = fabric.FabricTensor.sharded_1d_row(mesh, sb)
        pm = fabric.prepare_reduce("mean", fb, 0)
        got = pm.run()
        assert got.dtype == torch.bfloat16
        same_everywhere(got)
        np.testing.assert_allclose(got.float().cpu().numpy(), want_bf16_mean, rtol=1e-2, atol=1e-2)
        # the NaN rule across shards, fused and plain: first row of shard 1 is ignored, global row 0 wins
        xn = shard.clone()
        if rank == 1:
            xn[0, 2] = float("nan")
        if rank == 0:
            xn[0, 1] = float("nan")
        fn_ = fabric.FabricTensor.sharded_1d_row(mesh, xn)
        for prep in (fabric.prepare_reduce("max", fn_, 0), fabric.prepare_reduce("max", fn_, 0, fused=False)):
            r = prep.run().cpu().numpy()
            assert np.isnan(r[1]) and not np.isnan(r[2]) and not np.isnan(np.delete(r, 1)).any()
        one_off = fabric.amax(fn_, dim=0).cpu().numpy()
        assert np.isnan(one_off[1]) and not np.isnan(np.delete(one_off, 1)).any()
        # every rank holds the same combined result
        v = fabric.sum(ft).reshape(1)
        allv = [torch.empty_like(v) for _ in range(world)]
        dist.all_gather(allv, v)
        assert all(torch.equal(a, allv[0]) for a in allv)
        torch.cuda.synchronize()
        dist.destroy_process_group()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


@pytest.mark.parametrize("world", [2, 4, 8])
def test_nccl_sharded_ops(world):
    """One process per GPU over NCCL; the fused exchange kernels run over CUDA IPC mappings of
    every peer's exchange buffer, so 4 and 8 ranks cover the slot and flag indexing that 2 ranks
    cannot (a rank's own slot sits between peers' slots)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    errq = ctx.SimpleQueue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, errq)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    for p in procs:
        if p.is_alive():
            p.kill()
            errs.append((-1, "rank still alive after 300 s"))
    assert not errs, "\n".join(f"rank {r}:\n{t}" for r, t in errs)
    assert all(p.exitcode == 0 for p in procs)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_elementwise_with_one_operand_in_peer_memory():
    """The reference's vt::fabric_add / fabric_mul shape (src/vbt/cuda/fabric_elementwise.cu:
    820-1042): compute on the primary GPU, read one operand straight from a peer GPU's memory
    (plain loads over NVLink), write the result locally."""
    import oracle
    from vibetensor_b200 import ops
    if not torch.cuda.can_device_access_peer(0, 1):
        pytest.skip("no peer access between GPU 0 and GPU 1")
    rng = np.random.default_rng(5)
    a_np = rng.standard_normal((512, 300), dtype=np.float32)
    b_np = rng.standard_normal((512, 300), dtype=np.float32)
    a = torch.from_numpy(a_np).to("cuda:0")
    b = torch.from_numpy(b_np).to("cuda:1")
    with pytest.raises(ValueError, match="enable_peer_access"):
        ops.binary("add", a, b)           # refused on the host: nothing has opened GPU 1's memory yet
    ops.enable_peer_access(0, 1)
    ops.enable_peer_access(0, 1)          # idempotent
    torch.cuda.synchronize(0)
    torch.cuda.synchronize(1)
    port = oracle.port()
    with torch.cuda.device(0):
        for name in ("add", "mul"):
            out = torch.empty_like(a)
            ops.binary(name, a, b, out=out)   # b lives on GPU 1
            torch.cuda.synchronize(0)
            np.testing.assert_array_equal(out.cpu().numpy(), port.binary(name, a_np, b_np, oracle.F32))
        # bf16 with a broadcast remote operand, against the oracle
        ab_np, bb_np = oracle.f32_to_bf16_bits(a_np).reshape(a_np.shape), oracle.f32_to_bf16_bits(b_np[:1]).reshape(1, -1)
        ab = torch.from_numpy(ab_np.view(np.int16)).view(torch.bfloat16).to("cuda:0")
        bb = torch.from_numpy(bb_np.view(np.int16)).view(torch.bfloat16).to("cuda:1")
        out = ops.binary("add", ab, bb)
        torch.cuda.synchronize(0)
        assert out.device.index == 0
        got = out.cpu().view(torch.int16).numpy().view(np.uint16)
        np.testing.assert_array_equal(got, port.binary("add", ab_np, bb_np, oracle.BF16))
        # remote FIRST operand, local second, out= local, on a side stream of the compute device:
        # the launch goes to the stream of the device that owns the output
        side = torch.cuda.Stream(device=0)
        side.wait_stream(torch.cuda.current_stream(0))
        with torch.cuda.stream(side):
            out2 = torch.empty_like(a)
            ops.binary("sub", b, a, out=out2)          # b lives on GPU 1, a and out2 on GPU 0
        side.synchronize()
        np.testing.assert_array_equal(out2.cpu().numpy(), port.binary("sub", b_np, a_np, oracle.F32))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fabric_binary_modes_match_the_reference_contract():
    """vt::fabric_add / fabric_mul(a, b, compute_device, require_fabric, use_copy_fallback)
    (src/vbt/cuda/fabric_elementwise.cu:820-1042): same-device operands run the ordinary op; two
    devices use peer loads when the compute device can open the other's memory, the copy fallback
    when asked to (or when it cannot), and fail with a [Fabric] error when neither is allowed."""
    import oracle
    from vibetensor_b200 import _lib, ops
    port = oracle.port()
    rng = np.random.default_rng(6)
    a_np = rng.standard_normal((257, 130), dtype=np.float32)
    b_np = rng.standard_normal((257, 130), dtype=np.float32)
    a0, b0 = torch.from_numpy(a_np).to("cuda:0"), torch.from_numpy(b_np).to("cuda:0")
    b1 = torch.from_numpy(b_np).to("cuda:1")
    out, mode = ops.fabric_binary("add", a0, b0)
    assert mode == "local"
    np.testing.assert_array_equal(out.cpu().numpy(), port.binary("add", a_np, b_np, oracle.F32))
    p2p = torch.cuda.can_device_access_peer(0, 1)
    for name in ("add", "mul"):
        want = port.binary(name, a_np, b_np, oracle.F32)
        for compute in (0, 1):
            out, mode = ops.fabric_binary(name, a0, b1, compute_device=compute)
            torch.cuda.synchronize(compute)
            assert out.device.index == compute and mode == ("peer_load" if p2p else "copy_fallback")
            np.testing.assert_array_equal(out.cpu().numpy(), want)
            out, mode = ops.fabric_binary(name, a0, b1, compute_device=compute, use_copy_fallback="always")
            torch.cuda.synchronize(compute)
            assert mode == "copy_fallback"
            assert _lib.last_launch_info().family == 5 and _lib.last_launch_info().kernel == 2
            np.testing.assert_array_equal(out.cpu().numpy(), want)
    if p2p:
        out, mode = ops.fabric_binary("add", a0, b1, require_fabric=True, use_copy_fallback=False)
        assert mode == "peer_load"
    with pytest.raises(RuntimeError, match=r"\[Fabric\] vt::fabric_add: requires equal shapes"):
        ops.fabric_binary("add", a0, b1[:5])
    with pytest.raises(RuntimeError, match=r"\[Fabric\] vt::fabric_mul: requires equal dtypes"):
        ops.fabric_binary("mul", a0, b1.double().float().long())
    if torch.cuda.device_count() >= 3:
        with pytest.raises(RuntimeError, match="compute_device must be the device of one of the operands"):
            ops.fabric_binary("add", a0, b1, compute_device=2)
