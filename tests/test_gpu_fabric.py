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
        np.testing.assert_allclose(mb.float().cpu().numpy(), want, rtol=1e-2, atol=1e-2)
        # local ops keep the placement
        s2 = fabric.mul(ft, ft)
        assert torch.equal(s2.shard, shard * shard)
        loc = fabric.sum(ft, dim=1)
        np.testing.assert_allclose(loc.shard.cpu().numpy(), x[offs[rank]:offs[rank + 1]].sum(1), rtol=1e-5, atol=1e-5)
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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_rank_nccl_sharded_ops():
    import torch.multiprocessing as mp
    world = 2
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
        # bf16 with a broadcast remote operand
        ab = a.bfloat16()
        bb = b[:1].bfloat16()
        out = ops.binary("add", ab, bb)
        torch.cuda.synchronize(0)
        assert out.device.index == 0
        assert torch.equal(out, ab + bb.to("cuda:0"))
