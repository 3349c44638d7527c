"""Fabric: row-sharded tensors across the GPUs of one box, one process per GPU.

The reference's Fabric (python/vibetensor/fabric.py:206-533, :811-877) is a single process
that holds one shard per mesh device and loops over them; it has elementwise add / mul only
and no reductions.  Here each rank (``torch.distributed``, NCCL over NVLink) owns one shard
of a ``sharded_1d_row`` tensor -- rows ``[shard_offsets[r], shard_offsets[r+1])`` of the
global tensor -- and

* elementwise ops between tensors of the same placement are purely local kernel launches
  (no communication), as ``fabric.add`` / ``fabric.mul`` are in the reference;
* a reduction over the sharded dim is a local partial (FP32 or INT64, computed by
  ``vbt_b200_reduce_partial``) followed by ONE all-reduce of the partial on the same stream:
  4 bytes for a full sum / amax, ``4 * columns`` bytes for ``mean(dim=0)``;
* a reduction over a non-sharded dim is local and yields a tensor sharded the same way.

``FabricPlacement`` keeps the reference's invariants (kinds, offsets = prefix sums of rows,
``global_shape = (sum rows,) + tail``).

The compute backend is ``vibetensor_b200.ops`` (CUDA only).  ``local_ops=`` exists so the
multi-rank bookkeeping can be exercised by CPU ``gloo`` tests with a stand-in; nothing in
this module falls back to it on its own.
"""
from __future__ import annotations

import dataclasses
from typing import Optional, Sequence, Tuple

import torch
import torch.distributed as dist


class FabricError(RuntimeError):
    def __init__(self, msg: str):
        super().__init__("[Fabric] " + msg)


@dataclasses.dataclass(frozen=True)
class FabricMesh:
    """The ranks taking part (one CUDA device each); ``devices[r]`` is rank r's device index."""

    devices: Tuple[int, ...]
    group: Optional[object] = None  # torch.distributed process group, None = default

    def __post_init__(self):
        devs = tuple(int(d) for d in self.devices)
        if not devs:
            raise FabricError("FabricMesh.devices must not be empty")
        if any(d < 0 for d in devs):
            raise FabricError("FabricMesh.devices must be non-negative")
        object.__setattr__(self, "devices", devs)

    @property
    def world_size(self) -> int:
        return len(self.devices)

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group) if dist.is_initialized() else 0

    @staticmethod
    def from_world(group=None) -> "FabricMesh":
        """One mesh slot per rank of the process group; device index = local rank slot."""
        ws = dist.get_world_size(group) if dist.is_initialized() else 1
        return FabricMesh(tuple(range(ws)), group)


@dataclasses.dataclass(frozen=True)
class FabricPlacement:
    kind: str
    mesh: FabricMesh
    global_shape: Tuple[int, ...]
    shard_offsets: Tuple[int, ...]

    def __post_init__(self):
        if self.kind not in ("replicated", "sharded_1d_row"):
            raise FabricError(f"Invalid FabricPlacement.kind: {self.kind!r}")
        gs = tuple(int(s) for s in self.global_shape)
        so = tuple(int(s) for s in self.shard_offsets)
        if len(so) != self.mesh.world_size:
            raise FabricError("FabricPlacement.shard_offsets must have the same length as mesh.devices")
        if self.kind == "replicated":
            if any(o != 0 for o in so):
                raise FabricError("FabricPlacement(replicated) requires shard_offsets to be all zeros")
        else:
            if len(gs) < 1:
                raise FabricError("FabricPlacement(sharded_1d_row) requires global_shape to have rank >= 1")
            if so[0] != 0:
                raise FabricError("FabricPlacement(sharded_1d_row) requires shard_offsets[0] == 0")
            if any(c < p for p, c in zip(so, so[1:])):
                raise FabricError("FabricPlacement(sharded_1d_row) requires shard_offsets to be non-decreasing")
            if so[-1] > gs[0]:
                raise FabricError("FabricPlacement(sharded_1d_row) offsets exceed the global row count")
        object.__setattr__(self, "global_shape", gs)
        object.__setattr__(self, "shard_offsets", so)

    def rows_of(self, rank: int) -> int:
        if self.kind == "replicated":
            return self.global_shape[0] if self.global_shape else 1
        end = self.shard_offsets[rank + 1] if rank + 1 < len(self.shard_offsets) else self.global_shape[0]
        return end - self.shard_offsets[rank]


def _backend(local_ops, *tensors):
    if local_ops is not None:
        return local_ops
    for t in tensors:
        if not t.is_cuda:  # checked on every rank before any collective is entered
            raise ValueError("vibetensor_b200 ops take CUDA tensors (there is no CPU path)")
    from . import ops
    return ops


class FabricTensor:
    """This rank's shard plus the placement that says where it sits in the global tensor."""

    __vbt_fabric_tensor__ = True

    def __init__(self, placement: FabricPlacement, shard: torch.Tensor):
        if not isinstance(placement, FabricPlacement):
            raise FabricError("FabricTensor.placement must be a FabricPlacement")
        r = placement.mesh.rank
        if placement.kind == "sharded_1d_row":
            if shard.dim() < 1:
                raise FabricError("sharded_1d_row shards must have rank >= 1")
            if tuple(shard.shape[1:]) != tuple(placement.global_shape[1:]):
                raise FabricError("shard tail dims must match the global shape")
            if shard.shape[0] != placement.rows_of(r):
                raise FabricError("shard row count does not match the placement offsets")
        elif tuple(shard.shape) != tuple(placement.global_shape):
            raise FabricError("replicated shards must have the global shape")
        self.placement = placement
        self.shard = shard

    # ---- constructors (FabricTensor.replicated / sharded_1d_row of the reference) ----
    @staticmethod
    def replicated(mesh: FabricMesh, tensor: torch.Tensor) -> "FabricTensor":
        return FabricTensor(FabricPlacement("replicated", mesh, tuple(tensor.shape),
                                            (0,) * mesh.world_size), tensor)

    @staticmethod
    def sharded_1d_row(mesh: FabricMesh, local_shard: torch.Tensor) -> "FabricTensor":
        """Builds the placement from every rank's row count (one small all-gather on the host
        side of construction, not on the data path)."""
        rows = int(local_shard.shape[0]) if local_shard.dim() >= 1 else None
        if rows is None:
            raise FabricError("sharded_1d_row shards must have rank >= 1")
        ws = mesh.world_size
        if ws > 1:
            counts = [None] * ws
            dist.all_gather_object(counts, (rows, tuple(local_shard.shape[1:]), str(local_shard.dtype)),
                                   group=mesh.group)
            tails = {c[1] for c in counts}
            dts = {c[2] for c in counts}
            if len(tails) != 1:
                raise FabricError("sharded_1d_row shards must share their tail dims")
            if len(dts) != 1:
                raise FabricError("sharded_1d_row shards must share their dtype")
            row_counts = [c[0] for c in counts]
        else:
            row_counts = [rows]
        offs, acc = [], 0
        for c in row_counts:
            offs.append(acc)
            acc += c
        pl = FabricPlacement("sharded_1d_row", mesh, (acc,) + tuple(local_shard.shape[1:]), tuple(offs))
        return FabricTensor(pl, local_shard)

    @property
    def global_shape(self):
        return self.placement.global_shape

    @property
    def dtype(self):
        return self.shard.dtype

    def to_local_shard(self) -> torch.Tensor:
        return self.shard


def _same_placement(a: FabricTensor, b: FabricTensor, what: str):
    if a.placement.mesh.devices != b.placement.mesh.devices or a.placement.kind != b.placement.kind \
            or a.placement.shard_offsets != b.placement.shard_offsets \
            or a.placement.global_shape != b.placement.global_shape:
        raise FabricError(f"{what}: operands must share mesh and placement")
    if a.shard.dtype != b.shard.dtype:
        raise FabricError(f"{what}: dtype mismatch")


def _elementwise(name: str, a: FabricTensor, b: FabricTensor, local_ops=None) -> FabricTensor:
    _same_placement(a, b, "fabric." + name)
    out = _backend(local_ops, a.shard, b.shard).binary(name, a.shard, b.shard)
    return FabricTensor(a.placement, out)


def add(a: FabricTensor, b: FabricTensor, local_ops=None) -> FabricTensor:
    """fabric.add: per-shard vt::add, no communication (python/vibetensor/fabric.py:843-859)."""
    return _elementwise("add", a, b, local_ops)


def mul(a: FabricTensor, b: FabricTensor, local_ops=None) -> FabricTensor:
    return _elementwise("mul", a, b, local_ops)


_REDUCE_OP = {"sum": dist.ReduceOp.SUM, "mean": dist.ReduceOp.SUM, "max": dist.ReduceOp.MAX,
              "min": dist.ReduceOp.MIN}


def _all_reduce(t: torch.Tensor, name: str, mesh: FabricMesh):
    if mesh.world_size > 1:
        dist.all_reduce(t, op=_REDUCE_OP[name], group=mesh.group)
    return t


def _first_owner(placement: FabricPlacement) -> int:
    """The rank whose shard holds global row 0 (the first rank with any rows)."""
    for r in range(placement.mesh.world_size):
        if placement.rows_of(r) > 0:
            return r
    return 0


def _plan(name: str, ft: "FabricTensor", dim, keepdim: bool):
    if name not in _REDUCE_OP:
        raise FabricError(f"fabric.reduce: unsupported reduction {name!r}")
    nd = ft.shard.dim()
    dims = list(range(nd)) if dim is None else ([dim] if isinstance(dim, int) else list(dim))
    dims = sorted({d + nd if d < 0 else d for d in dims})
    if any(d < 0 or d >= nd for d in dims):
        raise ValueError(f"{name}: dim out of range")
    crosses = ft.placement.kind == "sharded_1d_row" and 0 in dims
    return dims, crosses


def _combine_extremum(name, partial, ft, be):
    """max / min of floating partials across ranks.  The single-GPU rule is "a NaN wins only at
    position 0 of the reduced slice"; across shards that position belongs to the first rank
    that has rows.  The other ranks computed their partial without the rule (so it cannot be a
    NaN that came from their own first row), and the partials are folded here in rank order
    from the owner on by the SAME reduction kernel -- the owner's partial sits at position 0
    of that fold -- instead of by the collective library's max, whose treatment of NaN is not
    part of its contract."""
    mesh = ft.placement.mesh
    ws = mesh.world_size
    if ws == 1:
        return partial
    flat = partial.contiguous().reshape(-1)
    gathered = torch.empty(ws * flat.numel(), dtype=partial.dtype, device=partial.device)
    dist.all_gather_into_tensor(gathered, flat, group=mesh.group)
    stacked = gathered.view((ws,) + tuple(partial.shape))
    return be.reduce(name, stacked[_first_owner(ft.placement):], [0], False)


def reduce(name: str, ft: FabricTensor, dim=None, keepdim: bool = False, local_ops=None):
    """sum / mean / max / min of a FabricTensor.

    * the reduced dims include dim 0 of a sharded_1d_row tensor: local partial, one exchange
      (all-reduce; all-gather + ordered fold for floating max / min), then for mean the scale by
      1 / global count and the cast to the input dtype -> a plain tensor, identical on every rank;
    * otherwise: local reduction -> FabricTensor sharded the same way.
    """
    dims, crosses = _plan(name, ft, dim, keepdim)
    x = ft.shard
    be = _backend(local_ops, x)
    if not crosses:
        out = be.reduce(name, x, dims, keepdim)
        if ft.placement.kind == "replicated":
            return out
        pl = FabricPlacement("sharded_1d_row", ft.placement.mesh,
                             (ft.placement.global_shape[0],) + tuple(out.shape[1:]),
                             ft.placement.shard_offsets)
        return FabricTensor(pl, out)
    local = "sum" if name == "mean" else name
    floating_ext = local in ("max", "min") and x.dtype.is_floating_point
    if x.shape[0] == 0:
        # an empty shard contributes the identity
        oshape = [1 if i in dims else s for i, s in enumerate(x.shape) if keepdim or i not in dims]
        pdt = torch.int64 if x.dtype == torch.int64 else torch.float32
        ident = {"sum": 0, "max": float("-inf") if pdt.is_floating_point else torch.iinfo(pdt).min,
                 "min": float("inf") if pdt.is_floating_point else torch.iinfo(pdt).max}[local]
        partial = torch.full(oshape, ident, dtype=pdt, device=x.device)
    else:
        first = ft.placement.mesh.rank == _first_owner(ft.placement)
        partial = be.reduce(local, x, dims, keepdim, partial=True, first_shard=first)
    if floating_ext:
        partial = _combine_extremum(local, partial, ft, be)
    else:
        _all_reduce(partial, name, ft.placement.mesh)
    if name == "mean":
        count = 1
        for d in dims:
            count *= ft.placement.global_shape[d]
        return be.scale_cast(partial, 1.0 / count if count else float("nan"), x.dtype)
    if partial.dtype != x.dtype:
        return be.scale_cast(partial, 1.0, x.dtype)
    return partial


class FabricComm:
    """Exchange buffers of the fused sharded reductions (``vbt_b200_reduce_exchange``): every
    rank allocates one small device buffer, the ranks swap handles to them with one
    ``all_gather_object`` and map each other's buffer.  Built collectively, once per mesh."""

    _by_mesh: dict = {}

    def __init__(self, mesh: FabricMesh, device: torch.device, slot_floats: int = 1 << 16):
        import ctypes
        from . import _lib
        self._lib, self._ct = _lib, ctypes
        self.mesh, self.device = mesh, device
        L = _lib.lib()
        self.ptr = ctypes.c_void_p()
        ok, err = True, ""
        try:
            _lib.check(L.vbt_b200_fabric_comm_create(device.index, mesh.rank, mesh.world_size, slot_floats,
                                                     ctypes.byref(self.ptr)))
            mine = ctypes.create_string_buffer(_lib.FABRIC_HANDLE_BYTES)
            _lib.check(L.vbt_b200_fabric_comm_handle(self.ptr, mine))
            payload = mine.raw
        except Exception as ex:  # every rank still has to take part in the exchange below
            ok, err, payload = False, str(ex), b""
        gathered = [None] * mesh.world_size
        dist.all_gather_object(gathered, (ok, payload), group=mesh.group)
        if ok and all(g[0] for g in gathered):
            try:
                _lib.check(L.vbt_b200_fabric_comm_connect(self.ptr, b"".join(g[1] for g in gathered)))
            except Exception as ex:
                ok, err = False, str(ex)
        else:
            ok = False
        flags = [None] * mesh.world_size
        dist.all_gather_object(flags, ok, group=mesh.group)
        self.ok = all(flags)
        self.error = err
        if not self.ok:
            self.close()

    @classmethod
    def get(cls, mesh: FabricMesh, device: torch.device) -> Optional["FabricComm"]:
        """The mesh's comm (created on first use; every rank must call this together), or None
        when some rank could not map its peers -- then the all-reduce path is used."""
        key = (mesh.devices, id(mesh.group), device.index)
        if key not in cls._by_mesh:
            comm = cls(mesh, device)
            cls._by_mesh[key] = comm if comm.ok else None
        return cls._by_mesh[key]

    def check(self) -> None:
        """Synchronises the current stream; raises if an exchange on this rank timed out."""
        self._lib.check(self._lib.lib().vbt_b200_fabric_comm_status(self.ptr, self._lib.stream_ptr(
            torch.empty(0, device=self.device))))

    def close(self) -> None:
        if self.ptr:
            self._lib.lib().vbt_b200_fabric_comm_destroy(self.ptr)
            self.ptr = self._ct.c_void_p()


class PreparedReduce:
    """A sharded reduction set up once and run many times: the reduction plan, tensor
    descriptors, partial / result buffers and workspace are built here, so a ``run()`` is the
    local kernel launch, the exchange, and (mean, 16-bit inputs) one scale-and-cast launch --
    no shape queries or allocations in between.  ``run()`` returns the same result tensor every
    time (it is overwritten by the next run).  The shard's storage must stay where it is; its
    contents may change between runs.  CUDA tensors only."""

    def __init__(self, name: str, ft: FabricTensor, dim=None, keepdim: bool = False, fused: Optional[bool] = None):
        """fused=None: one launch that reduces, exchanges over NVLink peer memory, scales and casts
        (vbt_b200_reduce_exchange) whenever every rank supports it for this layout, else the
        partial + all-reduce (+ scale-and-cast) form; False forces the latter."""
        from . import ops
        self.name = name
        self.ft = ft
        self.mesh = ft.placement.mesh
        dims, crosses = _plan(name, ft, dim, keepdim)
        if not crosses:
            raise FabricError("PreparedReduce is for reductions over the sharded dim")
        x = ft.shard
        _backend(None, x)
        if x.shape[0] == 0:
            raise FabricError("PreparedReduce needs a non-empty local shard")
        self._ops = ops
        local = "sum" if name == "mean" else name
        self._floating_ext = local in ("max", "min") and x.dtype.is_floating_point
        first = self.mesh.rank == _first_owner(ft.placement)
        self._local = ops.PreparedReduce(local, x, dims, keepdim, partial=True, first_shard=first)
        partial = self._local.out
        self._gathered = None
        self._fold = None
        if self._floating_ext and self.mesh.world_size > 1:
            ws = self.mesh.world_size
            self._gathered = torch.empty(ws * partial.numel(), dtype=partial.dtype, device=x.device)
            stacked = self._gathered.view((ws,) + tuple(partial.shape))
            self._fold = ops.PreparedReduce(local, stacked[_first_owner(ft.placement):], [0], False)
        src = self._fold.out if self._fold is not None else partial
        self._scale = None
        if name == "mean" or src.dtype != x.dtype:
            count = 1
            if name == "mean":
                for d in dims:
                    count *= ft.placement.global_shape[d]
            scale = (1.0 / count if count else float("nan")) if name == "mean" else 1.0
            self._scale = ops.PreparedScaleCast(src, scale, x.dtype)
        self.out = self._scale.out if self._scale is not None else src
        self.fused = None
        if fused is not False and self.mesh.world_size > 1 and x.dtype.is_floating_point:
            self._try_fused(local, x, dims, keepdim, first)

    def _try_fused(self, local, x, dims, keepdim, first):
        """Sets self.fused to a bound launch when ALL ranks can take the fused path."""
        import ctypes
        from . import _lib, ops
        comm = FabricComm.get(self.mesh, x.device)
        ok = comm is not None
        launch = None
        if ok:
            try:
                out = torch.empty(self.out.shape, dtype=x.dtype, device=x.device)
                dx, do, da = _lib.desc(x), _lib.desc(out), _lib.i64_array(dims)
                op = ops.REDUCE.index(local)
                nbytes = _lib.lib().vbt_b200_reduce_workspace_bytes(op, dx.ref, da, len(dims))
                ws = ops._reduce_workspace(nbytes, x.device)
                wp = ctypes.c_void_p(ws.data_ptr()) if ws is not None else None
                scale = 1.0
                if self.name == "mean":
                    count = 1
                    for d in dims:
                        count *= self.ft.placement.global_shape[d]
                    scale = 1.0 / count if count else float("nan")
                args = (op, do.ref, dx.ref, da, len(dims), int(keepdim), wp, nbytes, 1, comm.ptr,
                        _first_owner(self.ft.placement), scale)
                fn = _lib.lib().vbt_b200_reduce_exchange

                def launch():
                    _lib.check(fn(*args, _lib.stream_ptr(out)))
                    return out
                launch.keep = (dx, do, da, ws, out)
                launch()                      # a first call validates the layout (and runs the exchange once)
                torch.cuda.current_stream(x.device).synchronize()
                comm.check()
            except Exception:
                ok = False
        agreed = [None] * self.mesh.world_size
        dist.all_gather_object(agreed, ok, group=self.mesh.group)
        if all(agreed):
            self.fused = launch
            self.out = launch.keep[4]
            self.comm = comm
        elif any(agreed):
            # some ranks ran the trial exchange and some did not: their call counts differ now, so
            # this mesh stays on the all-reduce path from here on
            for key, val in list(FabricComm._by_mesh.items()):
                if val is comm:
                    FabricComm._by_mesh[key] = None

    def run(self, kernel_events=None) -> torch.Tensor:
        """kernel_events: an optional (start, end) pair of CUDA events recorded around the local
        reduction launch alone (for callers that time the kernel apart from the exchange)."""
        if self.fused is not None:
            if kernel_events is not None:
                kernel_events[0].record()
            out = self.fused()
            if kernel_events is not None:
                kernel_events[1].record()
            return out
        if kernel_events is not None:
            kernel_events[0].record()
        partial = self._local.run()
        if kernel_events is not None:
            kernel_events[1].record()
        if self.mesh.world_size > 1:
            if self._gathered is not None:
                dist.all_gather_into_tensor(self._gathered, partial.view(-1), group=self.mesh.group)
                self._fold.run()
            else:
                dist.all_reduce(partial, op=_REDUCE_OP[self.name], group=self.mesh.group)
        if self._scale is not None:
            self._scale.run()
        return self.out


def prepare_reduce(name: str, ft: FabricTensor, dim=None, keepdim: bool = False,
                   fused: Optional[bool] = None) -> PreparedReduce:
    return PreparedReduce(name, ft, dim, keepdim, fused)


def sum(ft, dim=None, keepdim=False, local_ops=None):  # noqa: A001
    return reduce("sum", ft, dim, keepdim, local_ops)


def mean(ft, dim=None, keepdim=False, local_ops=None):
    return reduce("mean", ft, dim, keepdim, local_ops)


def amax(ft, dim=None, keepdim=False, local_ops=None):
    return reduce("max", ft, dim, keepdim, local_ops)


def amin(ft, dim=None, keepdim=False, local_ops=None):
    return reduce("min", ft, dim, keepdim, local_ops)


def split_rows(total_rows: int, world_size: int) -> Sequence[Tuple[int, int]]:
    """(offset, rows) per rank for an even row split, remainder to the leading ranks."""
    base, rem = divmod(total_rows, world_size)
    out, off = [], 0
    for r in range(world_size):
        n = base + (1 if r < rem else 0)
        out.append((off, n))
        off += n
    return out
