"""N-split (output-feature) tensor parallelism of one INT4-G128 projection over the GPUs of a node.

The reference's weight layout shards along N with no re-packing: ``W_int4`` is ``[N][K/2]`` row-major and
``scales`` ``[N][K/128]`` (src/ops/linear.h:24), so rank r owns the contiguous rows ``[r N/g, (r+1) N/g)`` of
both, computes ``Y[:, slice]`` with the same kernel as the unsharded call, and one all-gather of ``[M, N]``
fp16 restores the full activation on every rank.  One process per GPU; the collective is NCCL through
``torch.distributed`` (gloo in the CPU tests).  The shard's result lands in slot ``rank`` of a
``[g][M][N/g]`` staging buffer, the all-gather runs in place on that buffer, and ``unstage`` turns it into
row-major ``[M][N]``.

``ColumnShardedLinear`` is the plain NCCL form (the baseline).  ``TpGroup`` is the product path: every rank owns an
exchange region mapped into all processes (CUDA IPC), the linear kernel's epilogue stores its slice straight into
every rank's activation buffer over NVLink and a flag per (receiver, sender) completes the exchange inside the
same launch; ``xinfer_b200.spec.SpecDecoder(tp=group)`` runs the whole speculative step that way (projections
N-split, KV cache and recurrent state split by sequence).
"""
from __future__ import annotations

import ctypes as C
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_rows(N: int, world: int, rank: int) -> Tuple[int, int]:
    """Rows ``[n0, n1)`` of a projection with N output features owned by ``rank``.

    Slices are equal (the all-gather wants equal counts) and even (the kernels pair rows), so N must be a
    multiple of ``2 * world``; projections that are not (the reference's N = 48 heads) stay replicated.
    """
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world {world}")
    if N <= 0 or N % (2 * world) != 0:
        raise ValueError(f"N={N} does not split into {world} even slices")
    per = N // world
    return rank * per, (rank + 1) * per


def can_shard(N: int, world: int) -> bool:
    return N > 0 and world >= 1 and N % (2 * world) == 0


class ColumnShardedLinear:
    """One rank's shard of ``linear_int4`` plus the all-gather that completes it.

    ``W_int4`` / ``scales`` / ``bias`` may be the full tensors (the shard is a view, no copy) or already the
    rank's slice (``sliced=True``).  ``compute`` is the per-shard linear; it defaults to the CUDA entry point
    and is replaceable so that the sharding and gathering can be tested on CPU ranks.
    """

    def __init__(self, W_int4: torch.Tensor, scales: torch.Tensor, bias: Optional[torch.Tensor], N: int, K: int,
                 rank: Optional[int] = None, world: Optional[int] = None, group=None, sliced: bool = False,
                 compute: Optional[Callable] = None, max_rows: int = 32):
        self.group = group
        self.world = dist.get_world_size(group) if world is None else world
        self.rank = dist.get_rank(group) if rank is None else rank
        self.N, self.K = N, K
        self.n0, self.n1 = shard_rows(N, self.world, self.rank)
        self.n_local = self.n1 - self.n0
        if sliced:
            self.W, self.S, self.b = W_int4, scales, bias
        else:
            self.W, self.S = W_int4[self.n0:self.n1], scales[self.n0:self.n1]
            self.b = None if bias is None else bias[self.n0:self.n1]
        if self.W.shape[0] != self.n_local or self.S.shape[0] != self.n_local:
            raise ValueError("weight shard has the wrong number of rows")
        self.max_rows = max_rows
        self._staging = torch.empty((self.world, max_rows, self.n_local), dtype=torch.float16, device=self.W.device)
        if compute is None:
            from . import ops
            compute = ops.linear_int4
        self._compute = compute

    def staging(self, M: int) -> torch.Tensor:
        """``[g][M][N/g]`` view of the staging buffer for M activation rows."""
        if not 1 <= M <= self.max_rows:
            raise ValueError(f"M={M} outside 1..{self.max_rows}")
        return self._staging.view(-1)[: self.world * M * self.n_local].view(self.world, M, self.n_local)

    def compute_local(self, X: torch.Tensor, M: int) -> torch.Tensor:
        """This rank's ``Y[:, n0:n1]`` into its slot of the staging buffer (no communication)."""
        st = self.staging(M)
        self._compute(st[self.rank], X, self.W, self.S, self.b, M, self.n_local, self.K)
        return st

    def gather(self, M: int) -> torch.Tensor:
        """All-gather of the staging buffer, in place: afterwards every rank holds every slot."""
        st = self.staging(M)
        if self.world > 1:
            mine = st[self.rank].reshape(-1)
            if dist.get_backend(self.group) != "nccl":
                mine = mine.clone()  # only NCCL defines the in-place form (input = own slot of the output)
            dist.all_gather_into_tensor(st.view(-1), mine, group=self.group)
        return st

    @staticmethod
    def unstage(st: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``[g][M][N/g]`` -> row-major ``[M][N]``."""
        g, M, n = st.shape
        if out is None:
            out = torch.empty((M, g * n), dtype=st.dtype, device=st.device)
        out.view(M, g, n).copy_(st.permute(1, 0, 2))
        return out

    def forward(self, X: torch.Tensor, M: int, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        self.compute_local(X, M)
        return self.unstage(self.gather(M), out)


class TpGroup:
    """This rank's end of the N-split exchange (``xinfer_tp_*`` in the C-ABI).

    Creates the rank's exchange region, all-gathers the IPC handles over ``torch.distributed`` (any backend: the
    blobs travel as CPU or CUDA byte tensors) and maps the peers' regions.  The current CUDA device must be the
    rank's own.  ``world == 1`` needs no process group.
    """

    def __init__(self, region_bytes: int, rank: Optional[int] = None, world: Optional[int] = None, group=None):
        from ._lib import check, lib
        self.group = group
        self.world = (dist.get_world_size(group) if dist.is_initialized() else 1) if world is None else world
        self.rank = (dist.get_rank(group) if dist.is_initialized() else 0) if rank is None else rank
        h = C.c_void_p()
        check(lib().xinfer_tp_create(self.rank, self.world, region_bytes, C.byref(h)), "tp_create")
        self._h = h
        if self.world > 1:
            nb = int(lib().xinfer_tp_handle_bytes())
            blob = (C.c_ubyte * nb)()
            check(lib().xinfer_tp_handle(self._h, blob), "tp_handle")
            mine = torch.tensor(list(bytes(blob)), dtype=torch.uint8)
            if dist.get_backend(group) == "nccl":
                mine = mine.cuda()
            gathered = [torch.empty_like(mine) for _ in range(self.world)]
            dist.all_gather(gathered, mine, group=group)
            allb = b"".join(bytes(t.cpu().numpy().tobytes()) for t in gathered)
            buf = C.create_string_buffer(allb, len(allb))
            check(lib().xinfer_tp_connect(self._h, C.cast(buf, C.c_void_p)), "tp_connect")
        else:
            check(lib().xinfer_tp_connect(self._h, None), "tp_connect")

    @property
    def handle(self):
        return self._h

    def close(self):
        from ._lib import lib
        if getattr(self, "_h", None):
            lib().xinfer_tp_destroy(self._h)
            self._h = None

    def alloc(self, nbytes: int) -> int:
        """Byte offset of a new buffer in the region (same on every rank when all allocate in the same order)."""
        from ._lib import check, lib
        off = C.c_size_t()
        check(lib().xinfer_tp_alloc(self._h, nbytes, C.byref(off)), "tp_alloc")
        return int(off.value)

    def read(self, offset: int, nbytes: int):
        """Host copy (numpy uint8) of ``nbytes`` of this rank's region at ``offset``; synchronises the device."""
        import numpy as np
        from ._lib import check, lib
        torch.cuda.synchronize()
        out = np.empty(nbytes, np.uint8)
        check(lib().xinfer_copy_device_to_host(out.ctypes.data_as(C.c_void_p), lib().xinfer_tp_ptr(self._h, offset), nbytes),
              "copy_device_to_host")
        return out

    def write(self, offset: int, array) -> None:
        import numpy as np
        from ._lib import check, lib
        a = np.ascontiguousarray(array)
        torch.cuda.synchronize()
        check(lib().xinfer_copy_host_to_device(lib().xinfer_tp_ptr(self._h, offset), a.ctypes.data_as(C.c_void_p), a.nbytes),
              "copy_host_to_device")

    def linear(self, y_offset: int, ldy: int, col0: int, X, W_local, scales_local, bias_local, M: int, n_local: int, K: int,
               rows_per_rank: int = 0, group_size: int = 128) -> int:
        """This rank's slice of ``linear_int4`` stored into every rank's Y (or the row owner's, rows_per_rank > 0)."""
        from ._lib import check, lib
        return check(lib().xinfer_tp_linear_int4_f16f16(
            self._h, torch.cuda.current_stream().cuda_stream, y_offset, ldy, col0, X.data_ptr(), W_local.data_ptr(),
            scales_local.data_ptr(), None if bias_local is None else bias_local.data_ptr(), M, n_local, K, group_size,
            rows_per_rank), "tp_linear_int4")

    def push(self, offset: int, nbytes: int) -> int:
        from ._lib import check, lib
        return check(lib().xinfer_tp_push(self._h, torch.cuda.current_stream().cuda_stream, offset, nbytes), "tp_push")

    def barrier(self) -> int:
        from ._lib import check, lib
        return check(lib().xinfer_tp_barrier(self._h, torch.cuda.current_stream().cuda_stream), "tp_barrier")

    def set_wait_limit(self, clocks: int) -> None:
        from ._lib import lib
        lib().xinfer_tp_set_wait_limit(self._h, clocks)

    def status(self) -> int:
        from ._lib import lib
        return int(lib().xinfer_tp_status(self._h))
