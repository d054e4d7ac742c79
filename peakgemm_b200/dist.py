"""Column-sharded GEMM across the GPUs of one node (one process per GPU, torch.distributed).

The reference project has no multi-GPU code.  The layout here follows from its data format: B is
stored [n, k] (PeakGemm/__init__.py:27-31), so rank r owns a CONTIGUOUS slab of B rows
[start_r, stop_r) and computes the column block C[:, start_r:stop_r] from a replicated A.  There is no
reduction across ranks (k is not split), so the GEMMs need no collective at all; an all-gather over
NCCL / NVLink runs only when the caller asks for a replicated C.

Layouts of a gathered C:
  "shard_major"  [world, m, n_local]: rank r's block is out[r]; what the all-gather produces natively.
  "row_major"    [m, n]: the reference's layout; costs one more device copy (a strided write per block).

With bands > 1 the rows of A are processed in bands: while NCCL gathers band i, the GEMM of band i+1 runs
(leave the collective a few SMs with max_sms).  The band buffers are gathered in place.

`gathered_fused` needs no collective at all: the GEMM kernel's epilogue stores each output box to every
rank's C through peer-mapped pointers (PeerMatrix), so the gather rides NVLink tile by tile under the math.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def column_shard(n: int, world: int, rank: int, multiple: int = 8) -> tuple[int, int]:
    """Rows [start, stop) of the stored B[n, k] (= columns of C) that `rank` owns.

    Blocks are contiguous, equal (ceil(n / world) rounded up to `multiple`) except possibly the last
    non-empty one; their union is [0, n) and every start is a multiple of `multiple` (16-byte alignment
    of a bf16/fp16 column block inside a full-width C).
    """
    if n < 0 or world < 1 or not (0 <= rank < world):
        raise ValueError("bad shard request")
    per = -(-n // world)
    per = -(-per // multiple) * multiple
    start = min(n, rank * per)
    return start, min(n, start + per)


def row_bands(m: int, bands: int, multiple: int = 256) -> list[tuple[int, int]]:
    """Splits [0, m) into at most `bands` contiguous row bands whose sizes are multiples of `multiple`
    (the pair kernel's tile height) except the last."""
    bands = max(1, bands)
    per = -(-m // bands)
    per = max(multiple, -(-per // multiple) * multiple)
    out, r = [], 0
    while r < m:
        out.append((r, min(m, r + per)))
        r += per
    return out or [(0, 0)]


class _DeviceArray:
    """Minimal __cuda_array_interface__ carrier so torch can wrap a raw device pointer (as int16 words)."""

    def __init__(self, ptr: int, n_words: int):
        self.__cuda_array_interface__ = {"shape": (n_words,), "typestr": "<i2", "data": (ptr, False), "version": 2}


class PeerMatrix:
    """A [rows, cols] 16-bit matrix allocated on every rank, whose copies on the OTHER ranks this rank's
    kernels can store into over NVLink (one node, one process per GPU).

    Each rank allocates its copy with pg_peer_alloc (cudaMalloc + CUDA IPC export) and opens every peer's
    handle with pg_peer_open while its own device is current, which is what makes the mapping valid for
    kernels of this device.  `local` is this rank's copy as a torch tensor; `ptrs[r]` is the device address of
    rank r's copy as seen from this process.  Nothing in this package loads from a peer's copy.
    """

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, group=None):
        from . import capi

        assert dist.is_initialized(), "PeerMatrix needs torch.distributed"
        assert dtype in (torch.bfloat16, torch.float16)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.rows, self.cols, self.dtype = rows, cols, dtype
        self._capi = capi
        self._own_ptr, handle = capi.peer_alloc(rows * cols * 2)
        everyone = [None] * self.world
        dist.all_gather_object(everyone, handle, group=group)
        self.ptrs, self._opened = [], []
        for r, h in enumerate(everyone):
            if r == self.rank:
                self.ptrs.append(self._own_ptr)
            else:
                p = capi.peer_open(h)
                self._opened.append(p)
                self.ptrs.append(p)
        self.local = torch.as_tensor(_DeviceArray(self._own_ptr, rows * cols),
                                     device=torch.device("cuda", torch.cuda.current_device())) \
            .view(dtype).view(rows, cols)
        dist.barrier(group=group)

    def block_ptr(self, r: int, col0: int) -> int:
        """Device address of element [0, col0] of rank r's copy."""
        return self.ptrs[r] + 2 * col0

    def close(self) -> None:
        """Unmaps the peers' copies and frees the local one (collective: every rank must call it)."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for p in self._opened:
            self._capi.peer_close(p)
        self._opened = []
        dist.barrier(group=self.group)
        if self._own_ptr:
            self.local = None
            self._capi.peer_free(self._own_ptr)
            self._own_ptr = 0


class MulticastMatrix:
    """A [rows, cols] 16-bit matrix allocated on every rank in torch's symmetric memory and bound to ONE multicast
    address: a store through that address is replicated by the NVLink switch into every rank's copy (NVLS).

    The allocation, the handle exchange and the multicast binding are torch.distributed._symmetric_memory's
    (plumbing); what this package adds is the kernel that stores through `multicast_ptr` (pg_hgemm_mcast).
    `local` is this rank's copy.  Raises if the group's GPUs offer no multicast (no NVSwitch).  Keep every rank
    alive until close(): a rank must not exit while its memory is bound and peers still store.
    """

    def __init__(self, rows: int, cols: int, dtype: torch.dtype, group=None):
        import torch.distributed._symmetric_memory as symm_mem

        assert dist.is_initialized(), "MulticastMatrix needs torch.distributed"
        assert dtype in (torch.bfloat16, torch.float16)
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        self.rows, self.cols, self.dtype = rows, cols, dtype
        dev = torch.device("cuda", torch.cuda.current_device())
        # The constructor is collective.  Each step that can fail on one rank alone is followed by an agreement, so
        # that either every rank goes on or every rank raises: nobody is left waiting in a rendezvous.
        self.local, err = None, ""
        try:
            self.local = symm_mem.empty(rows, cols, dtype=dtype, device=dev)
        except Exception as exc:  # noqa: BLE001  (allocation failure of any kind: the ranks must agree on it)
            err = repr(exc)
        self._agree(self.local is not None, f"symmetric allocation failed on a rank ({err})")
        self._handle = symm_mem.rendezvous(self.local, self.group)
        self.multicast_ptr = int(self._handle.multicast_ptr)
        self._agree(self.multicast_ptr != 0,
                    "this group's GPUs offer no NVLink multicast (NVLS): use PeerMatrix / gathered_fused")
        dist.barrier(group=self.group)

    def _agree(self, ok: bool, message: str) -> None:
        flag = torch.tensor([int(ok)], device=torch.device("cuda", torch.cuda.current_device()))
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=self.group)
        if int(flag.item()) == 0:
            self.local = None
            self._handle = None
            raise RuntimeError("multicast matrix: " + message)

    def close(self) -> None:
        """Collective: every rank's kernels have completed before any rank lets go of the memory."""
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._handle = None
        self.local = None
        dist.barrier(group=self.group)


def _default_gemm(c, a, b, ldc, max_sms):
    from . import capi   # the CUDA path; there is no fallback

    capi.hgemm(c, a, b, ldc=ldc, max_sms=max_sms)


class ShardedGemm:
    """C = A @ B^T with B sharded by rows (columns of C) over the ranks of `group`.

    `gemm(c, a, b, ldc, max_sms)` computes one block in place; it defaults to the sm_100a kernel through the
    C ABI.  Tests on CPU ranks (gloo) pass the oracle here to exercise the sharding and gather logic.
    """

    def __init__(self, n: int, group=None, gemm=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.n = n
        self.start, self.stop = column_shard(n, self.world, self.rank)
        self.gemm = gemm or _default_gemm

    @property
    def n_local(self) -> int:
        return self.stop - self.start

    def local(self, a: torch.Tensor, b_shard: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """This rank's column block, contiguous [m, n_local].  No communication."""
        m = a.shape[0]
        assert b_shard.shape[0] == self.n_local and b_shard.shape[1] == a.shape[1]
        if out is None:
            out = torch.empty(m, self.n_local, dtype=a.dtype, device=a.device)
        if self.n_local:
            self.gemm(out, a, b_shard, self.n_local, 0)
        return out

    def local_into_full(self, c_full: torch.Tensor, a: torch.Tensor, b_shard: torch.Tensor) -> torch.Tensor:
        """Writes this rank's block into columns [start, stop) of a full-width row-major C[m, n] (ldc = n)."""
        assert c_full.shape == (a.shape[0], self.n) and c_full.is_contiguous()
        if self.n_local:
            self.gemm(c_full[:, self.start:self.stop], a, b_shard, self.n, 0)
        return c_full

    def gathered_fused(self, c: "PeerMatrix", a: torch.Tensor, b_shard: torch.Tensor, max_sms: int = 0) -> torch.Tensor:
        """Replicated row-major C[m, n] with the gather fused into the GEMM: ONE kernel per rank whose epilogue
        stores every output box to the rank's own C and, over NVLink, to the same place in every peer's C
        (pg_hgemm_multi).  No all-gather, no re-layout; a stream-ordered barrier closes the step.  `c` is the
        PeerMatrix that holds the result on every rank; returns this rank's copy."""
        from . import capi

        assert (c.rows, c.cols) == (a.shape[0], self.n) and c.world == self.world and c.dtype == a.dtype
        if self.n_local:
            order = [self.rank] + [r for r in range(self.world) if r != self.rank]
            ptrs = [c.block_ptr(r, self.start) for r in order]
            capi.hgemm_multi(ptrs, a, b_shard, ldc=self.n, max_sms=max_sms)
        if self.world > 1:
            dist.barrier(group=self.group)      # NCCL: ordered on the stream behind this rank's GEMM
        return c.local

    def gathered_multicast(self, c: "MulticastMatrix", a: torch.Tensor, b_shard: torch.Tensor,
                           max_sms: int = 0) -> torch.Tensor:
        """Replicated row-major C[m, n] with the gather done by the NVLink switch: ONE kernel per rank whose epilogue
        writes this rank's column block through the multicast address of `c` (pg_hgemm_mcast, multimem.st), so each
        output byte leaves the GPU once and the switch delivers it to every rank's copy.  A stream-ordered barrier
        closes the step.  Returns this rank's copy."""
        from . import capi

        assert (c.rows, c.cols) == (a.shape[0], self.n) and c.world == self.world and c.dtype == a.dtype
        if self.n_local:
            capi.hgemm_mcast(c.local.data_ptr() + 2 * self.start, c.multicast_ptr + 2 * self.start, a, b_shard,
                             ldc=self.n, max_sms=max_sms)
        if self.world > 1:
            dist.barrier(group=self.group)      # NCCL: ordered on the stream behind this rank's GEMM
        return c.local

    def gathered(self, a: torch.Tensor, b_shard: torch.Tensor, layout: str = "row_major", bands: int = 1,
                 max_sms: int = 0) -> torch.Tensor:
        """Replicated C on every rank: local GEMM + all-gather of the column blocks (band-pipelined)."""
        if layout not in ("row_major", "shard_major"):
            raise ValueError(layout)
        m, w, nl = a.shape[0], self.world, self.n_local
        if w == 1:
            c = self.local(a, b_shard)
            return c if layout == "row_major" else c.view(1, m, nl)
        if self.n != nl * w:
            raise ValueError("gathered() needs equal shards: n must be a multiple of 8 * world")
        spans = row_bands(m, bands)
        # flat buffer: band after band, each band [world, rows_in_band, n_local] contiguous
        flat = torch.empty(w * m * nl, dtype=a.dtype, device=a.device)
        works, views = [], []
        for (r0, r1) in spans:
            band = flat[w * r0 * nl: w * r1 * nl].view(w, r1 - r0, nl)
            self.gemm(band[self.rank], a[r0:r1], b_shard, nl, max_sms if len(spans) > 1 else 0)
            works.append(dist.all_gather_into_tensor(band.view(-1), band[self.rank].reshape(-1), group=self.group,
                                                     async_op=True))
            views.append(band)
        for wk in works:
            wk.wait()
        if layout == "shard_major":
            if len(spans) == 1:
                return views[0]
            return torch.cat(views, dim=1)
        out = torch.empty(m, self.n, dtype=a.dtype, device=a.device)
        out3 = out.view(m, w, nl)
        for (r0, r1), band in zip(spans, views):
            out3[r0:r1].copy_(band.transpose(0, 1))      # block r -> columns [r*nl, (r+1)*nl)
        return out


# ------------------------------------------------------------------ RMSNorm ----

def row_shard(rows: int, world: int, rank: int) -> tuple[int, int]:
    """Rows [start, stop) of x (and dy, y, dx) that `rank` owns: contiguous blocks of ceil(rows / world) rows,
    the last non-empty one possibly shorter; their union is [0, rows)."""
    if rows < 0 or world < 1 or not (0 <= rank < world):
        raise ValueError("bad shard request")
    per = -(-rows // world)
    start = min(rows, rank * per)
    return start, min(rows, start + per)


def _default_rms_fwd(y, x, gamma, eps):
    from . import capi   # the CUDA path; there is no fallback

    capi.rmsnorm_fwd(y, x, gamma, eps)


def _default_rms_bwd(dx, dgamma, dy, x, gamma, eps):
    from . import capi

    ws = torch.empty(max(1, capi.rmsnorm_bwd_workspace_bytes(x.shape[0], x.shape[1]) // 4), device=x.device)
    capi.rmsnorm_bwd(dx, dgamma, dy, x, gamma, ws, eps)


class ShardedRmsNorm:
    """RMSNorm forward / backward with the ROWS of x sharded over the ranks of `group` (gamma replicated).

    The reference project has neither RMSNorm nor multi-GPU code; the split follows from the operator: every row
    is normalised on its own, so y and dx need no communication at all.  Only dgamma = sum over ALL rows of
    dy * xhat crosses ranks, and only when the caller wants the global sum:

      reduce="none"        dgamma holds this rank's partial sum (a data-parallel caller that reduces gradients
                           itself, bucketed with its other parameters, wants exactly this);
      reduce="all_reduce"  one all-reduce(SUM) of the [h] fp32 vector (16-32 KiB: latency-bound).  The order of
                           the additions is the collective library's: reproducible for a fixed world size and
                           algorithm, not specified otherwise;
      reduce="ordered"     all-gather of the partial vectors, summed in rank order on every rank: every rank gets
                           bit-identical dgamma, in an order that does not depend on the collective's algorithm.

    `fwd(y, x, gamma, eps)` and `bwd(dx, dgamma, dy, x, gamma, eps)` compute on this rank's rows in place; they
    default to the sm_100a kernels through the C ABI.  Tests on CPU ranks (gloo) pass the oracle here.
    """

    def __init__(self, rows: int, group=None, fwd=None, bwd=None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.rows = rows
        self.start, self.stop = row_shard(rows, self.world, self.rank)
        self.fwd = fwd or _default_rms_fwd
        self.bwd = bwd or _default_rms_bwd

    @property
    def rows_local(self) -> int:
        return self.stop - self.start

    def forward(self, x_local: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6,
                out: torch.Tensor | None = None) -> torch.Tensor:
        """y for this rank's rows.  No communication."""
        assert x_local.shape[0] == self.rows_local
        y = out if out is not None else torch.empty_like(x_local)
        if self.rows_local:
            self.fwd(y, x_local, gamma, eps)
        return y

    def backward(self, dy_local: torch.Tensor, x_local: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6,
                 reduce: str = "all_reduce"):
        """(dx for this rank's rows, dgamma [h] fp32 reduced as `reduce` says)."""
        if reduce not in ("none", "all_reduce", "ordered"):
            raise ValueError(reduce)
        assert x_local.shape[0] == self.rows_local and dy_local.shape == x_local.shape
        dx = torch.empty_like(x_local)
        dgamma = torch.zeros(x_local.shape[1], dtype=torch.float32, device=x_local.device)
        if self.rows_local:
            self.bwd(dx, dgamma, dy_local, x_local, gamma, eps)
        if self.world > 1 and reduce == "all_reduce":
            dist.all_reduce(dgamma, op=dist.ReduceOp.SUM, group=self.group)
        elif self.world > 1 and reduce == "ordered":
            parts = torch.empty(self.world, dgamma.numel(), dtype=torch.float32, device=dgamma.device)
            dist.all_gather_into_tensor(parts.view(-1), dgamma, group=self.group)
            total = parts[0].clone()
            for r in range(1, self.world):          # rank order, the same on every rank
                total += parts[r]
            dgamma = total
        return dx, dgamma
