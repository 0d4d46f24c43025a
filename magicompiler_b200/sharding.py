"""Column sharding of the packed gate/up weight across the GPUs of one box, and the row-parallel
down-projection that closes a full SwiGLU MLP.

Layout follows the reference's Llama example (example/training/llama3.py:168-170): ``w1``/``w3`` are
column-parallel with ``gather_output=False`` (rank r owns output columns ``[r*N/P, (r+1)*N/P)``), ``w2``
is row-parallel with ``input_is_parallel=True`` (rank r owns the matching input columns and the partial
products are summed with one all-reduce).  The fused op needs no collective: rank r multiplies the
replicated activations by its own packed shard ``cat(Wg[rows_r], Wu[rows_r])``.  The only exchange is the
reduction after the down-projection: NCCL's all-reduce or reduce-scatter, or ``reduce="peer_scatter"``, where
the down projection's own epilogue stores each row block into the memory of the GPU that owns it
(``PeerScatterReducer``).  No GPU ever READS another GPU's memory.
"""
from __future__ import annotations

from typing import Callable

import os

import torch
import torch.distributed as dist
import torch.nn.functional as F


def pack_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[N,K]`` gate_proj.weight and ``[N,K]`` up_proj.weight -> packed ``[2N,K]`` (gate rows first), contiguous."""
    if w_gate.shape != w_up.shape or w_gate.dim() != 2:
        raise ValueError(f"gate {tuple(w_gate.shape)} and up {tuple(w_up.shape)} must be equal 2-D shapes")
    if w_gate.dtype != w_up.dtype or w_gate.device != w_up.device:
        raise ValueError("gate and up weights must share dtype and device")
    return torch.cat([w_gate, w_up], dim=0).contiguous()


def shard_bounds(n: int, rank: int, world: int, multiple: int = 8) -> tuple[int, int]:
    """Half-open column range of rank ``rank``; every shard is a multiple of ``multiple`` columns."""
    if world < 1 or not (0 <= rank < world):
        raise ValueError(f"bad rank/world: {rank}/{world}")
    if n % (world * multiple) != 0:
        raise ValueError(f"N={n} cannot be cut into {world} shards that are multiples of {multiple}")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_gate_up(w_gate_up: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank ``rank``'s packed shard ``[2*N/P, K]`` of a packed ``[2N,K]`` weight (a copy, made once at load)."""
    if w_gate_up.dim() != 2 or w_gate_up.shape[0] % 2:
        raise ValueError("w_gate_up must be [2N, K]")
    n = w_gate_up.shape[0] // 2
    lo, hi = shard_bounds(n, rank, world)
    return torch.cat([w_gate_up[lo:hi], w_gate_up[n + lo:n + hi]], dim=0).contiguous()


def shard_down(w_down: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Rank ``rank``'s input-column shard ``[K_out, N/P]`` of down_proj.weight ``[K_out, N]``."""
    lo, hi = shard_bounds(w_down.shape[1], rank, world)
    return w_down[:, lo:hi].contiguous()


def _default_swiglu() -> Callable:
    from .ops import gemm_swiglu

    return gemm_swiglu


class ColumnParallelSwiGLU(torch.nn.Module):
    """Gate/up projection + SwiGLU of one rank: ``[..., K] -> [..., N/P]``, no communication."""

    def __init__(self, w_gate_up_full: torch.Tensor, rank: int = 0, world: int = 1,
                 swiglu_fn: Callable | None = None):
        super().__init__()
        self.rank, self.world = rank, world
        self.weight = torch.nn.Parameter(shard_gate_up(w_gate_up_full, rank, world), requires_grad=False)
        self._fn = swiglu_fn

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        fn = self._fn or _default_swiglu()
        return fn(x, self.weight)


def peer_slot_offset(dest_set: int, world: int, writer: int, rows: int, n_out: int) -> int:
    """Element offset, inside a receive buffer ``[2 sets][world slots][rows][n_out]``, of the slot that rank ``writer``
    fills in destination set ``dest_set`` (the same in every owner's buffer)."""
    if not (0 <= dest_set < 2 and 0 <= writer < world):
        raise ValueError(f"bad slot: set {dest_set}, writer {writer} of {world}")
    return ((dest_set * world + writer) * rows) * n_out


class PeerScatterReducer:
    """Reduce-scatter of a row-parallel GEMM whose data movement is the GEMM's own epilogue.

    Every rank holds a receive buffer ``[2 sets][world slots][M/world rows][n_out]`` in symmetric memory (mapped into
    all ranks of the group).  ``linear_reduce_scatter(h, w_down)`` runs ``h @ w_down.T`` on the tile kernels with the
    epilogue's TMA stores aimed at slot ``rank`` of the buffer of whichever GPU owns the row block
    (``magi_swiglu_gemm_nt_bf16_scatter``), waits for all ranks on the stream (a one-element NCCL all-reduce: it
    starts after this rank's GEMM has completed and ends only when every rank has joined, and a rank that never joins
    ends it with the process group's timeout error instead of an endless wait), and adds the ``world`` slots of its
    own buffer in rank order (``magi_swiglu_sum_slots_bf16``): deterministic, and the partial products cross NVLink
    while the tensor cores are still busy with later tiles instead of in a collective afterwards.
    Consecutive calls alternate between the two sets, so one barrier per call is enough: a peer can only start
    overwriting set s two calls later, which needs the barrier of the call in between, which this rank enters after
    its sum over set s.  Collective: all ranks of ``group`` construct it and call it in the same order.
    """

    _active: "PeerScatterReducer | None" = None  # whose destinations the library's two sets currently describe
    _shared: "dict[tuple, PeerScatterReducer]" = {}

    @classmethod
    def shared(cls, m: int, n_out: int, group=None, device: torch.device | None = None) -> "PeerScatterReducer":
        """One reducer per (group, shape, device) for all layers of a model: calls from different layers are just
        consecutive steps of the same reducer, so the buffers exist once and the library's destination sets are
        written once.  Collective on first use, like the constructor."""
        grp = group if group is not None else dist.group.WORLD
        dev = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        key = (id(grp), m, n_out, dev.index)
        red = cls._shared.get(key)
        if red is None:
            red = cls._shared[key] = cls(m, n_out, grp, dev)
        return red

    @classmethod
    def release_shared(cls) -> None:
        """Drop the shared reducers (before a process group is destroyed, say); their buffers go with them."""
        cls._shared.clear()
        cls._active = None

    def __init__(self, m: int, n_out: int, group=None, device: torch.device | None = None):
        # plain peer stores only: never bind the buffers to an NVLink multicast object
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.group = group if group is not None else dist.group.WORLD
        self.world, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        if m % (self.world * 32) or n_out % 64:
            raise ValueError(f"peer scatter needs M ({m}) to be a multiple of {self.world * 32} and the output width "
                             f"({n_out}) a multiple of 64")
        self.m, self.n_out, self.rows = m, n_out, m // self.world
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else device
        self.recv = symm_mem.empty((2, self.world, self.rows, n_out), dtype=torch.bfloat16, device=self.device)
        self.handle = symm_mem.rendezvous(self.recv, self.group)
        self.full = None  # [2 sets][M][n_out] in symmetric memory, made by the first linear_all_reduce
        self._full_handle = None
        self._token = torch.zeros(1, dtype=torch.float32, device=self.device)
        self.step = 0

    def _activate(self) -> None:
        if PeerScatterReducer._active is self:
            return
        from .ops import scatter_setup

        torch.cuda.current_stream(self.device).synchronize()  # no scattered GEMM may be running on the old sets
        bases = [int(p) for p in self.handle.buffer_ptrs]
        for dest_set in (0, 1):
            mine = 2 * peer_slot_offset(dest_set, self.world, self.rank, self.rows, self.n_out)  # bytes (bf16)
            scatter_setup(dest_set, [bases[o] + mine for o in range(self.world)], self.rows, self.n_out,
                          device=self.device.index)
        PeerScatterReducer._active = self

    def linear_reduce_scatter(self, h: torch.Tensor, w_down: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        """Rows ``[rank * M/world, (rank + 1) * M/world)`` of ``sum over ranks of h_r @ w_down_r.T``."""
        from .ops import gemm_nt_scatter, sum_slots

        if h.shape[0] != self.m or w_down.shape[0] != self.n_out:
            raise ValueError(f"built for [{self.m}, *] x [{self.n_out}, *], got {tuple(h.shape)} x {tuple(w_down.shape)}")
        self._activate()
        dest_set = self.step & 1
        self.step += 1
        gemm_nt_scatter(h, w_down, dest_set)
        dist.all_reduce(self._token, group=self.group)  # every rank's stores into every buffer have completed
        return sum_slots(self.recv[dest_set], out)

    def linear_all_reduce(self, h: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
        """The whole ``sum over ranks of h_r @ w_down_r.T`` on every rank: as ``linear_reduce_scatter``, but each rank's
        slot sum is stored into every rank's copy of the result (peer stores from the sum kernel) and a second barrier
        makes the whole result readable.  The returned ``[M, n_out]`` tensor is a view of one of two result buffers in
        symmetric memory: it is overwritten by the call after the next one."""
        from .ops import gemm_nt_scatter, sum_slots_bcast

        if h.shape[0] != self.m or w_down.shape[0] != self.n_out:
            raise ValueError(f"built for [{self.m}, *] x [{self.n_out}, *], got {tuple(h.shape)} x {tuple(w_down.shape)}")
        if self.full is None:  # collective, like the constructor
            import torch.distributed._symmetric_memory as symm_mem

            self.full = symm_mem.empty((2, self.m, self.n_out), dtype=torch.bfloat16, device=self.device)
            self._full_handle = symm_mem.rendezvous(self.full, self.group)
        self._activate()
        dest_set = self.step & 1
        self.step += 1
        gemm_nt_scatter(h, w_down, dest_set)
        dist.all_reduce(self._token, group=self.group)  # every rank's partial products have arrived
        block = (dest_set * self.m + self.rank * self.rows) * self.n_out * 2  # this rank's rows in a result buffer
        sum_slots_bcast(self.recv[dest_set], [int(p) + block for p in self._full_handle.buffer_ptrs])
        dist.all_reduce(self._token, group=self.group)  # every rank's rows have arrived in every result buffer
        return self.full[dest_set]


class TensorParallelSwiGLUMLP(torch.nn.Module):
    """Full SwiGLU MLP over ``world`` ranks: fused column-parallel gate/up, row-parallel down, one reduction.

    ``chunks`` > 1 cuts the rows into that many slices and reduces slice i asynchronously while slice i+1 is
    computed, so the NVLink transfer hides behind the GEMMs.

    ``reduce``: ``"all_reduce"`` (every rank gets the whole ``[M, K]`` result, fairscale's ``RowParallelLinear`` of
    example/training/llama3.py:169) or ``"reduce_scatter"`` (each rank keeps the rows ``owned_rows(M)`` of the sum —
    half the bytes on the links; the next layer all-gathers them or works row-sharded).  With reduce-scatter every
    slice's row count must be a multiple of ``world``.  ``"peer_scatter"`` gives the same rows with no collective
    kernel at all: the down projection's epilogue stores each row block into its owner's memory
    (``PeerScatterReducer``; ``chunks`` must be 1, M a multiple of ``32 * world``, the output width of 64).
    ``"peer_all_reduce"`` continues from there to the whole result on every rank: each rank's sum kernel stores its rows
    into every rank's result buffer (shared by all layers of that shape); the module returns a copy unless
    ``borrow_result=True``, in which case the tensor is overwritten by the second peer all-reduce after this one.

    ``down_fn(h, w_down)`` returns the partial down projection; if it has a true ``supports_out`` attribute it is
    called as ``down_fn(h, w_down, out=...)`` and writes straight into the result (``gemm_nt_out``).
    """

    def __init__(self, w_gate_up_full: torch.Tensor, w_down_full: torch.Tensor, rank: int = 0, world: int = 1,
                 group=None, chunks: int = 1, swiglu_fn: Callable | None = None, down_fn: Callable | None = None,
                 reduce: str = "all_reduce", borrow_result: bool = False):
        super().__init__()
        if reduce not in ("all_reduce", "reduce_scatter", "peer_scatter", "peer_all_reduce"):
            raise ValueError("reduce must be 'all_reduce', 'reduce_scatter', 'peer_scatter' or 'peer_all_reduce', "
                             f"got {reduce!r}")
        if reduce in ("peer_scatter", "peer_all_reduce") and max(1, int(chunks)) != 1:
            raise ValueError(f"{reduce} overlaps the transfer inside the kernel; chunks must be 1")
        self.borrow_result = bool(borrow_result)
        self.rank, self.world, self.group, self.chunks = rank, world, group, max(1, int(chunks))
        self.reduce = reduce
        self._down = down_fn  # (h [m, N/P], w_down [K_out, N/P]) -> [m, K_out]; None = library GEMM (torch.matmul)
        self.gate_up = ColumnParallelSwiGLU(w_gate_up_full, rank, world, swiglu_fn)
        self.w_down = torch.nn.Parameter(shard_down(w_down_full, rank, world), requires_grad=False)

    def _slices(self, m: int) -> list[tuple[int, int]]:
        step = -(-m // self.chunks) if m else 0
        return [(lo, min(m, lo + step)) for lo in range(0, m, step or 1)]

    def owned_rows(self, m: int) -> torch.Tensor:
        """Global row indices of this rank's output under ``reduce="reduce_scatter"``, in output order."""
        parts = []
        for lo, hi in self._slices(m):
            per = (hi - lo) // self.world
            parts.append(torch.arange(lo + self.rank * per, lo + (self.rank + 1) * per))
        return torch.cat(parts) if parts else torch.empty(0, dtype=torch.long)

    def _down_into(self, h: torch.Tensor, dst: torch.Tensor) -> None:
        if self._down is None:
            torch.matmul(h, self.w_down.t(), out=dst)  # plain library GEMM: partial sums of this rank
        elif getattr(self._down, "supports_out", False):
            self._down(h, self.w_down, out=dst)
        else:
            dst.copy_(self._down(h, self.w_down))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        m, k_out = x2.shape[0], self.w_down.shape[0]
        if self.reduce in ("peer_scatter", "peer_all_reduce") and self.world > 1:
            red = PeerScatterReducer.shared(m, k_out, self.group, x.device)
            if self.reduce == "peer_scatter":
                return red.linear_reduce_scatter(self.gate_up(x2), self.w_down)
            full = red.linear_all_reduce(self.gate_up(x2), self.w_down)
            # the reducer's result buffer is overwritten two calls later: hand out a copy unless the caller borrows it
            return (full if self.borrow_result else full.clone()).view(*lead, k_out)
        scatter = self.reduce in ("reduce_scatter", "peer_scatter") and self.world > 1
        slices = self._slices(m)
        if scatter and any((hi - lo) % self.world for lo, hi in slices):
            raise ValueError(f"reduce_scatter needs every row slice to be a multiple of {self.world} rows "
                             f"(M={m}, chunks={self.chunks})")
        partial = torch.empty((m, k_out), dtype=self.w_down.dtype, device=x.device)
        out = torch.empty((m // self.world, k_out), dtype=self.w_down.dtype, device=x.device) if scatter else partial
        works, done = [], 0
        for lo, hi in slices:
            self._down_into(self.gate_up(x2[lo:hi]), partial[lo:hi])
            if scatter:
                per = (hi - lo) // self.world
                works.append(dist.reduce_scatter_tensor(out[done:done + per], partial[lo:hi], op=dist.ReduceOp.SUM,
                                                        group=self.group, async_op=True))
                done += per
            elif self.world > 1:
                works.append(dist.all_reduce(partial[lo:hi], op=dist.ReduceOp.SUM, group=self.group, async_op=True))
        for wk in works:
            wk.wait()
        return out if scatter else out.view(*lead, k_out)


def reference_mlp(x: torch.Tensor, w_gate_up: torch.Tensor, w_down: torch.Tensor) -> torch.Tensor:
    """Unsharded eager MLP, the expression of the reference's TransformerMLP.forward
    (tests/model_definition.py:336-339) on the packed weight; used by tests as the comparison point."""
    n = w_gate_up.shape[0] // 2
    return F.linear(F.silu(F.linear(x, w_gate_up[:n])) * F.linear(x, w_gate_up[n:]), w_down)
