"""Column sharding of the packed weight and the row-parallel MLP, on CPU: shard algebra in-process and the
multi-rank path as two gloo ranks.  The kernel is replaced by the CPU oracle here (this is a test); what is
under test is the host logic around it — packing, shard bounds, chunked all-reduce, failure behaviour."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from magicompiler_b200 import (ColumnParallelSwiGLU, TensorParallelSwiGLUMLP, pack_gate_up, shard_bounds,
                               shard_down, shard_gate_up)
from magicompiler_b200.sharding import reference_mlp
from oracle import make_inputs, swiglu_gold


def _oracle_fn(x, w):
    return swiglu_gold(x.reshape(-1, x.shape[-1]).contiguous(), w, threads=2, want_eager=False)["gold_bf16"].view(
        *x.shape[:-1], w.shape[0] // 2)


def test_pack_and_shard_algebra():
    x, w = make_inputs(8, 64, 96, seed=3)
    n = 96
    assert torch.equal(pack_gate_up(w[:n], w[n:]), w)
    with pytest.raises(ValueError):
        pack_gate_up(w[:n], w[n:n + 8])
    for world in (1, 2, 4):
        cols = []
        for r in range(world):
            lo, hi = shard_bounds(n, r, world)
            s = shard_gate_up(w, r, world)
            assert s.shape == (2 * (hi - lo), 64) and s.is_contiguous()
            assert torch.equal(s[: hi - lo], w[lo:hi]) and torch.equal(s[hi - lo:], w[n + lo:n + hi])
            cols.append(_oracle_fn(x, s))
        # shards are independent units: concatenating their outputs IS the unsharded result, bit for bit
        assert torch.equal(torch.cat(cols, dim=1), _oracle_fn(x, w))
    with pytest.raises(ValueError):
        shard_bounds(96, 0, 5)       # 96 columns cannot be cut into 5 shards of multiples of 8
    with pytest.raises(ValueError):
        shard_bounds(96, 2, 2)
    wd = torch.randn(64, n)
    assert torch.equal(torch.cat([shard_down(wd, r, 4) for r in range(4)], dim=1), wd)


def test_single_rank_modules_match_reference_mlp():
    x, w, wd = make_inputs(24, 64, 96, seed=4, with_down=True)
    col = ColumnParallelSwiGLU(w, swiglu_fn=_oracle_fn)
    assert torch.equal(col(x), _oracle_fn(x, w))
    mlp = TensorParallelSwiGLUMLP(w, wd, chunks=3, swiglu_fn=_oracle_fn)
    got = mlp(x.view(2, 12, 64))
    ref = reference_mlp(x, w, wd).view(2, 12, 64)
    assert got.shape == ref.shape
    assert torch.allclose(got.float(), ref.float(), rtol=2e-2, atol=2e-2 * ref.float().abs().max().item())


def test_peer_scatter_mode_argument_rules():
    """reduce="peer_scatter": one chunk only; on one rank there is nothing to exchange and the plain path runs; its
    rows of the result are the ones NCCL's reduce-scatter would leave on the rank."""
    x, w, wd = make_inputs(64, 64, 128, seed=6, with_down=True)
    with pytest.raises(ValueError):
        TensorParallelSwiGLUMLP(w, wd, chunks=2, reduce="peer_scatter", swiglu_fn=_oracle_fn)
    with pytest.raises(ValueError):
        TensorParallelSwiGLUMLP(w, wd, chunks=2, reduce="peer_all_reduce", swiglu_fn=_oracle_fn)
    with pytest.raises(ValueError):
        TensorParallelSwiGLUMLP(w, wd, reduce="all_gather", swiglu_fn=_oracle_fn)
    one = TensorParallelSwiGLUMLP(w, wd, reduce="peer_scatter", swiglu_fn=_oracle_fn)
    ref = reference_mlp(x, w, wd)
    assert torch.allclose(one(x).float(), ref.float(), rtol=2e-2, atol=2e-2 * ref.float().abs().max().item())
    a = TensorParallelSwiGLUMLP(w, wd, rank=1, world=4, reduce="peer_scatter", swiglu_fn=_oracle_fn).owned_rows(64)
    b = TensorParallelSwiGLUMLP(w, wd, rank=1, world=4, reduce="reduce_scatter", swiglu_fn=_oracle_fn).owned_rows(64)
    assert torch.equal(a, b) and torch.equal(a, torch.arange(16, 32))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, chunks, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        x, w, wd = make_inputs(40, 64, 96, seed=9, with_down=True)  # same seed on every rank: X replicated
        # column-parallel op: no collective; gathering the shards reproduces the full output
        y_r = ColumnParallelSwiGLU(w, rank, world, swiglu_fn=_oracle_fn)(x)
        parts = [torch.empty_like(y_r) for _ in range(world)]
        dist.all_gather(parts, y_r)
        full = _oracle_fn(x, w)
        ok_cols = torch.equal(torch.cat(parts, dim=1), full)
        # full MLP: row-parallel down-projection + (chunked, asynchronous) all-reduce; fp32 so the sum is order-free enough
        mlp = TensorParallelSwiGLUMLP(w, wd.float(), rank, world, chunks=chunks,
                                      swiglu_fn=lambda a, b: _oracle_fn(a, b).float())
        z = mlp(x)
        ref = torch.matmul(full.float(), wd.float().t())
        ok_mlp = torch.allclose(z, ref, rtol=1e-4, atol=1e-4)
        # reduce-scatter form: each rank keeps its rows of every slice; a down_fn that writes into out= is used as such
        def down(h, wdown, out=None):
            return torch.matmul(h, wdown.t(), out=out)
        down.supports_out = True
        rs = TensorParallelSwiGLUMLP(w, wd.float(), rank, world, chunks=min(chunks, 2), reduce="reduce_scatter",
                                     swiglu_fn=lambda a, b: _oracle_fn(a, b).float(), down_fn=down)
        z_rs = rs(x)
        rows = rs.owned_rows(x.shape[0])
        ok_mlp = ok_mlp and list(z_rs.shape) == [20, 64] and torch.allclose(z_rs, ref[rows], rtol=1e-4, atol=1e-4)
        gathered = [torch.empty_like(rows) for _ in range(world)]
        dist.all_gather(gathered, rows)
        ok_mlp = ok_mlp and sorted(torch.cat(gathered).tolist()) == list(range(40))  # every row owned exactly once
        try:
            TensorParallelSwiGLUMLP(w, wd.float(), rank, world, chunks=3, reduce="reduce_scatter",
                                    swiglu_fn=lambda a, b: _oracle_fn(a, b).float())(x)  # slices of 14, 14, 12 rows
            ok_mlp = ok_mlp and world == 2  # 14 and 12 are multiples of 2
        except ValueError:
            ok_mlp = ok_mlp and world != 2
        q.put((rank, ok_cols, ok_mlp, list(z.shape)))
    except Exception as exc:  # report instead of leaving the parent to time out
        q.put((rank, False, False, [repr(exc)]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("chunks", [1, 3])
def test_two_gloo_ranks_column_shards_and_row_parallel_allreduce(chunks):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, chunks, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert [r[0] for r in res] == [0, 1]
    for _, ok_cols, ok_mlp, shape in res:
        assert ok_cols and ok_mlp and shape == [40, 64]


def _peer_protocol_rank(rank, world, port, bufs, q, leaver):
    """The host side of the fused reduce-scatter on CPU: shared-memory tensors stand in for symmetric memory, plain
    tensor writes for the epilogue's stores into the owners' slots, a gloo all-reduce of one element for the barrier.
    Same slot arithmetic (``peer_slot_offset``), same order (write, barrier, sum own slots in rank order), same
    alternation of the two destination sets, and ONE barrier per step; ranks are slowed down at different steps so
    that a set being overwritten before its owner has summed it would show up as a wrong result."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    import time

    from magicompiler_b200.sharding import peer_slot_offset

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=6))
    try:
        m, n_in, n_out = 96, 40, 64
        rows = m // world
        token = torch.zeros(1)
        ok, outcome = True, "done"
        for step in range(6):
            if rank == leaver and step == 3:
                outcome = "left"  # between steps: its writes of step 2 are complete, nothing of step 3 has started
                break
            g = torch.Generator().manual_seed(100 + step)
            h = torch.randn(world, m, n_in, generator=g)          # every rank can rebuild every rank's operands
            wd = torch.randn(world, n_out, n_in, generator=g)
            partial = h[rank] @ wd[rank].t()
            dest_set = step & 1
            if (step + rank) % 3 == 0:
                time.sleep(0.05)                                   # skew the ranks against each other
            for o in range(world):                                 # "epilogue stores": row block o into owner o's slot
                off = peer_slot_offset(dest_set, world, rank, rows, n_out)
                bufs[o].view(-1)[off:off + rows * n_out] = partial[o * rows:(o + 1) * rows].reshape(-1)
            try:
                dist.all_reduce(token)                             # the one barrier of the step
            except Exception as exc:
                outcome = "error:" + type(exc).__name__
                break
            acc = torch.zeros(rows, n_out)
            for r in range(world):                                 # own slots, rank order
                off = peer_slot_offset(dest_set, world, r, rows, n_out)
                acc += bufs[rank].view(-1)[off:off + rows * n_out].view(rows, n_out)
            want = sum(h[r] @ wd[r].t() for r in range(world))[rank * rows:(rank + 1) * rows]
            ok &= bool(torch.equal(acc, want))
        q.put((rank, ok, outcome))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


@pytest.mark.parametrize("world,leaver", [(2, -1), (3, -1), (2, 1)])
def test_peer_scatter_host_protocol(world, leaver):
    """Two destination sets and one barrier per step are enough (every step's sums are exact although the ranks run
    skewed); and a rank that leaves between steps ends the survivors' next barrier with an error, not a hang."""
    from magicompiler_b200.sharding import peer_slot_offset

    with pytest.raises(ValueError):
        peer_slot_offset(2, 2, 0, 8, 8)
    m, n_out = 96, 64
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    bufs = [torch.zeros(2 * world * (m // world) * n_out).share_memory_() for _ in range(world)]
    procs = [ctx.Process(target=_peer_protocol_rank, args=(r, world, port, bufs, q, leaver)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=180) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    for rank, ok, outcome in res:
        assert ok, res
        if leaver < 0:
            assert outcome == "done", res
        elif rank == leaver:
            assert outcome == "left", res
        else:
            assert outcome.startswith("error:"), res


def _failing_rank(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime

    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        if rank == 1:
            q.put((rank, "left"))  # leaves between steps, nothing in flight
            return
        t = torch.ones(4)
        try:
            dist.all_reduce(t)
            q.put((rank, "no-error"))
        except Exception as exc:  # the survivor learns of the loss as a host-side error, not a hang
            q.put((rank, "error:" + type(exc).__name__))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_rank_loss_surfaces_as_host_error():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failing_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert res[1] == "left" and res[0].startswith("error:"), res
