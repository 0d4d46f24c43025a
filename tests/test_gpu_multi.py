"""Two GPUs, one process each, NCCL: the column-sharded op and the tensor-parallel MLP against the unsharded
computation on one GPU.  Skipped on boxes with a single GPU."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, q):
    import torch.distributed as dist

    import magicompiler_b200 as mb
    from magicompiler_b200.sharding import reference_mlp
    from oracle import make_inputs

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        M, K, N = 1024, 512, 2048
        x, w, wd = make_inputs(M, K, N, seed=21, with_down=True)
        xd = x.to(dev)
        # column shards: no collective for the op; gathered shards are the unsharded result bit for bit
        y_r = mb.ColumnParallelSwiGLU(w, rank, world).to(dev)(xd)
        parts = [torch.empty_like(y_r) for _ in range(world)]
        dist.all_gather(parts, y_r)
        full = mb.gemm_swiglu(xd, w.to(dev))
        ok_cols = torch.equal(torch.cat(parts, dim=1), full)
        # full MLP, chunked all-reduce overlapping the next chunk's GEMMs
        ok_mlp = True
        ref = reference_mlp(xd, w.to(dev), wd.to(dev)).float()
        for chunks in (1, 4):
            z = mb.TensorParallelSwiGLUMLP(w, wd, rank, world, chunks=chunks).to(dev)(xd).float()
            ok_mlp &= bool(torch.allclose(z, ref, rtol=3e-2, atol=3e-2 * ref.abs().max().item()))
            # own down projection written in place, reduce-scatter instead of all-reduce: this rank's rows of the sum
            rs = mb.TensorParallelSwiGLUMLP(w, wd, rank, world, chunks=chunks, down_fn=mb.gemm_nt_out,
                                            reduce="reduce_scatter").to(dev)
            z_rs = rs(xd).float()
            rows = rs.owned_rows(M).to(dev)
            ok_mlp &= tuple(z_rs.shape) == (M // world, K)
            ok_mlp &= bool(torch.allclose(z_rs, ref[rows], rtol=3e-2, atol=3e-2 * ref.abs().max().item()))
        torch.cuda.synchronize()
        q.put((rank, ok_cols, ok_mlp, mb.device_status(rank)["code"]))
    except Exception as exc:  # report instead of leaving the parent to time out
        q.put((rank, False, False, repr(exc)))
    finally:
        dist.destroy_process_group()


def _rank_peer_scatter(rank, world, port, q):
    """The row-parallel down projection whose epilogue stores each row block into its owner's memory, three steps in a
    row (both destination sets, and the first one re-used): against NCCL-free expectations built from all-gathered
    partial products (bit for bit) and against the unsharded MLP."""
    import torch.distributed as dist

    import magicompiler_b200 as mb
    from magicompiler_b200.sharding import reference_mlp
    from oracle import make_inputs

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        M, K, N = 1024, 512, 2048
        _, w, wd = make_inputs(M, K, N, seed=22, with_down=True)
        mlp = mb.TensorParallelSwiGLUMLP(w, wd, rank, world, reduce="peer_scatter").to(dev)
        rows = mlp.owned_rows(M).to(dev)
        ok_exact, ok_ref = True, True
        for step in range(3):
            x, _, _ = make_inputs(M, K, N, seed=30 + step, with_down=True)
            xd = x.to(dev)
            z = mlp(xd)
            partial = mb.gemm_nt(mlp.gate_up(xd), mlp.w_down)             # this rank's partial product, whole
            parts = [torch.empty_like(partial) for _ in range(world)]
            dist.all_gather(parts, partial)
            acc = torch.zeros(M, K, dtype=torch.float32, device=dev)
            for p in parts:                                                # rank order, fp32, one rounding
                acc += p.float()
            ok_exact &= bool(torch.equal(z, acc.to(torch.bfloat16)[rows]))
            ref = reference_mlp(xd, w.to(dev), wd.to(dev)).float()
            ok_ref &= tuple(z.shape) == (M // world, K)
            ok_ref &= bool(torch.allclose(z.float(), ref[rows], rtol=3e-2, atol=3e-2 * ref.abs().max().item()))
        # ... and continued to an all-reduce: every rank's sum kernel stores its rows into every rank's result
        full = mb.TensorParallelSwiGLUMLP(w, wd, rank, world, reduce="peer_all_reduce").to(dev)
        for step in range(3):
            x, _, _ = make_inputs(M, K, N, seed=40 + step, with_down=True)
            xd = x.to(dev)
            z = full(xd).clone()
            partial = mb.gemm_nt(full.gate_up(xd), full.w_down)
            parts = [torch.empty_like(partial) for _ in range(world)]
            dist.all_gather(parts, partial)
            acc = torch.zeros(M, K, dtype=torch.float32, device=dev)
            for p in parts:
                acc += p.float()
            ok_exact &= tuple(z.shape) == (M, K) and bool(torch.equal(z, acc.to(torch.bfloat16)))
        torch.cuda.synchronize()
        q.put((rank, ok_exact, ok_ref, mb.device_status(rank)["code"]))
    except Exception as exc:  # report instead of leaving the parent to time out
        q.put((rank, False, False, repr(exc)))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_down_projection_scattered_by_its_epilogue():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank_peer_scatter, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    for rank, ok_exact, ok_ref, status in res:
        assert ok_exact and ok_ref and status == 0, res


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_column_shards_and_tensor_parallel_mlp():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=300) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    for rank, ok_cols, ok_mlp, status in res:
        assert ok_cols and ok_mlp and status == 0, res
