"""The scattered plain GEMM (row blocks of C leave the epilogue into per-owner buffers) and the slot sum that finishes
a reduce-scatter, through the C ABI on one GPU: here every "owner" buffer lives on the same device, which exercises
the same kernel path as buffers in peers' memory."""
import pytest
import torch

import magicompiler_b200 as mb
from magicompiler_b200 import ops

pytestmark = pytest.mark.gpu


def _rand(rows, cols, scale, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(rows, cols, generator=g, device="cuda") * scale).to(torch.bfloat16)


@pytest.mark.parametrize("world,rows,n,k", [(1, 512, 512, 256), (2, 256, 512, 1024), (4, 96, 128, 512),
                                            (8, 32, 1024, 320), (3, 1024, 2048, 512), (2, 160, 768, 192),
                                            (8, 2048, 8192, 448)])
@pytest.mark.parametrize("wide", [1, 0])
def test_scattered_gemm_equals_gemm_nt_row_blocks(world, rows, n, k, wide):
    """Both store-box widths (64 columns where the tile allows, 32 otherwise) against the plain GEMM, bit for bit."""
    from magicompiler_b200 import _loader

    a, b = _rand(world * rows, k, 1.0, 1), _rand(n, k, 0.05, 2)
    want = mb.gemm_nt(a, b)
    prev = _loader.set_tuning("scatter_wide", wide)
    try:
        _scatter_and_compare(a, b, want, world, rows, n)
    finally:
        _loader.set_tuning("scatter_wide", prev)
    assert mb.device_status(0)["code"] == 0


def _scatter_and_compare(a, b, want, world, rows, n):
    for dest_set in (0, 1):
        bufs = [torch.full((rows + 2, n), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
        ops.scatter_setup(dest_set, [t[1:].data_ptr() for t in bufs], rows, n)  # one guard row on either side
        ops.gemm_nt_scatter(a, b, dest_set)
        torch.cuda.synchronize()
        for o, t in enumerate(bufs):
            assert torch.equal(t[1:-1], want[o * rows:(o + 1) * rows]), (dest_set, o)
            assert torch.isnan(t[0]).all() and torch.isnan(t[-1]).all(), "rows outside the owner's block were written"


def test_scattered_gemm_with_padded_rows_of_the_destination():
    world, rows, n, k, ldc = 2, 128, 256, 256, 384
    a, b = _rand(world * rows, k, 1.0, 3), _rand(n, k, 0.05, 4)
    bufs = [torch.full((rows, ldc), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(world)]
    ops.scatter_setup(0, [t.data_ptr() for t in bufs], rows, n, ldc=ldc)
    ops.gemm_nt_scatter(a, b, 0)
    want = mb.gemm_nt(a, b)
    for o, t in enumerate(bufs):
        assert torch.equal(t[:, :n], want[o * rows:(o + 1) * rows])
        assert torch.isnan(t[:, n:]).all()


def test_scatter_argument_errors():
    buf = torch.empty(256, 512, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ValueError):
        ops.scatter_setup(2, [buf.data_ptr()], 256, 512)          # only sets 0 and 1 exist
    with pytest.raises(ValueError):
        ops.scatter_setup(0, [buf.data_ptr()], 100, 512)          # rows per owner must be a multiple of 32
    with pytest.raises(ValueError):
        ops.scatter_setup(0, [buf.data_ptr()], 256, 96)           # N must be a multiple of 64
    with pytest.raises(ValueError):
        ops.scatter_setup(0, [buf.data_ptr()] * 9, 32, 512)       # at most 8 owners
    ops.scatter_setup(0, [buf.data_ptr()], 256, 512)
    a, b = _rand(512, 128, 1.0, 5), _rand(512, 128, 0.05, 6)
    with pytest.raises(ValueError):
        ops.gemm_nt_scatter(a, b, 0)                              # set 0 was set up for 256 rows, not 512
    with pytest.raises(ValueError):
        ops.gemm_nt_scatter(a[:256], b[:256], 0)                  # ... and for N = 512


@pytest.mark.parametrize("slots,shape", [(1, (64, 64)), (2, (100, 264)), (8, (2048, 1024)), (5, (3, 8))])
def test_sum_slots_adds_in_fp32_in_slot_order(slots, shape):
    src = _rand(slots * shape[0], shape[1], 1.0, 7).view(slots, *shape).contiguous()
    acc = torch.zeros(shape, dtype=torch.float32, device="cuda")
    for s in range(slots):
        acc += src[s].float()
    assert torch.equal(ops.sum_slots(src), acc.to(torch.bfloat16))
    out = torch.empty(shape, dtype=torch.bfloat16, device="cuda")
    assert ops.sum_slots(src, out) is out and torch.equal(out, acc.to(torch.bfloat16))


def test_sum_slots_bcast_writes_the_same_sums_everywhere():
    slots, shape = 4, (256, 512)
    src = _rand(slots * shape[0], shape[1], 1.0, 8).view(slots, *shape).contiguous()
    want = ops.sum_slots(src)
    outs = [torch.full((shape[0] + 2, shape[1]), float("nan"), dtype=torch.bfloat16, device="cuda") for _ in range(8)]
    ops.sum_slots_bcast(src, [t[1:].data_ptr() for t in outs])
    torch.cuda.synchronize()
    for t in outs:
        assert torch.equal(t[1:-1], want) and torch.isnan(t[0]).all() and torch.isnan(t[-1]).all()
    with pytest.raises(ValueError):
        ops.sum_slots_bcast(src, [t.data_ptr() for t in outs] + [outs[0].data_ptr()])  # nine destinations
