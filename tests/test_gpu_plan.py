"""Block-plan kernel vs the CPU oracle: masks and every kept-block index list, bit-exact."""
import numpy as np
import pytest
import torch

from oracle import philox_mask as pm

pytestmark = pytest.mark.gpu

CASES = [  # (M, K, block_size, p, seed, offset)
    (1024, 1024, 128, 0.5, 0, 0),            # 8 x 8 grid (the 1024^3 CPU case)
    (4096, 4096, 128, 0.5, 0, 5),            # config 2 grid (32 x 32)
    (4096, 4096, 128, 0.0, 1, 0),
    (4096, 4096, 128, 0.999, 1, 0),          # whole rows dropped
    (262144, 576, 128, 0.5, 3, 1),           # config 3 im2col grid (2048 x 5, ragged K)
    (512, 1024, 128, 0.5, 4, 2),             # config 4 (4 x 8)
    (16384, 384, 128, 0.2, 5, 3), (16384, 1536, 128, 0.2, 5, 4),   # config 5 (128 x 3, 128 x 12)
    (128, 128, 128, 0.5, 6, 0), (384, 640, 128, 0.3, 7, 2**40 + 9),
    (1024, 2048, 256, 0.5, 8, 0), (1000, 1500, 512, 0.4, 9, 1),    # logical blocks larger than a tile
    (300, 392, 128, 0.4, 2**63 + 12345, 0),
    # beyond the 32-column / 3072-row fast path: the general kernel (wide, and tall)
    (1024, 8192, 128, 0.5, 10, 0), (640, 5120, 128, 0.3, 11, 1), (524288, 384, 128, 0.5, 12, 0),
    (393216, 4096, 128, 0.5, 13, 2),      # exactly 3072 rows x 32 columns: largest grid of the fast path
    # thousands of tiles: the cluster kernel (row slices that do not divide evenly; replicated logical blocks)
    (33024, 2048, 128, 0.5, 14, 1), (65536, 2048, 256, 0.3, 15, 0), (131072, 4096, 128, 0.9, 16, 3),
    (1048576, 512, 128, 0.5, 17, 0),      # 8192 x 4: slices of 1024 rows
    (3276800, 128, 128, 0.5, 18, 0),      # 25600 rows: past the cluster kernel's 24576, the general kernel again
]


def _check_plan(plan, mask, M, K, bs):
    tiles = pm.expand_to_tiles(mask, M, K, bs)
    R, C = tiles.shape
    assert (plan.R, plan.C) == (R, C)
    assert np.array_equal(plan.tile_mask.cpu().numpy().astype(bool), tiles)
    hdr = plan.header.cpu().numpy()
    kept = pm.kept_pairs(tiles)
    nnz = len(kept)
    assert hdr[0] == nnz and hdr[2] == R * C - nnz and hdr[3] == R and hdr[4] == C
    assert np.array_equal(plan.kept_pairs.cpu().numpy()[:nnz], kept)
    assert np.array_equal(plan.drop_pairs.cpu().numpy()[:R * C - nnz], np.argwhere(tiles).astype(np.int32))
    row_ptr, col_idx = pm.csr(tiles)
    col_ptr, row_idx = pm.csc(tiles)
    assert np.array_equal(plan.row_ptr.cpu().numpy(), row_ptr)
    assert np.array_equal(plan.col_idx.cpu().numpy()[:nnz], col_idx)
    assert np.array_equal(plan.col_ptr.cpu().numpy(), col_ptr)
    assert np.array_equal(plan.row_idx.cpu().numpy()[:nnz], row_idx)
    items = pm.sdd_items(tiles)
    assert hdr[1] == len(items)
    assert np.array_equal(plan.sdd_items.cpu().numpy()[:len(items)], items)
    assert hdr[5] == (np.diff(row_ptr).max() if R else 0) and hdr[6] == np.diff(col_ptr).max()
    for order, counts in ((plan.row_order, np.diff(row_ptr)), (plan.col_order, np.diff(col_ptr))):
        o = order.cpu().numpy()
        assert sorted(o.tolist()) == list(range(len(counts)))
        assert (np.diff(counts[o]) <= 0).all()          # heaviest first


@pytest.mark.parametrize("M,K,bs,p,seed,offset", CASES)
def test_plan_from_seed_bit_exact(built_lib, M, K, bs, p, seed, offset):
    from flash_dropout.cuda.binding_gemm import BlockPlan
    plan = BlockPlan.from_seed(M, K, bs, p, seed, offset, torch.device("cuda:0"))
    torch.cuda.synchronize()
    want = pm.block_mask(M, K, bs, p, seed % 2**64, offset)
    assert np.array_equal(plan.mask.cpu().numpy(), want)
    _check_plan(plan, want, M, K, bs)


@pytest.mark.parametrize("R,C,p", [(8, 8, 0.5), (32, 32, 0.1), (3, 5, 0.5), (2048, 5, 0.5), (1, 7, 0.9), (5, 1, 0.2)])
def test_plan_from_mask_any_strides(built_lib, R, C, p):
    from flash_dropout.cuda.binding_gemm import BlockPlan
    g = torch.Generator().manual_seed(R * 131 + C)
    mask = torch.rand(R, C, generator=g) < p
    dev = torch.device("cuda:0")
    for m in (mask.to(dev), mask.T.contiguous().to(dev).T):      # row-major and column-major masks
        plan = BlockPlan.from_mask(m, R * 128, C * 128, 128)
        torch.cuda.synchronize()
        _check_plan(plan, mask.numpy(), R * 128, C * 128, 128)
    planT = BlockPlan.from_mask(mask.to(dev).T, C * 128, R * 128, 128)   # mask.T as the reference passes for dW
    torch.cuda.synchronize()
    _check_plan(planT, mask.numpy().T, C * 128, R * 128, 128)


def test_docstring_mask_on_device(built_lib, golden):
    from flash_dropout.cuda.binding_gemm import BlockPlan
    from flash_dropout.functional.utils import mask_to_increment_table
    mask = torch.from_numpy(golden["inc0_mask"]).cuda()
    plan = BlockPlan.from_mask(mask, 3 * 128, 5 * 128, 128)
    assert plan.col_idx.cpu()[:7].tolist() == [0, 3, 1, 2, 4, 0, 2]
    table, row_indices, row_widths = mask_to_increment_table(mask, 16)
    assert table.cpu().tolist() == [0, 48, 16, 16, 32, 0, 32]
    assert row_indices.cpu().tolist() == [0, 2, 5] and row_widths.cpu().tolist() == [2, 3, 2]
    assert plan.row_ptr.cpu().tolist() == [0, 2, 5, 7]


def test_functional_mask_uses_device_draw(built_lib):
    from flash_dropout import random as sd_random
    from flash_dropout.functional.utils import blockwise_dropout_mask
    sd_random.manual_seed(42, subsequence=0)
    x = torch.empty(1024, 2048, device="cuda", dtype=torch.float16)
    m0 = blockwise_dropout_mask(x, 128, 0.5)
    m1 = blockwise_dropout_mask(x, 128, 0.5)
    assert m0.dtype == torch.bool and tuple(m0.shape) == (8, 16)
    assert np.array_equal(m0.cpu().numpy(), pm.block_mask(1024, 2048, 128, 0.5, 42, 0))
    assert np.array_equal(m1.cpu().numpy(), pm.block_mask(1024, 2048, 128, 0.5, 42, 1))
    sd_random.follow_torch_seed()


def test_device_counter_supplies_the_offset(built_lib):
    """Offset = base + counter read on the device; each launch increments the counter (CUDA-graph friendly)."""
    from flash_dropout.cuda.binding_gemm import BlockPlan
    dev = torch.device("cuda:0")
    counter = torch.full((1,), 5, dtype=torch.int64, device=dev)
    base = 3 << 40
    for i in range(3):
        plan = BlockPlan.from_device_counter(1024, 2048, 128, 0.5, 77, base, counter, dev)
        torch.cuda.synchronize()
        assert counter.item() == 6 + i
        assert np.array_equal(plan.mask.cpu().numpy(), pm.block_mask(1024, 2048, 128, 0.5, 77, base + 5 + i))


def test_plan_batch_equals_single_launches(built_lib):
    """One launch for several plans: masks and every list are what the single launches give, pass after pass."""
    from flash_dropout import random as sd_random
    from flash_dropout.cuda.binding_gemm import BlockPlan, PlanBatch
    dev = torch.device("cuda:0")
    shapes = [(512, 784, 128, 0.5), (512, 1024, 128, 0.5), (16384, 384, 128, 0.2), (16384, 1536, 256, 0.2), (300, 136, 128, 0.9)]
    sd_random.manual_seed(91, subsequence=2)
    sd_random.enable_device_counter(dev)
    counter = sd_random.device_counter(dev)
    seed, base = sd_random.seed_and_base()
    batch = PlanBatch(dev)
    side = torch.cuda.Stream(dev)
    drawn = 0
    try:
        for step in range(4):
            PlanBatch.active = batch
            if not batch.recording:
                # on the current stream, and (last pass) on a stream of its own that the first draw picks up again
                batch.launch(side if step == 3 else None)
            plans = [BlockPlan.draw(M, K, bs, p, dev) for M, K, bs, p in shapes]
            PlanBatch.active = None
            if batch.recording:
                batch.finalize()
            torch.cuda.synchronize()
            for i, ((M, K, bs, p), plan) in enumerate(zip(shapes, plans)):
                want = pm.block_mask(M, K, bs, p, seed, base + drawn + i)
                assert np.array_equal(plan.mask.cpu().numpy(), want), (step, i)
                ref = BlockPlan.from_mask(torch.from_numpy(want).to(dev), M, K, bs)
                nnz, n_items, n_drop = (int(v) for v in ref.header[:3].tolist())
                assert torch.equal(plan.header[:7], ref.header[:7]), (step, i)
                for name, n in (("row_ptr", None), ("col_ptr", None), ("col_idx", nnz), ("row_idx", nnz),
                                ("kept_pairs", nnz), ("drop_pairs", n_drop), ("sdd_items", n_items), ("tile_mask", None)):
                    assert torch.equal(getattr(plan, name)[:n], getattr(ref, name)[:n]), (step, i, name)
                # the heaviest-first orders are permutations sorted by kept count (ties in any order)
                keep = (plan.tile_mask == 0)
                for order, counts in ((plan.row_order, keep.sum(1)), (plan.col_order, keep.sum(0))):
                    o = order.long()
                    assert torch.equal(torch.sort(o).values, torch.arange(o.numel(), device=dev)), (step, i)
                    assert (counts[o][:-1] >= counts[o][1:]).all(), (step, i)
            drawn += len(shapes)
            assert counter.item() == drawn
    finally:
        PlanBatch.active = None
        sd_random.disable_device_counter()
        sd_random.follow_torch_seed()


def test_functional_mask_is_fresh_on_graph_replay(built_lib):
    """``blockwise_dropout_mask`` inside a captured region reads the device-side counter: every replay of the graph
    draws the next mask of the stream, not the one seen at capture."""
    from flash_dropout import random as sd_random
    from flash_dropout.functional.utils import blockwise_dropout_mask
    dev = torch.device("cuda:0")
    sd_random.manual_seed(5, subsequence=1)
    sd_random.enable_device_counter(dev)
    seed, base = sd_random.seed_and_base()
    try:
        x = torch.empty(1024, 2048, device=dev, dtype=torch.float16)
        out = torch.empty(8, 16, dtype=torch.bool, device=dev)
        side = torch.cuda.Stream(dev)
        side.wait_stream(torch.cuda.current_stream(dev))
        with torch.cuda.stream(side):
            out.copy_(blockwise_dropout_mask(x, 128, 0.5))                   # offset base + 0
        torch.cuda.current_stream(dev).wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out.copy_(blockwise_dropout_mask(x, 128, 0.5))
        for i in range(3):
            graph.replay()
            torch.cuda.synchronize()
            assert np.array_equal(out.cpu().numpy(), pm.block_mask(1024, 2048, 128, 0.5, seed, base + 1 + i)), i
    finally:
        sd_random.disable_device_counter()
        sd_random.follow_torch_seed()
