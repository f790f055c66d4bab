"""Data-parallel step on 2 CPU ranks (gloo): flat gradient buffer, bucketed all-reduce, per-rank mask streams."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG, REPO


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, scenario: str, out_dir: str) -> None:
    for p in (PKG, REPO):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=20))
    from flash_dropout import random as sd_random
    from flash_dropout.train import BasicNet, FlatGradDataParallel, train_step
    try:
        if scenario == "fail" and rank == 1:
            raise RuntimeError("injected failure on rank 1")       # host-side fault, before any collective
        torch.manual_seed(100 + rank)                               # different init per rank on purpose
        variant = "none" if scenario == "exact" else "blockwise[naive]"
        model = BasicNet(64, 2, 128, 10, dict(p=0.5, variant=variant, block_size=16)).double()
        dp = FlatGradDataParallel(model, bucket_bytes=32 << 10)     # several buckets
        assert len(dp.buckets) >= 2
        g = torch.Generator().manual_seed(7)
        x_all, y_all = torch.rand(16, 64, generator=g).double(), torch.randint(0, 10, (16,), generator=g)
        x, y = x_all[rank * 8:(rank + 1) * 8], y_all[rank * 8:(rank + 1) * 8]
        opt = torch.optim.SGD(model.parameters(), lr=0.1)
        before = [p.detach().clone() for p in model.parameters()]
        loss = train_step(model, dp, opt, lambda m: torch.nn.functional.cross_entropy(m(x), y))
        assert dp.grads_are_views()
        torch.save({"before": before, "after": [p.detach().clone() for p in model.parameters()],
                    "grad": dp.flat_grad.clone(), "loss": loss, "x": x_all, "y": y_all,
                    "rng": sd_random.get_state()}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


def _run(scenario: str, tmp_path) -> list:
    port = _free_port()
    mp.spawn(_worker, args=(2, port, scenario, str(tmp_path)), nprocs=2, join=True)
    return [torch.load(os.path.join(tmp_path, f"rank{r}.pt"), weights_only=False) for r in range(2)]


def test_two_ranks_equal_one_big_batch(tmp_path):
    r0, r1 = _run("exact", tmp_path)
    # parameters were broadcast from rank 0 and stay identical after the step
    for a, b in zip(r0["before"], r1["before"]):
        assert torch.equal(a, b)
    for a, b in zip(r0["after"], r1["after"]):
        assert torch.equal(a, b)
    assert torch.equal(r0["grad"], r1["grad"])
    # mean of the two half-batch gradients == gradient of the whole batch on one process
    sys.path.insert(0, PKG)
    from flash_dropout.train import BasicNet
    ref = BasicNet(64, 2, 128, 10, dict(p=0.5, variant="none", block_size=128)).double()
    with torch.no_grad():
        for p, b in zip(ref.parameters(), r0["before"]):
            p.copy_(b)
    torch.nn.functional.cross_entropy(ref(r0["x"]), r0["y"]).backward()
    want = torch.cat([p.grad.flatten() for p in reversed(list(ref.parameters()))])
    torch.testing.assert_close(r0["grad"], want, rtol=1e-9, atol=1e-12)


def test_ranks_draw_different_masks(tmp_path):
    r0, r1 = _run("masks", tmp_path)
    assert r0["rng"]["subsequence"] == 0 and r1["rng"]["subsequence"] == 1
    for a, b in zip(r0["after"], r1["after"]):       # still one model
        assert torch.equal(a, b)
    assert r0["loss"].item() != r1["loss"].item()


def test_failed_rank_is_reported(tmp_path):
    with pytest.raises(Exception, match="injected failure on rank 1|terminated|exit"):
        _run("fail", tmp_path)
