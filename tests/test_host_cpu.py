"""Host-side logic that needs no GPU: the op's argument checks, the module
mirror of the reference (names, parameter counts, FilterNorm arithmetic), the
harness model, and the batch partition under a 2-rank gloo group."""
import os
import socket
import sys

import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_op_refuses_cpu_tensors():
    from ddfnet_b200 import ddf
    x, cf, sf = torch.randn(1, 2, 6, 6), torch.randn(1, 2, 3, 3), torch.randn(1, 9, 6, 6)
    with pytest.raises(AssertionError, match="CUDA tensor"):
        ddf(x, cf, sf, 3, 1, 1, "mul")


def test_reference_import_path():
    import ddf as alias
    import ddfnet_b200
    assert alias.ddf is ddfnet_b200.ddf and alias.DDFPack is ddfnet_b200.DDFPack
    assert alias.DDFUpPack is ddfnet_b200.DDFUpPack


def test_ddfpack_state_dict_names_and_size():
    from ddfnet_b200 import DDFPack
    m = DDFPack(64, kernel_size=3, stride=2, se_ratio=0.2, kernel_combine="add")
    names = set(m.state_dict())
    assert names == {"spatial_branch.0.weight", "spatial_branch.0.bias",
                     "channel_branch.1.weight", "channel_branch.1.bias",
                     "channel_branch.3.weight", "channel_branch.3.bias",
                     "channel_branch.4.std"}
    assert m.spatial_branch[0].stride == (2, 2)
    assert m.channel_branch[1].out_channels == 12      # int(64 * 0.2)
    assert m.channel_branch[4].std.numel() == 64 * 9


def test_filternorm_arithmetic():
    from ddfnet_b200 import FilterNorm
    torch.manual_seed(0)
    x = torch.randn(2, 9, 5, 4, dtype=torch.float64)
    y = FilterNorm(1, 3, "spatial", "relu")(x)
    gain = 2 ** 0.5 / 3
    assert torch.allclose(y.mean(1), torch.zeros(2, 5, 4, dtype=torch.float64), atol=1e-12)
    assert torch.allclose(y.std(1), torch.full((2, 5, 4), gain, dtype=torch.float64), atol=1e-8)
    fn = FilterNorm(6, 3, "channel", "relu", running_std=True).double()
    z = fn(torch.randn(2, 54, 1, 1, dtype=torch.float64))
    z = (z / fn.std[None, :]).reshape(2, 6, 9)
    assert torch.allclose(z.mean(2), torch.zeros(2, 6, dtype=torch.float64), atol=1e-12)
    assert torch.allclose(z.std(2), torch.ones(2, 6, dtype=torch.float64), atol=1e-8)


def test_harness_model_matches_reference_model_table():
    from ddfnet_b200.resnet import MODELS
    m50 = MODELS["ddf_mul_resnet50"]()
    assert sum(p.numel() for p in m50.parameters()) == 16_843_748   # README.md:21: 16.8 M
    assert len(m50.ddf_layers()) == 16
    assert [l.stride for l in m50.ddf_layers()] == [1, 1, 1, 2, 1, 1, 1, 2, 1, 1, 1, 1, 1, 2, 1, 1]
    m101 = MODELS["ddf_add_resnet101"]()
    assert sum(p.numel() for p in m101.parameters()) == 28_146_912  # README.md:24: 28.1 M
    assert len(m101.ddf_layers()) == 33
    assert all(l.kernel_combine == "add" for l in m101.ddf_layers())
    assert float(m50.layer1[0].bn3.weight.min()) == 1.0             # gamma = 1 everywhere


def test_batch_slice_partition():
    from ddfnet_b200.shard import batch_slice
    for B in (1, 7, 256, 513):
        for N in (1, 2, 4, 8):
            parts = [batch_slice(B, r, N) for r in range(N)]
            assert parts[0][0] == 0 and parts[-1][1] == B
            assert all(a[1] == b[0] for a, b in zip(parts, parts[1:]))
            assert max(h - l for l, h in parts) - min(h - l for l, h in parts) <= 1
    with pytest.raises(ValueError):
        batch_slice(8, 2, 2)


def _rank_main(rank, world, port, batch, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from ddfnet_b200.shard import batch_slice, gather_batch
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    full = torch.arange(batch * 3, dtype=torch.float32).reshape(batch, 3)
    lo, hi = batch_slice(batch, rank, world)
    got = gather_batch(full[lo:hi] * 2, batch)       # each rank "processes" its slice
    q.put((rank, bool(torch.equal(got, full * 2))))
    dist.destroy_process_group()


@pytest.mark.parametrize("batch", [8, 7])
def test_two_rank_partition_and_gather(batch):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, batch, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert sorted(results) == [(0, True), (1, True)]
