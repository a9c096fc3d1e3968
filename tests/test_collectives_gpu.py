"""Every collective wrapper on a world of one (the reference's VoidCommunicator,
src/distributed/common/void_communicator.cc): a reduction over one rank is a copy, a gather
returns its input, whatever the reduction, the dtype or the rank_list.  Answers follow
tests/python/distributed/test_collective_communication.py with size 1."""
import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.float64, torch.int64, torch.int8, torch.uint8]


@pytest.fixture()
def world_of_one():
    from raf_b200 import distributed as dist

    dist.set_communicator(None)
    comm = dist.get_communicator()
    assert (comm.size, comm.rank) == (1, 0)
    yield dist
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", DTYPES)
def test_allreduce_allgather_reduce_scatter_copy(world_of_one, dtype):
    dist = world_of_one
    s = dist.comm_stream()
    base = torch.arange(24, device="cuda").reshape(6, 4).to(dtype)
    with torch.cuda.stream(s):
        for comp in ("sum", "prod", "min", "max", "avg"):
            if comp == "avg" and not dtype.is_floating_point:
                continue
            x = base.clone()
            assert dist.allreduce(x, comp, stream=s) is x
            assert torch.equal(x, base)
            y = dist.reduce_scatter(base.clone(), comp, stream=s)
            assert y.shape == base.shape and torch.equal(y, base)
        pair = dist.allreduce([base.clone(), base[:1].clone()], "sum", stream=s)
        assert torch.equal(pair[0], base) and torch.equal(pair[1], base[:1])
        for axis in (0, 1):
            y = dist.allgather(base, axis, stream=s)
            assert y.shape == base.shape and torch.equal(y, base)
        ys = dist.allgather([base, base[:2]], 0, stream=s)
        assert torch.equal(ys[0], base) and torch.equal(ys[1], base[:2])
    s.synchronize()


def test_group_forms_and_rank_list(world_of_one):
    dist = world_of_one
    s = dist.comm_stream()
    xs = [torch.randn(k, 3, device="cuda") for k in (1, 2, 5)]
    with torch.cuda.stream(s):
        ys = dist.group_reduce_scatter([x.clone() for x in xs], "sum", stream=s)
        outs = [torch.zeros_like(x) for x in xs]
        dist.group_allgather(xs, 0, outs, stream=s)
        # a rank_list that names this rank alone, and one that does not name it at all
        a = dist.allreduce(xs[0].clone(), "sum", rank_list=[[0]], stream=s)
        b = dist.allgather(xs[1], 0, rank_list=[[0]], stream=s)
    s.synchronize()
    for x, y, o in zip(xs, ys, outs):
        assert torch.equal(x, y) and torch.equal(x, o)
    assert torch.equal(a, xs[0]) and torch.equal(b, xs[1])
    with pytest.raises(Exception):
        dist.allreduce(xs[0].clone(), "sum", rank_list=[[0, 1]])  # rank 1 does not exist
    with pytest.raises(NotImplementedError):
        dist.group_allgather(xs, 1, outs)
    with pytest.raises(Exception):
        dist.allreduce(xs[0].clone(), "xor")


def test_streams_by_tag_are_stable(world_of_one):
    dist = world_of_one
    a, b = dist.get_stream("communicate"), dist.get_stream("communicate")
    assert a.cuda_stream == b.cuda_stream != 0
    assert dist.get_stream("compute").cuda_stream != a.cuda_stream
    assert dist.get_stream("fuse", 1).cuda_stream != dist.get_stream("fuse", 0).cuda_stream
    with pytest.raises(Exception):
        dist.get_stream(99)
