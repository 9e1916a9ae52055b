"""Explicit programs: parts, verbs and calls declared once, started, invoked several times (gloo ranks)."""
import torch


def _rank(rank, world, rdv):
    from mesh_b200.distributed.program import Mesh
    m = Mesh(device="cpu", copies=2)
    assert (m.rank, m.size) == (rank, world)
    # a tensor-parallel layer written by hand: x lives on rank 0, every rank holds a slice of W
    x = m.tensor(on=0, sections=[(4, 8)])[0]
    w = [m.constant(r, torch.full((8, 3), float(r + 1))) for r in range(world)]
    xs = m.broadcast(x, to=range(world))
    again = m.broadcast(x, to=range(world))
    assert [p.ident for p in xs] == [p.ident for p in again]                 # the second delivery shares the first receive
    ys = m.tensor(on=list(range(world)), sections=[(4, 3)] * world)
    m.map(lambda a, b: a @ b, [[xs[r], w[r]] for r in range(world)], [[ys[r]] for r in range(world)], workers=range(world))
    total = m.reduce(ys, to=0, op="sum")
    everywhere = m.all_reduce(ys, op="max")
    gathered = m.all_gather(ys)
    parts = [m.tensor(on=j, sections=[(2,)] * world) for j in range(world)]   # parts[j][i]: rank j's piece for rank i
    exchanged = m.all_to_all(parts)
    owned = m.reduce_scatter(parts, to=list(range(world)))
    m.sync_on_remote_fill([xs[r] for r in range(1, world)])
    m.start(wait_s=20.0)
    for i in range(3):                                                     # three invocations over two storage sets
        inv = m.invocation(i)
        if rank == 0:
            inv.part(x).fill_(float(i + 1))
        for i_to in range(world):
            inv.part(parts[rank][i_to]).fill_(float(10 * rank + i_to + i))
        inv.submit()
        assert m.result(i) == 0
        xv = torch.full((4, 8), float(i + 1))
        if rank == 0:
            want = sum(xv @ torch.full((8, 3), float(r + 1)) for r in range(world))
            assert torch.equal(inv.part(total), want)
        assert torch.equal(inv.part(everywhere[rank]), xv @ torch.full((8, 3), float(world)))
        for r in range(world):
            assert torch.equal(inv.part(gathered[rank][r]), xv @ torch.full((8, 3), float(r + 1)))
        for j in range(world):
            assert torch.equal(inv.part(exchanged[rank][j]), torch.full((2,), float(10 * j + rank + i)))
        assert torch.equal(inv.part(owned[rank]), torch.full((2,), float(sum(10 * j + rank + i for j in range(world)))))
    assert m.result(7) is None
    m.cancel()
    m.invocation(3).submit()
    from mesh_b200.runtime.rendezvous import ECANCELED
    assert m.result(3) == ECANCELED
    try:
        m.tensor(on=0, sections=[(1,)])
        raise AssertionError("declared after start")
    except RuntimeError:
        pass


def test_explicit_program_two_and_three_ranks():
    from mesh_b200.utils.launch import spawn_ranks
    for world in (2, 3):
        spawn_ranks(_rank, world, init_pg="gloo")


def test_call_refuses_parts_on_other_ranks():
    import pytest
    from mesh_b200.distributed.program import Mesh
    m = Mesh(rank=0, size=2)
    a, b = m.tensor(on=[0, 1], sections=[(2,), (2,)])
    with pytest.raises(ValueError):
        m.call(lambda u, v: u + v, [a, b], [a], on=0)
    with pytest.raises(ValueError):
        m.reduce([a, b], to=0, op="mean")


def _routed_rank(rank, world, rdv):
    """A delivery forced through a relay: 0 -> 2 goes by way of 1; the relay's copy is an ordinary part (a later
    delivery of the same part to the relay shares it), and the numbers arrive unchanged."""
    from mesh_b200.distributed.program import Mesh, Placement
    m = Mesh(device="cpu", copies=2, placement=Placement(routes={(0, 2): (1,)}))
    x = m.tensor(on=0, sections=[(5,)])[0]
    far = m.send(x, to=2)
    near = m.send(x, to=1)                      # the relay already holds it
    assert far.rank == 2 and near.rank == 1
    moves = [s for s in m.steps if s[0] == "move"]
    assert [[(a.rank, b.rank) for a, b in mv] for _, mv in moves] == [[(0, 1)], [(1, 2)]]
    direct = m.send(m.tensor(on=2, sections=[(5,)])[0], to=0)        # no route stated for (2, 0): the direct link
    assert [(a.rank, b.rank) for a, b in m.steps[-1][1]] == [(2, 0)]
    m.start(wait_s=20.0)
    for i in range(2):
        inv = m.invocation(i)
        if rank == 0:
            inv.part(x).copy_(torch.arange(5.0) + i)
        inv.submit()
        assert m.result(i) == 0
        if rank in (1, 2):
            assert torch.equal(inv.part(near if rank == 1 else far), torch.arange(5.0) + i)
    assert direct.rank == 0


def test_forced_relay_routes():
    from mesh_b200.utils.launch import spawn_ranks
    spawn_ranks(_routed_rank, 3, init_pg="gloo")
