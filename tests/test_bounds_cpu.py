from mesh_b200.utils.bounds import (Capability, Cut, Hop, Link, Placed, Topology, Work, b200_node, bounds, port_cut,
                                    tp_ffn_bounds)


def test_bounds_takes_the_largest_of_compute_memory_cut_and_path():
    topo = Topology().add(0, 1, Link("a", 8e9, 1e-6)).add(0, 1, Link("b", 8e9)).add(1, 2, Link("c", 16e9, 2e-6))
    caps = {0: Capability(1e12, 1e11), 1: Capability(1e12, 1e11), 2: Capability(2e12, 2e11)}
    placed = Placed(work={0: 3e12, 2: 1e12}, bytes={1: 5e10},
                    cuts={"left": Cut(frozenset({(0, 1)}), 4e9)}, path=[Hop((0, 1), 2e9), Hop((1, 2), 2e9)])
    b = bounds(Work(4e12, 1e11), placed, topo, caps)
    assert b.compute == 3.0                       # device 0 alone needs 3 s, the aggregate only 1 s
    assert b.memory == 0.5
    assert abs(b.cut["left"] - 2.0) < 1e-12       # 4 GB over 2 x 1 GB/s
    assert abs(b.path - (0.0 + 1.0 + 2e-6 + 1.0)) < 1e-9     # a link without a stated latency counts as 0: the hop takes the least
    assert b.max == 3.0 and b.binding() == "compute"
    assert abs(b.fraction(6.0) - 0.5) < 1e-12
    merged = topo.merging(Topology().add(0, 1, Link("d", 16e9)))
    assert len(merged.between(1, 0)) == 3


def test_b200_node_and_ffn_bounds():
    cap = {"nvlink_p2p_gbs": 770.0, "bf16_tflops_sustained": 1382.0, "hbm_gbs": 6529.0}
    topo, caps = b200_node(8, cap)
    assert len(topo.links) == 28
    c = port_cut(3, 8, 7.7e9)
    placed = Placed(cuts={"p": c})
    assert abs(bounds(Work(0, 0), placed, topo, caps).cut["p"] - 0.01) < 1e-9       # 7.7 GB through a 770 GB/s port
    b1 = tp_ffn_bounds(4096, 4096, 14336, 1, cap)
    b8 = tp_ffn_bounds(4096, 4096, 14336, 8, cap)
    assert b1.binding() == "compute" and abs(b1.max - 3 * 6 * 4096 * 4096 * 14336 / 1382e12) < 1e-6
    assert b8.max < b1.max / 7 and b8.binding() == "compute"
