import pytest

from elf_b200 import sequential_signatures
from elf_b200.registry import SCHEDULERS
from elf_b200.scheduling import add_comms
from elf_b200.scheduling.comm_scheduling import DirectedGraph, schedule_to_graph, topological_sort


def test_directed_graph_basic():
    g = DirectedGraph(3)
    g.add_edge(0, 1)
    g.add_edge(1, 2)
    assert g.has_edge(0, 1) and g.has_edge(1, 2) and not g.has_edge(0, 2)
    assert g.get_out_degree(0) == 1 and g.get_in_degree(1) == 1
    assert g.get_successors(0) == [1] and g.get_predecessors(2) == [1]
    g.remove_edge(1, 2)
    assert not g.has_edge(1, 2) and g.get_out_degree(1) == 0 and g.get_in_degree(2) == 0
    with pytest.raises(ValueError):
        g.add_edge(0, 0)
    with pytest.raises(ValueError):
        g.add_edge(0, 7)
    with pytest.raises(ValueError):
        DirectedGraph(0)


def test_cycle_detection_ignores_two_cycles():
    g1 = DirectedGraph(2)
    g1.add_edge(0, 1)
    g1.add_edge(1, 0)
    assert not g1.has_cycle()
    assert g1.has_bidirectional_edge(0, 1) and not g1.has_unidirectional_edge(0, 1)
    g2 = DirectedGraph(3)
    g2.add_edge(0, 1)
    g2.add_edge(1, 2)
    g2.add_edge(2, 0)
    assert g2.has_cycle()
    g3 = DirectedGraph(4)
    for a, b in [(0, 1), (1, 2), (0, 2), (2, 3)]:
        g3.add_edge(a, b)
    assert not g3.has_cycle()


def test_schedule_graph_is_acyclic_and_order_respects_it():
    placement = [0, 1, 2]
    sched = add_comms(SCHEDULERS["1f1b"](placement, 4), sequential_signatures(placement))
    graph = schedule_to_graph(sched)
    assert not graph.has_cycle()
    order = topological_sort(list(sched))
    index = {id(op): i for i, op in enumerate(sched)}
    pos = {index[id(op)]: i for i, op in enumerate(order)}
    for src in range(graph.num_nodes):
        for dst in graph.get_successors(src):  # src depends on dst
            if not graph.has_bidirectional_edge(src, dst):
                assert pos[dst] < pos[src]
