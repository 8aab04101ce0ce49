"""The schedule search (minimum cost sub-hypergraph, branch and bound) on hand built graphs, without a GPU.
The first three cases restate the reference's own tests of its hyper-path search
(test/compiler/algorithm/shortest_dag_hyperpath.cpp); the rest cover what this backend adds: edges with two
destinations, parallel edges (one per kernel variant), the 1 hour sentinel and the dispatch count pre-filter."""
import itertools
import random

import pytest

from denox_b200 import lib

HOUR_MS = 3600000.0


def fire(n_nodes, edges, inputs, order):
    avail = set(inputs)
    for e in order:
        s, d, _ = edges[e]
        assert set(s) <= avail, (e, s, avail)
        avail |= set(d)
    return avail


def test_chain_prefers_two_step_over_direct():
    edges = [([0], [1], 2.0), ([1], [2], 2.0), ([0], [2], 5.0)]
    order, cost = lib.select_min_cost(3, edges, [0], [2])
    assert order == [0, 1] and cost == 4.0
    assert 2 in fire(3, edges, [0], order)


def test_branching_two_tail_edge_beats_direct():
    edges = [([0], [1], 0.5), ([0], [2], 0.75), ([1, 2], [3], 1.0), ([0], [3], 3.0)]
    order, cost = lib.select_min_cost(4, edges, [0], [3])
    assert sorted(order) == [0, 1, 2] and order[-1] == 2 and abs(cost - 2.25) < 1e-12


def test_multi_source_single_step_and_unreachable():
    edges = [([0, 1], [2], 2.5)]
    assert lib.select_min_cost(3, edges, [0, 1], [2]) == ([0], 2.5)
    assert lib.select_min_cost(3, edges, [0], [2]) is None  # one source is not available


def test_edge_with_two_destinations():
    # 0 -conv-> 1 (full), 1 -pool-> 2, or one conv that writes both; 2 -> 3; {1, 3} -> 4
    edges = [([0], [1], 3.0), ([1], [2], 1.0), ([0], [1, 2], 3.2), ([2], [3], 1.0), ([1, 3], [4], 1.0)]
    order, cost = lib.select_min_cost(5, edges, [0], [4])
    assert order == [2, 3, 4] and abs(cost - 5.2) < 1e-12
    edges[2] = ([0], [1, 2], 4.5)  # the dual output conv is now slower than conv + pool
    order, cost = lib.select_min_cost(5, edges, [0], [4])
    assert sorted(order) == [0, 1, 3, 4] and abs(cost - 6.0) < 1e-12
    # the pre-filter keeps only the topology with the fewest dispatches, whatever the weights say
    order, cost = lib.select_min_cost(5, edges, [0], [4], min_dispatches=True)
    assert sorted(order) == [2, 3, 4] and abs(cost - 6.5) < 1e-12


def test_parallel_edges_and_unbenchmarked_sentinel():
    # three variants of one dispatch: timed, timed, never timed; then a second dispatch with only untimed variants
    edges = [([0], [1], 0.30), ([0], [1], 0.25), ([0], [1], HOUR_MS), ([1], [2], HOUR_MS + 0.001), ([1], [2], HOUR_MS)]
    order, cost = lib.select_min_cost(3, edges, [0], [2])
    assert order == [1, 4] and cost >= HOUR_MS  # a schedule with an untimed dispatch is recognisable by its cost


def test_unet_shaped_graph_with_skip_connections():
    # encoder 0->1->2->3, decoder {3 up, 2}->4, {4, 1}->5; each step has a fast and a slow variant; skip tensors
    # are needed by two consumers
    edges = []
    for (s, d) in [([0], [1]), ([1], [2]), ([2], [3]), ([3, 2], [4]), ([4, 1], [5])]:
        edges.append((s, d, 1.0))
        edges.append((s, d, 2.0))
    order, cost = lib.select_min_cost(6, edges, [0], [5])
    assert order == [0, 2, 4, 6, 8] and cost == 5.0


def test_against_brute_force_on_random_graphs():
    rnd = random.Random(7)
    for trial in range(40):
        n = rnd.randint(4, 7)
        edges = []
        for d in range(1, n):
            for _ in range(rnd.randint(1, 3)):
                k = rnd.randint(1, min(2, d))
                s = rnd.sample(range(d), k)
                dst = [d] + ([rnd.randrange(1, n)] if rnd.random() < 0.2 else [])
                dst = sorted(set(x for x in dst if x not in s and x >= max(s) + 0 and x != 0))
                if not dst or min(dst) <= max(s):
                    dst = [d]
                edges.append((s, dst, float(rnd.randint(1, 9))))
        best = None
        for r in range(1, len(edges) + 1):
            for sub in itertools.combinations(range(len(edges)), r):
                avail, progress = {0}, True
                used = set()
                while progress:
                    progress = False
                    for e in sub:
                        if e not in used and set(edges[e][0]) <= avail:
                            avail |= set(edges[e][1])
                            used.add(e)
                            progress = True
                if (n - 1) in avail and len(used) == len(sub):
                    c = sum(edges[e][2] for e in sub)
                    if best is None or c < best:
                        best = c
        got = lib.select_min_cost(n, edges, [0], [n - 1])
        if best is None:
            assert got is None
        else:
            order, cost = got
            assert abs(cost - best) < 1e-9, (trial, edges, cost, best)
            assert (n - 1) in fire(n, edges, [0], order)


def test_bad_arguments():
    import ctypes as C
    assert lib.L.dnxcu_select_min_cost(0, 0, None, None, None, None, None, None, 0, None, 0, 0, None, None, None) == lib.E_BAD_ARG


def test_populate_lists_fused_and_unfused_candidates(tmp_path):
    """With selection by cost alone the database gets the un-fused candidates too (basic-pool, basic-upsample,
    copy-transform, basic-activation); with the dispatch count pre-filter only the fused topology's."""
    from denox_b200 import nets
    net = nets.tiny_unet()
    a = lib.Db(tmp_path / "a.db")
    n_min = a.populate(net, 64, 128, device=-1)
    b = lib.Db(tmp_path / "b.db")
    n_all = b.populate(net, 64, 128, device=-1, options=lib.OPT_SELECT_BY_COST_ONLY)
    assert n_all > n_min > 4
    pool = lib.Dispatch()
    pool.variant, pool.c_a = lib.find_variant("basic-pool", "VEC=8"), 16
    pool.pc[0], pool.pc[1] = 128, 64
    n0 = len(b)
    b.add_result(pool, [1.0])
    assert len(b) == n0  # the stand-alone pool was a populated candidate already
    n0 = len(a)
    a.add_result(pool, [1.0])
    assert len(a) == n0 + 1  # ... and is not one where only the fewest-dispatch topology is kept
    a.close(); b.close()
