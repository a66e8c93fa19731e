"""The session's stream planner (csrc/runtime/stream_plan.cc) on hand-made graphs: pure host logic."""
import random


def _plan(nodes, streams):
    from ogle_b200 import session
    return session.plan_streams(nodes, streams)


def _span(i, size=100):
    return (1000 * i, 1000 * i + size)


def test_chain_stays_on_one_stream():
    # node k reads tensor k and writes tensor k+1
    nodes = [([_span(k)], [_span(k + 1)]) for k in range(6)]
    lanes, waits, branches = _plan(nodes, 4)
    assert lanes == [0] * 6 and branches == 0 and all(w == [] for w in waits)


def test_one_stream_is_file_order():
    nodes = [([_span(0)], [_span(k + 1)]) for k in range(5)]
    lanes, waits, branches = _plan(nodes, 1)
    assert lanes == [0] * 5 and branches == 0 and all(w == [] for w in waits)


def test_head_branches_off_and_joins():
    # backbone 0 -> 1 -> 2 -> 3; head A reads the output of node 1; head B reads the output of node 3;
    # the concat reads both heads
    t = {name: _span(i) for i, name in enumerate(["in", "f1", "f2", "f3", "f4", "ha", "hb", "out"])}
    nodes = [([t["in"]], [t["f1"]]), ([t["f1"]], [t["f2"]]), ([t["f2"]], [t["f3"]]), ([t["f3"]], [t["f4"]]),
             ([t["f2"]], [t["ha"]]),            # head A: depends on node 1 only
             ([t["f4"]], [t["hb"]]),            # head B: continues the backbone's stream
             ([t["ha"], t["hb"]], [t["out"]])]
    lanes, waits, branches = _plan(nodes, 3)
    assert lanes[:4] == [0, 0, 0, 0]
    assert lanes[4] != 0 and waits[4] == [1] and branches == 1
    assert lanes[5] == 0 and waits[5] == []
    # the concat continues the stream of its latest producer and waits for the other
    assert lanes[6] == 0 and waits[6] == [4]


def test_aliases_and_hazards_are_dependencies():
    a, b = (0, 400), (1000, 1400)
    nodes = [([], [a]),                     # 0 writes a
             ([(0, 100)], [b]),             # 1 reads a piece of a (an alias), writes b
             ([], [(300, 500)]),            # 2 overwrites the end of a: must follow 0 (write after write), not 1 (no overlap)
             ([b], [(0, 50)])]              # 3 overwrites what 1 read: write after read on node 1, and after write on 0
    lanes, waits, _ = _plan(nodes, 4)
    assert _reaches(lanes, waits, 1, 0) and _reaches(lanes, waits, 2, 0) and _reaches(lanes, waits, 3, 1)


def _reaches(lanes, waits, i, j):
    """True when the plan orders node i after node j (same stream, a wait, or transitively)."""
    seen, todo = set(), [i]
    while todo:
        k = todo.pop()
        if k == j:
            return True
        if k in seen or k < j:
            continue
        seen.add(k)
        todo.extend(waits[k])
        prev = [p for p in range(k) if lanes[p] == lanes[k]]
        if prev:
            todo.append(prev[-1])
    return False


def test_random_graphs_keep_every_hazard_ordered():
    rng = random.Random(7)
    for trial in range(40):
        n = rng.randint(2, 24)
        tensors = [_span(i, rng.randint(10, 1500)) for i in range(n + 3)]     # some spans overlap their neighbour
        nodes = []
        for i in range(n):
            reads = [tensors[rng.randrange(0, i + 3)] for _ in range(rng.randint(1, 3))]
            writes = [tensors[rng.randrange(3, n + 3)]]
            nodes.append((reads, writes))
        for streams in (2, 3, 8):
            lanes, waits, _ = _plan(nodes, streams)
            assert all(0 <= l < streams for l in lanes)

            def hit(xs, ys):
                return any(x[0] < y[1] and y[0] < x[1] for x in xs for y in ys)
            for i in range(n):
                assert all(j < i and lanes[j] != lanes[i] for j in waits[i])
                for j in range(i):
                    if hit(nodes[j][1], nodes[i][0]) or hit(nodes[j][1], nodes[i][1]) or hit(nodes[j][0], nodes[i][1]):
                        assert _reaches(lanes, waits, i, j), (trial, streams, i, j)
