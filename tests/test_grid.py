"""Rank <-> coordinate mapping and group membership for every factorisation of 8
(pure functions, no process group)."""

import itertools

from axonn_b200.communication import coords_of, grid_groups, rank_of


def factorisations(n, k):
    if k == 1:
        yield (n,)
        return
    for f in range(1, n + 1):
        if n % f == 0:
            for rest in factorisations(n // f, k - 1):
                yield (f,) + rest


def test_coords_roundtrip_and_layout():
    for G_inter, G_data, r, c, d in factorisations(8, 5):
        seen = set()
        for w in range(8):
            co = coords_of(w, G_inter, G_data, r, c, d)
            assert 0 <= co.col < c and 0 <= co.row < r and 0 <= co.depth < d
            assert 0 <= co.inter < G_inter and 0 <= co.data < G_data
            assert rank_of(co.data, co.inter, co.depth, co.row, co.col, G_inter, G_data, r, c, d) == w
            # column index is the fastest varying coordinate
            assert co.intra == co.depth * r * c + co.row * c + co.col
            seen.add((co.data, co.inter, co.depth, co.row, co.col))
        assert len(seen) == 8


def test_groups_partition_world():
    for G_inter, G_data, r, c, d in factorisations(8, 5):
        lay = grid_groups(G_inter, G_data, r, c, d)
        sizes = {"data": G_data, "intra": r * c * d, "inner": c, "outer": r, "depth": d, "pipe": G_inter}
        for name, size in sizes.items():
            flat = list(itertools.chain.from_iterable(lay[name]))
            assert sorted(flat) == list(range(8)), (name, lay[name])
            assert all(len(g) == size for g in lay[name])
        # members of an inner group differ only in the column coordinate, etc.
        for name, attr in (("inner", "col"), ("outer", "row"), ("depth", "depth"), ("data", "data"),
                           ("pipe", "inter")):
            for g in lay[name]:
                cs = [coords_of(w, G_inter, G_data, r, c, d) for w in g]
                for field in ("data", "inter", "depth", "row", "col"):
                    vals = {getattr(x, field) for x in cs}
                    if field == attr:
                        assert len(vals) == len(g)
                    else:
                        assert len(vals) == 1


def test_reference_example_layout():
    # world 8, r=c=d=2: rank 5 = depth 1, row 0, col 1
    co = coords_of(5, 1, 1, 2, 2, 2)
    assert (co.depth, co.row, co.col) == (1, 0, 1)
