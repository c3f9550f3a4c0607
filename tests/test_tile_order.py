"""Tile order of the GEMM kernels, checked on the host: whatever the grouping, every (row block, column block)
is visited exactly once, shards come in the documented order, and a group keeps its row blocks together."""
import ctypes as C
import itertools

import pytest

from xccl_b200 import _capi as K

COMM_NONE, COMM_AG, COMM_RS = 0, 1, 2


def _order(tiles_m, tiles_n, tp, rank, comm, group_rows):
    L = K.load()
    fn = L.xccl_tp_tile_order
    fn.restype = C.c_int
    fn.argtypes = [C.c_int] * 6 + [C.POINTER(C.c_int)] * 3 + [C.c_int]
    n = tiles_m * tiles_n
    mb, nb, sh = (C.c_int * n)(), (C.c_int * n)(), (C.c_int * n)()
    assert fn(tiles_m, tiles_n, tp, rank, comm, group_rows, mb, nb, sh, n) == n
    return list(zip(mb, nb, sh))


@pytest.mark.parametrize("tiles_m,tiles_n", [(1, 1), (7, 3), (32, 32), (33, 5), (64, 224)])
@pytest.mark.parametrize("group_rows", [0, 1, 5, 8, 12, 16, 100])
def test_plain_gemm_visits_every_tile_once(tiles_m, tiles_n, group_rows):
    order = _order(tiles_m, tiles_n, 1, 0, COMM_NONE, group_rows)
    assert sorted((m, n) for m, n, _ in order) == sorted(itertools.product(range(tiles_m), range(tiles_n)))
    gr = group_rows if group_rows > 0 else 16
    # tiles of one group are contiguous in the walk and a group spans at most gr row blocks
    groups = [m // gr for m, _, _ in order]
    assert groups == sorted(groups)


@pytest.mark.parametrize("tp,mbs", [(2, 16), (4, 8), (8, 4), (8, 3), (4, 7)])
@pytest.mark.parametrize("comm", [COMM_AG, COMM_RS])
@pytest.mark.parametrize("group_rows", [0, 2, 3, 8, 12])
def test_sharded_modes_visit_every_tile_once_in_shard_order(tp, mbs, comm, group_rows):
    tiles_m, tiles_n = tp * mbs, 9
    for rank in range(tp):
        order = _order(tiles_m, tiles_n, tp, rank, comm, group_rows)
        assert sorted((m, n) for m, n, _ in order) == sorted(itertools.product(range(tiles_m), range(tiles_n)))
        for m, _, s in order:
            assert m // mbs == s                       # a tile's shard owns its rows
        shards = [s for _, _, s in order]
        first = rank if comm == COMM_AG else (rank + 1) % tp
        want = [(first + i) % tp for i in range(tp) for _ in range(mbs * tiles_n)]
        assert shards == want                          # allgather starts with the local shard, reduce-scatter ends with it


def _order_ramp(tiles_m, tiles_n, tp, rank, comm, group_rows):
    L = K.load()
    fn = L.xccl_tp_tile_order_ramp
    fn.restype = C.c_int
    fn.argtypes = [C.c_int] * 7 + [C.POINTER(C.c_int)] * 3 + [C.c_int]
    n = tiles_m * tiles_n
    mb, nb, sh = (C.c_int * n)(), (C.c_int * n)(), (C.c_int * n)()
    assert fn(tiles_m, tiles_n, tp, rank, comm, group_rows, 1, mb, nb, sh, n) == n
    return list(zip(mb, nb, sh))


@pytest.mark.parametrize("tiles_m,tiles_n,tp", [(16, 224, 1), (1, 3, 1), (7, 5, 1), (33, 4, 1), (16, 28, 2), (16, 9, 8), (12, 7, 4)])
@pytest.mark.parametrize("group_rows", [0, 1, 3, 8, 100])
def test_ramped_order_for_rows_arriving_from_the_host(tiles_m, tiles_n, tp, group_rows):
    """Group heights 1, 1, 2, 4, ... up to the configured one: every tile once, the rows needed grow with the walk
    (the first tiles_n tiles touch row block 0 only), other shards keep their order."""
    comm = COMM_NONE if tp == 1 else COMM_AG
    for rank in range(tp):
        order = _order_ramp(tiles_m, tiles_n, tp, rank, comm, group_rows)
        assert sorted((m, n) for m, n, _ in order) == sorted(itertools.product(range(tiles_m), range(tiles_n)))
        mbs = tiles_m // tp
        base = rank * mbs if tp > 1 else 0
        local = [m - base for m, _, s in order[:mbs * tiles_n]]
        assert all(0 <= m < mbs for m in local)
        assert local[:tiles_n] == [0] * tiles_n
        # the highest row block needed so far never jumps by more than a doubling of what has been walked
        hi, seen = 0, []
        for m in local:
            hi = max(hi, m)
            seen.append(hi)
        assert seen == sorted(seen)
        gr = group_rows if group_rows > 0 else (16 if tp == 1 else mbs)
        starts = [i for i in range(0, len(local), tiles_n)]
        heights = []
        i = 0
        while i < len(local):
            g = local[i]
            h = 1
            while g + h < mbs and (i + h) < len(local) and local[i + h] == g + h:
                h += 1
            heights.append(h)
            i += h * tiles_n
        ramp = [1, 1, 2, 4, 8, 16, 32, 64]
        for k, h in enumerate(heights[:-1]):
            assert h == min(ramp[min(k, 7)], gr, mbs), (heights, gr)
        if tp > 1:
            plain = _order(tiles_m, tiles_n, tp, rank, comm, group_rows)
            assert order[mbs * tiles_n:] == plain[mbs * tiles_n:]


@pytest.mark.parametrize("tp,mbs,tiles_n", [(4, 8, 28), (8, 4, 28), (8, 2, 5), (2, 3, 7)])
def test_phase_order_of_the_allgather_while_every_shard_is_arriving(tp, mbs, tiles_n):
    """group_ramp = 2: row block c of every shard (local first) x all column blocks, then c + 1."""
    L = K.load()
    fn = L.xccl_tp_tile_order_ramp
    fn.restype = C.c_int
    fn.argtypes = [C.c_int] * 7 + [C.POINTER(C.c_int)] * 3 + [C.c_int]
    tiles_m = tp * mbs
    n = tiles_m * tiles_n
    for rank in range(tp):
        mb, nb, sh = (C.c_int * n)(), (C.c_int * n)(), (C.c_int * n)()
        assert fn(tiles_m, tiles_n, tp, rank, COMM_AG, 0, 2, mb, nb, sh, n) == n
        order = list(zip(mb, nb, sh))
        assert sorted((m, c) for m, c, _ in order) == sorted(itertools.product(range(tiles_m), range(tiles_n)))
        for t, (m, c, s) in enumerate(order):
            assert m // mbs == s
            assert m % mbs == t // (tiles_n * tp)            # the phase
            assert s == (rank + t % tp) % tp                  # shards rotate fastest, the local one first
            assert c == (t % (tiles_n * tp)) // tp
