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
