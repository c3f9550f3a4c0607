"""Algorithm-selection thresholds: derived from sweep rows by the benchmark, stored as a small text table,
read back by the NVLink team (XCCL_TEAM_NVLINK_TUNING_FILE). All of it runs without a GPU."""
import ctypes as C

from xccl_b200 import _capi as K
from xccl_b200.bench.collectives import selection_table


def _rows():
    out = []
    times = {  # bytes -> {alg: us}
        1024: {"one_shot": 19.0, "two_shot": 39.0, "nvls": 28.0},
        262144: {"one_shot": 24.0, "two_shot": 46.0, "nvls": 33.0},
        1048576: {"one_shot": 36.0, "two_shot": 47.0, "nvls": 34.0, "direct": 35.0},
        4194304: {"one_shot": 73.0, "two_shot": 53.0, "nvls": 42.0, "direct": 40.0},
        67108864: {"two_shot": 242.0, "nvls": 238.0, "direct": 209.0},
    }
    for b, algs in times.items():
        for alg, us in algs.items():
            out.append({"coll": "allreduce", "impl": "nvlink", "alg": alg, "dtype": "float32", "gpus": 8, "bytes": b, "us": us})
        out.append({"coll": "allreduce", "impl": "nccl", "alg": "nccl", "dtype": "float32", "gpus": 8, "bytes": b, "us": 1.0})
    return out


def test_selection_table_from_sweep_rows():
    tab = selection_table(_rows())
    assert tab == {8: {"one_shot_max": 262144, "nvls_min": 1048576, "direct_min": 4194304}}


def test_tuning_file_lookup(tmp_path):
    L = K.load()
    fn = L.xccl_nvlink_tuning_lookup
    fn.restype = C.c_int
    fn.argtypes = [C.c_char_p, C.c_int] + [C.POINTER(C.c_longlong)] * 3
    f = tmp_path / "table.txt"
    f.write_text("# team_size one_shot_max nvls_min direct_min\n4 1048576 131072 -1\n8 262144 1048576 4194304\n8 131072 -1\n")
    a, b, c = C.c_longlong(-1), C.c_longlong(-1), C.c_longlong(-1)
    assert fn(str(f).encode(), 4, C.byref(a), C.byref(b), C.byref(c)) == 2
    assert (a.value, b.value, c.value) == (1048576, 131072, -1)
    a, b, c = C.c_longlong(-1), C.c_longlong(-1), C.c_longlong(-1)
    assert fn(str(f).encode(), 8, C.byref(a), C.byref(b), C.byref(c)) == 1     # the last matching line wins
    assert a.value == 131072
    assert fn(str(f).encode(), 2, C.byref(a), C.byref(b), C.byref(c)) == 0     # no line for this team size
    assert fn(b"/nonexistent/table", 8, C.byref(a), C.byref(b), C.byref(c)) == 0
