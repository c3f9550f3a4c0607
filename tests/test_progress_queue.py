"""The two progress queues driven directly: the list queue of single-thread contexts and the lock-free queue of
thread-multiple contexts (two pools of XCCL_LF_TASKS_QUEUE_SIZE slots, overflow list behind them), the latter with
several threads enqueuing and progressing at once. Reference: src/core/xccl_tasks_queue.c:3-43,
src/core/xccl_lock_free_tasks_queue.c:3-121 (which has no test of its own)."""
import ctypes as C

import pytest

from xccl_b200 import _capi as K


def _selftest(mode, slots, producers, per_thread, polls):
    fn = K.load().xccl_progress_queue_selftest
    fn.restype = C.c_long
    fn.argtypes = [C.c_uint, C.c_int, C.c_int, C.c_int, C.c_int, C.c_double]
    return fn(mode, slots, producers, per_thread, polls, 60.0)


def test_single_thread_queue_completes_every_task_once():
    assert _selftest(K.THREAD_SINGLE, 8, 1, 500, 3) == 500


@pytest.mark.parametrize("slots", [1, 8, 128])
@pytest.mark.parametrize("producers,per_thread", [(1, 300), (4, 200), (8, 100)])
def test_lock_free_queue_under_concurrent_producers(slots, producers, per_thread):
    """More tasks in flight than 2 x slots: the overflow list is used; every task completes exactly once and is never
    progressed by two threads at the same time."""
    assert _selftest(K.THREAD_MULTIPLE, slots, producers, per_thread, 5) == producers * per_thread
