"""Background batch preparation: same batches as the direct calls, in order, overlapped, and cleanly shut down."""
import threading
import time

from superscaler_b200.data.prefetch import Prefetcher


def test_batches_are_those_of_the_wrapped_function_and_are_built_ahead():
    calls, lock = [], threading.Lock()

    def fn(i):
        with lock:
            calls.append(i)
        time.sleep(0.05)
        return {"i": i}

    fn.valid = "held-out"
    p = Prefetcher(fn, workers=3, stop=8)
    assert p.valid == "held-out" and p.test is None and p.fn is fn
    t0 = time.time()
    got = [p(i)["i"] for i in range(8)]
    took = time.time() - t0
    assert got == list(range(8))
    assert sorted(calls) == list(range(8))                # every batch built exactly once, none past the end
    assert took < 8 * 0.05 * 0.8                          # three at a time, not one after the other
    p.close()


def test_a_jump_ahead_drops_the_skipped_batches_and_errors_reach_the_caller():
    def fn(i):
        if i == 5:
            raise ValueError("bad batch")
        return i

    p = Prefetcher(fn, workers=2)
    assert p(0) == 0
    assert p(3) == 3 and all(j > 3 for j in p.pending)
    assert p(4) == 4
    try:
        p(5)
    except ValueError as e:
        assert "bad batch" in str(e)
    else:
        raise AssertionError("the worker's exception was swallowed")
    p.close()
    assert not p.pending
