"""The native inner loops of the cost model against their Python definitions: equal bit for bit on random stages."""
import random

import pytest

from superscaler_b200.search import cost_model as cm

pytestmark = pytest.mark.skipif(cm._native is None, reason="host helper not built")


def _python_only(fn, *args):
    native, cm._native = cm._native, None
    try:
        return fn(*args)
    finally:
        cm._native = native


def _random_stage(rng, n):
    acts = [rng.choice([0.0, 0.125, 1.5, 64.0, 96.25, 384.0]) * rng.random() for _ in range(n)]
    kinds = [rng.choice([0, 0, 0, 1, 2]) for _ in range(n)]
    ends = [int(rng.random() < 0.15) for _ in range(n - 1)]
    return acts, kinds, ends


def test_saved_and_peak_accounts_equal_python():
    rng = random.Random(7)
    for _ in range(300):
        n = rng.randint(2, 60)
        acts, kinds, ends = _random_stage(rng, n)
        rc = [int(rng.random() < 0.6) for _ in range(n)]
        for fn in (cm.CostModel._saved_fast, cm.CostModel._peak_fast):
            assert fn(rc, acts, kinds, ends) == _python_only(fn, rc, acts, kinds, ends)


def test_choose_recompute_equals_python():
    """Drives CostModel._choose_recompute through a stub that supplies the tables it reads."""
    rng = random.Random(11)

    class Stub(cm.CostModel):
        def __init__(self, acts, kinds, ends, mem):
            self.opt = cm.CostOptions(memory_limit=1000.0, never_recompute=("never-op",))
            self._arr, self._mem = (acts, kinds, ends), mem
            self._name_ids, self._groups_cache = {}, {}

        def _act_arrays(self, ops, mbs, tp, algo):
            return self._arr

        def stage_memory_cached(self, *a):
            return self._mem

    names = ["enc-1st-layernorm", "qkv", "score", "never-op", "dense", "blk-conv1", "blk-relu", "mlp", "gelu"]
    for _ in range(300):
        n = rng.randint(2, 80)
        ops = [rng.choice(names) for _ in range(n)]
        acts, kinds, ends = _random_stage(rng, n)
        stub = Stub(acts, kinds, ends, 1000.0 + rng.random() * 3000.0)
        args = (ops, 4, [1] * n, [1] * n, rng.randint(0, 3), [0] * n)
        got = stub._choose_recompute(*args)
        want = _python_only(stub._choose_recompute, *args)
        assert list(got) == list(want)
