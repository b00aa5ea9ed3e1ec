"""GPU parity against the live oracle over randomly drawn configurations: scene sets, batch sizes
(odd ones included), one or two groups, fixed and rotating scenes, both action mixes and every
plan switch of the generator.  The draw is seeded; the run stops after a time budget, so the
number of configurations depends on the box (several hundred on a B200 host)."""
import random
import time

import pytest

from oracle import pyoracle
from test_gpu_live_oracle import _compare_run

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not pyoracle.available(), reason="oracle libraries not built")]

ALL_SCENES = ["c0", "c1", "d0"] + [f"m{i:02d}" for i in range(16)]


def _draw(rng):
    k = rng.choice([1, 1, 2, 3, 4, 8, 16])
    names = rng.sample(ALL_SCENES, k)
    groups = rng.choice([1, 1, 2])
    if groups == 2 and k > 1 and k % 2:
        names, k = names[:-1], k - 1
    per = rng.choice([3, 17, 64, 250, 512, 1024, 2048, 4096])
    n = min(per * k, 65536)
    n -= n % (k * groups)
    if n <= 0:
        return None
    steps = rng.choice([20, 40]) if n > 8192 else rng.choice([60, 150])
    kw = dict(seed=rng.randrange(1, 10 ** 6), mix=rng.choice(["uniform", "policy"]), threads=16,
              check_state_every=max(10, steps // 3))
    if groups == 2:
        kw["double_buffered"] = True
    flag = rng.choice([None, None, "two_launches", "global_memory", "small_smem"])
    if flag:
        kw[flag] = True
    if k >= 4 and rng.random() < 0.3:
        half = k // 2
        kw["num_active"] = (half - half % groups) or groups
        if rng.random() < 0.5:
            kw["swap_interval"] = rng.choice([3, 16])
    form = rng.choice([None, None, 1, 2])
    if form is not None:
        kw["force_batched"] = form
    return names, n, steps, kw


def test_random_configurations_match_the_oracle():
    rng = random.Random(20240611)
    t0 = time.time()
    ran = 0
    while time.time() - t0 < 25.0:
        cfg = _draw(rng)
        if cfg is None:
            continue
        names, n, steps, kw = cfg
        try:
            _compare_run(names, n, steps, **kw)
        except AssertionError as e:
            raise AssertionError(f"{names} n={n} steps={steps} {kw}: {e}") from e
        ran += 1
    assert ran >= 10
