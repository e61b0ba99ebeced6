"""The tcgen05 (tensor memory) building blocks: one int8 MMA must give the exact integer product."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [64, 128])
def test_one_tcgen05_int8_mma_is_exact(n):
    from tachyon_b200 import build, cuda

    build.build()
    ctx = cuda.Context(0)
    rng = np.random.default_rng(n)
    a = rng.integers(-127, 128, size=(128, 32), dtype=np.int8)
    b = rng.integers(-127, 128, size=(n, 32), dtype=np.int8)
    got = ctx.umma_selftest(a, b)
    want = a.astype(np.int32) @ b.astype(np.int32).T
    assert np.array_equal(got, want)
    ctx.close()
