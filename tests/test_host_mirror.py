"""CPU tests of the host side: the numpy mirror of Tachyon's `Matrix` against
the oracle's restatement of the same quantizers (two independent statements of
src/kernels.rs:135-149 and 180-242 must give the same bytes), the synthetic
generator, and that the C-ABI library loads and exports every declared symbol."""
import os
import re

import numpy as np
import pytest

from refgen import lcg_data, xorshift_data
from tachyon_b200 import synth, weights, workloads
from tachyon_b200.q4 import quantize_q4_matrix


def test_q8_weight_mirror_matches_oracle(oracle):
    w = synth.normal(0, 3, 96 * 1024, scale=0.02)
    s, q = weights.quantize_q8_weights(w)
    s2, q2 = oracle.quantize_q8_weights(w)
    assert np.array_equal(s, s2) and np.array_equal(q, q2)
    # zeros, halves (round away from zero) and a huge block
    w = np.concatenate([np.zeros(32, np.float32), np.arange(-16, 16, dtype=np.float32) * 0.5,
                        np.full(32, 3e38, np.float32)])
    s, q = weights.quantize_q8_weights(w)
    s2, q2 = oracle.quantize_q8_weights(w)
    assert np.array_equal(s, s2) and np.array_equal(q, q2)


def test_q8_activation_mirror_matches_oracle(oracle):
    x = synth.normal(1, 1, 64 * 1024)
    d, q = weights.quantize_q8_activations(x)
    d2, q2 = oracle.quantize_q8(x)
    assert np.array_equal(d, d2) and np.array_equal(q, q2)


def test_bf16_mirror_matches_oracle(oracle):
    w = synth.normal(0, 2, 4096, scale=0.02)
    got = weights.f32_to_bf16(w)
    want = np.array([oracle.f32_to_bf16(float(v)) for v in w], np.uint16)
    assert np.array_equal(got, want)
    assert np.array_equal(weights.bf16_to_f32(got), np.array([oracle.bf16_to_f32(int(b)) for b in got], np.float32))


@pytest.mark.parametrize("rows,cols,gen", [(37, 352, "xor"), (8, 1536, "normal"), (1, 352, "kat")])
def test_q4_mirror_matches_oracle(oracle, rows, cols, gen):
    if gen == "xor":
        data = xorshift_data(rows * cols, 1)
    elif gen == "normal":
        data = synth.normal(0, 4, rows * cols, scale=0.02)
    else:  # the partial super-block / constant-block case of src/kernels.rs:1743-1749
        data = lcg_data(cols, 5)
        data[3 * 32:4 * 32] = 0.25
        data[9 * 32:10 * 32] = 0.0
    s, q = quantize_q4_matrix(data, rows, cols)
    s2, q2 = oracle.quantize_q4_matrix(data, rows, cols)
    assert np.array_equal(s, s2) and np.array_equal(q, q2)
    assert s.size == rows * weights.q4_words(cols)


def test_generator_is_counter_based_and_standard_normal():
    a = synth.normal(0, 1, 100_000)
    assert np.array_equal(a[5000:6000], synth.normal(0, 1, 1000, start=5000))
    assert not np.array_equal(a[:1000], synth.normal(0, 2, 1000))
    assert not np.array_equal(a[:1000], synth.normal(1, 1, 1000))
    assert not np.array_equal(a[:1000], synth.normal(0, 1, 1000, layer=1))
    assert abs(float(a.mean())) < 0.02 and abs(float(a.std()) - 1.0) < 0.02
    ids = synth.token_ids(0, 10_000, 49155)
    assert ids.max() < 49155 and len(np.unique(ids)) > 8000
    bias = synth.zipf_router_bias(0, 64)
    p = np.exp(bias.astype(np.float64))
    assert abs(p.sum() - 1.0) < 1e-5 and p.max() / p.min() > 20


def test_workload_byte_counts():
    # One expert's gate_up + down as stored: 8.5 and 4.625 bits per weight.
    assert workloads.expert_bytes(workloads.GRANITE_1B) == 1_671_168
    assert workloads.expert_bytes(workloads.GRANITE_3B_Q8) == 2_506_752
    assert workloads.expert_bytes(workloads.SKEW) == 6_684_672
    assert workloads.expert_bytes(workloads.GRANITE_3B) == 1_363_968
    lw = workloads.layer_weights(workloads.MoeShape("tiny", 64, 4, 2, 32), threads=1)
    assert lw.gate_up.rows == 4 * 64 and lw.down.rows == 4 * 64 and lw.router.kind == weights.KIND_BF16


def test_library_loads_and_exports_every_declared_symbol():
    from tachyon_b200 import build, cuda

    build.build()
    lib = cuda.load()
    header = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include",
                               "tachyon_cuda.h")).read()
    declared = set(re.findall(r"\b(tc_[a-z0-9_]+)\s*\(", header))
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared but not exported"
    assert declared == set(cuda.SYMBOLS), declared ^ set(cuda.SYMBOLS)


def test_no_device_fails_loudly():
    """Without a GPU the context refuses to exist: there is no CPU fallback."""
    import ctypes

    from tachyon_b200 import build, cuda

    build.build()
    lib = cuda.load()
    err = ctypes.create_string_buffer(256)
    # Skip when a device is actually present (the GPU box runs the parity tests instead).
    h = lib.tc_create(0, err, len(err))
    if h:
        lib.tc_destroy(h)
        pytest.skip("a CUDA device is present")
    assert err.value
    with pytest.raises(cuda.TachyonCudaError):
        cuda.Context(0)


def test_rust_glue_binds_only_declared_entry_points():
    """The `extern "C"` block of the Rust glue (tachyon_b200/rust/src/gpu/cuda/mod.rs) names
    entry points that the header declares and the ctypes mirror binds, and its build script
    lists every .cu source of the library."""
    import glob
    import re

    from tachyon_b200 import cuda

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    rust = open(os.path.join(root, "tachyon_b200", "rust", "src", "gpu", "cuda", "mod.rs")).read()
    block = rust[rust.index('extern "C" {'):]
    block = block[:block.index("\n}\n")]
    bound = set(re.findall(r"fn (tc_\w+)\(", block))
    assert len(bound) > 20
    header = open(os.path.join(root, "include", "tachyon_cuda.h")).read()
    for name in bound:
        assert re.search(r"\b" + name + r"\(", header), name
        assert name in cuda.SYMBOLS, name
    build_rs = open(os.path.join(root, "tachyon_b200", "rust", "build_cuda.rs")).read()
    listed = set(re.findall(r'^    "(\w+)",$', build_rs, flags=re.M))
    have = {os.path.basename(p)[:-3] for p in glob.glob(os.path.join(root, "tachyon_b200", "csrc", "*.cu"))}
    assert listed == have, (listed ^ have)
