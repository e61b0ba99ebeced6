"""The device-side weight quantizers (Matrix::from_f32 on the GPU) against the CPU
quantizers: integer and byte work, so the buffers must be equal bit for bit."""
import numpy as np
import pytest

from refgen import xorshift_data
from tachyon_b200 import synth, weights
from test_gpu_parity import ctx  # noqa: F401

pytestmark = pytest.mark.gpu


def device_matrix(ctx, data, rows, cols, fmt):
    from tachyon_b200 import cuda

    dm = cuda.DeviceMatrix.quantize(ctx, data, rows, cols, fmt)
    m = dm.to_host()
    dm.free()
    return m


@pytest.mark.parametrize("rows,cols", [(37, 352), (64, 1024), (5, 32), (96, 2048)])
def test_q8_and_bf16_bytes_equal_the_cpu_quantizers(oracle, ctx, rows, cols):
    data = (xorshift_data(rows * cols, rows + cols) * np.float32(0.05)).astype(np.float32)
    data[3 * cols:3 * cols + 32] = 0.0            # an all-zero block: scale 0
    data[cols + 5] = np.float32(70000.0)          # a scale beyond f16's range
    got = device_matrix(ctx, data, rows, cols, "q8")
    s, q = oracle.quantize_q8_weights(data)
    assert np.array_equal(got.scales, s) and np.array_equal(got.data, q)
    host = weights.Matrix.from_f32(data, rows, cols, "q8")
    assert np.array_equal(got.scales, host.scales) and np.array_equal(got.data, host.data)
    bf = device_matrix(ctx, data, rows, cols, "bf16")
    assert np.array_equal(bf.data, weights.f32_to_bf16(data))


@pytest.mark.parametrize("rows,cols", [(37, 352), (16, 1024), (3, 32), (24, 1536), (8, 2048)])
def test_q4_bytes_equal_the_cpu_quantizer(oracle, ctx, rows, cols):
    """Partial last super-block (352 columns = 11 blocks), constant blocks, a zero row."""
    data = synth.normal(3, 7, rows * cols, 0, scale=0.02)
    data[:32] = np.float32(0.125)                 # a constant block: all offset
    data[2 * cols:3 * cols] = 0.0 if rows > 2 else data[2 * cols:3 * cols]  # a zero row
    got = device_matrix(ctx, data, rows, cols, "q4")
    s, q = oracle.quantize_q4_matrix(data, rows, cols, None, 4)
    assert np.array_equal(got.data, q)
    assert np.array_equal(got.scales, s)


def test_layer_from_device_quantized_matrices_equals_the_uploaded_one(oracle, ctx):
    """A layer built from matrices quantized on the device gives the same block output as one
    built from the host-quantized matrices (they are the same bytes)."""
    from tachyon_b200 import cuda, workloads
    from tachyon_b200.workloads import MoeShape

    shape = MoeShape("dq", 512, 8, 2, 128, fmt="q8")
    h, e, i = shape.hidden, shape.experts, shape.inter
    raw = {name: synth.normal(9, stream, rows * cols, 0, scale=0.02)
           for name, stream, rows, cols in [("router", 2, e, h), ("gate_up", 3, e * 2 * i, h), ("down", 4, e * h, i)]}
    x = workloads.hidden_states(shape, 20, seed=9)
    outs = []
    for fmt in ("q8", "q4"):
        dm = [cuda.DeviceMatrix.quantize(ctx, raw["router"], e, h, "bf16"),
              cuda.DeviceMatrix.quantize(ctx, raw["gate_up"], e * 2 * i, h, fmt),
              cuda.DeviceMatrix.quantize(ctx, raw["down"], e * h, i, fmt)]
        on_device = cuda.MoeLayer(ctx, dm[0], dm[1], dm[2], shape.topk, 20)
        uploaded = cuda.MoeLayer(ctx, dm[0].to_host(), dm[1].to_host(), dm[2].to_host(), shape.topk, 20)
        ys = []
        for layer in (on_device, uploaded):
            xd, yd = ctx.to_device(x), ctx.to_device(np.zeros_like(x))
            layer.forward(xd, yd)
            ctx.sync()
            ys.append(yd.get())
        assert np.array_equal(ys[0], ys[1])
        host = [weights.Matrix.from_f32(raw["gate_up"], e * 2 * i, h, fmt)] if fmt == "q8" else []
        for m in host:
            assert np.array_equal(m.data, dm[1].to_host().data)
        outs.append(ys[0])
        uploaded.free()
        on_device.free()
    assert np.all(np.isfinite(outs[0])) and np.all(np.isfinite(outs[1]))
