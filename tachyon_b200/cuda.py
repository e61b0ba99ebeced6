"""ctypes binding of ``libtachyon_cuda.so`` (include/tachyon_cuda.h) and the thin
host-side objects over it. The names follow Tachyon's GPU backend
(src/gpu/mod.rs): a ``Context`` owns the device, ``DeviceMatrix`` is
``GpuMatrix``, ``MoeLayer.forward`` is ``GpuBackend::moe``.

There is no CPU fallback: loading fails loudly if the library is missing, and
every compute call runs CUDA kernels or raises ``TachyonCudaError``.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from .weights import KIND_BF16, Matrix

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "lib", "libtachyon_cuda.so")

# Every symbol include/tachyon_cuda.h declares: (restype, argtypes).
_vp, _sz, _i, _f, _u64 = C.c_void_p, C.c_size_t, C.c_int, C.c_float, C.c_uint64
SYMBOLS = {
    "tc_create": (_vp, [_i, C.c_char_p, _sz]),
    "tc_destroy": (None, [_vp]),
    "tc_device_name": (None, [_vp, C.c_char_p, _sz]),
    "tc_last_error": (_sz, [_vp, C.c_char_p, _sz]),
    "tc_sync": (_i, [_vp]),
    "tc_stream": (_vp, [_vp]),
    "tc_set_arithmetic": (_i, [_vp, _i]),
    "tc_set_prefill_threshold": (_i, [_vp, _i]),
    "tc_set_launch_overlap": (_i, [_vp, _i]),
    "tc_set_decode_block": (_i, [_vp, _i]),
    "tc_profile_phases": (_i, [_vp, _i]),
    "tc_profile_read_phases": (_i, [_vp, _vp]),
    "tc_malloc": (_vp, [_vp, _sz]),
    "tc_free": (None, [_vp, _vp]),
    "tc_upload": (_i, [_vp, _vp, _vp, _sz]),
    "tc_download": (_i, [_vp, _vp, _vp, _sz]),
    "tc_memset": (_i, [_vp, _vp, _i, _sz]),
    "tc_copy": (_i, [_vp, _vp, _vp, _sz]),
    "tc_host_alloc": (_vp, [_vp, _sz]),
    "tc_host_free": (None, [_vp, _vp]),
    "tc_profile_enable": (_i, [_vp, _i]),
    "tc_profile_read": (_i, [_vp, _vp, _vp]),
    "tc_matrix_upload": (_vp, [_vp, _i, _sz, _sz, _vp, _sz, _vp, _sz]),
    "tc_matrix_quantize": (_vp, [_vp, _i, _sz, _sz, _vp]),
    "tc_matrix_download": (_i, [_vp, _vp, _sz, _vp, _sz]),
    "tc_matrix_free": (None, [_vp]),
    "tc_moe_layer_create": (_vp, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _i]),
    "tc_moe_layer_free": (None, [_vp]),
    "tc_moe_layer_detach_experts": (_i, [_vp]),
    "tc_moe_set_router_bias": (_i, [_vp, _vp]),
    "tc_moe_forward": (_i, [_vp, _vp, _i, _vp]),
    "tc_moe_block": (_i, [_vp, _vp, _f, _i, _vp]),
    "tc_moe_forward_host": (_i, [_vp, _vp, _i, _vp]),
    "tc_moe_last_routing": (_i, [_vp, _vp, _vp, _vp, _vp]),
    "tc_moe_last_dispatch": (_i, [_vp, _vp, _vp]),
    "tc_ep_unique_id": (_i, [C.c_char_p]),
    "tc_ep_init": (_i, [_vp, C.c_char_p, _i, _i]),
    "tc_ep_expert_range": (_i, [_i, _i, _i, C.POINTER(C.c_int), C.POINTER(C.c_int)]),
    "tc_ep_set_uniform_batch": (_i, [_vp, _i]),
    "tc_ep_enable_peer_exchange": (_i, [_vp, _i, _i, _i]),
    "tc_ep_set_wait_limit": (_i, [_vp, C.c_uint32]),
    "tc_ep_test_mute_signals": (_i, [_vp, _i]),
    "tc_ep_barrier": (_i, [_vp]),
    "tc_moe_ep_layer_create": (_vp, [_vp, _i, _i, _i, _i, _vp, _vp, _vp, _i]),
    "tc_umma_selftest": (_i, [_vp, _vp, _vp, _i, _vp]),
    "tc_int8_peak": (_i, [_vp, _i, C.POINTER(C.c_double), C.POINTER(C.c_float)]),
    "tc_dispatch_static": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _vp]),
    "tc_rmsnorm": (_i, [_vp, _vp, _vp, _f, _i, _i, _vp]),
    "tc_capture_begin": (_i, [_vp]),
    "tc_capture_end": (_vp, [_vp]),
    "tc_graph_launch": (_i, [_vp]),
    "tc_graph_free": (None, [_vp]),
    "tc_timer_start": (_i, [_vp]),
    "tc_timer_stop_ms": (_f, [_vp]),
    "tc_launch_count": (_u64, [_vp]),
}


class TachyonCudaError(RuntimeError):
    pass


_lib = None


def load() -> C.CDLL:
    """Loads the shared library (built in-tree by ``tachyon_b200.build``)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise TachyonCudaError(
                f"{LIB_PATH} is missing: build it with `python -m tachyon_b200.build` "
                "(there is no CPU fallback)")
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data_as(C.c_void_p)
    return C.c_void_p(int(a))


class Context:
    """One device, one stream (``tc_ctx``). Driven by one thread at a time."""

    def __init__(self, device: int = 0):
        self.lib = load()
        err = C.create_string_buffer(1024)
        self.handle = self.lib.tc_create(device, err, len(err))
        if not self.handle:
            raise TachyonCudaError(f"CUDA setup failed: {err.value.decode()}")
        self.device = device

    def close(self):
        if getattr(self, "handle", None):
            self.lib.tc_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc, what: str):
        if rc != 0:
            buf = C.create_string_buffer(1024)
            self.lib.tc_last_error(self.handle, buf, len(buf))
            raise TachyonCudaError(f"{what}: {buf.value.decode()}")

    def last_error(self) -> str:
        buf = C.create_string_buffer(1024)
        self.lib.tc_last_error(self.handle, buf, len(buf))
        return buf.value.decode()

    @property
    def name(self) -> str:
        buf = C.create_string_buffer(256)
        self.lib.tc_device_name(self.handle, buf, len(buf))
        return buf.value.decode()

    ARITH_FAST, ARITH_CPU_LANES = 0, 1

    def set_arithmetic(self, mode: int):
        """ARITH_FAST (default) or ARITH_CPU_LANES (bit-identical to the CPU path)."""
        self._check(self.lib.tc_set_arithmetic(self.handle, mode), "tc_set_arithmetic")

    def set_launch_overlap(self, on: bool):
        """Programmatic dependent launch between the kernels of a block (default on)."""
        self._check(self.lib.tc_set_launch_overlap(self.handle, int(on)), "tc_set_launch_overlap")

    def set_decode_block(self, on: bool):
        """Decode-size blocks (up to 128 tokens) as one kernel (default on) or as four."""
        self._check(self.lib.tc_set_decode_block(self.handle, int(on)), "tc_set_decode_block")

    def profile_phases(self, on: bool):
        self._check(self.lib.tc_profile_phases(self.handle, int(on)), "tc_profile_phases")

    PHASES = ("wait_previous", "route", "gate_up", "down", "combine")

    def read_phases(self) -> dict:
        """Microseconds CTA 0 of the last one-kernel block spent up to each phase boundary."""
        ns = np.zeros(6, np.uint64)
        self._check(self.lib.tc_profile_read_phases(self.handle, _ptr(ns)), "tc_profile_read_phases")
        d = np.diff(ns.astype(np.int64)) / 1e3
        return {name: float(v) for name, v in zip(self.PHASES, d)}

    def set_prefill_threshold(self, avg_tokens_per_expert: int):
        """Average tokens per expert from which the tcgen05 kernels take over (default 32; 0 = always)."""
        self._check(self.lib.tc_set_prefill_threshold(self.handle, avg_tokens_per_expert),
                    "tc_set_prefill_threshold")

    def sync(self):
        self._check(self.lib.tc_sync(self.handle), "tc_sync")

    def stream(self) -> int:
        return self.lib.tc_stream(self.handle) or 0

    def malloc(self, nbytes: int) -> int:
        p = self.lib.tc_malloc(self.handle, nbytes)
        if not p:
            raise TachyonCudaError(f"tc_malloc({nbytes}): {self.last_error()}")
        return p

    def free(self, dev: int):
        self.lib.tc_free(self.handle, dev)

    def upload(self, dev: int, host: np.ndarray):
        host = np.ascontiguousarray(host)
        self._check(self.lib.tc_upload(self.handle, dev, _ptr(host), host.nbytes), "tc_upload")

    def download(self, host: np.ndarray, dev: int):
        assert host.flags["C_CONTIGUOUS"]
        self._check(self.lib.tc_download(self.handle, _ptr(host), dev, host.nbytes), "tc_download")

    def memset(self, dev: int, value: int, nbytes: int):
        self._check(self.lib.tc_memset(self.handle, dev, value, nbytes), "tc_memset")

    def copy(self, dst: "DeviceArray", src: "DeviceArray"):
        assert dst.nbytes == src.nbytes
        self._check(self.lib.tc_copy(self.handle, dst.ptr, src.ptr, src.nbytes), "tc_copy")

    def copy_bytes(self, dst: int, src: int, nbytes: int):
        """Device to device on the context's stream (can be captured)."""
        self._check(self.lib.tc_copy(self.handle, dst, src, nbytes), "tc_copy")

    def pinned(self, shape, dtype=np.float32) -> np.ndarray:
        """A numpy array over page-locked host memory (kept alive by the context)."""
        dtype = np.dtype(dtype)
        n = int(np.prod(shape))
        p = self.lib.tc_host_alloc(self.handle, n * dtype.itemsize)
        if not p:
            raise TachyonCudaError(f"tc_host_alloc: {self.last_error()}")
        buf = (C.c_byte * (n * dtype.itemsize)).from_address(p)
        return np.frombuffer(buf, dtype=dtype).reshape(shape)

    PROFILE_STAGES = ("route", "dispatch", "gate_up", "quant_hidden", "down", "combine", "rmsnorm", "decode_block")

    def profile_enable(self, on: bool):
        self._check(self.lib.tc_profile_enable(self.handle, int(on)), "tc_profile_enable")

    def profile_read(self) -> dict:
        ms = np.zeros(8, np.float32)
        n = np.zeros(8, np.uint64)
        self._check(self.lib.tc_profile_read(self.handle, _ptr(ms), _ptr(n)), "tc_profile_read")
        return {name: (float(ms[i]), int(n[i])) for i, name in enumerate(self.PROFILE_STAGES)}

    def to_device(self, host: np.ndarray) -> "DeviceArray":
        arr = DeviceArray(self, host.shape, host.dtype)
        self.upload(arr.ptr, host)
        return arr

    def empty(self, shape, dtype=np.float32) -> "DeviceArray":
        return DeviceArray(self, shape, dtype)

    def rmsnorm(self, x: "DeviceArray", weight: "DeviceArray", eps: float, out: "DeviceArray"):
        t, n = x.shape
        self._check(self.lib.tc_rmsnorm(self.handle, x.ptr, weight.ptr, eps, t, n, out.ptr), "tc_rmsnorm")

    def dispatch_static(self, ids: "DeviceArray", t: int, experts: int, topk: int, counts: "DeviceArray",
                        offsets: "DeviceArray", perm: "DeviceArray", pos: "DeviceArray",
                        slot_token: "DeviceArray", active: "DeviceArray"):
        """The token -> expert dispatch with its scratch inside the library: allocates nothing.
        At most 16384 tokens and 256 experts; every buffer is the caller's."""
        self._check(self.lib.tc_dispatch_static(self.handle, ids.ptr, t, experts, topk, counts.ptr, offsets.ptr,
                                                perm.ptr, pos.ptr, slot_token.ptr, active.ptr),
                    "tc_dispatch_static")

    def int8_peak(self, min_ms: float = 50.0) -> dict:
        """Dense int8 tensor-core rate in Pop/s, from a run of at least min_ms milliseconds."""
        batches, ops, ms = 64, C.c_double(0.0), C.c_float(0.0)
        while True:
            self._check(self.lib.tc_int8_peak(self.handle, batches, C.byref(ops), C.byref(ms)), "tc_int8_peak")
            if ms.value >= min_ms or batches >= (1 << 24):
                break
            batches = int(batches * max(2.0, 1.2 * min_ms / max(ms.value, 1e-3)))
        return {"pops": ops.value / (ms.value * 1e-3) / 1e15, "ms": ms.value, "mma_per_sm": batches * 32,
                "shape": "tcgen05.mma kind::i8 m128 n256 k32, cta_group::1, operands resident in shared memory"}

    def umma_selftest(self, a_rows: np.ndarray, b_rows: np.ndarray) -> np.ndarray:
        """a_rows i8[128, 32] x b_rows i8[n, 32]^T through one tcgen05 MMA; returns i32[128, n]."""
        a_rows = np.ascontiguousarray(a_rows, np.int8)
        b_rows = np.ascontiguousarray(b_rows, np.int8)
        n = b_rows.shape[0]
        out = np.empty((128, n), np.int32)
        self._check(self.lib.tc_umma_selftest(self.handle, _ptr(a_rows), _ptr(b_rows), n, _ptr(out)),
                    "tc_umma_selftest")
        return out

    def capture_begin(self):
        self._check(self.lib.tc_capture_begin(self.handle), "tc_capture_begin")

    def capture_end(self) -> "Graph":
        g = self.lib.tc_capture_end(self.handle)
        if not g:
            raise TachyonCudaError(f"tc_capture_end: {self.last_error()}")
        return Graph(self, g)

    def timer_start(self):
        self._check(self.lib.tc_timer_start(self.handle), "tc_timer_start")

    def timer_stop_ms(self) -> float:
        ms = self.lib.tc_timer_stop_ms(self.handle)
        if ms < 0:
            raise TachyonCudaError(f"tc_timer_stop_ms: {self.last_error()}")
        return ms

    def launch_count(self) -> int:
        return int(self.lib.tc_launch_count(self.handle))


class DeviceArray:
    """A typed device buffer (``tc_malloc``), freed with its owner."""

    def __init__(self, ctx: Context, shape, dtype):
        self.ctx = ctx
        self.shape = tuple(int(s) for s in (shape if hasattr(shape, "__len__") else (shape,)))
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        self.ptr = ctx.malloc(max(self.nbytes, 1))

    def get(self) -> np.ndarray:
        out = np.empty(self.shape, self.dtype)
        if self.nbytes:
            self.ctx.download(out, self.ptr)
        return out

    def set(self, host: np.ndarray):
        host = np.ascontiguousarray(host, self.dtype)
        assert host.nbytes == self.nbytes
        self.ctx.upload(self.ptr, host)

    def free(self):
        if self.ptr and self.ctx.handle:
            self.ctx.free(self.ptr)
        self.ptr = 0

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Graph:
    def __init__(self, ctx: Context, handle):
        self.ctx, self.handle = ctx, handle

    def launch(self):
        self.ctx._check(self.ctx.lib.tc_graph_launch(self.handle), "tc_graph_launch")

    def free(self):
        if self.handle:
            self.ctx.lib.tc_graph_free(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class DeviceMatrix:
    """A ``Matrix`` uploaded byte for byte (``GpuMatrix::upload``, src/gpu/mod.rs:222-251)."""

    def __init__(self, ctx: Context, m: Matrix):
        self.ctx, self.kind, self.rows, self.cols = ctx, m.kind, m.rows, m.cols
        scales = None if m.scales is None else np.ascontiguousarray(m.scales)
        data = np.ascontiguousarray(m.data)
        self.nbytes = data.nbytes + (0 if scales is None else scales.nbytes)
        self.handle = ctx.lib.tc_matrix_upload(
            ctx.handle, m.kind, m.rows, m.cols, _ptr(scales), 0 if scales is None else scales.nbytes,
            _ptr(data), data.nbytes)
        if not self.handle:
            raise TachyonCudaError(f"tc_matrix_upload: {ctx.last_error()}")

    @classmethod
    def quantize(cls, ctx: Context, data: np.ndarray, rows: int, cols: int, fmt: str) -> "DeviceMatrix":
        """``Matrix::from_f32`` (src/weights.rs:82-105) on the device: uploads the f32 values and
        quantizes them there with Tachyon's own quantizers; same bytes as the host path."""
        from .weights import KIND_Q4, KIND_Q8

        kind = {"bf16": KIND_BF16, "q8": KIND_Q8, "int8": KIND_Q8, "q4": KIND_Q4, "int4": KIND_Q4}[fmt.lower()]
        data = np.ascontiguousarray(data, np.float32).reshape(-1)
        assert data.size == rows * cols
        self = cls.__new__(cls)
        self.ctx, self.kind, self.rows, self.cols = ctx, kind, rows, cols
        self.handle = ctx.lib.tc_matrix_quantize(ctx.handle, kind, rows, cols, _ptr(data))
        if not self.handle:
            raise TachyonCudaError(f"tc_matrix_quantize: {ctx.last_error()}")
        nb = cols // 32
        self.nbytes = {KIND_BF16: rows * cols * 2, KIND_Q8: rows * cols + rows * nb * 2,
                       KIND_Q4: rows * cols // 2 + rows * (-(-nb // 8) * 5) * 4}[kind]
        return self

    def to_host(self) -> Matrix:
        """The matrix's buffers copied back: a host ``Matrix`` with the same bytes."""
        from .weights import KIND_Q4, KIND_Q8

        nb = self.cols // 32
        if self.kind == KIND_BF16:
            scales, data = None, np.empty(self.rows * self.cols, np.uint16)
        elif self.kind == KIND_Q8:
            scales, data = np.empty(self.rows * nb, np.uint16), np.empty(self.rows * self.cols, np.int8)
        else:
            scales = np.empty(self.rows * (-(-nb // 8) * 5), np.uint32)
            data = np.empty(self.rows * self.cols // 2, np.uint8)
        rc = self.ctx.lib.tc_matrix_download(self.handle, _ptr(scales), 0 if scales is None else scales.nbytes,
                                             _ptr(data), data.nbytes)
        self.ctx._check(rc, "tc_matrix_download")
        return Matrix(self.kind, self.rows, self.cols, scales, data)

    def free(self):
        if self.handle and self.ctx.handle:
            self.ctx.lib.tc_matrix_free(self.handle)
        self.handle = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class MoeLayer:
    """One Granite MoE block on the device (``tc_moe_layer``)."""

    def __init__(self, ctx: Context, router: Matrix, gate_up: Matrix, down: Matrix, experts_per_token: int,
                 max_tokens: int):
        assert router.kind == KIND_BF16
        self.ctx = ctx
        self.hidden, self.experts = router.cols, router.rows
        self.inter, self.topk = down.cols, experts_per_token
        self.max_tokens = max_tokens
        # (Matrices already on the device, e.g. quantized there, are taken as they are.)
        self.router = router if isinstance(router, DeviceMatrix) else DeviceMatrix(ctx, router)
        self.gate_up = gate_up if isinstance(gate_up, DeviceMatrix) else DeviceMatrix(ctx, gate_up)
        self.down = down if isinstance(down, DeviceMatrix) else DeviceMatrix(ctx, down)
        self.weight_bytes = self.router.nbytes + self.gate_up.nbytes + self.down.nbytes
        self.handle = ctx.lib.tc_moe_layer_create(
            ctx.handle, self.hidden, self.experts, self.topk, self.inter, self.router.handle,
            self.gate_up.handle, self.down.handle, max_tokens)
        if not self.handle:
            raise TachyonCudaError(f"tc_moe_layer_create: {ctx.last_error()}")

    def detach_experts(self):
        """Drops the expert matrices as uploaded (the layer computes from its own re-tiled copies;
        only ``ARITH_CPU_LANES`` reads the uploaded ones again, and is refused from here on)."""
        self.ctx._check(self.ctx.lib.tc_moe_layer_detach_experts(self.handle), "tc_moe_layer_detach_experts")
        for m in (self.gate_up, self.down):
            m.free()

    def set_router_bias(self, bias):
        b = None if bias is None else np.ascontiguousarray(bias, np.float32)
        self.ctx._check(self.ctx.lib.tc_moe_set_router_bias(self.handle, _ptr(b)), "tc_moe_set_router_bias")

    def forward(self, x: DeviceArray, y: DeviceArray, t: int | None = None):
        """y[t, hidden] += moe(x[t, hidden]) on the device; returns without waiting."""
        t = x.shape[0] if t is None else t
        self.ctx._check(self.ctx.lib.tc_moe_forward(self.handle, x.ptr, t, y.ptr), "tc_moe_forward")

    def block(self, norm_weight: DeviceArray, eps: float, y: DeviceArray, t: int | None = None):
        """y[t, hidden] += moe(rmsnorm(y, norm_weight, eps)): the MLP block on the residual stream."""
        t = y.shape[0] if t is None else t
        self.ctx._check(self.ctx.lib.tc_moe_block(self.handle, norm_weight.ptr, eps, t, y.ptr), "tc_moe_block")

    def forward_host(self, x: np.ndarray, y: np.ndarray):
        """The same through host buffers (copies in and out, waits); y is updated in place."""
        x = np.ascontiguousarray(x, np.float32)
        assert y.dtype == np.float32 and y.flags["C_CONTIGUOUS"] and y.shape == x.shape
        self.ctx._check(self.ctx.lib.tc_moe_forward_host(self.handle, _ptr(x), x.shape[0], _ptr(y)),
                        "tc_moe_forward_host")

    def last_routing(self, t: int):
        ids = np.empty((t, self.topk), np.uint32)
        gates = np.empty((t, self.topk), np.float32)
        counts = np.empty(self.experts, np.uint32)
        logits = np.empty((t, self.experts), np.float32)
        self.ctx._check(self.ctx.lib.tc_moe_last_routing(self.handle, _ptr(ids), _ptr(gates), _ptr(counts),
                                                       _ptr(logits)), "tc_moe_last_routing")
        return ids, gates, counts, logits

    def last_dispatch(self, t: int):
        offsets = np.empty(self.experts + 1, np.uint32)
        perm = np.empty(t * self.topk, np.uint32)
        self.ctx._check(self.ctx.lib.tc_moe_last_dispatch(self.handle, _ptr(offsets), _ptr(perm)),
                        "tc_moe_last_dispatch")
        return offsets, perm

    def free(self):
        if getattr(self, "handle", None) and self.ctx.handle:
            self.ctx.lib.tc_moe_layer_free(self.handle)
        self.handle = None
        for m in (self.router, self.gate_up, self.down):
            m.free()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass
