"""Shared helpers for the parity tests: run a graph through the runtime and through the oracle."""

import torch

from oracle import metrics
from oracle.backend import OracleBuilder
from ttmlir_b200 import graphs

# Tolerances (floating point): PCC >= 0.999 and |got - want| <= atol + rtol*|want| with
# atol 1e-2 / rtol 2^-7 (one bf16 ulp) for bf16 results, atol 1e-4 / rtol 1e-4 for f32.
# Integer, quantized and index results must be bit-exact.
TOL = {torch.bfloat16: (0.999, 1e-2, 2.0 ** -7), torch.float16: (0.999, 1e-2, 2.0 ** -7),
       torch.float32: (0.999, 1e-4, 1e-4)}


def assert_matches(got: torch.Tensor, want: torch.Tensor, what: str = "", tol=None):
    assert list(got.shape) == list(want.shape), f"{what}: shape {list(got.shape)} != {list(want.shape)}"
    assert got.dtype == want.dtype, f"{what}: dtype {got.dtype} != {want.dtype}"
    if not want.is_floating_point():
        bad = (got != want).sum().item()
        assert bad == 0, f"{what}: {bad} of {want.numel()} integer elements differ"
        return
    pcc, atol, rtol = tol or TOL[want.dtype]
    ok, report = metrics.check_close(want, got, pcc, atol, rtol)
    assert ok, f"{what}: {report}"


def run_program(rt, device, binary_bytes, inputs, program=0):
    """ttrt-style run: load, to_layout every input, submit, to_host every output."""
    binary = rt.Binary.load_from_memory(binary_bytes)
    rt.set_compatible_device_runtime(binary)
    ins = []
    for i, t in enumerate(inputs):
        h = rt.from_torch(t)
        ins.append(rt.to_layout(h, device, rt.get_layout(binary, program, i)))
    outs = rt.submit(device, binary, program, ins)
    res = []
    for o in outs:
        hs = rt.to_host(o, untilize=True)
        res.append(rt.to_torch(hs[0]))
    return res


def oracle_results(graph_fn, inputs, mesh_shape=(1, 1), **kw):
    ob = OracleBuilder(inputs, mesh_shape=mesh_shape)
    graph_fn(ob, **kw)
    return ob.results()


def check_graph(rt, device, graph_fn, inputs, what, tol=None, **kw):
    buf = graphs.build_binary(graph_fn, **kw)
    got = run_program(rt, device, buf, inputs)
    want = oracle_results(graph_fn, inputs, **kw)
    assert len(got) == len(want)
    for i, (g, w) in enumerate(zip(got, want)):
        assert_matches(g, w, f"{what} output {i}", tol)
    return got, want


# Pooling cases recorded in tests/golden (pool/<name>) over an NHWC [2, 9, 11, 8] activation:
# name -> (kind, kernel, stride, padding in flatbuffer order (h, w) or (top, left, bottom, right),
#          dilation, ceil_mode, count_include_pad)
POOL_CASES = {
    "max_k2s2": ("max", (2, 2), (2, 2), (0, 0), (1, 1), False, True),
    "max_k3s2p1": ("max", (3, 3), (2, 2), (1, 1), (1, 1), False, True),
    "max_k3s2p1_ceil": ("max", (3, 3), (2, 2), (1, 1), (1, 1), True, True),
    "max_k3s1_dil2": ("max", (3, 3), (1, 1), (1, 1), (2, 2), False, True),
    "max_asym": ("max", (3, 2), (2, 1), (1, 2, 0, 1), (1, 1), False, True),
    "max_asym_ceil": ("max", (3, 3), (2, 2), (0, 0, 1, 1), (1, 1), True, True),
    "avg_k2s2": ("avg", (2, 2), (2, 2), (0, 0), (1, 1), False, True),
    "avg_k3s2p1": ("avg", (3, 3), (2, 2), (1, 1), (1, 1), False, True),
    "avg_k3s2p1_nopad": ("avg", (3, 3), (2, 2), (1, 1), (1, 1), False, False),
    "avg_k3s2p1_ceil": ("avg", (3, 3), (2, 2), (1, 1), (1, 1), True, True),
    "avg_k3s2p1_ceil_nopad": ("avg", (3, 3), (2, 2), (1, 1), (1, 1), True, False),
    "avg_asym": ("avg", (3, 3), (2, 2), (1, 2, 0, 1), (1, 1), False, True),
    "avg_asym_nopad": ("avg", (3, 3), (2, 2), (1, 2, 0, 1), (1, 1), False, False),
    "avg_bigpad": ("avg", (2, 2), (2, 2), (2, 2), (1, 1), False, True),
    "avg_bigpad_nopad": ("avg", (2, 2), (2, 2), (2, 2), (1, 1), False, False),
}


def pool_on(b, x, case, batch=2, height=9, width=11, channels=8):
    """Emits (or, on the oracle builder, computes) one POOL_CASES entry on the flattened activation `x`."""
    kind, kernel, stride, padding, dilation, ceil, include = POOL_CASES[case]
    if kind == "max":
        return b.max_pool2d(x, batch, height, width, channels, kernel, stride, padding, dilation, ceil)
    return b.avg_pool2d(x, batch, height, width, channels, kernel, stride, padding, ceil, include)


DTYPE_NAME = {torch.float32: "Float32", torch.bfloat16: "BFloat16", torch.float16: "Float16", torch.int32: "Int32",
              torch.int8: "Int8", torch.uint8: "UInt8"}


def run_body(rt, device, body, inputs, mesh_shape=(1, 1)):
    """Runs `body(b, *values)` (returning one value or a tuple) on the GPU and on the oracle."""
    def graph(b):
        vals = [b.input(list(t.shape), DTYPE_NAME[t.dtype]) for t in inputs]
        out = body(b, *vals)
        b.output(*(out if isinstance(out, (tuple, list)) else (out,)))
    buf = graphs.build_binary(graph, mesh_shape=mesh_shape)
    got = run_program(rt, device, buf, inputs)
    want = oracle_results(graph, inputs, mesh_shape=mesh_shape)
    return got, want


class KernelHarness:
    """Raw access to the kernel-level C ABI (include/ttb_kernels.h) for tests: device buffers
    from torch CPU tensors, one stream, explicit copies."""

    def __init__(self, rt):
        import ctypes
        self.ct = ctypes
        self.lib = rt.lib
        self.rt = rt
        self._check(self.lib.ttb_set_device(0))
        s = ctypes.c_void_p()
        self._check(self.lib.ttb_stream_create(ctypes.byref(s)))
        self.stream = s
        self._bufs = []

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.ttb_last_error().decode())

    def upload(self, t: torch.Tensor):
        t = t.contiguous()
        p = self.ct.c_void_p()
        n = t.numel() * t.element_size()
        self._check(self.lib.ttb_malloc(self.ct.byref(p), self.ct.c_size_t(max(n, 16)), self.stream))
        self._check(self.lib.ttb_memcpy_h2d(p, self.ct.c_void_p(t.data_ptr()), self.ct.c_size_t(n), self.stream))
        self._check(self.lib.ttb_stream_sync(self.stream))
        self._bufs.append(p)
        return p

    def empty(self, shape, dtype):
        return self.upload(torch.zeros(shape, dtype=dtype))

    def download(self, p, shape, dtype):
        out = torch.empty(shape, dtype=dtype)
        n = out.numel() * out.element_size()
        self._check(self.lib.ttb_memcpy_d2h(self.ct.c_void_p(out.data_ptr()), p, self.ct.c_size_t(n), self.stream))
        self._check(self.lib.ttb_stream_sync(self.stream))
        return out

    def sync(self):
        self._check(self.lib.ttb_stream_sync(self.stream))

    def close(self):
        for p in self._bufs:
            self.lib.ttb_free(p, self.stream)
        self._bufs = []
        self.lib.ttb_stream_sync(self.stream)
        self.lib.ttb_stream_destroy(self.stream)


class TeacherForcedOracle(OracleBuilder):
    """The oracle run op by op on the GPU's own operands.

    `gpu_outputs` maps an op's location string (as the debug hooks report it, 'loc("name")') to the
    tensor the GPU produced there.  Every graph op that carries a `loc` is evaluated by the oracle on
    the values handed on so far, compared with the GPU's output of the same op (the comparison goes to
    `self.report[name]`), and then REPLACED by the GPU's output, so that the next op sees exactly what
    the GPU's next kernel saw.  What is measured per op is then the arithmetic of that one kernel, not
    the accumulated effect of earlier single-ulp rounding differences."""

    PASS_THROUGH = {"input", "output", "results"}

    def __init__(self, inputs, gpu_outputs, mesh_shape=(1, 1)):
        super().__init__(inputs, mesh_shape=mesh_shape)
        self._gpu = gpu_outputs
        self.report = {}

    def __getattribute__(self, name):
        attr = super().__getattribute__(name)
        if name.startswith("_") or name in TeacherForcedOracle.PASS_THROUGH or not callable(attr):
            return attr

        def wrapped(*args, **kw):
            res = attr(*args, **kw)
            loc = kw.get("loc")
            got = self._gpu.get(f'loc("{loc}")') if loc else None
            if got is None or not hasattr(res, "t") or isinstance(res.t, list):
                return res
            want = res.t
            got = got.reshape(want.shape)
            self.report[loc] = op_error(got, want)
            return type(res)(got)
        return wrapped


def op_error(got: torch.Tensor, want: torch.Tensor) -> dict:
    """Error of one op's output in units that do not depend on its magnitude: the share of elements that
    are bit-equal, the largest error in bf16 ulps of the element it belongs to (beyond an absolute 1e-2),
    and the Pearson correlation."""
    if not want.is_floating_point():
        return {"equal": float((got == want).float().mean().item()), "max_ulps": 0.0 if torch.equal(got, want) else float("inf"),
                "pcc": 1.0 if torch.equal(got, want) else 0.0}
    g, w = got.float(), want.float()
    err = (g - w).abs()
    ulp = torch.maximum(w.abs(), g.abs()) * 2.0 ** -7          # a bf16 ulp is between 2^-8 and 2^-7 of the magnitude
    beyond = torch.clamp(err - 1e-2, min=0.0) / torch.clamp(ulp, min=1e-30)
    return {"equal": float((got == want).float().mean().item()), "max_ulps": float(beyond.max().item()),
            "max_abs": float(err.max().item()), "pcc": float(metrics.get_pcc(want, got))}
