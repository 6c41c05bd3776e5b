"""Authoring TTNN flatbuffers (.ttnn) without the tt-mlir compiler.

The reference produces these files with `ttmlir-opt --ttir-to-ttnn-backend-pipeline` followed by
`ttmlir-translate --ttnn-to-flatbuffer` (lib/Target/TTNN/TTNNToFlatbuffer.cpp); neither tool can
be built where this repo is developed, so this module writes the same wire format directly.
It mirrors what the serialiser emits for the optimizer-off pipeline:

* one `TensorRef` table per SSA value, ids assigned in emission order, the same table shared by
  the producing op's `out` and every consumer (TTNNToFlatbuffer.cpp:141-167 and
  include/ttmlir/Target/Utils/FlatbufferObjectCache.h);
* device tensors are DRAM / interleaved / tile (32x32), host tensors row-major (1x1);
* a `GetDeviceOp` first, a `DeallocateOp` after the last use of every intermediate
  (lib/Dialect/TTNN/Pipelines/TTNNPipelines.cpp:521), `debug_info` = a printed op,
  `loc_info` = the op's location string (include/ttmlir/Target/Utils/FuncOpToProgram.h:191-196);
* multi-device programs carry `mesh_shape` and start / end with DistributeTensorOp /
  AggregateTensorOp the way `ttir.mesh_shard` lowers (lib/Conversion/TTIRToTTNN/TTIRToTTNN.cpp:2753-2888).

What it cannot reproduce is the schema hash (see schema/ttnn_schema.py).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

from .schema.fbs import Writer
from .schema.ttnn_schema import FILE_IDENTIFIER, S, SCHEMA_HASH

ITEMSIZE = {"Float32": 4, "Float16": 2, "BFloat16": 2, "UInt32": 4, "UInt16": 2, "UInt8": 1, "Int32": 4, "Int8": 1}


class Value:
    """An SSA value: shape, dtype and the TensorRef dict every user shares."""

    def __init__(self, ref: dict, shape: Sequence[int], dtype: str, on_device: bool):
        self.ref = ref
        self.shape = list(shape)
        self.dtype = dtype
        self.on_device = on_device

    @property
    def id(self) -> int:
        return self.ref["global_id"]

    def __repr__(self):
        return f"%{self.id}:{self.dtype}{self.shape}"


def _volume(shape):
    v = 1
    for d in shape:
        v *= d
    return v


def _norm(dim, rank):
    return dim + rank if dim < 0 else dim


def _broadcast(a, b):
    out = []
    ra, rb = list(reversed(a)), list(reversed(b))
    for i in range(max(len(a), len(b))):
        x = ra[i] if i < len(ra) else 1
        y = rb[i] if i < len(rb) else 1
        if x != y and x != 1 and y != 1:
            raise ValueError(f"shapes {a} and {b} do not broadcast")
        out.append(max(x, y))
    return list(reversed(out))


class ProgramBuilder:
    def __init__(self, binary: "BinaryBuilder", name: str, mesh_shape: Tuple[int, int] = (1, 1)):
        self._bin = binary
        self.name = name
        self.mesh_shape = tuple(mesh_shape)
        self.inputs: List[Value] = []
        self.outputs: List[Value] = []
        self.ops: List[dict] = []
        self._op_values: List[Tuple[List[Value], List[Value]]] = []
        self.private = False
        self.goldens = {}                  # key -> [GoldenDeviceTensor], see golden()
        self.index = len(binary.programs)  # position in the binary = the id other programs call it by
        self.device_ref = {"global_id": binary.next_id()}
        self._emit("GetDeviceOp", {"mesh": self.mesh_shape, "offset": (0, 0),
                                   "chip_ids": list(range(self.mesh_shape[0] * self.mesh_shape[1])),
                                   "out": self.device_ref}, [], [], "get_device")

    # ---- plumbing ---------------------------------------------------------------------------
    def _value(self, shape, dtype, on_device=True, tile=None) -> Value:
        if tile is None:
            tile = on_device
        multi = self.mesh_shape[0] * self.mesh_shape[1] > 1 and on_device
        ref = {
            "global_id": self._bin.next_id(),
            "desc": {
                "shape": list(shape),
                "mesh_shape": list(self.mesh_shape) if multi else [1, 1],
                "layout": {
                    "oob_val": "Undef",
                    "memory_desc": {
                        "storage_type": "Device" if on_device else "Host",
                        "tile_shape": (32, 32) if tile else (1, 1),
                        "data_type": dtype,
                        "memory_config": {"tensor_memory_layout": "Interleaved", "buffer_type": "DRAM"}
                        if on_device else None,
                    },
                },
                "shard_status": "Unsharded",
                "local_shape": list(shape),
            },
        }
        return Value(ref, shape, dtype, on_device)

    def _emit(self, op_type: str, table: dict, ins: List[Value], outs: List[Value], loc: Optional[str]):
        idx = len(self.ops)
        loc = loc or f"{op_type}_{idx}"
        ins_s = ", ".join(f"%{v.id}" for v in ins)
        outs_s = ", ".join(f"%{v.id}" for v in outs)
        snake = op_type[:-2] if op_type.endswith("Op") else op_type
        dbg = f'{outs_s + " = " if outs_s else ""}"ttnn.{snake}"({ins_s})'
        self.ops.append({"type": (op_type, table), "debug_info": dbg, "loc_info": f'loc("{loc}")'})
        self._op_values.append((ins, outs))

    def _mc(self):
        return {"tensor_memory_layout": "Interleaved", "buffer_type": "DRAM"}

    # ---- program interface ------------------------------------------------------------------
    def input(self, shape, dtype: str, on_device: bool = True) -> Value:
        v = self._value(shape, dtype, on_device)
        self.inputs.append(v)
        return v

    def output(self, *values: Value):
        self.outputs.extend(values)

    # ---- layout / creation -------------------------------------------------------------------
    def to_device(self, x: Value, loc=None) -> Value:
        out = self._value(x.shape, x.dtype, True, tile=False)
        self._emit("ToDeviceOp", {"in": x.ref, "device": self.device_ref, "memcfg": self._mc(), "out": out.ref},
                   [x], [out], loc)
        return out

    def from_device(self, x: Value, loc=None) -> Value:
        out = self._value(x.shape, x.dtype, False)
        self._emit("FromDeviceOp", {"in": x.ref, "out": out.ref}, [x], [out], loc)
        return out

    def to_layout(self, x: Value, layout: str = "Tile", dtype: Optional[str] = None, on_device: Optional[bool] = None,
                  loc=None) -> Value:
        dev = x.on_device if on_device is None else on_device
        out = self._value(x.shape, dtype or x.dtype, dev, tile=(layout == "Tile"))
        self._emit("ToLayoutOp", {"in": x.ref, "layout": layout, "dtype": dtype, "memcfg": self._mc() if dev else None,
                                  "out": out.ref}, [x], [out], loc)
        return out

    def typecast(self, x: Value, dtype: str, loc=None) -> Value:
        out = self._value(x.shape, dtype)
        self._emit("TypecastOp", {"in": x.ref, "dtype": dtype, "memcfg": self._mc(), "out": out.ref}, [x], [out], loc)
        return out

    def full(self, shape, value, dtype: str, loc=None) -> Value:
        out = self._value(shape, dtype)
        fv = ("FP", {"value": float(value)}) if isinstance(value, float) else ("I32", {"value": int(value)})
        self._emit("FullOp", {"device": self.device_ref, "shape": list(shape), "fill_value": fv, "dtype": dtype,
                              "layout": "Tile", "memcfg": self._mc(), "out": out.ref}, [], [out], loc)
        return out

    def zeros(self, shape, dtype: str, loc=None) -> Value:
        out = self._value(shape, dtype)
        self._emit("NamedFullOp", {"type": "Zeros", "device": self.device_ref, "shape": list(shape), "dtype": dtype,
                                   "layout": "Tile", "memcfg": self._mc(), "out": out.ref}, [], [out], loc)
        return out

    def ones(self, shape, dtype: str, loc=None) -> Value:
        out = self._value(shape, dtype)
        self._emit("NamedFullOp", {"type": "Ones", "device": self.device_ref, "shape": list(shape), "dtype": dtype,
                                   "layout": "Tile", "memcfg": self._mc(), "out": out.ref}, [], [out], loc)
        return out

    def constant(self, data: bytes, shape, dtype: str, loc=None) -> Value:
        assert len(data) == _volume(shape) * ITEMSIZE[dtype]
        out = self._value(shape, dtype)
        self._emit("ConstantOp", {"device": self.device_ref, "input": data, "input_dtype": dtype, "dtype": dtype,
                                  "layout": "Tile", "memcfg": self._mc(), "out": out.ref}, [], [out], loc)
        return out

    def arange(self, start, end, step, dtype: str, loc=None) -> Value:
        n = max(0, int(math.ceil((end - start) / step)))
        out = self._value([n], dtype)
        self._emit("ArangeOp", {"device": self.device_ref, "start": float(start), "end": float(end),
                                "step": float(step), "dtype": dtype, "layout": "Tile", "memcfg": self._mc(),
                                "out": out.ref}, [], [out], loc)
        return out

    def deallocate(self, x: Value, force: bool = False):
        self._emit("DeallocateOp", {"in": x.ref, "force": force}, [x], [], None)

    # ---- eltwise --------------------------------------------------------------------------------
    def unary(self, kind: str, x: Value, param: Optional[float] = None, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        t = {"type": kind, "in": x.ref, "memory_config": self._mc(), "out": out.ref}
        if param is not None:
            t["params"] = ("EltwiseOpWithFloatParams", {"parameter": float(param)})
        self._emit("EltwiseUnaryOp", t, [x], [out], loc)
        return out

    def relu(self, x, loc=None): return self.unary("Relu", x, loc=loc)
    def silu(self, x, loc=None): return self.unary("Silu", x, loc=loc)
    def exp(self, x, loc=None): return self.unary("Exp", x, loc=loc)
    def neg(self, x, loc=None): return self.unary("Neg", x, loc=loc)
    def sigmoid(self, x, loc=None): return self.unary("Sigmoid", x, loc=loc)

    def clamp(self, x: Value, lo: float, hi: float, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("EltwiseUnaryCompositeOp", {
            "type": "ClampScalar", "in": x.ref, "memory_config": self._mc(), "out": out.ref,
            "params": ("ClampScalarOpParams", {"min": ("FP", {"value": float(lo)}), "max": ("FP", {"value": float(hi)})})},
            [x], [out], loc)
        return out

    def binary(self, kind: str, a: Value, b: Value, dtype: Optional[str] = None, loc=None) -> Value:
        out = self._value(_broadcast(a.shape, b.shape), dtype or a.dtype)
        composite = kind in S.enums["EltwiseBinaryCompositeOpType"].values
        if composite:
            self._emit("EltwiseBinaryCompositeOp", {"type": kind, "lhs": a.ref, "rhs": b.ref,
                                                    "memory_config": self._mc(), "out": out.ref}, [a, b], [out], loc)
        else:
            self._emit("EltwiseBinaryOp", {"type": kind, "lhs": a.ref, "rhs": b.ref, "output_dtype": dtype,
                                           "memory_config": self._mc(), "out": out.ref}, [a, b], [out], loc)
        return out

    def add(self, a, b, loc=None): return self.binary("Add", a, b, loc=loc)
    def multiply(self, a, b, loc=None): return self.binary("Multiply", a, b, loc=loc)
    def subtract(self, a, b, loc=None): return self.binary("Subtract", a, b, loc=loc)
    def divide(self, a, b, loc=None): return self.binary("Divide", a, b, loc=loc)
    def maximum(self, a, b, loc=None): return self.binary("Maximum", a, b, loc=loc)

    def where(self, c: Value, a: Value, b: Value, loc=None) -> Value:
        out = self._value(_broadcast(_broadcast(c.shape, a.shape), b.shape), a.dtype)
        self._emit("EltwiseTernaryWhereOp", {"first": c.ref, "second": a.ref, "third": b.ref,
                                             "memory_config": self._mc(), "out": out.ref}, [c, a, b], [out], loc)
        return out

    # ---- quantization ---------------------------------------------------------------------------
    @staticmethod
    def _scale(s):
        return ("PerAxisScale", {"scale": s.ref}) if isinstance(s, Value) else ("PerTensorScale", {"scale": float(s)})

    @staticmethod
    def _zp(z):
        return ("PerAxisZeroPoint", {"zero_point": z.ref}) if isinstance(z, Value) else \
            ("PerTensorZeroPoint", {"zero_point": int(z)})

    def quantize(self, x: Value, scale, zero_point, out_dtype: str = "Int32", axis: Optional[int] = None, loc=None):
        out = self._value(x.shape, out_dtype)
        ins = [x] + [p for p in (scale, zero_point) if isinstance(p, Value)]
        self._emit("EltwiseQuantizationOp", {
            "type": "Quantize", "in": x.ref, "axis": axis, "output_dtype": out_dtype, "memory_config": self._mc(),
            "out": out.ref,
            "params": ("QuantizeDequantizeOpParams", {"scale": self._scale(scale), "zero_point": self._zp(zero_point)})},
            ins, [out], loc)
        return out

    def dequantize(self, x: Value, scale, zero_point, out_dtype: str = "Float32", axis: Optional[int] = None, loc=None):
        out = self._value(x.shape, out_dtype)
        ins = [x] + [p for p in (scale, zero_point) if isinstance(p, Value)]
        self._emit("EltwiseQuantizationOp", {
            "type": "Dequantize", "in": x.ref, "axis": axis, "output_dtype": out_dtype, "memory_config": self._mc(),
            "out": out.ref,
            "params": ("QuantizeDequantizeOpParams", {"scale": self._scale(scale), "zero_point": self._zp(zero_point)})},
            ins, [out], loc)
        return out

    def requantize(self, x: Value, in_scale, in_zp, out_scale, out_zp, out_dtype: Optional[str] = None,
                   axis: Optional[int] = None, loc=None):
        out = self._value(x.shape, out_dtype or x.dtype)
        ins = [x] + [p for p in (in_scale, in_zp, out_scale, out_zp) if isinstance(p, Value)]
        self._emit("EltwiseQuantizationOp", {
            "type": "Requantize", "in": x.ref, "axis": axis, "output_dtype": out_dtype or x.dtype,
            "memory_config": self._mc(), "out": out.ref,
            "params": ("RequantizeOpParams", {"in_scale": self._scale(in_scale), "in_zero_point": self._zp(in_zp),
                                              "out_scale": self._scale(out_scale), "out_zero_point": self._zp(out_zp)})},
            ins, [out], loc)
        return out

    # ---- contractions ------------------------------------------------------------------------------
    @staticmethod
    def _mm_shape(a, b, ta, tb):
        a, b = list(a), list(b)
        if len(a) == 1:
            a = [1] + a
        if len(b) == 1:
            b = b + [1]
        m, k = (a[-1], a[-2]) if ta else (a[-2], a[-1])
        kb, n = (b[-1], b[-2]) if tb else (b[-2], b[-1])
        if k != kb:
            raise ValueError(f"matmul inner dims differ: {k} vs {kb}")
        batch = _broadcast(a[:-2], b[:-2])
        return batch + [m, n]

    def matmul(self, a: Value, b: Value, transpose_a=False, transpose_b=False, activation: Optional[str] = None,
               out_dtype: Optional[str] = None, loc=None) -> Value:
        """`out_dtype` differs from the operands' type for a matmul on quantized (8-bit integer) operands,
        whose result is the Int32 accumulator (lib/Dialect/TTIR/IR/TTIROps.cpp:1516-1577 does the same for
        the quantized convolution)."""
        out = self._value(self._mm_shape(a.shape, b.shape, transpose_a, transpose_b), out_dtype or a.dtype)
        self._emit("MatmulOp", {"a": a.ref, "b": b.ref, "out": out.ref, "transpose_a": transpose_a,
                                "transpose_b": transpose_b, "activation": activation}, [a, b], [out], loc)
        return out

    def linear(self, a: Value, b: Value, bias: Optional[Value] = None, transpose_a=False, transpose_b=False,
               activation: Optional[str] = None, loc=None) -> Value:
        out = self._value(self._mm_shape(a.shape, b.shape, transpose_a, transpose_b), a.dtype)
        self._emit("LinearOp", {"a": a.ref, "b": b.ref, "bias": bias.ref if bias else None, "out": out.ref,
                                "transpose_a": transpose_a, "transpose_b": transpose_b, "activation": activation},
                   [a, b] + ([bias] if bias else []), [out], loc)
        return out

    def conv2d(self, x: Value, w: Value, bias: Optional[Value], batch: int, height: int, width: int, stride=(1, 1),
               padding=(0, 0, 0, 0), dilation=(1, 1), groups: int = 1, out_dtype: Optional[str] = None, loc=None) -> Value:
        """x is [1, 1, N*H*W, C] (the flattened form the compiler emits) or [N, H, W, C];
        w is [O, C/groups, kH, kW]; bias [1, 1, 1, O].  Output keeps x's rank.  `out_dtype` "Int32" for a
        convolution on quantized (8-bit integer) operands, whose result is the accumulator."""
        o, cg, kh, kw = getattr(w, "filter_shape", w.shape)   # a prepared weight remembers its filter's shape
        c = cg * groups
        pad = list(padding) if len(padding) == 4 else [padding[0], padding[1], padding[0], padding[1]]
        ho = (height + pad[0] + pad[2] - dilation[0] * (kh - 1) - 1) // stride[0] + 1
        wo = (width + pad[1] + pad[3] - dilation[1] * (kw - 1) - 1) // stride[1] + 1
        oshape = [1, 1, batch * ho * wo, o] if x.shape[:2] == [1, 1] and len(x.shape) == 4 and x.shape[2] == batch * height * width \
            else [batch, ho, wo, o]
        out = self._value(oshape, out_dtype or x.dtype)
        self._emit("Conv2dOp", {
            "input": x.ref, "weight": w.ref, "bias": bias.ref if bias else None, "out": out.ref,
            "device": self.device_ref, "in_channels": c, "out_channels": o, "batch_size": batch,
            "input_height": height, "input_width": width, "kernel_size": [kh, kw], "stride": list(stride),
            "padding": pad, "dilation": list(dilation), "groups": groups, "output_dtype": out_dtype or x.dtype},
            [x, w] + ([bias] if bias else []), [out], loc)
        return out

    # ---- normalisation / reduction ------------------------------------------------------------------
    def softmax(self, x: Value, dim: int = -1, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("SoftmaxOp", {"in": x.ref, "out": out.ref, "dimension": dim, "numeric_stable": True}, [x], [out], loc)
        return out

    def rms_norm(self, x: Value, weight: Optional[Value], bias: Optional[Value] = None, epsilon: float = 1e-5,
                 loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("RMSNormOp", {"input": x.ref, "weight": weight.ref if weight else None,
                                 "bias": bias.ref if bias else None, "epsilon": float(epsilon),
                                 "memory_config": self._mc(), "out": out.ref},
                   [x] + [v for v in (weight, bias) if v], [out], loc)
        return out

    def reduce(self, kind: str, x: Value, dims: Optional[Sequence[int]], keep_dim: bool, loc=None) -> Value:
        rank = len(x.shape)
        ds = sorted(_norm(d, rank) for d in dims) if dims else list(range(rank))
        shape = [1 if i in ds else s for i, s in enumerate(x.shape)] if keep_dim else \
            [s for i, s in enumerate(x.shape) if i not in ds]
        out = self._value(shape, x.dtype)
        self._emit("ReductionOp", {"type": kind, "in": x.ref, "out": out.ref, "dim_arg": list(dims) if dims else None,
                                   "keep_dim": keep_dim}, [x], [out], loc)
        return out

    # ---- data movement -----------------------------------------------------------------------------------
    def reshape(self, x: Value, shape, loc=None) -> Value:
        shape = list(shape)
        if -1 in shape:
            known = _volume([s for s in shape if s != -1])
            shape[shape.index(-1)] = _volume(x.shape) // known
        assert _volume(shape) == _volume(x.shape)
        out = self._value(shape, x.dtype)
        self._emit("ReshapeOp", {"in": x.ref, "out": out.ref, "shape": shape, "memory_config": self._mc()}, [x], [out], loc)
        return out

    def permute(self, x: Value, perm, loc=None) -> Value:
        out = self._value([x.shape[p] for p in perm], x.dtype)
        self._emit("PermuteOp", {"in": x.ref, "permutation": list(perm), "memory_config": self._mc(), "pad_value": 0.0,
                                 "out": out.ref}, [x], [out], loc)
        return out

    def transpose(self, x: Value, d0: int, d1: int, loc=None) -> Value:
        shape = list(x.shape)
        a, b = _norm(d0, len(shape)), _norm(d1, len(shape))
        shape[a], shape[b] = shape[b], shape[a]
        out = self._value(shape, x.dtype)
        self._emit("TransposeOp", {"in": x.ref, "out": out.ref, "dim0": d0, "dim1": d1}, [x], [out], loc)
        return out

    def concat(self, xs: Sequence[Value], dim: int, loc=None) -> Value:
        shape = list(xs[0].shape)
        d = _norm(dim, len(shape))
        shape[d] = sum(v.shape[d] for v in xs)
        out = self._value(shape, xs[0].dtype)
        self._emit("ConcatOp", {"inputs": [v.ref for v in xs], "out": out.ref, "dim": dim, "memory_config": self._mc()},
                   list(xs), [out], loc)
        return out

    def slice(self, x: Value, begins, ends, step=None, loc=None) -> Value:
        step = list(step) if step else [1] * len(x.shape)
        shape = [(e - b + s - 1) // s for b, e, s in zip(begins, ends, step)]
        out = self._value(shape, x.dtype)
        self._emit("SliceOp", {"type": "SliceStaticOp", "in": x.ref, "out": out.ref, "step": step,
                               "params": ("SliceStaticOpParams", {"begins": list(begins), "ends": list(ends)})},
                   [x], [out], loc)
        return out

    def repeat(self, x: Value, repeats, loc=None) -> Value:
        out = self._value([s * r for s, r in zip(x.shape, repeats)], x.dtype)
        self._emit("RepeatOp", {"in": x.ref, "out": out.ref, "repeat_dims": list(repeats), "memcfg": self._mc()},
                   [x], [out], loc)
        return out

    def repeat_interleave(self, x: Value, repeats: int, dim: int, loc=None) -> Value:
        shape = list(x.shape)
        shape[_norm(dim, len(shape))] *= repeats
        out = self._value(shape, x.dtype)
        self._emit("RepeatInterleaveOp", {"input": x.ref, "out": out.ref, "repeats": repeats, "dim": dim,
                                          "memory_config": self._mc()}, [x], [out], loc)
        return out

    # ---- transformer ------------------------------------------------------------------------------------------
    def concatenate_heads(self, x: Value, loc=None) -> Value:
        b, h, s, d = x.shape
        out = self._value([b, s, h * d], x.dtype)
        self._emit("ConcatenateHeadsOp", {"in": x.ref, "out": out.ref, "memcfg": self._mc()}, [x], [out], loc)
        return out

    def split_query_key_value_and_split_heads(self, x: Value, kv: Optional[Value], num_heads: int,
                                              num_kv_heads: Optional[int] = None, transpose_key: bool = False, loc=None):
        b, s, hidden = x.shape
        hkv = num_kv_heads if num_kv_heads is not None else num_heads
        d = hidden // num_heads if kv is not None else hidden // (num_heads + 2 * hkv)
        q = self._value([b, num_heads, s, d], x.dtype)
        k = self._value([b, hkv, d, s] if transpose_key else [b, hkv, s, d], x.dtype)
        v = self._value([b, hkv, s, d], x.dtype)
        self._emit("SplitQueryKeyValueAndSplitHeadsOp", {
            "in": x.ref, "kv_input": kv.ref if kv else None, "q_out": q.ref, "k_out": k.ref, "v_out": v.ref,
            "num_heads": num_heads, "num_kv_heads": num_kv_heads, "transpose_key": transpose_key,
            "memcfg": self._mc()}, [x] + ([kv] if kv else []), [q, k, v], loc)
        return q, k, v

    def rotary_embedding(self, x: Value, cos: Value, sin: Value, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("RotaryEmbeddingOp", {"input": x.ref, "cos_cache": cos.ref, "sin_cache": sin.ref, "out": out.ref,
                                         "memcfg": self._mc()}, [x, cos, sin], [out], loc)
        return out

    def scaled_dot_product_attention(self, q: Value, k: Value, v: Value, is_causal: bool = True,
                                     mask: Optional[Value] = None, scale: Optional[float] = None, loc=None) -> Value:
        out = self._value(q.shape, q.dtype)
        self._emit("ScaledDotProductAttentionOp", {
            "query": q.ref, "key": k.ref, "value": v.ref, "is_causal": is_causal,
            "attention_mask": mask.ref if mask else None, "scale": scale, "out": out.ref, "memcfg": self._mc()},
            [q, k, v] + ([mask] if mask else []), [out], loc)
        return out

    # ---- mesh ----------------------------------------------------------------------------------------------------
    def _axis_size(self, cluster_axis: int) -> int:
        return self.mesh_shape[cluster_axis]

    def distribute(self, x: Value, shard_dim: Optional[int], cluster_axis: int = 1, on_device: bool = True, loc=None) -> Value:
        """ttir.mesh_shard full_to_shard: shard `shard_dim` over `cluster_axis`, or replicate (None)."""
        n = self._axis_size(cluster_axis)
        placements = [("Replicate", -1), ("Replicate", -1)]
        shape = list(x.shape)
        if shard_dim is not None:
            placements[cluster_axis] = ("Shard", shard_dim)
            assert shape[shard_dim] % n == 0
            shape[shard_dim] //= n
        out = self._value(shape, x.dtype, on_device)
        self._emit("DistributeTensorOp", {
            "in": x.ref, "out": out.ref, "device": self.device_ref,
            "mapper_config": {"placements": placements, "mesh_shape_override": list(self.mesh_shape)}},
            [x], [out], loc)
        return out

    def aggregate(self, x: Value, shard_dim: Optional[int], cluster_axis: int = 1, loc=None) -> Value:
        """ttir.mesh_shard shard_to_full: concatenate `shard_dim` over `cluster_axis`, or take one replica."""
        n = self._axis_size(cluster_axis)
        shape = list(x.shape)
        if shard_dim is None:
            dims, override = [0], [1]
        else:
            rank = len(shape)
            other = next(d for d in range(rank - 1, -1, -1) if d != shard_dim) if rank > 1 else 0
            dims, override = [other, other], [1, 1]
            dims[cluster_axis] = shard_dim
            override[cluster_axis] = n
            shape[shard_dim] *= n
        out = self._value(shape, x.dtype, False)
        self._emit("AggregateTensorOp", {"in": x.ref, "out": out.ref, "device": self.device_ref,
                                         "composer_config": {"dims": dims, "mesh_shape_override": override}},
                   [x], [out], loc)
        return out

    def all_reduce(self, x: Value, reduce_type: int = 0, cluster_axis: int = 1, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("AllReduceOp", {"in": x.ref, "out": out.ref, "reduce_type": reduce_type, "cluster_axis": cluster_axis,
                                   "memory_config": self._mc()}, [x], [out], loc)
        return out

    def all_gather(self, x: Value, dim: int, cluster_axis: int = 1, loc=None) -> Value:
        shape = list(x.shape)
        shape[_norm(dim, len(shape))] *= self._axis_size(cluster_axis)
        out = self._value(shape, x.dtype)
        self._emit("AllGatherOp", {"in": x.ref, "out": out.ref, "all_gather_dim": dim, "cluster_axis": cluster_axis,
                                   "memory_config": self._mc()}, [x], [out], loc)
        return out

    def reduce_scatter(self, x: Value, dim: int, reduce_type: int = 0, cluster_axis: int = 1, loc=None) -> Value:
        shape = list(x.shape)
        d = _norm(dim, len(shape))
        assert shape[d] % self._axis_size(cluster_axis) == 0
        shape[d] //= self._axis_size(cluster_axis)
        out = self._value(shape, x.dtype)
        self._emit("ReduceScatterOp", {"in": x.ref, "out": out.ref, "scatter_dim": dim, "reduce_type": reduce_type,
                                       "cluster_axis": cluster_axis, "memory_config": self._mc()}, [x], [out], loc)
        return out

    def mesh_partition(self, x: Value, dim: int, cluster_axis: int = 1, loc=None) -> Value:
        shape = list(x.shape)
        d = _norm(dim, len(shape))
        shape[d] //= self._axis_size(cluster_axis)
        out = self._value(shape, x.dtype)
        self._emit("MeshPartitionOp", {"in": x.ref, "out": out.ref, "dim": dim, "cluster_axis": cluster_axis,
                                       "memory_config": self._mc()}, [x], [out], loc)
        return out

    def cpu_op(self, ins: Sequence[Value], out_shape, out_dtype: str, func_name: str, loc=None) -> Value:
        """A CPU-hoisted call, as the compiler emits for ttir ops tagged for host execution."""
        out = self._value(out_shape, out_dtype, False)
        self._emit("CpuOp", {"ins": [v.ref for v in ins], "outs": [out.ref], "func_name": func_name, "dylib_id": 0},
                   list(ins), [out], loc)
        return out

    # ---- wider op set: normalisation, pooling, embedding, argmax, pad, cumsum ------------------------------------
    def layer_norm(self, x: Value, weight: Optional[Value] = None, bias: Optional[Value] = None, epsilon: float = 1e-5,
                   loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        ins = [v for v in (x, weight, bias) if v is not None]
        self._emit("LayerNormOp", {"input": x.ref, "weight": weight.ref if weight else None,
                                   "bias": bias.ref if bias else None, "epsilon": float(epsilon),
                                   "memory_config": self._mc(), "out": out.ref}, ins, [out], loc)
        return out

    def argmax(self, x: Value, dim: Optional[int] = None, keep_dim: bool = False, loc=None) -> Value:
        rank = len(x.shape)
        if dim is None:
            shape = [1] * rank if keep_dim else []
        else:
            d = _norm(dim, rank)
            shape = [1 if i == d else s for i, s in enumerate(x.shape)] if keep_dim else \
                [s for i, s in enumerate(x.shape) if i != d]
        out = self._value(shape, "Int32")
        self._emit("ReductionArgMaxOp", {"in": x.ref, "out": out.ref, "dim": dim, "keep_dim": keep_dim,
                                         "memcfg": self._mc()}, [x], [out], loc)
        return out

    def cumsum(self, x: Value, dim: int, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("CumSumOp", {"in": x.ref, "out": out.ref, "dim": dim, "memcfg": self._mc()}, [x], [out], loc)
        return out

    def cumprod(self, x: Value, dim: int, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("CumProdOp", {"in": x.ref, "out": out.ref, "dim": dim, "memcfg": self._mc()}, [x], [out], loc)
        return out

    def prod(self, x: Value, dim: Optional[int] = None, keep_dim: bool = False, loc=None) -> Value:
        """Product over one dimension, or over all of them (dim None), as ::ttnn::prod takes it."""
        if dim is None:
            shape = [1] * len(x.shape) if keep_dim else []
        else:
            d = dim % len(x.shape)
            shape = [s if i != d else 1 for i, s in enumerate(x.shape)] if keep_dim else [s for i, s in enumerate(x.shape) if i != d]
        out = self._value(shape, x.dtype)
        self._emit("ReductionProdOp", {"in": x.ref, "out": out.ref, "dim_arg": dim, "keep_dim": keep_dim, "memcfg": self._mc()},
                   [x], [out], loc)
        return out

    def batch_norm_inference(self, x: Value, mean: Value, var: Value, weight: Optional[Value], bias: Optional[Value],
                             epsilon: float = 1e-5, loc=None) -> Value:
        """x is [N, C, ...]; statistics and parameters have C entries."""
        out = self._value(x.shape, x.dtype)
        ins = [x, mean, var] + [t for t in (weight, bias) if t is not None]
        self._emit("BatchNormInferenceOp", {
            "input": x.ref, "running_mean": mean.ref, "running_var": var.ref, "epsilon": epsilon,
            "weight": weight.ref if weight else None, "bias": bias.ref if bias else None, "memory_config": self._mc(),
            "out": out.ref}, ins, [out], loc)
        return out

    def upsample(self, x: Value, scale, mode: str = "nearest", loc=None) -> Value:
        """x is NHWC; scale an integer or (scale_h, scale_w)."""
        sy, sx = (scale, scale) if isinstance(scale, int) else scale
        out = self._value([x.shape[0], x.shape[1] * sy, x.shape[2] * sx, x.shape[3]], x.dtype)
        sf = ("UniformScale2D", {"scale": scale}) if isinstance(scale, int) else ("NonUniformScale2D", {"scale": [sy, sx]})
        self._emit("UpsampleOp", {"in": x.ref, "scale_factor": sf, "mode": mode, "memory_config": self._mc(), "out": out.ref},
                   [x], [out], loc)
        return out

    def group_norm(self, x: Value, weight: Optional[Value], bias: Optional[Value], num_groups: int, epsilon: float = 1e-5,
                   loc=None) -> Value:
        """x is channels-last [N, 1, H*W, C]; weight / bias have C entries."""
        out = self._value(x.shape, x.dtype)
        self._emit("GroupNormOp", {
            "input": x.ref, "weight": weight.ref if weight else None, "bias": bias.ref if bias else None,
            "num_groups": num_groups, "epsilon": epsilon, "memory_config": self._mc(), "out": out.ref},
            [x] + [t for t in (weight, bias) if t is not None], [out], loc)
        return out

    def conv_transpose2d(self, x: Value, w: Value, bias: Optional[Value], batch: int, height: int, width: int, stride=(1, 1),
                         padding=(0, 0), output_padding=(0, 0), dilation=(1, 1), groups: int = 1, loc=None) -> Value:
        """x is [1, 1, N*H*W, C] or [N, H, W, C]; w is [C, O/groups, kH, kW]; bias [1, 1, 1, O]."""
        c, og, kh, kw = getattr(w, "filter_shape", w.shape)
        o = og * groups
        ho = (height - 1) * stride[0] - 2 * padding[0] + dilation[0] * (kh - 1) + output_padding[0] + 1
        wo = (width - 1) * stride[1] - 2 * padding[1] + dilation[1] * (kw - 1) + output_padding[1] + 1
        flat = x.shape[:2] == [1, 1] and len(x.shape) == 4 and x.shape[2] == batch * height * width
        out = self._value([1, 1, batch * ho * wo, o] if flat else [batch, ho, wo, o], x.dtype)
        self._emit("ConvTranspose2dOp", {
            "input": x.ref, "weight": w.ref, "bias": bias.ref if bias else None, "out": out.ref, "device": self.device_ref,
            "in_channels": c, "out_channels": o, "batch_size": batch, "input_height": height, "input_width": width,
            "kernel_size": [kh, kw], "stride": list(stride), "padding": list(padding), "output_padding": list(output_padding),
            "dilation": list(dilation), "groups": groups, "output_dtype": x.dtype, "memory_config": self._mc()},
            [x, w] + ([bias] if bias else []), [out], loc)
        return out

    def conv1d(self, x: Value, w: Value, bias: Optional[Value], batch: int, length: int, stride: int = 1, padding=(0, 0),
               dilation: int = 1, groups: int = 1, loc=None) -> Value:
        """x is [N, L, C]; w is [O, C/groups, K]; bias [1, 1, O]."""
        o, cg, k = w.shape
        lo = (length + padding[0] + padding[1] - dilation * (k - 1) - 1) // stride + 1
        out = self._value([batch, lo, o], x.dtype)
        self._emit("Conv1dOp", {
            "input": x.ref, "weight": w.ref, "bias": bias.ref if bias else None, "out": out.ref, "device": self.device_ref,
            "in_channels": cg * groups, "out_channels": o, "batch_size": batch, "input_length": length, "kernel_size": k,
            "stride": stride, "padding": list(padding), "dilation": dilation, "groups": groups, "output_dtype": x.dtype},
            [x, w] + ([bias] if bias else []), [out], loc)
        return out

    def bitcast_convert(self, x: Value, dtype: str, loc=None) -> Value:
        out = self._value(x.shape, dtype)
        self._emit("BitcastConvertOp", {"in": x.ref, "dtype": dtype, "memcfg": self._mc(), "out": out.ref}, [x], [out], loc)
        return out

    def nlp_concat_heads(self, x: Value, loc=None) -> Value:
        b, h, s_, d = x.shape
        out = self._value([b, 1, s_, h * d], x.dtype)
        self._emit("NLPConcatHeadsOp", {"in": x.ref, "out": out.ref, "memcfg": self._mc()}, [x], [out], loc)
        return out

    # ---- further ops of real model flatbuffers: copies, debug markers, decode-step head ops, random ops
    def assign(self, x: Value, dtype: Optional[str] = None, loc=None) -> Value:
        out = self._value(x.shape, dtype or x.dtype)
        t = {"input": x.ref, "output": out.ref, "output_memory_config": self._mc()}
        if dtype:
            t["output_dtype"] = dtype
        self._emit("AssignOp", t, [x], [out], loc)
        return out

    def pow_scalar(self, x: Value, exponent, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        rhs = ("FP", {"value": float(exponent)}) if isinstance(exponent, float) else ("I32", {"value": int(exponent)})
        self._emit("EltwiseBinaryCompositeScalarOp", {"type": "PowScalar", "lhs": x.ref, "rhs": rhs, "memory_config": self._mc(),
                                                      "out": out.ref}, [x], [out], loc)
        return out

    def _marker(self, op_type: str, x: Value, key: str, text: str, loc=None) -> Value:
        out = self._value(x.shape, x.dtype, x.on_device)
        self._emit(op_type, {"operand": x.ref, "result": out.ref, key: text}, [x], [out], loc)
        return out

    def annotate(self, x: Value, annotation: str, loc=None) -> Value: return self._marker("AnnotateOp", x, "annotation", annotation, loc)
    def region_start(self, x: Value, region_id: str, loc=None) -> Value: return self._marker("RegionStartOp", x, "region_id", region_id, loc)
    def region_end(self, x: Value, region_id: str, loc=None) -> Value: return self._marker("RegionEndOp", x, "region_id", region_id, loc)

    def breakpoint(self, x: Value, loc=None) -> None: self._emit("BreakpointOp", {"operand": x.ref}, [x], [], loc)
    def print_message(self, x: Value, message: str, loc=None) -> None: self._emit("PrintOp", {"operand": x.ref, "message": message}, [x], [], loc)

    def memory_snapshot(self, x: Value, file_path: str, loc=None) -> None:
        self._emit("MemorySnapshotOp", {"operand": x.ref, "file_path": file_path}, [x], [], loc)

    def dump_tensor(self, x: Value, file_path: str, loc=None) -> None:
        self._emit("DumpTensorOp", {"file_path": file_path, "in": x.ref}, [x], [], loc)

    def load_tensor(self, file_path: str, shape, dtype: str, on_device: bool = True, loc=None) -> Value:
        out = self._value(shape, dtype, on_device)
        t = {"file_path": file_path, "out": out.ref}
        if on_device:
            t["device"] = self.device_ref
        self._emit("LoadTensorOp", t, [], [out], loc)
        return out

    def nlp_create_qkv_heads_decode(self, x: Value, num_heads: int, num_kv_heads: Optional[int] = None,
                                    batch_offset: Optional[Value] = None, slice_size: Optional[int] = None, loc=None):
        """x is [1, 1, batch, (num_heads + 2 * num_kv_heads) * head_dim]; q is [1, batch, num_heads, head_dim]."""
        _, _, b, hidden = x.shape
        hkv = num_kv_heads if num_kv_heads is not None else num_heads
        d = hidden // (num_heads + 2 * hkv)
        nb = slice_size if slice_size is not None else b
        q, k, v = (self._value([1, nb, h, d], x.dtype) for h in (num_heads, hkv, hkv))
        t = {"input": x.ref, "q_out": q.ref, "k_out": k.ref, "v_out": v.ref, "num_heads": num_heads, "memcfg": self._mc()}
        if num_kv_heads is not None:
            t["num_kv_heads"] = num_kv_heads
        if slice_size is not None:
            t["slice_size"] = slice_size
            t["batch_offset"] = batch_offset.ref
        self._emit("NLPCreateQKVHeadsDecodeOp", t, [x] + ([batch_offset] if batch_offset is not None else []), [q, k, v], loc)
        return q, k, v

    def nlp_concat_heads_decode(self, x: Value, num_heads: int, loc=None) -> Value:
        _, b, _, d = x.shape
        out = self._value([1, 1, b, num_heads * d], x.dtype)
        self._emit("NLPConcatHeadsDecodeOp", {"in": x.ref, "out": out.ref, "num_heads": num_heads, "memcfg": self._mc()}, [x], [out], loc)
        return out

    def rotary_embedding_llama(self, x: Value, cos: Value, sin: Value, trans_mat: Value, is_decode_mode: bool = False, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("RotaryEmbeddingLlamaOp", {"input": x.ref, "cos_cache": cos.ref, "sin_cache": sin.ref, "trans_mat": trans_mat.ref,
                                              "is_decode_mode": is_decode_mode, "out": out.ref, "memcfg": self._mc()},
                   [x, cos, sin, trans_mat], [out], loc)
        return out

    def max_pool2d_with_indices(self, x: Value, batch: int, height: int, width: int, channels: int, kernel=(2, 2), stride=(2, 2),
                                padding=(0, 0), dilation=(1, 1), ceil_mode: bool = False, index_dtype: str = "Int32", loc=None):
        ho, wo = self.pool_out_hw("MaxPool2d", height, width, kernel, stride, padding, dilation, ceil_mode)
        out = self._value([1, 1, batch * ho * wo, channels], x.dtype)
        idx = self._value([1, 1, batch * ho * wo, channels], index_dtype)
        self._emit("MaxPool2dWithIndicesOp", {
            "in": x.ref, "result": out.ref, "result_indices": idx.ref, "batch_size": batch, "input_height": height,
            "input_width": width, "channels": channels, "kernel_size": list(kernel), "stride": list(stride),
            "padding": list(padding), "dilation": list(dilation), "memory_config": self._mc(), "ceil_mode": ceil_mode},
            [x], [out, idx], loc)
        return out, idx

    def dropout(self, x: Value, prob: float, scale: Optional[float] = None, seed: int = 0, use_per_device_seed: bool = True,
                loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        scale = 1.0 / (1.0 - prob) if scale is None else scale
        self._emit("DropoutOp", {"in": x.ref, "prob": prob, "scale": scale, "seed": seed, "use_per_device_seed": use_per_device_seed,
                                 "memory_config": self._mc(), "out": out.ref}, [x], [out], loc)
        return out

    def rand(self, shape, dtype: str, low: float = 0.0, high: float = 1.0, seed: int = 0, loc=None) -> Value:
        out = self._value(shape, dtype)
        self._emit("RandOp", {"device": self.device_ref, "size": list(shape), "low": low, "high": high, "seed": seed, "dtype": dtype,
                              "layout": "Tile", "memcfg": self._mc(), "out": out.ref}, [], [out], loc)
        return out

    def batch_norm_training(self, x: Value, mean: Value, var: Value, weight: Optional[Value], bias: Optional[Value],
                            epsilon: float = 1e-5, momentum: float = 0.1, loc=None) -> Value:
        """x is [N, C, ...]; `mean` / `var` are the running statistics, updated in place."""
        out = self._value(x.shape, x.dtype)
        ins = [x, mean, var] + [t for t in (weight, bias) if t is not None]
        self._emit("BatchNormTrainingOp", {
            "input": x.ref, "running_mean": mean.ref, "running_var": var.ref, "epsilon": epsilon, "momentum": momentum,
            "weight": weight.ref if weight else None, "bias": bias.ref if bias else None, "memory_config": self._mc(),
            "out": out.ref}, ins, [out], loc)
        return out

    def dit_rms_norm_unary_fused(self, x: Value, weight: Optional[Value] = None, bias: Optional[Value] = None,
                                 residual: Optional[Value] = None, epsilon: float = 1e-5, activation: Optional[str] = None,
                                 loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        opt = lambda v: v.ref if v is not None else None
        self._emit("DitRMSNormUnaryFusedOp", {
            "input": x.ref, "weight": opt(weight), "bias": opt(bias), "residual_input": opt(residual), "epsilon": epsilon,
            "activation": activation, "memory_config": self._mc(), "out": out.ref},
            [x] + [t for t in (weight, bias, residual) if t is not None], [out], loc)
        return out

    def distributed_rms_norm(self, x: Value, weight: Optional[Value] = None, residual: Optional[Value] = None,
                             cluster_axis: int = 1, epsilon: float = 1e-5, loc=None) -> Value:
        """x holds this device's slice of the normalised (last) dimension; weight its slice of gamma."""
        out = self._value(x.shape, x.dtype)
        opt = lambda v: v.ref if v is not None else None
        self._emit("DistributedRMSNormOp", {
            "input": x.ref, "weight": opt(weight), "residual": opt(residual), "cluster_axis": cluster_axis, "epsilon": epsilon,
            "memory_config": self._mc(), "out": out.ref, "semaphore": {"global_id": 0}},
            [x] + [t for t in (weight, residual) if t is not None], [out], loc)
        return out

    def rms_norm_pre_all_gather(self, x: Value, residual: Optional[Value] = None, dtype: Optional[str] = None, loc=None) -> Value:
        out = self._value(list(x.shape[:-1]) + [32], dtype or x.dtype)
        self._emit("RMSNormPreAllGatherOp", {"input": x.ref, "dtype": dtype or x.dtype, "residual": residual.ref if residual else None,
                                             "memory_config": self._mc(), "out": out.ref},
                   [x] + ([residual] if residual else []), [out], loc)
        return out

    def layer_norm_pre_all_gather(self, x: Value, residual: Optional[Value] = None, dtype: Optional[str] = None, loc=None) -> Value:
        out = self._value(list(x.shape[:-1]) + [64], dtype or x.dtype)
        self._emit("LayerNormPreAllGatherOp", {"input": x.ref, "residual_input": residual.ref if residual else None,
                                               "dtype": dtype or x.dtype, "memory_config": self._mc(), "out": out.ref},
                   [x] + ([residual] if residual else []), [out], loc)
        return out

    def layer_norm_post_all_gather(self, x: Value, stats: Value, weight: Optional[Value] = None, bias: Optional[Value] = None,
                                   epsilon: float = 1e-12, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        opt = lambda v: v.ref if v is not None else None
        self._emit("LayerNormPostAllGatherOp", {
            "input": x.ref, "stats": stats.ref, "weight": opt(weight), "bias": opt(bias), "epsilon": epsilon,
            "memory_config": self._mc(), "out": out.ref}, [x, stats] + [t for t in (weight, bias) if t is not None], [out], loc)
        return out

    def create_global_semaphore(self, initial_value: int = 0, loc=None) -> None:
        self._emit("CreateGlobalSemaphoreOp", {"initial_value": initial_value, "out": {"global_id": 0}}, [], [], loc)

    def reset_global_semaphore(self, value: int = 0, loc=None) -> None:
        self._emit("ResetGlobalSemaphoreOp", {"semaphore": {"global_id": 0}, "value": value}, [], [], loc)

    def flash_mla_prefill(self, q: Value, k: Value, head_dim_v: int, v: Optional[Value] = None, mask: Optional[Value] = None,
                          is_causal: bool = True, scale: Optional[float] = None, loc=None) -> Value:
        """q [B, H, S, Dqk], k [B, Hkv, Skv, Dqk]; values are k[..., :head_dim_v] unless `v` is given."""
        out = self._value(list(q.shape[:3]) + [head_dim_v], q.dtype)
        t = {"query": q.ref, "key": k.ref, "value": v.ref if v is not None else None,
             "attention_mask": mask.ref if mask is not None else None, "head_dim_v": head_dim_v, "is_causal": is_causal,
             "out": out.ref, "memcfg": self._mc()}
        if scale is not None:
            t["scale"] = scale
        self._emit("FlashMlaPrefillOp", t, [q, k] + [x for x in (v, mask) if x is not None], [out], loc)
        return out

    def indexer_score_dsa(self, q: Value, k: Value, weights: Value, chunk_start_idx: int = 0, cluster_axis: Optional[int] = None,
                          loc=None) -> Value:
        """q [B, Hi, Sq, D], k [B, 1, T, D], weights [B, Hi, Sq, 1] -> scores [B, 1, Sq, T]."""
        out = self._value([q.shape[0], 1, q.shape[2], k.shape[2]], q.dtype)
        t = {"query": q.ref, "key": k.ref, "weights": weights.ref, "chunk_start_idx": chunk_start_idx, "out": out.ref}
        if cluster_axis is not None:
            t["cluster_axis"] = cluster_axis
        self._emit("IndexerScoreDsaOp", t, [q, k, weights], [out], loc)
        return out

    def paged_flash_multi_latent_attention_decode(self, q: Value, k_cache: Value, head_dim_v: int, page_table: Value,
                                                  v_cache: Optional[Value] = None, cur_pos: Optional[Value] = None,
                                                  mask: Optional[Value] = None, is_causal: bool = True,
                                                  scale: Optional[float] = None, loc=None) -> Value:
        """q [1, B, H, D], k_cache [blocks, Hkv, block, D], page_table [B, blocks per user], cur_pos [B]."""
        out = self._value(list(q.shape[:3]) + [head_dim_v], q.dtype)
        opt = lambda x: x.ref if x is not None else None
        t = {"query": q.ref, "key": k_cache.ref, "value": opt(v_cache), "head_dim_v": head_dim_v, "page_table": page_table.ref,
             "is_causal": is_causal, "attention_mask": opt(mask), "cur_pos_tensor": opt(cur_pos), "out": out.ref, "memcfg": self._mc()}
        if scale is not None:
            t["scale"] = scale
        self._emit("PagedFlashMultiLatentAttentionDecodeOp", t,
                   [q, k_cache, page_table] + [x for x in (v_cache, cur_pos, mask) if x is not None], [out], loc)
        return out

    def chunked_scaled_dot_product_attention(self, q: Value, k_cache: Value, v_cache: Value, page_table: Value, chunk_start_idx: Value,
                                             scale: Optional[float] = None, loc=None) -> Value:
        """q [B, H, Sq, D] (positions chunk_start ..), caches [blocks, Hkv, block, D], page_table [B, blocks per user]."""
        out = self._value(q.shape, q.dtype)
        t = {"query": q.ref, "key": k_cache.ref, "value": v_cache.ref, "page_table": page_table.ref,
             "chunk_start_idx": chunk_start_idx.ref, "out": out.ref, "memcfg": self._mc()}
        if scale is not None:
            t["scale"] = scale
        self._emit("ChunkedScaledDotProductAttentionOp", t, [q, k_cache, v_cache, page_table, chunk_start_idx], [out], loc)
        return out

    def conv3d(self, x: Value, w: Value, bias: Optional[Value], batch: int, depth: int, height: int, width: int, stride=(1, 1, 1),
               padding=(0, 0, 0), groups: int = 1, padding_mode: str = "zeros", loc=None) -> Value:
        """x is [1, 1, N*D*H*W, C] or [N, D, H, W, C]; w is [O, C/groups, kD, kH, kW]; bias [1, 1, 1, 1, O]."""
        o, cg, kd, kh, kw = getattr(w, "filter_shape", w.shape)
        od, oh, ow = ((s + 2 * p - k) // st + 1 for s, p, k, st in zip((depth, height, width), padding, (kd, kh, kw), stride))
        flat = len(x.shape) == 4
        out = self._value([1, 1, batch * od * oh * ow, o] if flat else [batch, od, oh, ow, o], x.dtype)
        self._emit("Conv3dOp", {
            "input": x.ref, "weight": w.ref, "bias": bias.ref if bias else None, "out": out.ref, "device": self.device_ref,
            "in_channels": cg * groups, "out_channels": o, "batch_size": batch, "input_depth": depth, "input_height": height,
            "input_width": width, "kernel_size": [kd, kh, kw], "stride": list(stride), "padding": list(padding),
            "padding_mode": padding_mode, "groups": groups, "output_dtype": x.dtype, "memory_config": self._mc()},
            [x, w] + ([bias] if bias else []), [out], loc)
        return out

    def prepare_conv3d_weights(self, w: Value, groups: int = 1, c_in_block: int = 32, alignment: int = 32, loc=None) -> Value:
        o, cg, kd, kh, kw = w.shape
        out = self._value([kd * kh * kw * cg, o], w.dtype)
        out.filter_shape = list(w.shape)
        self._emit("PrepareConv3dWeightsOp", {"weight_tensor": w.ref, "out": out.ref, "groups": groups, "c_in_block": c_in_block,
                                              "alignment": alignment, "device": self.device_ref}, [w], [out], loc)
        return out

    def gelu_backward(self, grad: Value, x: Value, approximate: str = "none", loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("ExperimentalEltwiseBinaryBackwardOp", {"type": "GeluBW", "grad": grad.ref, "input": x.ref, "approximate": approximate,
                                                           "memory_config": self._mc(), "out": out.ref}, [grad, x], [out], loc)
        return out

    def embedding_backward(self, indices: Value, weight: Value, in_grad: Value, loc=None) -> Value:
        out = self._value(weight.shape, in_grad.dtype)
        self._emit("EmbeddingBackwardOp", {"input": indices.ref, "weight": weight.ref, "in_grad": in_grad.ref, "memcfg": self._mc(),
                                           "out": out.ref}, [indices, weight, in_grad], [out], loc)
        return out

    def adamw(self, param: Value, grad: Value, exp_avg: Value, exp_avg_sq: Value, max_exp_avg_sq: Optional[Value] = None,
              lr: float = 1e-3, beta1: float = 0.9, beta2: float = 0.999, beta1_pow: float = 0.9, beta2_pow: float = 0.999,
              epsilon: float = 1e-8, weight_decay: float = 0.0, stochastic_rounding: bool = False, loc=None) -> None:
        """Updates param, exp_avg, exp_avg_sq (and max_exp_avg_sq) in place."""
        ins = [param, grad, exp_avg, exp_avg_sq] + ([max_exp_avg_sq] if max_exp_avg_sq is not None else [])
        self._emit("AdamWOp", {
            "param": param.ref, "grad": grad.ref, "exp_avg": exp_avg.ref, "exp_avg_sq": exp_avg_sq.ref,
            "max_exp_avg_sq": max_exp_avg_sq.ref if max_exp_avg_sq is not None else None, "lr": lr, "beta1": beta1, "beta2": beta2,
            "beta1_pow": beta1_pow, "beta2_pow": beta2_pow, "epsilon": epsilon, "weight_decay": weight_decay,
            "stochastic_rounding": stochastic_rounding}, ins, [], loc)

    # ---- mixture of experts (generic flow: dispatch -> remap -> sparse matmuls -> combine)
    def all_to_all_dispatch(self, x: Value, expert_indices: Value, expert_mapping: Value, cluster_axis: int = 1, loc=None):
        """x [B, 1, S, H] and expert_indices [B, 1, S, K] hold this device's tokens; expert_mapping is the replicated
        [1, 1, E, D] one-hot table.  Returns dispatched [1, B*D, S, H] and metadata [1, B*D, S, K]."""
        n = self._axis_size(cluster_axis)
        b, _, s_, h = x.shape
        k = expert_indices.shape[-1]
        disp = self._value([1, b * n, s_, h], x.dtype)
        meta = self._value([1, b * n, s_, k], expert_indices.dtype)
        self._emit("AllToAllDispatchOp", {
            "input_tensor": x.ref, "expert_indices": expert_indices.ref, "expert_mapping": expert_mapping.ref,
            "dispatched": disp.ref, "metadata": meta.ref, "num_devices": n, "cluster_axis": cluster_axis,
            "memory_config": self._mc()}, [x, expert_indices, expert_mapping], [disp, meta], loc)
        return disp, meta

    def all_to_all_dispatch_metadata(self, x: Value, expert_indices: Value, expert_scores: Value, expert_mapping: Value,
                                     cluster_axis: int = 1, loc=None):
        """x [1, 1, M, H], expert_indices / expert_scores [1, 1, M, K]; expert_mapping [1, 1, D, E] holds the owning
        device of every expert.  Returns dispatched [1, D*M, H], indices [1, D*M, K], scores [1, D*M, K]."""
        n = self._axis_size(cluster_axis)
        m, h, k = x.shape[-2], x.shape[-1], expert_indices.shape[-1]
        disp = self._value([1, n * m, h], x.dtype)
        idx = self._value([1, n * m, k], expert_indices.dtype)
        scr = self._value([1, n * m, k], expert_scores.dtype)
        self._emit("AllToAllDispatchMetadataOp", {
            "input_tensor": x.ref, "expert_indices": expert_indices.ref, "expert_scores": expert_scores.ref,
            "expert_mapping": expert_mapping.ref, "dispatched": disp.ref, "indices": idx.ref, "scores": scr.ref,
            "num_devices": n, "cluster_axis": cluster_axis, "memory_config": self._mc(),
            "cross_device_semaphore": {"global_id": 0}}, [x, expert_indices, expert_scores, expert_mapping], [disp, idx, scr], loc)
        return disp, idx, scr

    def topk_router_gpt(self, x: Value, weight: Value, bias: Value, k: int, index_dtype: str = "UInt16", loc=None):
        """x [B, H], weight [H, E], bias [B, E] -> expert_indices [B, k], expert_weights [B, k]."""
        b, e = x.shape[0], weight.shape[1]
        idx = self._value([b, k], index_dtype)
        wts = self._value([b, k], x.dtype)
        self._emit("TopKRouterGptOp", {"input": x.ref, "weight": weight.ref, "bias": bias.ref, "k": k, "num_experts": e,
                                       "expert_indices": idx.ref, "expert_weights": wts.ref}, [x, weight, bias], [idx, wts], loc)
        return idx, wts

    def all_to_all_combine(self, x: Value, expert_metadata: Value, expert_mapping: Value, num_experts_per_tok: int,
                           cluster_axis: int = 1, output_shard_dim: int = 1, loc=None) -> Value:
        """x [E_local, B*D, S, H] -> [K, B, S, H] (this device's tokens, one slice per selected expert)."""
        n = self._axis_size(cluster_axis)
        _, bg, sg, h = x.shape
        shape = [num_experts_per_tok, bg // n, sg, h] if output_shard_dim == 1 else [num_experts_per_tok, bg, sg // n, h]
        out = self._value(shape, x.dtype)
        self._emit("AllToAllCombineOp", {
            "input_tensor": x.ref, "expert_metadata": expert_metadata.ref, "expert_mapping": expert_mapping.ref, "out": out.ref,
            "num_devices": n, "cluster_axis": cluster_axis, "num_experts_per_tok": num_experts_per_tok,
            "output_shard_dim": output_shard_dim, "memory_config": self._mc()}, [x, expert_metadata, expert_mapping], [out], loc)
        return out

    def moe_expert_token_remap(self, topk: Value, expert_mapping: Value, expert_metadata: Value, reduction_size: int = 32,
                               reduced_dtype: Optional[str] = None, loc=None):
        """topk [1, T_b, S, E] -> mapping [1, T_b, S, E_local], reduced [1, 1, ceil(T_b*S / reduction_size), E_local]."""
        _, tb, s_, e = topk.shape
        d = expert_mapping.shape[-1]
        el = e // d
        mapping = self._value([1, tb, s_, el], topk.dtype)
        reduced = self._value([1, 1, (tb * s_ + reduction_size - 1) // reduction_size, el], reduced_dtype or topk.dtype)
        self._emit("MoeExpertTokenRemapOp", {
            "topk_tensor": topk.ref, "expert_mapping": expert_mapping.ref, "expert_metadata": expert_metadata.ref,
            "mapping": mapping.ref, "reduced": reduced.ref, "reduction_size": reduction_size, "memory_config": self._mc()},
            [topk, expert_mapping, expert_metadata], [mapping, reduced], loc)
        return mapping, reduced

    def sparse_matmul(self, a: Value, b: Value, sparsity: Value, is_input_a_sparse: bool = False, is_input_b_sparse: bool = True,
                      nnz: Optional[int] = None, loc=None) -> Value:
        _, e, _, n = b.shape
        if is_input_a_sparse:
            shape = [a.shape[0], e, a.shape[2], n]
        else:
            shape = [a.shape[0], a.shape[1], 1, e, a.shape[2], n]
        out = self._value(shape, a.dtype)
        t = {"a": a.ref, "b": b.ref, "sparsity": sparsity.ref, "out": out.ref, "is_input_a_sparse": is_input_a_sparse,
             "is_input_b_sparse": is_input_b_sparse, "memory_config": self._mc(), "dtype": a.dtype}
        if nnz is not None:
            t["nnz"] = nnz
        self._emit("SparseMatmulOp", t, [a, b, sparsity], [out], loc)
        return out

    def all_reduce_async(self, x: Value, reduce_type: int = 0, cluster_axis: int = 1, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        self._emit("AllReduceAsyncOp", {"in": x.ref, "out": out.ref, "reduce_type": reduce_type, "cluster_axis": cluster_axis,
                                        "memory_config": self._mc()}, [x], [out], loc)
        return out

    def point_to_point(self, x: Value, sender_coord, receiver_coord, output: Optional[Value] = None, loc=None) -> Value:
        out = self._value(x.shape, x.dtype)
        t = {"in": x.ref, "out": out.ref, "sender_coord": list(sender_coord), "receiver_coord": list(receiver_coord)}
        if output is not None:
            t["optional_output_tensor"] = output.ref
        self._emit("PointToPointOp", t, [x] + ([output] if output is not None else []), [out], loc)
        return out

    def prepare_conv_transpose2d_weights(self, w: Value, batch: int, height: int, width: int, stride=(1, 1), padding=(0, 0),
                                         output_padding=(0, 0), dilation=(1, 1), groups: int = 1, has_bias: bool = True,
                                         loc=None) -> Value:
        """Like prepare_conv2d_weights, for [C_in, C_out / groups, kH, kW] filters."""
        c, og, kh, kw = w.shape
        up = lambda v: (v + 31) // 32 * 32
        out = self._value([1, 1, up(kh * kw * c), up(og * groups)], w.dtype)
        out.filter_shape = list(w.shape)
        self._emit("PrepareConvTranspose2dWeightsOp", {
            "weight_tensor": w.ref, "out": out.ref, "input_memory_config": self._mc(), "input_tensor_layout": "Tile",
            "weights_format": "IOHW", "in_channels": c, "out_channels": og * groups, "batch_size": batch, "input_height": height,
            "input_width": width, "kernel_size": [kh, kw], "stride": list(stride), "padding": list(padding),
            "output_padding": list(output_padding), "dilation": list(dilation), "has_bias": has_bias, "groups": groups,
            "device": self.device_ref, "input_dtype": w.dtype}, [w], [out], loc)
        return out

    def prepare_conv_transpose2d_bias(self, bias: Value, in_channels: int, batch: int, height: int, width: int, kernel=(1, 1),
                                      stride=(1, 1), padding=(0, 0), dilation=(1, 1), groups: int = 1, loc=None) -> Value:
        o = bias.shape[-1]
        out = self._value([1, 1, 1, (o + 31) // 32 * 32], bias.dtype)
        self._emit("PrepareConvTranspose2dBiasOp", {
            "bias_tensor": bias.ref, "out": out.ref, "input_memory_config": self._mc(), "input_tensor_layout": "Tile",
            "in_channels": in_channels, "out_channels": o, "batch_size": batch, "input_height": height, "input_width": width,
            "kernel_size": list(kernel), "stride": list(stride), "padding": list(padding), "dilation": list(dilation),
            "groups": groups, "device": self.device_ref, "input_dtype": bias.dtype}, [bias], [out], loc)
        return out

    def prepare_conv2d_weights(self, w: Value, batch: int, height: int, width: int, stride=(1, 1), padding=(0, 0, 0, 0),
                               dilation=(1, 1), groups: int = 1, has_bias: bool = True, loc=None) -> Value:
        """The op the compiler's optimizer puts in front of conv2d.  The declared result shape is TTNN's prepared
        layout ([1, 1, kH*kW*C rounded up to 32, O rounded up to 32]); the value remembers the filter's own shape so
        that conv2d can still be described."""
        o, cg, kh, kw = w.shape
        up = lambda v: (v + 31) // 32 * 32
        out = self._value([1, 1, up(kh * kw * cg * groups), up(o)], w.dtype)
        out.filter_shape = list(w.shape)
        pad = list(padding) if len(padding) == 4 else [padding[0], padding[1], padding[0], padding[1]]
        self._emit("PrepareConv2dWeightsOp", {
            "weight_tensor": w.ref, "out": out.ref, "input_memory_config": self._mc(), "input_tensor_layout": "Tile",
            "weights_format": "OIHW", "in_channels": cg * groups, "out_channels": o, "batch_size": batch,
            "input_height": height, "input_width": width, "kernel_size": [kh, kw], "stride": list(stride), "padding": pad,
            "dilation": list(dilation), "has_bias": has_bias, "groups": groups, "device": self.device_ref,
            "input_dtype": w.dtype, "output_dtype": w.dtype}, [w], [out], loc)
        return out

    def prepare_conv2d_bias(self, bias: Value, w_shape, batch: int, height: int, width: int, stride=(1, 1),
                            padding=(0, 0, 0, 0), dilation=(1, 1), groups: int = 1, loc=None) -> Value:
        o, cg, kh, kw = w_shape
        out = self._value([1, 1, 32, (o + 31) // 32 * 32], bias.dtype)
        pad = list(padding) if len(padding) == 4 else [padding[0], padding[1], padding[0], padding[1]]
        self._emit("PrepareConv2dBiasOp", {
            "bias_tensor": bias.ref, "out": out.ref, "input_memory_config": self._mc(), "input_tensor_layout": "Tile",
            "in_channels": cg * groups, "out_channels": o, "batch_size": batch, "input_height": height, "input_width": width,
            "kernel_size": [kh, kw], "stride": list(stride), "padding": pad, "dilation": list(dilation), "groups": groups,
            "device": self.device_ref, "input_dtype": bias.dtype, "output_dtype": bias.dtype}, [bias], [out], loc)
        return out

    def embedding(self, indices: Value, weight: Value, loc=None) -> Value:
        out = self._value(list(indices.shape) + [weight.shape[-1]], weight.dtype)
        self._emit("EmbeddingOp", {"input": indices.ref, "weight": weight.ref, "out": out.ref}, [indices, weight], [out], loc)
        return out

    @staticmethod
    def pool_out_hw(kind, h, w, kernel, stride, padding, dilation=(1, 1), ceil_mode=False):
        """Output extent of Pool2dOp, following torch's rule the way the reference's CPU twin applies
        it: four paddings (top, left, bottom, right) -- and, for the average, two paddings larger than
        half the kernel -- are applied to the input by hand before pooling."""
        if len(padding) == 4:
            pt, pl, pb, pr = padding
            by_hand = True
        else:
            pt = pb = padding[0]
            pl = pr = padding[1]
            by_hand = False
        if kind == "AvgPool2d":
            dilation = (1, 1)
            by_hand = not ((pt == pb and pl == pr) and not (pt > kernel[0] // 2 or pl > kernel[1] // 2))

        def extent(n, k, lo, hi, s, d):
            if by_hand:
                n, lo, hi = n + lo + hi, 0, 0
            num = n + lo + hi - d * (k - 1) - 1 + (s - 1 if ceil_mode else 0)
            out = num // s + 1
            if ceil_mode and (out - 1) * s >= n + lo:
                out -= 1
            return out
        return (extent(h, kernel[0], pt, pb, stride[0], dilation[0]), extent(w, kernel[1], pl, pr, stride[1], dilation[1]))

    def _pool2d(self, kind, x, batch, height, width, channels, kernel, stride, padding, dilation, ceil_mode, extra, loc):
        ho, wo = self.pool_out_hw(kind, height, width, kernel, stride, padding, dilation, ceil_mode)
        out = self._value([1, 1, batch * ho * wo, channels], x.dtype)
        self._emit("Pool2dOp", {
            "type": kind, "in": x.ref, "out": out.ref, "batch_size": batch, "input_height": height, "input_width": width,
            "channels": channels, "kernel_size": list(kernel), "stride": list(stride), "padding": list(padding),
            "dilation": list(dilation), "extra_params": extra, "memory_config": self._mc(), "ceil_mode": ceil_mode},
            [x], [out], loc)
        return out

    def max_pool2d(self, x: Value, batch: int, height: int, width: int, channels: int, kernel=(2, 2), stride=(2, 2),
                   padding=(0, 0), dilation=(1, 1), ceil_mode: bool = False, loc=None) -> Value:
        """`x` is the flattened NHWC activation [1, 1, N*H*W, C]; `padding` is (h, w) or (top, left, bottom, right)."""
        return self._pool2d("MaxPool2d", x, batch, height, width, channels, kernel, stride, padding, dilation, ceil_mode,
                            ("MaxPool2dExtraParams", {}), loc)

    def avg_pool2d(self, x: Value, batch: int, height: int, width: int, channels: int, kernel=(2, 2), stride=(2, 2),
                   padding=(0, 0), ceil_mode: bool = False, count_include_pad: bool = True, loc=None) -> Value:
        return self._pool2d("AvgPool2d", x, batch, height, width, channels, kernel, stride, padding, (1, 1), ceil_mode,
                            ("AvgPool2dExtraParams", {"count_include_pad": count_include_pad}), loc)

    def global_avg_pool2d(self, x: Value, loc=None) -> Value:
        n, _, _, c = x.shape
        out = self._value([n, 1, 1, c], x.dtype)
        self._emit("GlobalAvgPool2dOp", {"in": x.ref, "out": out.ref, "memory_config": self._mc()}, [x], [out], loc)
        return out

    def pad(self, x: Value, padding: Sequence[int], value: float = 0.0, loc=None) -> Value:
        """`padding` = (low_0, high_0, low_1, high_1, ...), one pair per dimension."""
        assert len(padding) == 2 * len(x.shape)
        shape = [s + padding[2 * i] + padding[2 * i + 1] for i, s in enumerate(x.shape)]
        out = self._value(shape, x.dtype)
        self._emit("PadOp", {"in": x.ref, "out": out.ref, "padding": list(padding), "value": float(value),
                             "use_multicore": True, "memcfg": self._mc()}, [x], [out], loc)
        return out

    # ---- KV cache and decode attention ----------------------------------------------------------------------------
    def fill_cache(self, cache: Value, x: Value, batch_offset: int = 0, loc=None) -> Value:
        """In place: cache[batch_offset + b, h, :S] = x[b, h].  Returns `cache` (the op has no result)."""
        self._emit("FillCacheOp", {"cache": cache.ref, "input": x.ref, "batch_offset": batch_offset}, [cache, x], [], loc)
        return cache

    def update_cache(self, cache: Value, x: Value, update_index: Value, batch_offset: int = 0, loc=None) -> Value:
        """In place: cache[batch_offset + b, h, update_index[0]] = x[0, h, b].  Returns `cache`."""
        self._emit("UpdateCacheOp", {"cache": cache.ref, "input": x.ref, "update_index": update_index.ref,
                                     "batch_offset": batch_offset}, [cache, x, update_index], [], loc)
        return cache

    def scaled_dot_product_attention_decode(self, q: Value, k: Value, v: Value, cur_pos: Optional[Value] = None,
                                            mask: Optional[Value] = None, is_causal: bool = True,
                                            scale: Optional[float] = None, loc=None) -> Value:
        out = self._value(q.shape, q.dtype)
        ins = [x for x in (q, k, v, mask, cur_pos) if x is not None]
        self._emit("ScaledDotProductAttentionDecodeOp", {
            "query": q.ref, "key": k.ref, "value": v.ref, "is_causal": is_causal,
            "attention_mask": mask.ref if mask else None, "cur_pos_tensor": cur_pos.ref if cur_pos else None,
            "scale": scale, "out": out.ref, "memcfg": self._mc()}, ins, [out], loc)
        return out

    def paged_update_cache(self, cache: Value, x: Value, update_index: Value, page_table: Optional[Value] = None,
                           share_cache: bool = False, loc=None) -> Value:
        """In place: token s of user b of x [users, seq, heads, D] goes to position update_index[b] + s of the
        paged cache [blocks, heads, block_size, D].  Returns `cache`."""
        ins = [cache, x, update_index] + ([page_table] if page_table else [])
        self._emit("PagedUpdateCacheOp", {"cache": cache.ref, "input": x.ref, "update_index": update_index.ref,
                                          "share_cache": share_cache, "page_table": page_table.ref if page_table else None},
                   ins, [], loc)
        return cache

    def paged_fill_cache(self, cache: Value, x: Value, page_table: Value, batch_idx: Optional[Value] = None, loc=None) -> Value:
        """In place: x [users, heads, seq, D] fills the pages of the users' page-table rows.  Returns `cache`."""
        ins = [cache, x, page_table] + ([batch_idx] if batch_idx else [])
        self._emit("PagedFillCacheOp", {"cache": cache.ref, "input": x.ref, "page_table": page_table.ref,
                                        "batch_idx_tensor": batch_idx.ref if batch_idx else None}, ins, [], loc)
        return cache

    def paged_scaled_dot_product_attention_decode(self, q: Value, k: Value, v: Value, page_table: Value,
                                                  cur_pos: Optional[Value] = None, mask: Optional[Value] = None,
                                                  is_causal: bool = True, scale: Optional[float] = None, loc=None) -> Value:
        """q [B, 1, H, D] against paged k / v [blocks, Hkv, block_size, D] read through page_table [B, pages]."""
        out = self._value(q.shape, q.dtype)
        ins = [x for x in (q, k, v, page_table, mask, cur_pos) if x is not None]
        self._emit("PagedScaledDotProductAttentionDecodeOp", {
            "query": q.ref, "key": k.ref, "value": v.ref, "page_table": page_table.ref, "is_causal": is_causal,
            "attention_mask": mask.ref if mask else None, "cur_pos_tensor": cur_pos.ref if cur_pos else None,
            "scale": scale, "out": out.ref, "memcfg": self._mc()}, ins, [out], loc)
        return out

    # ---- indexing ---------------------------------------------------------------------------------------------------
    def gather(self, x: Value, index: Value, dim: int, loc=None) -> Value:
        out = self._value(index.shape, x.dtype)
        self._emit("GatherOp", {"input": x.ref, "index": index.ref, "out": out.ref, "dim": dim, "memory_config": self._mc()},
                   [x, index], [out], loc)
        return out

    def scatter(self, x: Value, index: Value, src: Value, dim: int, reduce_type: Optional[str] = None, loc=None) -> Value:
        """reduce_type None (plain scatter) or "Sum" / "Max" / "Min" / "Prod"."""
        out = self._value(x.shape, x.dtype)
        self._emit("ScatterOp", {"input": x.ref, "out": out.ref, "index": index.ref, "source": src.ref, "dim": dim,
                                 "memory_config": self._mc(), "scatter_reduce_type": reduce_type or "Invalid"},
                   [x, index, src], [out], loc)
        return out

    def sort(self, x: Value, dim: int = -1, descending: bool = False, stable: bool = True, index_dtype: str = "Int32", loc=None):
        values, indices = self._value(x.shape, x.dtype), self._value(x.shape, index_dtype)
        self._emit("SortOp", {"in": x.ref, "dim": dim, "descending": descending, "stable": stable, "memcfg": self._mc(),
                              "outputs": [values.ref, indices.ref]}, [x], [values, indices], loc)
        return values, indices

    def topk(self, x: Value, k: int, dim: int = -1, largest: bool = True, index_dtype: str = "Int32", loc=None):
        shape = list(x.shape)
        shape[_norm(dim, len(shape))] = k
        values, indices = self._value(shape, x.dtype), self._value(shape, index_dtype)
        self._emit("TopKOp", {"input_tensor": x.ref, "k": k, "dim": dim, "largest": largest, "sorted": True,
                              "memcfg": self._mc(), "outputs": [values.ref, indices.ref]}, [x], [values, indices], loc)
        return values, indices

    def sampling(self, values: Value, indices: Value, k: Value, p: Value, temp: Value, seed: Optional[int] = None, loc=None) -> Value:
        """One sampled candidate per row of values / indices [batch, candidates]; result [batch] Int32."""
        out = self._value([values.shape[-2]], "Int32")
        self._emit("SamplingOp", {"input_values": values.ref, "input_indices": indices.ref, "k": k.ref, "p": p.ref, "temp": temp.ref,
                                  "seed": seed, "out": out.ref}, [values, indices, k, p, temp], [out], loc)
        return out

    # ---- sub-programs: const-eval, calls, traces -------------------------------------------------------------
    def input_like(self, v: Value, on_device: Optional[bool] = None) -> Value:
        return self.input(v.shape, v.dtype, v.on_device if on_device is None else on_device)

    def empty(self, shape, dtype: str, loc=None) -> Value:
        out = self._value(shape, dtype)
        self._emit("EmptyOp", {"shape": list(shape), "dtype": dtype, "layout": "Tile", "device": self.device_ref,
                               "memcfg": self._mc(), "out": out.ref}, [], [out], loc)
        return out

    def _results_like(self, callee: "ProgramBuilder") -> List[Value]:
        return [self._value(v.shape, v.dtype, v.on_device) for v in callee.outputs]

    def load_cached(self, callee: "ProgramBuilder", inputs: Sequence[Value], program_hash: Optional[str] = None,
                    loc=None) -> List[Value]:
        """`ttcore.load_cached(@callee, [inputs])`: the results of a const-eval function, computed on
        first use and cached by the runtime (lib/Target/TTNN/TTNNToFlatbuffer.cpp emits LoadCachedOp
        with the callee's position in the binary and a hash of its body)."""
        outs = self._results_like(callee)
        if program_hash is None:
            import hashlib
            program_hash = hashlib.sha256(repr([op["type"] for op in callee.ops]).encode()).hexdigest()
        self._emit("LoadCachedOp", {"inputs": [v.ref for v in inputs], "callee_name": callee.name,
                                    "program_idx": callee.index, "outputs": [v.ref for v in outs],
                                    "program_hash": program_hash}, list(inputs), outs, loc)
        return outs

    def func_call(self, callee: "ProgramBuilder", inputs: Sequence[Value], loc=None) -> List[Value]:
        outs = self._results_like(callee)
        self._emit("FuncCallOp", {"program_id": callee.index, "inputs": [v.ref for v in inputs],
                                  "outputs": [v.ref for v in outs]}, list(inputs), outs, loc)
        return outs

    def begin_trace_capture(self, loc=None) -> Value:
        tid = self._value([], "UInt32", False)
        self._emit("BeginTraceCaptureOp", {"device": self.device_ref, "trace_id": tid.ref, "cq_id": 0}, [], [tid], loc)
        return tid

    def end_trace_capture(self, trace_id: Value, loc=None):
        self._emit("EndTraceCaptureOp", {"device": self.device_ref, "trace_id": trace_id.ref, "cq_id": 0},
                   [trace_id], [], loc)

    def execute_trace(self, trace_id: Value, blocking: bool = False, loc=None):
        self._emit("ExecuteTraceOp", {"device": self.device_ref, "trace_id": trace_id.ref, "cq_id": 0,
                                      "blocking": blocking}, [trace_id], [], loc)

    def write_tensor(self, host: Value, device: Value, blocking: bool = False, loc=None):
        self._emit("WriteTensorOp", {"host_tensor": host.ref, "device_tensor": device.ref, "blocking": blocking,
                                     "cq_id": 0}, [host, device], [], loc)

    def copy(self, src: Value, dst: Value, loc=None):
        self._emit("CopyOp", {"src": src.ref, "dst": dst.ref}, [src, dst], [], loc)

    def capture_or_execute_trace(self, capture: "ProgramBuilder", execute: "ProgramBuilder", allocate: "ProgramBuilder",
                                 inputs: Sequence[Value], results_like: Sequence[Value], loc=None) -> List[Value]:
        outs = [self._value(v.shape, v.dtype, True) for v in results_like]
        self._emit("CaptureOrExecuteTraceOp", {
            "device": self.device_ref, "capture_program_id": capture.index, "execute_program_id": execute.index,
            "allocate_slots_program_id": allocate.index, "inputs": [v.ref for v in inputs],
            "outputs": [v.ref for v in outs]}, list(inputs), outs, loc)
        return outs

    # ---- finishing -----------------------------------------------------------------------------------------------------
    def _with_deallocs(self) -> List[dict]:
        """Inserts a DeallocateOp after the last use of every op result that is not a program output."""
        keep = {v.id for v in self.outputs} | {v.id for v in self.inputs}
        last_use: Dict[int, int] = {}
        produced: Dict[int, Value] = {}
        for i, (ins, outs) in enumerate(self._op_values):
            for v in ins:
                last_use[v.id] = i
            for v in outs:
                produced[v.id] = v
                last_use.setdefault(v.id, i)
        ops: List[dict] = []
        for i, op in enumerate(self.ops):
            ops.append(op)
            if op["type"][0] == "DeallocateOp":
                continue
            for vid, at in last_use.items():
                if at == i and vid in produced and vid not in keep:
                    v = produced[vid]
                    ops.append({"type": ("DeallocateOp", {"in": v.ref, "force": False}),
                                "debug_info": f'"ttnn.deallocate"(%{vid})', "loc_info": f'loc("dealloc_{vid}")'})
        return ops

    def golden(self, key: str, tensor, device: int = 0) -> None:
        """Embeds a golden tensor under `key` in the program's debug info, as the compiler's builders do
        (include/ttmlir/Target/Common/debug_info.fbs:5-31): "input_<i>" / "output_<i>" for program
        arguments and results, an op's location string for intermediates.  `tensor` is a torch tensor."""
        import torch
        names = {torch.float32: "Float32", torch.bfloat16: "BFloat16", torch.float16: "Float16", torch.int32: "Int32",
                 torch.uint8: "UInt8", torch.int8: "Int8", torch.uint16: "UInt16", torch.uint32: "UInt32"}
        t = tensor.contiguous()
        entry = {"name": key, "shape": [int(d) for d in t.shape], "stride": [int(x) for x in t.stride()],
                 "dtype": names[t.dtype], "data": bytes(t.view(torch.uint8).reshape(-1).numpy().tobytes())}
        self.goldens.setdefault(key, []).append({"device": int(device), "value": entry})

    def table(self, auto_dealloc: bool = True) -> dict:
        t = {
            "name": self.name,
            "inputs": [v.ref for v in self.inputs],
            "outputs": [v.ref for v in self.outputs],
            "operations": self._with_deallocs() if auto_dealloc else self.ops,
            "private": self.private,
            "mesh_shape": self.mesh_shape,
        }
        if self.goldens:
            t["debug_info"] = {"golden_info": {"golden_map": [{"key": k, "value": v} for k, v in self.goldens.items()]}}
        return t


class BinaryBuilder:
    def __init__(self, version=(0, 1, 0), git_hash: str = "b200-authored", system_desc: Optional[dict] = None):
        self.version = version
        self.git_hash = git_hash
        # the system the binary is "compiled for" (what ttrt compares with the machine's own descriptor);
        # None leaves the field out
        self.system_desc = system_desc
        self._next = 0
        self.programs: List[ProgramBuilder] = []
        self.auto_dealloc = True

    def next_id(self) -> int:
        i = self._next
        self._next += 1
        return i

    def program(self, name: str = "main", mesh_shape=(1, 1)) -> ProgramBuilder:
        p = ProgramBuilder(self, name, mesh_shape)
        self.programs.append(p)
        return p

    def private_program(self, name: str, mesh_shape=(1, 1)) -> ProgramBuilder:
        p = self.program(name, mesh_shape)
        p.private = True
        return p

    def hoist_trace(self, main: ProgramBuilder, name: str, inputs: Sequence[Value], body, index: int = 0) -> List[Value]:
        """Wraps `body` in a trace the way the compiler's trace hoisting does
        (lib/Dialect/TTNN/Transforms/TTNNTraceHoistTransform.cpp): four private programs

          trace_<i>_<name>                 (inputs..., output slots...)       the traced function; stores its
                                                                              results into the slots with CopyOp
          allocate_slots_trace_<i>_<name>  (device-resident inputs) -> input slots..., output slots...
          run_and_capture_trace_<i>_<name> (host-staged inputs..., input slots..., output slots...) -> trace id
          execute_trace_<i>_<name>         (trace id)

        and a CaptureOrExecuteTraceOp in `main`.  `inputs` are values of `main`: the ones on device
        (parameters, constants, const-eval results) are their own slots, the ones on host are staged
        into freshly allocated slots; device-resident inputs come first, as in the compiler's order.
        `body(program, args) -> results` emits the traced ops."""
        inputs = sorted(inputs, key=lambda v: 0 if v.on_device else 1)  # stable: resident first
        resident = [v for v in inputs if v.on_device]
        staged = [v for v in inputs if not v.on_device]
        mesh = main.mesh_shape

        fn = self.private_program(f"trace_{index}_{name}", mesh)
        args = [fn.input(v.shape, v.dtype, True) for v in inputs]
        results = list(body(fn, args))
        fn_slots = [fn.input(r.shape, r.dtype, True) for r in results]
        for r, slot in zip(results, fn_slots):
            fn.copy(r, slot)

        alloc = self.private_program(f"allocate_slots_trace_{index}_{name}", mesh)
        a_in = [alloc.input_like(v) for v in resident]
        a_slots = a_in + [alloc.empty(v.shape, v.dtype) for v in staged] + [alloc.empty(r.shape, r.dtype) for r in results]
        alloc.output(*a_slots)

        cap = self.private_program(f"run_and_capture_trace_{index}_{name}", mesh)
        c_host = [cap.input(v.shape, v.dtype, False) for v in staged]
        c_in = [cap.input(v.shape, v.dtype, True) for v in inputs]
        c_out = [cap.input(r.shape, r.dtype, True) for r in results]
        for h, slot in zip(c_host, c_in[len(resident):]):
            cap.write_tensor(h, slot)
        cap.func_call(fn, c_in + c_out)       # once normally: everything lazily set up is set up
        tid = cap.begin_trace_capture()
        cap.func_call(fn, c_in + c_out)       # once recording
        cap.end_trace_capture(tid)
        cap.execute_trace(tid)                # replay: the output slots hold this call's results
        cap.output(tid)

        exe = self.private_program(f"execute_trace_{index}_{name}", mesh)
        e_tid = exe.input([], "UInt32", False)
        exe.execute_trace(e_tid)

        return main.capture_or_execute_trace(cap, exe, alloc, inputs, results)

    def finish(self) -> bytes:
        w = Writer(S)
        root = w.create_table("TTNNBinary", {
            "version": self.version,
            "schema_hash": SCHEMA_HASH,
            "ttmlir_git_hash": self.git_hash,
            "system_desc": self.system_desc,
            "mlir": {"name": "ttnn", "source": ""},
            "programs": [p.table(self.auto_dealloc) for p in self.programs],
        })
        return w.finish(root, FILE_IDENTIFIER, size_prefixed=True)
