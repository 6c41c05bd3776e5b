"""Op-level CPU restatement of the reference semantics (see the package docstring for sources).

Every function takes and returns torch CPU tensors in the graph's storage dtype.  `_hoist`
applies the CPU-hoist rounding model: widen floats to f32 / integers to i32, run the op, narrow
to the result dtype (lib/Dialect/TTIR/Transforms/HoistCPUOps/HoistCPUOps.cpp:78-93).
Each op cites the reference function it follows; ttir_cpu.py = tools/tt-alchemist/templates/
python/local/ttir_cpu.py, mapping.py = tools/golden/mapping.py.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F


def _widen(t: torch.Tensor) -> torch.Tensor:
    if t.is_floating_point():
        return t.to(torch.float32)
    if t.dtype == torch.bool:
        return t
    return t.to(torch.int32)


def _hoist(fn, out_dtype, *tensors, **kw):
    res = fn(*[_widen(t) if isinstance(t, torch.Tensor) else t for t in tensors], **kw)
    return res.to(out_dtype)


# ---- eltwise (ttir_cpu.py:94-330) -------------------------------------------------------------
UNARY = {
    "Abs": torch.abs, "Ceil": torch.ceil, "Cos": torch.cos, "Floor": torch.floor,
    "Gelu": lambda t: F.gelu(t), "IsFinite": lambda t: torch.isfinite(t).to(t.dtype),
    "LogicalNot": lambda t: torch.logical_not(t).to(t.dtype), "Neg": torch.neg, "Relu": torch.relu,
    "Sqrt": lambda t: torch.sqrt(t.double()).to(t.dtype),  # correctly rounded, ttir_cpu.py:218-224
    "Rsqrt": torch.rsqrt, "Sigmoid": torch.sigmoid, "Sin": torch.sin,
    "Reciprocal": torch.reciprocal, "Sign": torch.sign, "Tan": torch.tan, "Tanh": torch.tanh,
    "Atan": torch.atan, "Exp": torch.exp, "Erf": torch.erf, "Erfc": torch.erfc, "Log": torch.log,
    "Expm1": torch.expm1, "Relu6": F.relu6, "Silu": F.silu, "Hardsigmoid": F.hardsigmoid,
    "Mish": lambda t: t * torch.tanh(F.softplus(t)),  # ttir_cpu.py:174
   
    "Acos": torch.acos, "Asin": torch.asin, "Asinh": torch.asinh,
    "Cbrt": lambda t: torch.sign(t) * torch.pow(torch.abs(t), 1.0 / 3.0), "Log1p": torch.log1p,
}


def unary(kind: str, x: torch.Tensor, param: Optional[float] = None) -> torch.Tensor:
    if kind == "LeakyRelu":
        return _hoist(lambda t: F.leaky_relu(t, param if param is not None else 0.01), x.dtype, x)
    if kind == "BitwiseNot":
        return torch.bitwise_not(x)
    return _hoist(UNARY[kind], x.dtype, x)


def _cmp(fn):
    return lambda a, b: fn(a, b)


BINARY = {
    "Add": torch.add, "Multiply": torch.mul, "Subtract": torch.sub, "Divide": torch.div,
    "Maximum": torch.maximum, "Minimum": torch.minimum, "Pow": torch.pow, "Atan2": torch.atan2,
    "Remainder": torch.remainder,
    "Equal": torch.eq, "NotEqual": torch.ne, "GreaterEqual": torch.ge, "GreaterThan": torch.gt,
    "LessEqual": torch.le, "LessThan": torch.lt,
    "LogicalAnd": torch.logical_and, "LogicalOr": torch.logical_or, "LogicalXor": torch.logical_xor,
    "BitwiseAnd": torch.bitwise_and, "BitwiseOr": torch.bitwise_or, "BitwiseXor": torch.bitwise_xor,
}


def binary(kind: str, a: torch.Tensor, b: torch.Tensor, out_dtype=None) -> torch.Tensor:
    out_dtype = out_dtype or a.dtype
    return _hoist(BINARY[kind], out_dtype, a, b)


def where(c, a, b):
    return torch.where(c != 0, a, b)


def clamp(x, lo, hi):
    return _hoist(lambda t: torch.clamp(t, lo, hi), x.dtype, x)


def typecast(x, dtype):  # ttir_cpu.py:498
    return x.to(dtype)


# ---- quantization (mapping.py:2534-2582; formulas include/ttmlir/Dialect/TTIR/IR/TTIROps.td:6010-6137) --
def _qdtype(container: torch.dtype, clamp_i8: bool):
    if container == torch.int8 or (container == torch.int32 and clamp_i8):
        return torch.qint8
    if container == torch.uint8:
        return torch.quint8
    return torch.qint32


def quantize(x: torch.Tensor, scale: float, zero_point: int, container: torch.dtype = torch.int32,
             clamp_i8: bool = True) -> torch.Tensor:
    q = torch.quantize_per_tensor(x.to(torch.float32), scale, zero_point, _qdtype(container, clamp_i8)).int_repr()
    return q.to(container)


def dequantize(q: torch.Tensor, scale: float, zero_point: int, out_dtype=torch.float32) -> torch.Tensor:
    # torch.dequantize(q) = (q - zp) * scale in f32
    return ((q.to(torch.int32) - zero_point).to(torch.float32) * torch.tensor(scale, dtype=torch.float32)).to(out_dtype)


def requantize(q: torch.Tensor, in_scale: float, in_zp: int, out_scale: float, out_zp: int,
               container: Optional[torch.dtype] = None, clamp_i8: bool = True) -> torch.Tensor:
    # golden: quantize(dequantize(q)) with the new parameters
    return quantize(dequantize(q, in_scale, in_zp), out_scale, out_zp, container or q.dtype, clamp_i8)


def quantize_per_axis(x, scales: torch.Tensor, zps: Optional[torch.Tensor], axis: int, container=torch.int32,
                      clamp_i8: bool = True):
    zps = zps if zps is not None else torch.zeros_like(scales, dtype=torch.int32)
    q = torch.quantize_per_channel(x.to(torch.float32), scales.to(torch.float32).double(), zps.to(torch.int64), axis,
                                   _qdtype(container, clamp_i8)).int_repr()
    return q.to(container)


def dequantize_per_axis(q, scales: torch.Tensor, zps: Optional[torch.Tensor], axis: int, out_dtype=torch.float32):
    shape = [1] * q.dim()
    shape[axis] = -1
    z = zps.to(torch.int32).reshape(shape) if zps is not None else 0
    return ((q.to(torch.int32) - z).to(torch.float32) * scales.to(torch.float32).reshape(shape)).to(out_dtype)


# ---- contractions (ttir_cpu.py:509-521; f32 accumulation per lib/Conversion/TTIRToLinalg/TTIRToLinalg.cpp:542-549) --
def matmul(a, b, transpose_a=False, transpose_b=False, activation=None):
    def fn(x, y):
        if transpose_a:
            x = x.transpose(-2, -1)
        if transpose_b:
            y = y.transpose(-2, -1)
        return _act(torch.matmul(x, y), activation)
    return _hoist(fn, a.dtype, a, b)


def int_matmul(a, b, transpose_a=False, transpose_b=False, out_dtype=torch.int32):
    """Matmul on quantized (integer) operands with an Int32 accumulator, which is what the CPU-hoist
    path computes after widening integers to i32 (HoistCPUOps.cpp:78-93) and what the quantized
    convolution's i32 result type prescribes (lib/Dialect/TTIR/IR/TTIROps.cpp:1516-1577).  Evaluated in
    f64, which is exact here: |a b| <= 2^14 per product and sums stay far below 2^53."""
    x, y = a.to(torch.float64), b.to(torch.float64)
    if transpose_a:
        x = x.transpose(-2, -1)
    if transpose_b:
        y = y.transpose(-2, -1)
    return torch.matmul(x, y).to(torch.int64).to(out_dtype)


def linear(a, b, bias=None, transpose_a=False, transpose_b=False, activation=None):
    def fn(x, y, z=None):
        if transpose_a:
            x = x.transpose(-2, -1)
        if transpose_b:
            y = y.transpose(-2, -1)
        r = torch.matmul(x, y)
        if z is not None:
            r = r + z
        return _act(r, activation)
    if bias is None:
        return _hoist(fn, a.dtype, a, b)
    return _hoist(fn, a.dtype, a, b, bias)


def _act(t, name):
    if not name:
        return t
    return {"relu": torch.relu, "silu": F.silu, "gelu": F.gelu, "sigmoid": torch.sigmoid}[name](t)


def conv2d(x, w, bias, batch, height, width, stride=(1, 1), padding=(0, 0, 0, 0), dilation=(1, 1), groups=1):
    """NHWC activations (any view with N*H*W*C elements), OIHW weights, bias [1,1,1,O]
    (ttir_cpu.py:772-815).  Returns a tensor shaped like the input view ([1,1,P,O] or [N,Ho,Wo,O])."""
    c = w.shape[1] * groups
    flat = x.dim() == 4 and x.shape[0] == 1 and x.shape[1] == 1 and x.shape[2] == batch * height * width

    def fn(xx, ww, bb=None):
        t = xx.reshape(batch, height, width, c).permute(0, 3, 1, 2)
        pt, pl, pb, pr = padding
        t = F.pad(t, (pl, pr, pt, pb))
        r = F.conv2d(t, ww, bias=bb.reshape(-1) if bb is not None else None, stride=tuple(stride), padding=0,
                     dilation=tuple(dilation), groups=groups)
        r = r.permute(0, 2, 3, 1)
        return r.reshape(1, 1, -1, r.shape[-1]) if flat else r
    if bias is None:
        return _hoist(fn, x.dtype, x, w)
    return _hoist(fn, x.dtype, x, w, bias)


def int_conv2d(x, w, batch, height, width, stride=(1, 1), padding=(0, 0, 0, 0), dilation=(1, 1), groups=1,
               out_dtype=torch.int32):
    """conv2d on quantized (integer) operands with an Int32 accumulator (the result type the compiler
    gives the quantized convolution, lib/Dialect/TTIR/IR/TTIROps.cpp:1516-1577).  Same layouts as conv2d;
    evaluated in f64, which is exact for these magnitudes."""
    c = w.shape[1] * groups
    flat = x.dim() == 4 and x.shape[0] == 1 and x.shape[1] == 1 and x.shape[2] == batch * height * width
    t = x.to(torch.float64).reshape(batch, height, width, c).permute(0, 3, 1, 2)
    pt, pl, pb, pr = padding
    t = F.pad(t, (pl, pr, pt, pb))
    r = F.conv2d(t, w.to(torch.float64), stride=tuple(stride), padding=0, dilation=tuple(dilation), groups=groups)
    r = r.permute(0, 2, 3, 1).to(torch.int64).to(out_dtype)
    return r.reshape(1, 1, -1, r.shape[-1]) if flat else r.contiguous()


# ---- normalisation / reductions -------------------------------------------------------------------
def softmax(x, dim=-1):  # ttir_cpu.py:585
    return _hoist(lambda t: F.softmax(t, dim=dim), x.dtype, x)


def rms_norm(x, weight=None, bias=None, epsilon=1e-5):  # mapping.py:1221-1290
    r = F.rms_norm(x.float(), normalized_shape=(x.shape[-1],), weight=weight, eps=epsilon)
    if bias is not None:
        r = torch.add(r, bias.float())
    return r.to(x.dtype)


def reduce(kind, x, dims, keep_dim):  # ttir_cpu.py:374-397
    dims = tuple(dims) if dims else tuple(range(x.dim()))

    def fn(t):
        if kind == "Sum":
            return torch.sum(t, dim=dims, keepdim=keep_dim)
        if kind == "Mean":
            return torch.mean(t, dim=dims, keepdim=keep_dim)
        r = t
        for d in sorted((d % t.dim() for d in dims), reverse=True):
            r = (torch.max if kind == "Max" else torch.min)(r, dim=d, keepdim=keep_dim).values
        return r
    return _hoist(fn, x.dtype, x)


# ---- data movement (ttir_cpu.py:449-495, 824-877) -----------------------------------------------------
def layer_norm(x, weight=None, bias=None, epsilon=1e-5):  # ttir_cpu.py layer_norm: F.layer_norm over weight.shape
    shape = tuple(weight.shape) if weight is not None else (x.shape[-1],)
    return _hoist(lambda t, w=None, b=None: F.layer_norm(t, shape, weight=w, bias=b, eps=epsilon), x.dtype, x, weight, bias)


def argmax(x, dim=None, keep_dim=False):  # ttir_cpu.py argmax: torch.argmax, Int32 result
    if dim is None:
        idx = torch.argmax(x.flatten())
        return (idx.reshape([1] * x.dim()) if keep_dim else idx).to(torch.int32)
    return torch.argmax(x, dim=dim, keepdim=keep_dim).to(torch.int32)


def cumsum(x, dim):  # ttir_cpu.py cumsum
    return torch.cumsum(x, dim=dim).to(x.dtype)


def cumprod(x, dim):  # tools/golden/mapping.py:4308-4314 (torch.cumprod, result in the input's type)
    return torch.cumprod(x, dim=dim).to(x.dtype)


def prod(x, dim=None, keep_dim=False):
    """tools/golden/mapping.py:2858-2900 (torch.prod over one dim, or over all).  16-bit floats are widened to f32 for
    the op and narrowed once, as every CPU-hoisted op is (torch itself would keep a bf16 running product)."""
    xf = x.float() if x.dtype in (torch.bfloat16, torch.float16) else x
    if dim is None:
        r = torch.prod(xf)
        r = r.reshape([1] * x.dim()) if keep_dim else r
    else:
        r = torch.prod(xf, dim=dim, keepdim=keep_dim)
    return r.to(x.dtype)


def batch_norm_inference(x, mean, var, weight, bias, epsilon):
    """tools/golden/mapping.py:4948-4976 with the channel dimension at 1: torch's inference batch norm, evaluated in
    f32 (the CPU-hoist rounding model: widen, one op, narrow)."""
    r = F.batch_norm(x.float(), running_mean=mean.float(), running_var=var.float(),
                     weight=None if weight is None else weight.float(), bias=None if bias is None else bias.float(),
                     training=False, eps=epsilon)
    return r.to(x.dtype)


def upsample2d(x, scale, mode="nearest"):
    """tools/golden/mapping.py:3552-3578: NHWC in, torch.nn.functional.interpolate on the channels-first view, NHWC
    out.  The golden transposes dims 1 and 3 (H and C) and hands interpolate the (H_out, W_out) of the result, which
    is the intended NHWC upsampling for square inputs with one scale; this restatement permutes properly so that
    non-square inputs and two scales mean what ::ttnn::upsample computes."""
    sy, sx = (scale, scale) if isinstance(scale, int) else scale
    nchw = x.permute(0, 3, 1, 2).float()
    out = F.interpolate(nchw, size=(x.shape[1] * sy, x.shape[2] * sx), mode=mode,
                        **({"align_corners": False} if mode == "bilinear" else {}))
    return out.permute(0, 2, 3, 1).contiguous().to(x.dtype)


def group_norm(x, weight, bias, num_groups, epsilon):
    """tools/golden/mapping.py:1541-1574: channels-last [N, 1, H*W, C] in, torch group_norm on the NCHW view in f32."""
    w = None if weight is None else weight.float().reshape(-1)
    b = None if bias is None else bias.float().reshape(-1)
    r = F.group_norm(x.float().permute(0, 3, 1, 2), num_groups=num_groups, weight=w, bias=b, eps=epsilon)
    return r.permute(0, 2, 3, 1).contiguous().to(x.dtype)


def conv_transpose2d(x, w, bias, batch, height, width, stride, padding, output_padding, dilation, groups):
    """tools/golden/mapping.py:804-893: NHWC (possibly flattened) in, torch conv_transpose2d on the NCHW view with f32
    accumulation, NHWC out in the input's form."""
    c = w.shape[0]
    nchw = x.reshape(batch, height, width, c).permute(0, 3, 1, 2).float()
    r = F.conv_transpose2d(nchw, w.float(), None if bias is None else bias.float().reshape(-1), stride=tuple(stride),
                           padding=tuple(padding), output_padding=tuple(output_padding), dilation=tuple(dilation), groups=groups)
    r = r.permute(0, 2, 3, 1).contiguous().to(x.dtype)
    return r.reshape(1, 1, -1, r.shape[-1]) if x.dim() == 4 and x.shape[0] == 1 and x.shape[1] == 1 and batch * height * width == x.shape[2] else r


def conv1d(x, w, bias, stride, padding, dilation, groups):
    """tools/golden/mapping.py:502-574: NLC in, torch conv1d on the NCL view (asymmetric padding applied first), NLC out."""
    ncl = F.pad(x.float().permute(0, 2, 1), [padding[0], padding[1]])
    r = F.conv1d(ncl, w.float(), None if bias is None else bias.float().reshape(-1), stride=stride, padding=0, dilation=dilation,
                 groups=groups)
    return r.permute(0, 2, 1).contiguous().to(x.dtype)


def embedding(indices, weight):  # ttir_cpu.py embedding: leading 1-dims of the table are dropped
    w = weight
    while w.dim() > 2 and w.shape[0] == 1:
        w = w.squeeze(0)
    return F.embedding(indices.long(), w)


def _nchw(x, batch, height, width, channels):  # ttir_cpu.py _pool_to_nchw
    return x.reshape(batch, height, width, channels).permute(0, 3, 1, 2)


def max_pool2d(x, batch, height, width, channels, kernel, stride, padding, dilation=(1, 1), ceil_mode=False):
    """ttir_cpu.py max_pool2d / _pool_padding.  `padding` in flatbuffer order: (h, w) or (top, left,
    bottom, right); four paddings are applied as -inf data before pooling.  Result flattened like
    the TTNN op's: [1, 1, N*Ho*Wo, C]."""
    def fn(t):
        t = _nchw(t, batch, height, width, channels)
        if len(padding) == 4:
            pt, pl, pb, pr = padding
            t = F.pad(t, (pl, pr, pt, pb), mode="constant", value=float("-inf"))
            pad = 0
        else:
            pad = tuple(padding)
        y = F.max_pool2d(t, kernel_size=tuple(kernel), stride=tuple(stride), padding=pad, dilation=tuple(dilation),
                         ceil_mode=ceil_mode)
        return y.permute(0, 2, 3, 1).reshape(1, 1, -1, channels)
    return _hoist(fn, x.dtype, x)


def avg_pool2d(x, batch, height, width, channels, kernel, stride, padding, ceil_mode=False, count_include_pad=True):
    """ttir_cpu.py avg_pool2d: symmetric padding up to half the kernel goes to torch; anything else is
    applied by hand (zeros), with sum / count when padding must not be counted."""
    if len(padding) == 4:
        pt, pl, pb, pr = padding
    else:
        pt = pb = padding[0]
        pl = pr = padding[1]
    ks, st = tuple(kernel), tuple(stride)
    symmetric = pt == pb and pl == pr
    exceeds = pt > ks[0] // 2 or pl > ks[1] // 2

    def fn(t):
        t = _nchw(t, batch, height, width, channels)
        if symmetric and not exceeds:
            y = F.avg_pool2d(t, ks, st, (pt, pl), ceil_mode, count_include_pad)
        elif not count_include_pad and not symmetric:
            ones = F.pad(torch.ones_like(t), (pl, pr, pt, pb))
            tp = F.pad(t, (pl, pr, pt, pb))
            y = F.avg_pool2d(tp, ks, st, 0, ceil_mode, True) / F.avg_pool2d(ones, ks, st, 0, ceil_mode, True).clamp(min=1e-8)
        else:
            y = F.avg_pool2d(F.pad(t, (pl, pr, pt, pb)), ks, st, 0, ceil_mode, count_include_pad)
        return y.permute(0, 2, 3, 1).reshape(1, 1, -1, channels)
    return _hoist(fn, x.dtype, x)


def global_avg_pool2d(x):  # ttir_cpu.py global_avg_pool2d, NHWC in and out
    return _hoist(lambda t: F.adaptive_avg_pool2d(t.permute(0, 3, 1, 2), (1, 1)).permute(0, 2, 3, 1), x.dtype, x)


def pad(x, padding, value=0.0):  # ttir_cpu.py pad: (low, high) per dimension, outermost first
    pairs = [(padding[i], padding[i + 1]) for i in range(0, len(padding), 2)]
    flat = []
    for lo, hi in reversed(pairs):
        flat.extend([lo, hi])
    return F.pad(x, tuple(flat), value=value)


def fill_cache(cache, x, batch_offset=0):
    """mapping.py:3582-3611 (fill_cache_golden), with the batch offset the TTNN op takes: the input's
    users land at cache[batch_offset : batch_offset + users]; rows up to the next multiple of the
    32-row tile are zeroed when the cache has them."""
    out = cache.clone()
    users, _, seq, _ = x.shape
    pad = (seq + 31) // 32 * 32
    out[batch_offset:batch_offset + users, :, :seq, :] = x
    if seq < pad <= cache.shape[2]:
        out[batch_offset:batch_offset + users, :, seq:pad, :] = 0
    return out


def update_cache(cache, x, update_index, batch_offset=0):
    """mapping.py:3614-3670 (update_cache_golden): cache[batch_offset + b, h, idx, :] = x[0, h, b, :]."""
    out = cache.clone()
    idx = int(update_index.flatten()[0].item())
    users = x.shape[2]
    out[batch_offset:batch_offset + users, :, idx, :] = x[0].permute(1, 0, 2)
    return out


def sdpa_decode(q, k, v, cur_pos=None, mask=None, is_causal=True, scale=None):
    """mapping.py:2417-2482 (sdpa_decode_golden): q [1, B, H, D], k / v [B, Hkv, S, D]; the mask
    [B|1, 1, H|1, S] is added before the scale; causal = keys after cur_pos[b] are -inf."""
    qq = q.float().squeeze(0).unsqueeze(2)                      # [B, H, 1, D]
    kk, vv = k.float(), v.float()
    rep = qq.shape[1] // kk.shape[1]
    if rep > 1:
        kk = torch.repeat_interleave(kk, rep, dim=1)
        vv = torch.repeat_interleave(vv, rep, dim=1)
    qk = torch.matmul(qq, kk.transpose(-2, -1))                 # [B, H, 1, S]
    if mask is not None:
        qk = qk + mask.float().permute(0, 2, 1, 3)
    elif is_causal and cur_pos is not None:
        cm = torch.zeros((qk.shape[0], 1, 1, qk.shape[3]), dtype=torch.float32)
        for i in range(qk.shape[0]):
            cm[i, :, :, int(cur_pos[i].item()) + 1:] = float("-inf")
        qk = qk + cm
    if scale is not None:
        qk = qk * scale
    out = torch.matmul(torch.softmax(qk, dim=-1), vv)           # [B, H, 1, D]
    return out.squeeze(2).unsqueeze(0).to(q.dtype)


def concatenate_heads(x):
    b, h, s, d = x.shape
    return x.permute(0, 2, 1, 3).reshape(b, s, h * d)


def split_qkv(x, kv, num_heads, num_kv_heads=None, transpose_key=False):
    hkv = num_kv_heads if num_kv_heads is not None else num_heads
    b, s = x.shape[0], x.shape[1]
    d = x.shape[-1] // (num_heads + 2 * hkv) if kv is None else x.shape[-1] // num_heads
    if kv is None:
        q, k, v = x[:, :, :num_heads * d], x[:, :, num_heads * d:(num_heads + hkv) * d], x[:, :, (num_heads + hkv) * d:]
    else:
        q, k, v = x, kv[:, :, :hkv * d], kv[:, :, hkv * d:]
    q = q.reshape(b, s, num_heads, d).permute(0, 2, 1, 3).contiguous()
    k = k.reshape(b, s, hkv, d).permute(0, 2, 1, 3).contiguous()
    v = v.reshape(b, s, hkv, d).permute(0, 2, 1, 3).contiguous()
    if transpose_key:
        k = k.transpose(-2, -1).contiguous()
    return q, k, v


def rotary_embedding(x, cos, sin):
    """x*cos + rotate_half(x)*sin (lib/Dialect/TTNN/Transforms/Fusing/RoPEFusingPattern.cpp:49-51);
    one op, so f32 math and a single rounding."""
    def fn(t, c, s):
        half = t.shape[-1] // 2
        rot = torch.cat((-t[..., half:], t[..., :half]), dim=-1)
        c = c.reshape(t.shape[-2], t.shape[-1])
        s = s.reshape(t.shape[-2], t.shape[-1])
        return t * c + rot * s
    return _hoist(fn, x.dtype, x, cos, sin)


def sdpa(q, k, v, is_causal=True, mask=None, scale=None):  # mapping.py:8398-8500
    hq, hkv = q.shape[1], k.shape[1]
    if hq != hkv:
        k = torch.repeat_interleave(k, hq // hkv, dim=1)
        v = torch.repeat_interleave(v, hq // hkv, dim=1)
    if scale is None:
        scale = 1.0 / (float(q.shape[-1]) ** 0.5)
    qk = torch.matmul(q.float(), k.float().transpose(-2, -1))
    qk = torch.mul(qk, scale)
    if is_causal and mask is None:
        sq, sk = qk.shape[-2], qk.shape[-1]
        qk = torch.add(qk, torch.triu(torch.full((sq, sk), float("-inf")), diagonal=1))
    if mask is not None:
        qk = torch.add(qk, mask.float())
    w = torch.softmax(qk, dim=-1)
    return torch.matmul(w, v.float()).to(q.dtype)


# ---- mesh (mapping.py:4189-4235, 5658-5794); a distributed value is a list of shards ------------------
def mesh_shard_full_to_shard(x: torch.Tensor, n: int, shard_dim: Optional[int]) -> List[torch.Tensor]:
    if shard_dim is None:
        return [x.clone() for _ in range(n)]
    return [c.contiguous() for c in torch.chunk(x, n, dim=shard_dim)]


def mesh_shard_shard_to_full(shards: Sequence[torch.Tensor], shard_dim: Optional[int]) -> torch.Tensor:
    if shard_dim is None:
        return shards[0].clone()
    return torch.cat(list(shards), dim=shard_dim)


REDUCE = {0: lambda xs: torch.sum(torch.stack(xs), 0), 1: lambda xs: torch.mean(torch.stack(xs), 0),
          2: lambda xs: torch.amax(torch.stack(xs), 0), 3: lambda xs: torch.amin(torch.stack(xs), 0)}


def all_reduce(shards, reduce_type=0):
    dt = shards[0].dtype
    r = REDUCE[reduce_type]([s.float() for s in shards]).to(dt)
    return [r.clone() for _ in shards]


def all_gather(shards, dim):
    g = torch.cat(list(shards), dim=dim)
    return [g.clone() for _ in shards]


def reduce_scatter(shards, dim, reduce_type=0):
    dt = shards[0].dtype
    r = REDUCE[reduce_type]([s.float() for s in shards]).to(dt)
    return [c.contiguous() for c in torch.chunk(r, len(shards), dim=dim)]


def point_to_point(shards, sender, receiver, output=None):
    """::ttnn::point_to_point (runtime/lib/ttnn/operations/ccl/point_to_point.cpp): every coordinate keeps its shard of
    the output tensor (the input when none is given), the receiver's becomes the sender's shard of the input."""
    base = output if output is not None else shards
    out = [s.clone() for s in base]
    out[receiver] = shards[sender].clone()
    return out


def mesh_partition(shards, dim):
    n = len(shards)
    return [torch.chunk(s, n, dim=dim)[i].contiguous() for i, s in enumerate(shards)]


# ---- indexing ops (mapping.py:5384-5437, 5624-5640, 5927-5958) ------------------------------------------
def gather(x, index, dim):  # ttir_gather_golden: torch.gather with 64-bit indices
    return torch.gather(x, dim, index.to(torch.int64))


def scatter(x, index, src, dim, reduce_type=None):
    """ttir_scatter_golden: plain scatter (reduce type Invalid) or scatter_reduce with sum / prod / amax /
    amin, the input's own values included."""
    idx = index.to(torch.int64)
    if reduce_type in (None, "Invalid"):
        return torch.scatter(x, dim, idx, src)
    return torch.scatter_reduce(x, dim, idx, src, reduce={"Sum": "sum", "Prod": "prod", "Max": "amax", "Min": "amin"}[reduce_type])


def sort(x, dim=-1, descending=False, stable=True):  # ttir_sort_golden; indices narrowed to Int32 (the device width)
    values, indices = torch.sort(x, dim=dim, descending=descending, stable=stable)
    return values, indices.to(torch.int32)


def topk(x, k, dim=-1, largest=True):  # ttir_topk_golden: always sorted; ties keep torch.topk's order
    values, indices = torch.topk(x, k=k, dim=dim, largest=largest, sorted=True)
    return values, indices.to(torch.int32)


# ---- paged kv-cache (mapping.py:8745-8844, 8926-9007) ---------------------------------------------------
def paged_update_cache(cache, x, update_index, page_table=None):
    """ttir_paged_update_cache_golden: cache [blocks, heads, block_size, d], x [batch, seq, heads, d];
    token s of user b lands at position update_index[b] + s, in the physical block the page table
    names (indices clamped into range)."""
    out = cache.clone()
    blocks, _, block_size, _ = cache.shape
    for b in range(x.shape[0]):
        for s in range(x.shape[1]):
            pos = int(update_index[b].item()) + s
            blk, off = pos // block_size, pos % block_size
            if page_table is not None:
                blk = int(page_table[b, min(max(blk, 0), page_table.shape[1] - 1)].item())
            blk = min(max(blk, 0), blocks - 1)
            out[blk, :, off, :] = x[b, s]
    return out


def paged_fill_cache(cache, x, page_table, batch_idx=None):
    """ttir_paged_fill_cache_golden: x [batch, heads, seq, d]; user b uses page-table row batch_idx[b]."""
    out = cache.clone()
    blocks, _, block_size, _ = cache.shape
    for b in range(x.shape[0]):
        row = int(batch_idx.reshape(-1)[b].item()) if batch_idx is not None else b
        row = min(max(row, 0), page_table.shape[0] - 1)
        for pos in range(x.shape[2]):
            col = min(pos // block_size, page_table.shape[1] - 1)
            blk = min(max(int(page_table[row, col].item()), 0), blocks - 1)
            out[blk, :, pos % block_size, :] = x[b, :, pos, :]
    return out


def paged_sdpa_decode(q, k_cache, v_cache, page_table, cur_pos=None, is_causal=True, scale=None, mask=None):
    """ttir_paged_sdpa_decode_golden: q [B, 1, H, D]; caches [blocks, Hkv, block_size, D]; keys after
    cur_pos[b] get the most negative f32 (pre-scaled, as the golden has it) and the softmax runs in f32."""
    b, sq, h, d = q.shape
    blocks, hkv, block_size, _ = k_cache.shape
    per_user = page_table.shape[-1]
    seq = per_user * block_size
    flat = page_table.long().reshape(-1).clamp(0, blocks - 1)

    def unpage(c):
        t = c[flat].reshape(b, per_user, hkv, block_size, c.shape[-1])
        return t.transpose(1, 2).reshape(b, hkv, seq, c.shape[-1]).float()
    kk, vv = unpage(k_cache), unpage(v_cache)
    if h // hkv > 1:
        kk = kk.repeat_interleave(h // hkv, dim=1)
        vv = vv.repeat_interleave(h // hkv, dim=1)
    m = None
    if mask is not None:
        m = mask.float().permute(0, 2, 1, 3)
    elif is_causal and cur_pos is not None:
        m = torch.zeros((b, h, sq, seq), dtype=torch.float32)
        for i in range(b):
            m[i, :, :, int(cur_pos[i].item()) + 1:] = torch.finfo(torch.float32).min
    if m is not None:
        m = m * (scale if scale is not None else d ** -0.5)
    o = F.scaled_dot_product_attention(q.float().permute(0, 2, 1, 3), kk, vv, attn_mask=m, scale=scale, is_causal=False)
    return o.permute(0, 2, 1, 3).to(q.dtype)


def pow_scalar(x: torch.Tensor, exponent) -> torch.Tensor:
    """tools/golden/mapping.py:10447-10450 (torch.pow(lhs, exponent)); evaluated in f32, one rounding."""
    return torch.pow(x.float(), float(exponent)).to(x.dtype)


def batch_norm_training(x, running_mean, running_var, weight, bias, eps: float, momentum: float):
    """tools/golden/mapping.py:4979-5063: batch mean and biased batch variance over every dimension but 1 normalise x
    ((x - mean) / sqrt(var + eps) * weight + bias); the running statistics become
    momentum * batch + (1 - momentum) * running.  Returns (y, new_running_mean, new_running_var)."""
    dt = x.dtype
    xf = x.float()
    dims = [0] + list(range(2, xf.ndim))
    shape = [1, -1] + [1] * (xf.ndim - 2)
    mean = xf.mean(dim=dims)
    var = ((xf - mean.reshape(shape)) ** 2).sum(dim=dims) / (xf.numel() // xf.shape[1])
    y = (xf - mean.reshape(shape)) / torch.sqrt(var.reshape(shape) + eps)
    if weight is not None:
        y = y * weight.float().reshape(shape)
    if bias is not None:
        y = y + bias.float().reshape(shape)
    new_mean = mean * momentum + running_mean.float().reshape(-1) * (1 - momentum)
    new_var = var * momentum + running_var.float().reshape(-1) * (1 - momentum)
    return y.to(dt), new_mean.reshape(running_mean.shape).to(dt), new_var.reshape(running_var.shape).to(dt)


def max_pool2d_with_indices(x, batch, height, width, channels, kernel, stride, padding, dilation, ceil_mode):
    """tools/golden/mapping.py:5339-5378: torch max_pool2d(return_indices=True) on the NCHW view of NHWC data; the
    index is iy * W + ix inside the image's plane.  Returns flattened [1, 1, N*Ho*Wo, C] values and indices."""
    t = x.reshape(batch, height, width, channels).permute(0, 3, 1, 2).float()
    pad = (padding[0], padding[1])
    y, idx = torch.nn.functional.max_pool2d(t, kernel_size=tuple(kernel), stride=tuple(stride), padding=pad, dilation=tuple(dilation),
                                            ceil_mode=ceil_mode, return_indices=True)
    y = y.permute(0, 2, 3, 1).reshape(1, 1, -1, channels).to(x.dtype)
    return y, idx.permute(0, 2, 3, 1).reshape(1, 1, -1, channels)


def rotary_embedding_llama(x, cos, sin, trans_mat, is_decode_mode: bool):
    """::ttnn::experimental::rotary_embedding_llama (runtime/lib/ttnn/operations/transformer/rotary_embedding_llama.cpp):
    y = x * cos + (x @ T) * sin, the 32 x 32 matrix T applied to every 32-wide piece of the head dimension.  Prefill: x
    [1, heads, seq, D], caches [1, 1, seq, D]; decode: x [1, batch, heads, D], caches [1, batch, 1, D].  f32, one rounding."""
    xf, d = x.float(), x.shape[-1]
    t = trans_mat.float().reshape(-1, 32)[:32]
    rot = (xf.reshape(*x.shape[:-1], d // 32, 32) @ t).reshape(x.shape)
    c, s = cos.float(), sin.float()
    if not is_decode_mode:
        c, s = c[..., : x.shape[-2], :], s[..., : x.shape[-2], :]
    return (xf * c + rot * s).to(x.dtype)


def nlp_create_qkv_heads_decode(x, num_heads, num_kv_heads, batch_offset=0, slice_size=None):
    """::ttnn::experimental::nlp_create_qkv_heads_decode: [1, 1, B, (Hq + 2 Hkv) D] -> q [1, B, Hq, D], k, v [1, B, Hkv, D]."""
    b, hidden = x.shape[2], x.shape[3]
    hkv = num_heads if num_kv_heads is None else num_kv_heads
    d = hidden // (num_heads + 2 * hkv)
    rows = x.reshape(b, hidden)
    if slice_size is not None:
        rows = rows[batch_offset: batch_offset + slice_size]
    n = rows.shape[0]
    q = rows[:, : num_heads * d].reshape(1, n, num_heads, d)
    k = rows[:, num_heads * d: (num_heads + hkv) * d].reshape(1, n, hkv, d)
    v = rows[:, (num_heads + hkv) * d:].reshape(1, n, hkv, d)
    return q.contiguous(), k.contiguous(), v.contiguous()


def nlp_concat_heads_decode(x, num_heads):
    """::ttnn::experimental::nlp_concat_heads_decode: [1, B, padded heads, D] -> [1, 1, B, num_heads * D]."""
    return x[:, :, :num_heads, :].reshape(1, 1, x.shape[1], num_heads * x.shape[3]).contiguous()


FUSED_ACTIVATIONS = {
    "relu": torch.nn.functional.relu, "relu6": torch.nn.functional.relu6, "silu": torch.nn.functional.silu,
    "mish": torch.nn.functional.mish, "sigmoid": torch.sigmoid, "hardsigmoid": torch.nn.functional.hardsigmoid,
    "tanh": torch.tanh, "log": torch.log, "softplus": torch.nn.functional.softplus, "gelu": torch.nn.functional.gelu,
    "sqrt": torch.sqrt,
}


def dit_rms_norm_unary_fused(x, weight, bias, residual, eps: float, activation):
    """tools/golden/mapping.py:1291-1326: act(rms_norm(x + residual, weight) + bias), f32 throughout, one rounding."""
    xf = x.float() if residual is None else x.float() + residual.float()
    y = xf * torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    if weight is not None:
        y = y * weight.float().reshape(-1)
    if bias is not None:
        y = y + bias.float().reshape(-1)
    if activation:
        name = activation[:-7] if activation.endswith("_approx") else activation
        y = FUSED_ACTIVATIONS[name](y)
    return y.to(x.dtype)


def distributed_rms_norm(shards, weights, residuals, eps: float):
    """tools/golden/mapping.py:1329-1415: the shards are slices of the last dimension; the RMS statistics are those
    of the concatenated rows, weight slices apply locally, each device keeps its slice of the result."""
    xs = [s.float() if residuals is None else s.float() + r.float() for s, r in zip(shards, residuals or shards)]
    total = sum(x.square().sum(dim=-1, keepdim=True) for x in xs)
    n = sum(x.shape[-1] for x in xs)
    scale = torch.rsqrt(total / n + eps)
    out = []
    for i, x in enumerate(xs):
        y = x * scale
        if weights is not None:
            y = y * weights[i].float().reshape(-1)
        out.append(y.to(shards[i].dtype))
    return out


def rms_norm_pre_all_gather(x, residual, dtype):
    """tools/golden/mapping.py:7800-7826: [..., 32] with E(x^2) of the local row in column 0."""
    xf = x.float() if residual is None else x.float() + residual.float()
    out = torch.zeros(list(x.shape[:-1]) + [32])
    out[..., :1] = xf.square().mean(dim=-1, keepdim=True)
    return out.to(dtype)


def layer_norm_pre_all_gather(x, residual, dtype):
    """tools/golden/mapping.py:7852-7888: [..., 64] with sum(x^2) in column 0 and sum(x) in column 32."""
    xf = x.float() if residual is None else x.float() + residual.float()
    out = torch.zeros(list(x.shape[:-1]) + [64])
    out[..., :1] = xf.square().sum(dim=-1, keepdim=True)
    out[..., 32:33] = xf.sum(dim=-1, keepdim=True)
    return out.to(dtype)


def layer_norm_post_all_gather(x, stats, weight, bias, eps: float):
    """::ttnn::layer_norm_post_all_gather: mean and variance of the whole distributed row rebuilt from the gathered
    [..., 64 * devices] statistics normalise the local slice.  With one device this is the reference golden
    (tools/golden/mapping.py:7891-7921, layer_norm of the shard)."""
    blocks = stats.shape[-1] // 64
    st = stats.float().reshape(*stats.shape[:-1], blocks, 64)
    n = x.shape[-1] * blocks
    mean = st[..., 32].sum(dim=-1, keepdim=True) / n
    var = (st[..., 0].sum(dim=-1, keepdim=True) / n - mean * mean).clamp_min(0.0)
    y = (x.float() - mean) * torch.rsqrt(var + eps)
    if weight is not None:
        y = y * weight.float().reshape(-1)
    if bias is not None:
        y = y + bias.float().reshape(-1)
    return y.to(x.dtype)


# ---- mixture of experts (mapping.py:1596-1760, 2030-2186; ::ttnn::all_to_all_dispatch / all_to_all_combine /
# moe_expert_token_remap / sparse_matmul).  expert_mapping is the [1, 1, E, D] one-hot ownership table; a device numbers
# its experts in ascending global order.
def _local_experts(mapping, device):
    m = mapping.reshape(mapping.shape[-2], mapping.shape[-1])
    return [e for e in range(m.shape[0]) if int(m[e, device]) != 0]


def all_to_all_dispatch(xs, indices, mapping):
    """Per device: the global token grid (devices concatenated along the batch) with the rows that selected none of
    the device's experts cleared, and everybody's expert indices.  Routed rows are what
    ttir_all_to_all_dispatch_metadata_golden (mapping.py:1656-1760) places."""
    to_grid = lambda t: t.permute(1, 0, 2, 3) if t.shape[1] == 1 else t.permute(2, 0, 1, 3)
    full = torch.cat([to_grid(x) for x in xs], dim=1)
    meta = torch.cat([to_grid(i) for i in indices], dim=1)
    out = []
    for d in range(len(xs)):
        mine = torch.tensor(_local_experts(mapping, d), dtype=torch.int64)
        routed = torch.isin(meta.to(torch.int64), mine).any(dim=-1, keepdim=True)
        out.append(torch.where(routed, full, torch.zeros_like(full)))
    return out, [meta.clone() for _ in xs]


def all_to_all_combine(xs, metadata, mapping, k, seq_sharded=False):
    """Per destination device p: out[slot, b, s, :] = the row of the expert named by metadata[token, slot], taken from
    the device that owns it (mapping.py:2030-2150; the token is the destination's own one of the global grid)."""
    n = len(xs)
    owners = {}
    for d in range(n):
        for le, e in enumerate(_local_experts(mapping, d)):
            owners[e] = (d, le)
    _, bg, sg, h = xs[0].shape
    b, s_ = (bg, sg // n) if seq_sharded else (bg // n, sg)
    outs = []
    for p in range(n):
        md = metadata[p] if isinstance(metadata, list) else metadata
        out = torch.zeros(k, b, s_, h, dtype=xs[0].dtype)
        for bi in range(b):
            for si in range(s_):
                gb, gs = (bi, p * s_ + si) if seq_sharded else (p * b + bi, si)
                for slot in range(k):
                    e = int(md[0, gb, gs, slot])
                    if e in owners:
                        d, le = owners[e]
                        out[slot, bi, si] = xs[d][le, gb, gs]
        outs.append(out)
    return outs


def moe_expert_token_remap(topk, mapping, metadata, device, reduction_size):
    """mapping[t, le] = topk[t, e] for the experts in metadata[t] that `device` owns; reduced[block, le] = 1 when a
    token of the block of `reduction_size` tokens selected local expert le (::ttnn::moe_expert_token_remap; the
    reference golden, mapping.py:2153-2186, only fixes the shapes)."""
    mine = _local_experts(mapping, device)
    e_total = topk.shape[-1]
    tk = topk.reshape(-1, e_total)
    md = metadata.reshape(tk.shape[0], -1)
    out = torch.zeros(tk.shape[0], len(mine), dtype=topk.dtype)
    for t in range(tk.shape[0]):
        for e in md[t].tolist():
            if e in mine:
                out[t, mine.index(e)] = tk[t, e]
    blocks = (tk.shape[0] + reduction_size - 1) // reduction_size
    red = torch.zeros(blocks, len(mine))
    for blk in range(blocks):
        rows = md[blk * reduction_size: (blk + 1) * reduction_size]
        for le, e in enumerate(mine):
            red[blk, le] = float((rows == e).any())
    return out.reshape(*topk.shape[:-1], len(mine)), red.reshape(1, 1, blocks, len(mine))


def sparse_matmul(a, b, sparsity, a_sparse: bool):
    """tools/golden/mapping.py:1596-1624 (dense products) with the skipped blocks cleared; f32 accumulation, one rounding."""
    af, bf = a.float(), b.float()
    if a_sparse:
        out = torch.matmul(af, bf)                                           # [A, E, M, N]
        mask = sparsity.reshape(a.shape[0], b.shape[1], 1, 1)
    else:
        out = torch.einsum("abmk,xekn->abxemn", af, bf)                      # [A, B, 1, E, M, N]
        mask = sparsity.reshape(a.shape[0], a.shape[1], 1, b.shape[1], 1, 1)
    return torch.where(mask.float() != 0, out, torch.zeros_like(out)).to(a.dtype)


def all_to_all_dispatch_metadata(xs, indices, scores, owner):
    """tools/golden/mapping.py:1656-1760: per device the global token list [1, T, H] with the rows routed to it (an
    expert of the token lives there; owner[e] = device of expert e), and everybody's indices and scores."""
    h, k = xs[0].shape[-1], indices[0].shape[-1]
    full = torch.cat([x.reshape(-1, h) for x in xs])
    idx = torch.cat([i.reshape(-1, k) for i in indices])
    scr = torch.cat([s_.reshape(-1, k) for s_ in scores])
    own = owner.reshape(-1, owner.shape[-1])[0].to(torch.int64)
    target = own[idx.to(torch.int64)]                                          # [T, K] device per selected expert
    outs = []
    for d in range(len(xs)):
        routed = (target == d).any(dim=-1, keepdim=True)
        outs.append(torch.where(routed, full, torch.zeros_like(full)).reshape(1, -1, h))
    return outs, [idx.reshape(1, -1, k).clone() for _ in xs], [scr.reshape(1, -1, k).clone() for _ in xs]


def topk_router_gpt(x, weight, bias, k):
    """tools/golden/mapping.py:5960-5992: logits = x @ weight (in the input's 16-bit type) + bias, the k largest per
    row in descending order, softmax over those k."""
    logits = torch.matmul(x.float(), weight.float()).to(x.dtype) + bias
    values, idx = torch.topk(logits, k=k, dim=-1, largest=True, sorted=True)
    return idx, torch.softmax(values.float(), dim=-1).to(x.dtype)


def conv3d(x, w, bias, batch, depth, height, width, stride, padding, groups, padding_mode="zeros"):
    """tools/golden/mapping.py:714-801: torch conv3d on the NCDHW view of NDHWC data, symmetric padding; "replicate"
    repeats the edge values.  f32, one rounding; the result keeps the input's flattened / 5-D form."""
    c = x.numel() // (batch * depth * height * width)
    t = x.reshape(batch, depth, height, width, c).permute(0, 4, 1, 2, 3).float()
    if padding_mode == "replicate" and any(padding):
        t = torch.nn.functional.pad(t, (padding[2], padding[2], padding[1], padding[1], padding[0], padding[0]), mode="replicate")
        padding = (0, 0, 0)
    y = torch.nn.functional.conv3d(t, w.float(), bias.float().reshape(-1) if bias is not None else None, stride=tuple(stride),
                                   padding=tuple(padding), groups=groups)
    y = y.permute(0, 2, 3, 4, 1).contiguous()
    return (y.reshape(1, 1, -1, y.shape[-1]) if x.ndim == 4 else y).to(x.dtype)


def gelu_backward(grad, x, approximate="none"):
    """tools/golden/mapping.py:4379-4383 (aten.gelu_backward), evaluated in f32, one rounding."""
    return torch.ops.aten.gelu_backward(grad.float(), x.float(), approximate=approximate).to(x.dtype)


def embedding_backward(indices, weight_shape, in_grad):
    """tools/golden/mapping.py:5875-5912: index_add_ of the gradient rows into a zero table; accumulated in f32 here."""
    vocab, dim = weight_shape[-2], weight_shape[-1]
    acc = torch.zeros(vocab, dim)
    acc.index_add_(0, indices.to(torch.int64).flatten(), in_grad.float().reshape(-1, dim))
    return acc.reshape(list(weight_shape)).to(in_grad.dtype)


def adamw(param, grad, exp_avg, exp_avg_sq, max_exp_avg_sq, lr, beta1, beta2, beta1_pow, beta2_pow, eps, weight_decay):
    """tools/golden/mapping.py:1155-1218 (tt-train's CPUAdamW).  Returns (param, exp_avg, exp_avg_sq[, max_exp_avg_sq])."""
    g = grad.float()
    m = exp_avg.float() * beta1 + g * (1.0 - beta1)
    v = exp_avg_sq.float() * beta2 + (g * g) * (1.0 - beta2)
    vv = torch.maximum(max_exp_avg_sq.float(), v) if max_exp_avg_sq is not None else v
    denom = torch.sqrt(vv / (1.0 - beta2_pow)) + eps
    p = param.float()
    r = (p - (m / (1.0 - beta1_pow)) / denom * lr) - p * (lr * weight_decay)
    out = (r.to(param.dtype), m.to(exp_avg.dtype), v.to(exp_avg_sq.dtype))
    return out + ((vv.to(max_exp_avg_sq.dtype),) if max_exp_avg_sq is not None else ())


def chunked_sdpa(q, k_cache, v_cache, page_table, chunk_start, scale=None):
    """tools/golden/mapping.py:8847-8912: un-page K and V through the page table, expand grouped heads, row j of the
    chunk (absolute position chunk_start + j) sees keys 0 .. chunk_start + j; f32 softmax, one rounding."""
    b, nh, sq, d = q.shape
    nblocks, nkv, bs, _ = k_cache.shape
    per_user = page_table.shape[-1]
    pt = page_table.to(torch.int64).reshape(-1).clamp(0, nblocks - 1)
    unpage = lambda c: c[pt].reshape(b, per_user, nkv, bs, d).transpose(1, 2).reshape(b, nkv, per_user * bs, d).float()
    k, v = unpage(k_cache), unpage(v_cache)
    if nh // nkv > 1:
        k, v = k.repeat_interleave(nh // nkv, dim=1), v.repeat_interleave(nh // nkv, dim=1)
    seq = per_user * bs
    allowed = torch.arange(seq).view(1, seq) <= (chunk_start + torch.arange(sq)).view(sq, 1)
    mask = torch.zeros(1, 1, sq, seq).masked_fill_(~allowed.view(1, 1, sq, seq), torch.finfo(torch.float32).min)
    return torch.nn.functional.scaled_dot_product_attention(q.float(), k, v, attn_mask=mask, scale=scale).to(q.dtype)


def flash_mla_prefill(q, k, v, mask, head_dim_v, is_causal, scale=None):
    """tools/golden/mapping.py:8662-8692: attention whose values are the first head_dim_v key columns unless given;
    a mask switches the causal flag off; f32, one rounding."""
    vt = k[..., :head_dim_v] if v is None else v
    kf, vf = k.float(), vt.float()
    rep = q.shape[1] // k.shape[1]
    if rep > 1:
        kf, vf = kf.repeat_interleave(rep, dim=1), vf.repeat_interleave(rep, dim=1)
    return torch.nn.functional.scaled_dot_product_attention(
        q.float(), kf, vf, attn_mask=mask.float() if mask is not None else None, is_causal=is_causal and mask is None, scale=scale).to(q.dtype)


def indexer_score_dsa(q, k, weights, offset):
    """tools/golden/mapping.py:8695-8742: score[b, 0, s, t] = sum_h relu(q[b, h, s] . k[b, 0, t]) * weights[b, h, s, 0] in f32,
    -inf for keys t > offset + s, one rounding to the query's type."""
    qk = torch.relu(torch.einsum("bhsd,btd->bhst", q.float(), k.float()[:, 0]))
    score = (qk * weights.float()).sum(dim=1, keepdim=True)
    sq, t = q.shape[2], k.shape[2]
    visible = (torch.arange(sq).view(1, 1, sq, 1) + offset) >= torch.arange(t).view(1, 1, 1, t)
    return score.masked_fill(~visible, float("-inf")).to(q.dtype)


def paged_mla_decode(q, k_cache, v_cache, page_table, cur_pos, mask, head_dim_v, is_causal=True, scale=None):
    """tools/golden/mapping.py:8275-8365: q [1, B, H, D]; the latent cache is un-paged through the page table, values are
    its first head_dim_v columns unless a value cache is given, user b sees keys 0 .. cur_pos[b]; scale defaults to 1."""
    qf = q.permute(1, 2, 0, 3).float()
    b, nh, _, d = qf.shape
    nblocks, nkv, bs, _ = k_cache.shape
    per_user = page_table.shape[-1]
    pt = page_table.to(torch.int64).reshape(-1)
    seq = per_user * bs
    unpage = lambda c: c[pt].reshape(b, per_user, nkv, bs, c.shape[-1]).transpose(1, 2).reshape(b, nkv, seq, c.shape[-1]).float()
    k = unpage(k_cache)
    v = unpage(v_cache) if v_cache is not None else k[..., :head_dim_v]
    rep = nh // nkv
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    am = None
    if mask is not None:
        am = mask.float()
    elif is_causal and cur_pos is not None:
        am = torch.zeros(b, nh, 1, seq)
        for i in range(b):
            am[i, :, :, int(cur_pos[i]) + 1:] = torch.finfo(torch.float32).min
    out = torch.nn.functional.scaled_dot_product_attention(qf, k, v, attn_mask=am, scale=1.0 if scale is None else scale)
    return out.permute(2, 0, 1, 3).to(q.dtype)
