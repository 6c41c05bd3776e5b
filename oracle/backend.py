"""Eager CPU evaluation of a graph written against the ProgramBuilder interface.

A graph function (tt-mlir_b200/graphs.py) takes a builder `b` and calls b.input / b.matmul /
b.output ...  Given a `ProgramBuilder` it emits a TTNN flatbuffer; given this `OracleBuilder`
it computes the reference result with oracle/ops.py.  Both therefore describe the same graph.
Multi-device values are lists with one tensor per mesh coordinate.
"""

from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from . import ops

TORCH_DTYPE = {"Float32": torch.float32, "Float16": torch.float16, "BFloat16": torch.bfloat16, "Int32": torch.int32,
               "UInt8": torch.uint8, "Int8": torch.int8, "UInt16": torch.uint16, "UInt32": torch.uint32}
NAME_OF = {v: k for k, v in TORCH_DTYPE.items()}


class OValue:
    def __init__(self, t):
        self.t = t  # torch.Tensor or list of per-device tensors

    @property
    def first(self) -> torch.Tensor:
        return self.t[0] if isinstance(self.t, list) else self.t

    @property
    def shape(self):
        return list(self.first.shape)

    @property
    def dtype(self) -> str:
        return NAME_OF[self.first.dtype]


def _map(fn, *vals):
    """Applies fn per device when any operand is distributed."""
    n = max((len(v.t) for v in vals if isinstance(v, OValue) and isinstance(v.t, list)), default=0)
    if n == 0:
        res = fn(*[v.t if isinstance(v, OValue) else v for v in vals])
        return tuple(OValue(r) for r in res) if isinstance(res, tuple) else OValue(res)
    out = []
    for i in range(n):
        args = [(v.t[i] if isinstance(v.t, list) else v.t) if isinstance(v, OValue) else v for v in vals]
        out.append(fn(*args))
    if isinstance(out[0], tuple):
        return tuple(OValue([o[k] for o in out]) for k in range(len(out[0])))
    return OValue(out)


class OracleBuilder:
    def __init__(self, inputs: Sequence[torch.Tensor], mesh_shape=(1, 1), quant_clamp_i8: bool = True):
        self._inputs = list(inputs)
        self._next_input = 0
        self.mesh_shape = tuple(mesh_shape)
        self.outputs: List[OValue] = []
        self.clamp_i8 = quant_clamp_i8

    # ---- program interface
    def input(self, shape, dtype: str, on_device: bool = True) -> OValue:
        t = self._inputs[self._next_input]
        self._next_input += 1
        assert list(t.shape) == list(shape), f"input {self._next_input - 1}: {list(t.shape)} vs {list(shape)}"
        assert t.dtype == TORCH_DTYPE[dtype]
        return OValue(t)

    def output(self, *values: OValue):
        self.outputs.extend(values)

    def results(self):
        return [v.t for v in self.outputs]

    # ---- layout / creation
    def to_device(self, x, loc=None): return x
    def from_device(self, x, loc=None): return x

    def to_layout(self, x, layout="Tile", dtype=None, on_device=None, loc=None):
        return _map(lambda t: t.to(TORCH_DTYPE[dtype]), x) if dtype else x

    def typecast(self, x, dtype, loc=None):
        return _map(lambda t: ops.typecast(t, TORCH_DTYPE[dtype]), x)

    def full(self, shape, value, dtype, loc=None):
        return OValue(torch.full(list(shape), value, dtype=TORCH_DTYPE[dtype]))

    def zeros(self, shape, dtype, loc=None): return OValue(torch.zeros(list(shape), dtype=TORCH_DTYPE[dtype]))
    def ones(self, shape, dtype, loc=None): return OValue(torch.ones(list(shape), dtype=TORCH_DTYPE[dtype]))

    def constant(self, data: bytes, shape, dtype, loc=None):
        return OValue(torch.frombuffer(bytearray(data), dtype=TORCH_DTYPE[dtype]).reshape(list(shape)).clone())

    def arange(self, start, end, step, dtype, loc=None):
        return OValue(torch.arange(start, end, step, dtype=torch.float64).to(TORCH_DTYPE[dtype]))

    def deallocate(self, x, force=False): pass

    # ---- eltwise
    def unary(self, kind, x, param=None, loc=None): return _map(lambda t: ops.unary(kind, t, param), x)
    def relu(self, x, loc=None): return self.unary("Relu", x)
    def silu(self, x, loc=None): return self.unary("Silu", x)
    def exp(self, x, loc=None): return self.unary("Exp", x)
    def neg(self, x, loc=None): return self.unary("Neg", x)
    def sigmoid(self, x, loc=None): return self.unary("Sigmoid", x)
    def clamp(self, x, lo, hi, loc=None): return _map(lambda t: ops.clamp(t, lo, hi), x)

    def binary(self, kind, a, b, dtype=None, loc=None):
        return _map(lambda x, y: ops.binary(kind, x, y, TORCH_DTYPE[dtype] if dtype else None), a, b)

    def add(self, a, b, loc=None): return self.binary("Add", a, b)
    def multiply(self, a, b, loc=None): return self.binary("Multiply", a, b)
    def subtract(self, a, b, loc=None): return self.binary("Subtract", a, b)
    def divide(self, a, b, loc=None): return self.binary("Divide", a, b)
    def maximum(self, a, b, loc=None): return self.binary("Maximum", a, b)
    def where(self, c, a, b, loc=None): return _map(ops.where, c, a, b)

    # ---- quantization
    def quantize(self, x, scale, zero_point, out_dtype="Int32", axis=None, loc=None):
        dt = TORCH_DTYPE[out_dtype]
        if isinstance(scale, OValue):
            return _map(lambda t, s, z=None: ops.quantize_per_axis(t, s, z, axis, dt, self.clamp_i8), x, scale,
                        *([zero_point] if isinstance(zero_point, OValue) else []))
        return _map(lambda t: ops.quantize(t, scale, zero_point, dt, self.clamp_i8), x)

    def dequantize(self, x, scale, zero_point, out_dtype="Float32", axis=None, loc=None):
        dt = TORCH_DTYPE[out_dtype]
        if isinstance(scale, OValue):
            return _map(lambda t, s, z=None: ops.dequantize_per_axis(t, s, z, axis, dt), x, scale,
                        *([zero_point] if isinstance(zero_point, OValue) else []))
        return _map(lambda t: ops.dequantize(t, scale, zero_point, dt), x)

    def requantize(self, x, in_scale, in_zp, out_scale, out_zp, out_dtype=None, axis=None, loc=None):
        dt = TORCH_DTYPE[out_dtype] if out_dtype else None
        return _map(lambda t: ops.requantize(t, in_scale, in_zp, out_scale, out_zp, dt, self.clamp_i8), x)

    # ---- contractions
    def matmul(self, a, b, transpose_a=False, transpose_b=False, activation=None, out_dtype=None, loc=None):
        if out_dtype is not None and not TORCH_DTYPE[out_dtype].is_floating_point:
            return _map(lambda x, y: ops.int_matmul(x, y, transpose_a, transpose_b, TORCH_DTYPE[out_dtype]), a, b)
        return _map(lambda x, y: ops.matmul(x, y, transpose_a, transpose_b, activation), a, b)

    def linear(self, a, b, bias=None, transpose_a=False, transpose_b=False, activation=None, loc=None):
        if bias is None:
            return _map(lambda x, y: ops.linear(x, y, None, transpose_a, transpose_b, activation), a, b)
        return _map(lambda x, y, z: ops.linear(x, y, z, transpose_a, transpose_b, activation), a, b, bias)

    def conv2d(self, x, w, bias, batch, height, width, stride=(1, 1), padding=(0, 0, 0, 0), dilation=(1, 1), groups=1,
               out_dtype=None, loc=None):
        pad = list(padding) if len(padding) == 4 else [padding[0], padding[1], padding[0], padding[1]]
        if out_dtype is not None and not TORCH_DTYPE[out_dtype].is_floating_point:
            return _map(lambda t, ww: ops.int_conv2d(t, ww, batch, height, width, stride, pad, dilation, groups,
                                                     TORCH_DTYPE[out_dtype]), x, w)
        if bias is None:
            return _map(lambda t, ww: ops.conv2d(t, ww, None, batch, height, width, stride, pad, dilation, groups), x, w)
        return _map(lambda t, ww, bb: ops.conv2d(t, ww, bb, batch, height, width, stride, pad, dilation, groups), x, w, bias)

    # ---- normalisation / reduction
    def softmax(self, x, dim=-1, loc=None): return _map(lambda t: ops.softmax(t, dim), x)

    def rms_norm(self, x, weight, bias=None, epsilon=1e-5, loc=None):
        args = [v for v in (weight, bias) if v is not None]
        if weight is not None and bias is not None:
            return _map(lambda t, w, b: ops.rms_norm(t, w, b, epsilon), x, weight, bias)
        if weight is not None:
            return _map(lambda t, w: ops.rms_norm(t, w, None, epsilon), x, weight)
        return _map(lambda t: ops.rms_norm(t, None, None, epsilon), x)

    def layer_norm(self, x, weight=None, bias=None, epsilon=1e-5, loc=None):
        vals = [v for v in (x, weight, bias) if v is not None]

        def fn(*ts):
            it = iter(ts)
            t = next(it)
            w = next(it) if weight is not None else None
            b = next(it) if bias is not None else None
            return ops.layer_norm(t, w, b, epsilon)
        return _map(fn, *vals)

    def argmax(self, x, dim=None, keep_dim=False, loc=None): return _map(lambda t: ops.argmax(t, dim, keep_dim), x)
    def cumsum(self, x, dim, loc=None): return _map(lambda t: ops.cumsum(t, dim), x)
    def cumprod(self, x, dim, loc=None): return _map(lambda t: ops.cumprod(t, dim), x)
    def prod(self, x, dim=None, keep_dim=False, loc=None): return _map(lambda t: ops.prod(t, dim, keep_dim), x)

    def batch_norm_inference(self, x, mean, var, weight, bias, epsilon=1e-5, loc=None):
        if weight is None and bias is None:
            return _map(lambda t, m, v: ops.batch_norm_inference(t, m, v, None, None, epsilon), x, mean, var)
        return _map(lambda t, m, v, w, b: ops.batch_norm_inference(t, m, v, w, b, epsilon), x, mean, var, weight, bias)

    def upsample(self, x, scale, mode="nearest", loc=None): return _map(lambda t: ops.upsample2d(t, scale, mode), x)

    def group_norm(self, x, weight, bias, num_groups, epsilon=1e-5, loc=None):
        return _map(lambda t, w, b: ops.group_norm(t, w, b, num_groups, epsilon), x, weight, bias)

    def conv_transpose2d(self, x, w, bias, batch, height, width, stride=(1, 1), padding=(0, 0), output_padding=(0, 0),
                         dilation=(1, 1), groups=1, loc=None):
        return _map(lambda t, wt, b: ops.conv_transpose2d(t, wt, b, batch, height, width, stride, padding, output_padding, dilation,
                                                          groups), x, w, bias)

    def conv1d(self, x, w, bias, batch, length, stride=1, padding=(0, 0), dilation=1, groups=1, loc=None):
        return _map(lambda t, wt, b: ops.conv1d(t, wt, b, stride, padding, dilation, groups), x, w, bias)

    def bitcast_convert(self, x, dtype, loc=None):
        return _map(lambda t: t.view(TORCH_DTYPE[dtype]), x)

    def nlp_concat_heads(self, x, loc=None):
        return _map(lambda t: t.permute(0, 2, 1, 3).reshape(t.shape[0], 1, t.shape[2], t.shape[1] * t.shape[3]), x)

    def assign(self, x, dtype=None, loc=None): return _map(lambda t: t.clone().to(TORCH_DTYPE[dtype]) if dtype else t.clone(), x)
    def pow_scalar(self, x, exponent, loc=None): return _map(lambda t: ops.pow_scalar(t, exponent), x)
    def annotate(self, x, annotation, loc=None): return x
    def region_start(self, x, region_id, loc=None): return x
    def region_end(self, x, region_id, loc=None): return x
    def breakpoint(self, x, loc=None): return None
    def print_message(self, x, message, loc=None): return None
    def memory_snapshot(self, x, file_path, loc=None): return None

    def nlp_create_qkv_heads_decode(self, x, num_heads, num_kv_heads=None, batch_offset=None, slice_size=None, loc=None):
        off = int(batch_offset.t.reshape(-1)[0]) if batch_offset is not None else 0
        q, k, v = ops.nlp_create_qkv_heads_decode(x.t, num_heads, num_kv_heads, off, slice_size)
        return OValue(q), OValue(k), OValue(v)

    def nlp_concat_heads_decode(self, x, num_heads, loc=None): return _map(lambda t: ops.nlp_concat_heads_decode(t, num_heads), x)

    def rotary_embedding_llama(self, x, cos, sin, trans_mat, is_decode_mode=False, loc=None):
        return _map(lambda t, c, s, m: ops.rotary_embedding_llama(t, c, s, m, is_decode_mode), x, cos, sin, trans_mat)

    def max_pool2d_with_indices(self, x, batch, height, width, channels, kernel=(2, 2), stride=(2, 2), padding=(0, 0), dilation=(1, 1),
                                ceil_mode=False, index_dtype="Int32", loc=None):
        y, idx = ops.max_pool2d_with_indices(x.t, batch, height, width, channels, kernel, stride, padding, dilation, ceil_mode)
        return OValue(y), OValue(idx.to(TORCH_DTYPE[index_dtype]))

    def batch_norm_training(self, x, mean, var, weight, bias, epsilon=1e-5, momentum=0.1, loc=None):
        y, m, v = ops.batch_norm_training(x.t, mean.t, var.t, weight.t if weight is not None else None,
                                          bias.t if bias is not None else None, epsilon, momentum)
        mean.t, var.t = m, v                                    # the running statistics are updated in place
        return OValue(y)

    def prepare_conv_transpose2d_weights(self, w, *a, **k): return w
    def prepare_conv_transpose2d_bias(self, bias, *a, **k): return bias
    # the preparation ops change nothing a CPU evaluation can see
    def prepare_conv2d_weights(self, w, *a, **k): return w
    def prepare_conv2d_bias(self, bias, *a, **k): return bias
    def embedding(self, indices, weight, loc=None): return _map(ops.embedding, indices, weight)

    def max_pool2d(self, x, batch, height, width, channels, kernel=(2, 2), stride=(2, 2), padding=(0, 0), dilation=(1, 1),
                   ceil_mode=False, loc=None):
        return _map(lambda t: ops.max_pool2d(t, batch, height, width, channels, kernel, stride, padding, dilation, ceil_mode), x)

    def avg_pool2d(self, x, batch, height, width, channels, kernel=(2, 2), stride=(2, 2), padding=(0, 0), ceil_mode=False,
                   count_include_pad=True, loc=None):
        return _map(lambda t: ops.avg_pool2d(t, batch, height, width, channels, kernel, stride, padding, ceil_mode,
                                             count_include_pad), x)

    def global_avg_pool2d(self, x, loc=None): return _map(ops.global_avg_pool2d, x)
    def pad(self, x, padding, value=0.0, loc=None): return _map(lambda t: ops.pad(t, padding, value), x)

    def fill_cache(self, cache, x, batch_offset=0, loc=None): return _map(lambda c, t: ops.fill_cache(c, t, batch_offset), cache, x)

    def update_cache(self, cache, x, update_index, batch_offset=0, loc=None):
        return _map(lambda c, t, i: ops.update_cache(c, t, i, batch_offset), cache, x, update_index)

    def scaled_dot_product_attention_decode(self, q, k, v, cur_pos=None, mask=None, is_causal=True, scale=None, loc=None):
        vals = [x for x in (q, k, v, cur_pos, mask) if x is not None]

        def fn(*ts):
            it = iter(ts)
            qq, kk, vv = next(it), next(it), next(it)
            cp = next(it) if cur_pos is not None else None
            mk = next(it) if mask is not None else None
            return ops.sdpa_decode(qq, kk, vv, cp, mk, is_causal, scale)
        return _map(fn, *vals)

    def paged_update_cache(self, cache, x, update_index, page_table=None, share_cache=False, loc=None):
        if page_table is None:
            return _map(lambda c, t, i: ops.paged_update_cache(c, t, i, None), cache, x, update_index)
        return _map(lambda c, t, i, pt: ops.paged_update_cache(c, t, i, pt), cache, x, update_index, page_table)

    def paged_fill_cache(self, cache, x, page_table, batch_idx=None, loc=None):
        if batch_idx is None:
            return _map(lambda c, t, pt: ops.paged_fill_cache(c, t, pt, None), cache, x, page_table)
        return _map(lambda c, t, pt, bi: ops.paged_fill_cache(c, t, pt, bi), cache, x, page_table, batch_idx)

    def paged_scaled_dot_product_attention_decode(self, q, k, v, page_table, cur_pos=None, mask=None, is_causal=True, scale=None,
                                                  loc=None):
        vals = [x for x in (q, k, v, page_table, cur_pos, mask) if x is not None]

        def fn(*ts):
            it = iter(ts)
            qq, kk, vv, pt = next(it), next(it), next(it), next(it)
            cp = next(it) if cur_pos is not None else None
            mk = next(it) if mask is not None else None
            return ops.paged_sdpa_decode(qq, kk, vv, pt, cp, is_causal, scale, mk)
        return _map(fn, *vals)

    def gather(self, x, index, dim, loc=None): return _map(lambda t, i: ops.gather(t, i, dim), x, index)

    def scatter(self, x, index, src, dim, reduce_type=None, loc=None):
        return _map(lambda t, i, u: ops.scatter(t, i, u, dim, reduce_type), x, index, src)

    def sort(self, x, dim=-1, descending=False, stable=True, index_dtype="Int32", loc=None):
        def fn(t):
            v, i = ops.sort(t, dim, descending, stable)
            return v, i.to(TORCH_DTYPE[index_dtype])
        return _map(fn, x)

    def topk(self, x, k, dim=-1, largest=True, index_dtype="Int32", loc=None):
        def fn(t):
            v, i = ops.topk(t.float(), k, dim, largest)
            return v.to(t.dtype), i.to(TORCH_DTYPE[index_dtype])
        return _map(fn, x)

    def sampling(self, values, indices, k, p, temp, seed=None, loc=None):
        """The reference's golden draws with torch.multinomial (tools/golden/mapping.py:6008-6018): a result that
        no other generator can reproduce.  The oracle returns the most probable candidate, which equals the
        device's answer only where the support is a single candidate; tests compare distributions otherwise."""
        def fn(v, i):
            return torch.gather(i, 1, v.float().argmax(dim=1, keepdim=True)).squeeze(1).to(torch.int32)
        return _map(fn, values, indices)

    def reduce(self, kind, x, dims, keep_dim, loc=None): return _map(lambda t: ops.reduce(kind, t, dims, keep_dim), x)

    # ---- data movement
    def reshape(self, x, shape, loc=None): return _map(lambda t: t.reshape(list(shape)), x)
    def permute(self, x, perm, loc=None): return _map(lambda t: t.permute(list(perm)).contiguous(), x)
    def transpose(self, x, d0, d1, loc=None): return _map(lambda t: t.transpose(d0, d1).contiguous(), x)

    def concat(self, xs, dim, loc=None):
        return _map(lambda *ts: torch.cat(list(ts), dim=dim), *xs)

    def slice(self, x, begins, ends, step=None, loc=None):
        step = step or [1] * len(begins)
        return _map(lambda t: t[tuple(slice(b, e, s) for b, e, s in zip(begins, ends, step))].contiguous(), x)

    def repeat(self, x, repeats, loc=None): return _map(lambda t: t.repeat(*repeats), x)
    def repeat_interleave(self, x, repeats, dim, loc=None): return _map(lambda t: torch.repeat_interleave(t, repeats, dim=dim), x)

    # ---- transformer
    def concatenate_heads(self, x, loc=None): return _map(ops.concatenate_heads, x)

    def split_query_key_value_and_split_heads(self, x, kv, num_heads, num_kv_heads=None, transpose_key=False, loc=None):
        if kv is None:
            return _map(lambda t: ops.split_qkv(t, None, num_heads, num_kv_heads, transpose_key), x)
        return _map(lambda t, u: ops.split_qkv(t, u, num_heads, num_kv_heads, transpose_key), x, kv)

    def rotary_embedding(self, x, cos, sin, loc=None): return _map(ops.rotary_embedding, x, cos, sin)

    def scaled_dot_product_attention(self, q, k, v, is_causal=True, mask=None, scale=None, loc=None):
        if mask is None:
            return _map(lambda a, b, c: ops.sdpa(a, b, c, is_causal, None, scale), q, k, v)
        return _map(lambda a, b, c, m: ops.sdpa(a, b, c, is_causal, m, scale), q, k, v, mask)

    # ---- mesh
    def _n(self, cluster_axis): return self.mesh_shape[cluster_axis]

    def distribute(self, x, shard_dim, cluster_axis=1, on_device=True, loc=None):
        return OValue(ops.mesh_shard_full_to_shard(x.t, self._n(cluster_axis), shard_dim))

    def aggregate(self, x, shard_dim, cluster_axis=1, loc=None):
        return OValue(ops.mesh_shard_shard_to_full(x.t, shard_dim))

    def all_reduce(self, x, reduce_type=0, cluster_axis=1, loc=None): return OValue(ops.all_reduce(x.t, reduce_type))
    def dit_rms_norm_unary_fused(self, x, weight=None, bias=None, residual=None, epsilon=1e-5, activation=None, loc=None):
        return _map(lambda t, w, b, r: ops.dit_rms_norm_unary_fused(t, w, b, r, epsilon, activation), x, weight, bias, residual)

    def distributed_rms_norm(self, x, weight=None, residual=None, cluster_axis=1, epsilon=1e-5, loc=None):
        if not isinstance(x.t, list):
            return OValue(ops.distributed_rms_norm([x.t], [weight.t] if weight is not None else None,
                                                   [residual.t] if residual is not None else None, epsilon)[0])
        per = lambda v: (v.t if isinstance(v.t, list) else [v.t] * len(x.t)) if v is not None else None
        return OValue(ops.distributed_rms_norm(x.t, per(weight), per(residual), epsilon))

    def rms_norm_pre_all_gather(self, x, residual=None, dtype=None, loc=None):
        return _map(lambda t, r: ops.rms_norm_pre_all_gather(t, r, TORCH_DTYPE[dtype] if dtype else t.dtype), x, residual)

    def layer_norm_pre_all_gather(self, x, residual=None, dtype=None, loc=None):
        return _map(lambda t, r: ops.layer_norm_pre_all_gather(t, r, TORCH_DTYPE[dtype] if dtype else t.dtype), x, residual)

    def layer_norm_post_all_gather(self, x, stats, weight=None, bias=None, epsilon=1e-12, loc=None):
        return _map(lambda t, st, w, b: ops.layer_norm_post_all_gather(t, st, w, b, epsilon), x, stats, weight, bias)

    def create_global_semaphore(self, initial_value=0, loc=None): return None
    def reset_global_semaphore(self, value=0, loc=None): return None

    def all_to_all_dispatch(self, x, expert_indices, expert_mapping, cluster_axis=1, loc=None):
        per = lambda v: v.t if isinstance(v.t, list) else [v.t]
        mp = expert_mapping.first
        disp, meta = ops.all_to_all_dispatch(per(x), per(expert_indices), mp)
        return (OValue(disp), OValue(meta)) if isinstance(x.t, list) else (OValue(disp[0]), OValue(meta[0]))

    def flash_mla_prefill(self, q, k, head_dim_v, v=None, mask=None, is_causal=True, scale=None, loc=None):
        return _map(lambda qt, kt, vt, mt: ops.flash_mla_prefill(qt, kt, vt, mt, head_dim_v, is_causal, scale), q, k, v, mask)

    def indexer_score_dsa(self, q, k, weights, chunk_start_idx=0, cluster_axis=None, loc=None):
        """Every device's causal window starts behind the query rows of the devices before it along the axis that
        carries the sequence (all devices in row-major order when no axis is named)."""
        sq = q.first.shape[2]
        if not isinstance(q.t, list):
            return OValue(ops.indexer_score_dsa(q.t, k.first, weights.first, chunk_start_idx))
        per = lambda v, i: v.t[i] if isinstance(v.t, list) else v.t
        coord = lambda i: i if cluster_axis is None else (i // self.mesh_shape[1] if cluster_axis == 0 else i % self.mesh_shape[1])
        return OValue([ops.indexer_score_dsa(q.t[i], per(k, i), per(weights, i), chunk_start_idx + coord(i) * sq) for i in range(len(q.t))])

    def paged_flash_multi_latent_attention_decode(self, q, k_cache, head_dim_v, page_table, v_cache=None, cur_pos=None, mask=None,
                                                  is_causal=True, scale=None, loc=None):
        return _map(lambda qt, kc, pt, vc, cp, mt: ops.paged_mla_decode(qt, kc, vc, pt, cp, mt, head_dim_v, is_causal, scale),
                    q, k_cache, page_table, v_cache, cur_pos, mask)

    def chunked_scaled_dot_product_attention(self, q, k_cache, v_cache, page_table, chunk_start_idx, scale=None, loc=None):
        start = int(chunk_start_idx.first.reshape(-1)[0])
        return _map(lambda t, kc, vc, pt: ops.chunked_sdpa(t, kc, vc, pt, start, scale), q, k_cache, v_cache, page_table)

    def conv3d(self, x, w, bias, batch, depth, height, width, stride=(1, 1, 1), padding=(0, 0, 0), groups=1, padding_mode="zeros", loc=None):
        return _map(lambda t, wt, b: ops.conv3d(t, wt, b, batch, depth, height, width, stride, padding, groups, padding_mode), x, w, bias)

    def prepare_conv3d_weights(self, w, *a, **k): return w
    def gelu_backward(self, grad, x, approximate="none", loc=None): return _map(lambda g, t: ops.gelu_backward(g, t, approximate), grad, x)
    def embedding_backward(self, indices, weight, in_grad, loc=None):
        return _map(lambda i, w, g: ops.embedding_backward(i, list(w.shape), g), indices, weight, in_grad)

    def adamw(self, param, grad, exp_avg, exp_avg_sq, max_exp_avg_sq=None, lr=1e-3, beta1=0.9, beta2=0.999, beta1_pow=0.9, beta2_pow=0.999,
              epsilon=1e-8, weight_decay=0.0, stochastic_rounding=False, loc=None):
        res = ops.adamw(param.t, grad.t, exp_avg.t, exp_avg_sq.t, max_exp_avg_sq.t if max_exp_avg_sq is not None else None, lr, beta1, beta2,
                        beta1_pow, beta2_pow, epsilon, weight_decay)
        param.t, exp_avg.t, exp_avg_sq.t = res[0], res[1], res[2]              # updated in place
        if max_exp_avg_sq is not None:
            max_exp_avg_sq.t = res[3]

    def all_to_all_dispatch_metadata(self, x, expert_indices, expert_scores, expert_mapping, cluster_axis=1, loc=None):
        per = lambda v: v.t if isinstance(v.t, list) else [v.t]
        d, i, s_ = ops.all_to_all_dispatch_metadata(per(x), per(expert_indices), per(expert_scores), expert_mapping.first)
        pack = (lambda v: OValue(v)) if isinstance(x.t, list) else (lambda v: OValue(v[0]))
        return pack(d), pack(i), pack(s_)

    def topk_router_gpt(self, x, weight, bias, k, index_dtype="UInt16", loc=None):
        def fn(t, w, b):
            idx, wts = ops.topk_router_gpt(t, w, b, k)
            return idx.to(TORCH_DTYPE[index_dtype]), wts
        return _map(fn, x, weight, bias)

    def all_to_all_combine(self, x, expert_metadata, expert_mapping, num_experts_per_tok, cluster_axis=1, output_shard_dim=1, loc=None):
        per = lambda v: v.t if isinstance(v.t, list) else [v.t]
        md = expert_metadata.t if isinstance(expert_metadata.t, list) else expert_metadata.t
        outs = ops.all_to_all_combine(per(x), md, expert_mapping.first, num_experts_per_tok, seq_sharded=output_shard_dim == 2 and len(per(x)) > 1)
        return OValue(outs) if isinstance(x.t, list) else OValue(outs[0])

    def moe_expert_token_remap(self, topk, expert_mapping, expert_metadata, reduction_size=32, reduced_dtype=None, loc=None):
        def fn(i, t, md):
            m, r = ops.moe_expert_token_remap(t, expert_mapping.first, md, i, reduction_size)
            return m, r.to(TORCH_DTYPE[reduced_dtype] if reduced_dtype else t.dtype)
        if isinstance(topk.t, list) or isinstance(expert_metadata.t, list):
            n = len(topk.t) if isinstance(topk.t, list) else len(expert_metadata.t)
            pick = lambda v, i: v.t[i] if isinstance(v.t, list) else v.t
            res = [fn(i, pick(topk, i), pick(expert_metadata, i)) for i in range(n)]
            return OValue([r[0] for r in res]), OValue([r[1] for r in res])
        m, r = fn(0, topk.t, expert_metadata.t)
        return OValue(m), OValue(r)

    def sparse_matmul(self, a, b, sparsity, is_input_a_sparse=False, is_input_b_sparse=True, nnz=None, loc=None):
        return _map(lambda x, w, sp: ops.sparse_matmul(x, w, sp, is_input_a_sparse), a, b, sparsity)

    def all_reduce_async(self, x, reduce_type=0, cluster_axis=1, loc=None): return OValue(ops.all_reduce(x.t, reduce_type))

    def point_to_point(self, x, sender_coord, receiver_coord, output=None, loc=None):
        lin = lambda c: c[0] * self.mesh_shape[1] + c[1]
        return OValue(ops.point_to_point(x.t, lin(sender_coord), lin(receiver_coord), output.t if output is not None else None))

    def all_gather(self, x, dim, cluster_axis=1, loc=None): return OValue(ops.all_gather(x.t, dim))
    def reduce_scatter(self, x, dim, reduce_type=0, cluster_axis=1, loc=None): return OValue(ops.reduce_scatter(x.t, dim, reduce_type))
    def mesh_partition(self, x, dim, cluster_axis=1, loc=None): return OValue(ops.mesh_partition(x.t, dim))
