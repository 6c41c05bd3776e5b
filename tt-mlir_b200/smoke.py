"""One small invocation of the hot path on cuda:0, checked against the CPU oracle: a decoder
block (rms_norm, linear on the tensor cores, rotary embedding, attention, SwiGLU) and the
quantization chain, each through Binary -> to_layout -> submit -> to_host."""

from __future__ import annotations

import os
import sys

import torch


def run() -> None:
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    from . import graphs, runtime_api as rt
    from oracle import metrics
    from oracle.backend import OracleBuilder

    if rt.get_num_available_devices() == 0:
        raise RuntimeError("smoke() needs a CUDA device; this backend has no CPU fallback")
    device = rt.open_mesh_device(rt.MeshDeviceOptions(mesh_shape=[1, 1]))
    try:
        def through_runtime(graph_fn, inputs, **kw):
            binary = rt.Binary.load_from_memory(graphs.build_binary(graph_fn, **kw))
            rt.set_compatible_device_runtime(binary)
            ins = [rt.to_layout(rt.from_torch(t), device, rt.get_layout(binary, 0, i)) for i, t in enumerate(inputs)]
            outs = rt.submit(device, binary, 0, ins)
            return [rt.to_torch(rt.to_host(o, untilize=True)[0]) for o in outs]

        def through_oracle(graph_fn, inputs, **kw):
            ob = OracleBuilder(inputs)
            graph_fn(ob, **kw)
            return ob.results()

        before = rt.launch_count()
        kw = dict(rows=256, cols=512, keep_intermediates=True)
        ins = graphs.quant_chain_inputs(256, 512)
        got, want = through_runtime(graphs.quant_chain_graph, ins, **kw), through_oracle(graphs.quant_chain_graph, ins, **kw)
        for g, w in zip(got, want):
            if not torch.equal(g, w):
                raise AssertionError("quantization chain differs from the oracle")

        kw = dict(seq=256, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024)
        ins = graphs.decoder_block_inputs(**kw)
        got, want = through_runtime(graphs.decoder_block_graph, ins, **kw)[0], through_oracle(graphs.decoder_block_graph, ins, **kw)[0]
        ok, report = metrics.check_close(want, got, 0.999, 2e-2, 2.0 ** -6)
        if not ok:
            raise AssertionError("decoder block differs from the oracle: " + report)
        launched = rt.launch_count() - before
        if launched <= 0:
            raise AssertionError("no kernel of this library was launched")
        print(f"smoke ok: quant chain bit-exact, decoder block {report}, {launched} kernel launches")
    finally:
        rt.close_mesh_device(device)
