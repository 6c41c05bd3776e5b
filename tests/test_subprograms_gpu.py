"""Const-eval functions (LoadCachedOp), calls (FuncCallOp) and traces (CaptureOrExecuteTraceOp and
the ops of its capture / execute programs) on the GPU: same results as the plain programs, and
the caching behaviour the reference documents (operations/cache/load_cached.cpp,
operations/trace/capture_or_execute_trace.cpp)."""

import pytest
import torch

from helpers import assert_matches, oracle_results
from ttmlir_b200 import graphs

pytestmark = pytest.mark.gpu


def _to_device_inputs(rt, device, binary, tensors, program=0):
    return [rt.to_layout(rt.from_torch(t), device, rt.get_layout(binary, program, i)) for i, t in enumerate(tensors)]


def _read(rt, outs):
    return [rt.to_torch(rt.to_host(o, untilize=True)[0]) for o in outs]


def test_const_eval_is_computed_once_and_follows_its_inputs(rt, device):
    kw = dict(m=256, k=512, n=384)
    ins = graphs.w8_linear_inputs(**kw)
    want = oracle_results(graphs.w8_linear_graph, ins, **kw)[0]
    binary = rt.Binary.load_from_memory(graphs.w8_linear_const_eval_binary(**kw))
    rt.clear_const_eval_cache()
    rt.clear_stats()
    dev_ins = _to_device_inputs(rt, device, binary, ins)
    launches = []
    for _ in range(3):
        before = rt.launch_count()
        got = _read(rt, rt.submit(device, binary, 0, dev_ins))[0]
        launches.append(rt.launch_count() - before)
        assert_matches(got, want, "w8 linear through a const-eval function")
    assert rt.get_stat("ConstEvalCacheMiss") == 1 and rt.get_stat("ConstEvalCacheHit") == 2
    assert rt.const_eval_cache_size() == 1
    assert launches[1] == launches[2] and launches[1] < launches[0]      # the dequantization ran once
    # a second binary with the same function shares the entry
    other = rt.Binary.load_from_memory(graphs.w8_linear_const_eval_binary(**kw))
    assert_matches(_read(rt, rt.submit(device, other, 0, dev_ins))[0], want, "second binary")
    assert rt.get_stat("ConstEvalCacheHit") == 3
    # new weights: other tensors, other versions -> evaluated again, with the new values
    ins2 = graphs.w8_linear_inputs(seed=7, **kw)
    want2 = oracle_results(graphs.w8_linear_graph, ins2, **kw)[0]
    dev_ins2 = _to_device_inputs(rt, device, binary, ins2)
    assert_matches(_read(rt, rt.submit(device, binary, 0, dev_ins2))[0], want2, "new weights")
    assert rt.get_stat("ConstEvalCacheMiss") == 2 and rt.const_eval_cache_size() == 2
    # overwriting a weight in place renews its version: evaluated again
    rt.memcpy(dev_ins2[1], dev_ins[1])
    rt.memcpy(dev_ins2[2], dev_ins[2])
    mixed = [ins2[0], ins[1], ins[2], ins2[3]]
    want3 = oracle_results(graphs.w8_linear_graph, mixed, **kw)[0]
    assert_matches(_read(rt, rt.submit(device, binary, 0, dev_ins2))[0], want3, "weights overwritten in place")
    assert rt.get_stat("ConstEvalCacheMiss") == 3
    # entries die with the tensors they were computed from
    del dev_ins2
    import gc
    gc.collect()
    assert rt.const_eval_cache_size() == 1
    rt.clear_const_eval_cache()
    assert rt.const_eval_cache_size() == 0


def test_traced_mlp_replays_with_new_inputs(rt, device):
    kw = dict(batch=128, d_in=784, d_hidden=256, d_out=10)
    binary = rt.Binary.load_from_memory(graphs.mlp_traced_binary(**kw))
    plain = rt.Binary.load_from_memory(graphs.build_binary(graphs.mlp_graph, **kw))
    rt.clear_stats()
    base = graphs.mlp_inputs(**kw)
    params = _to_device_inputs(rt, device, binary, base)[1:]
    plain_params = _to_device_inputs(rt, device, plain, base)[1:]
    replay_launches = None
    for step in range(4):
        x = graphs.mlp_inputs(seed=100 + step, **kw)[0]
        want = oracle_results(graphs.mlp_graph, [x] + base[1:], **kw)[0]
        hx = rt.to_layout(rt.from_torch(x), device, rt.get_layout(binary, 0, 0))        # stays on host
        before = rt.launch_count()
        got = _read(rt, rt.submit(device, binary, 0, [hx] + params))[0]
        n = rt.launch_count() - before
        assert_matches(got, want, f"traced mlp step {step}")
        ref = _read(rt, rt.submit(device, plain, 0, [rt.to_layout(rt.from_torch(x), device, rt.get_layout(plain, 0, 0))]
                                  + plain_params))[0]
        assert torch.equal(got, ref), "the replay and the plain program differ"
        if step >= 1:
            # a replay enqueues one graph: none of this library's launchers run on the host
            assert n == 0
            replay_launches = n
    assert replay_launches == 0
    assert rt.get_stat("TraceCacheMiss") == 1 and rt.get_stat("CapturedTrace") == 1 and rt.get_stat("ExecutedTrace") == 3


def test_trace_follows_replaced_parameters_and_can_be_released(rt, device):
    kw = dict(batch=32, d_in=64, d_hidden=48, d_out=10)
    binary = rt.Binary.load_from_memory(graphs.mlp_traced_binary(**kw))
    rt.clear_stats()
    a = graphs.mlp_inputs(seed=1, **kw)
    b = graphs.mlp_inputs(seed=2, **kw)
    pa = _to_device_inputs(rt, device, binary, a)
    pb = _to_device_inputs(rt, device, binary, b)
    want_a = oracle_results(graphs.mlp_graph, a, **kw)[0]
    want_b = oracle_results(graphs.mlp_graph, b, **kw)[0]
    assert_matches(_read(rt, rt.submit(device, binary, 0, pa))[0], want_a, "capture")
    assert_matches(_read(rt, rt.submit(device, binary, 0, pa))[0], want_a, "replay")
    # other parameter tensors: their contents are copied into the slots the trace reads
    assert_matches(_read(rt, rt.submit(device, binary, 0, pb))[0], want_b, "replay with replaced parameters")
    assert rt.get_stat("CapturedTrace") == 1
    rt.release_trace(device, binary.id, 0)
    assert_matches(_read(rt, rt.submit(device, binary, 0, pb))[0], want_b, "captured again after release")
    assert rt.get_stat("CapturedTrace") == 2


def test_func_call_runs_a_private_program(rt, device):
    from ttmlir_b200.ttnn_builder import BinaryBuilder
    bb = BinaryBuilder()
    main = bb.program("main")
    x = main.input([64, 96], "Float32")
    y = main.input([64, 96], "Float32")
    fn = bb.private_program("helper")
    fx, fy = fn.input([64, 96], "Float32"), fn.input([64, 96], "Float32")
    fn.output(fn.relu(fn.add(fx, fy)), fn.multiply(fx, fy))
    s, p = main.func_call(fn, [x, y])
    main.output(main.subtract(s, p))
    binary = rt.Binary.load_from_memory(bb.finish())
    tx, ty = torch.randn(64, 96), torch.randn(64, 96)
    got = _read(rt, rt.submit(device, binary, 0, _to_device_inputs(rt, device, binary, [tx, ty])))[0]
    assert_matches(got, torch.relu(tx + ty) - tx * ty, "func_call")


def test_failed_recording_leaves_the_device_usable(rt, device):
    """A program that asks for something a recording cannot hold (here: a device-to-host read)
    fails with a message; the stream leaves recording mode and later submits work."""
    from ttmlir_b200.ttnn_builder import BinaryBuilder
    bb = BinaryBuilder()
    main = bb.program("main")
    x = main.input([32, 32], "Float32")
    tid = main.begin_trace_capture()
    h = main.from_device(main.relu(x))
    main.end_trace_capture(tid)
    main.output(h)
    binary = rt.Binary.load_from_memory(bb.finish())
    tx = torch.randn(32, 32)
    with pytest.raises(RuntimeError):
        rt.submit(device, binary, 0, _to_device_inputs(rt, device, binary, [tx]))
    plain = rt.Binary.load_from_memory(graphs.build_binary(graphs.mlp_graph))
    ins = graphs.mlp_inputs()
    got = _read(rt, rt.submit(device, plain, 0, _to_device_inputs(rt, device, plain, ins)))[0]
    assert_matches(got, oracle_results(graphs.mlp_graph, ins)[0], "after a failed recording")


def test_traced_decoder_block_equals_the_plain_program(rt, device):
    """The decoder block (tensor-core GEMMs with fused epilogues, grouped and SwiGLU launches, rotary
    embedding through strides, tcgen05 attention) recorded as one CUDA graph: replays with new
    activations give bit for bit what the plain program gives."""
    kw = dict(seq=256, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024)
    traced = rt.Binary.load_from_memory(graphs.decoder_block_traced_binary(**kw))
    plain = rt.Binary.load_from_memory(graphs.build_binary(graphs.decoder_block_graph, **kw))
    base = graphs.decoder_block_inputs(**kw)
    t_in = _to_device_inputs(rt, device, traced, base)
    p_in = _to_device_inputs(rt, device, plain, base)
    rt.clear_stats()
    for step in range(3):
        x = graphs.decoder_block_inputs(seed=50 + step, **kw)[0]
        hx = rt.to_layout(rt.from_torch(x), device, rt.get_layout(traced, 0, 0))
        dx = rt.to_layout(rt.from_torch(x), device, rt.get_layout(plain, 0, 0))
        before = rt.launch_count()
        got = _read(rt, rt.submit(device, traced, 0, [hx] + t_in[1:]))[0]
        launches = rt.launch_count() - before
        ref = _read(rt, rt.submit(device, plain, 0, [dx] + p_in[1:]))[0]
        assert torch.equal(got, ref), f"step {step}: replay and plain program differ"
        if step:
            assert launches == 0
    want = oracle_results(graphs.decoder_block_graph, [x] + base[1:], **kw)[0]
    assert_matches(got, want, "traced decoder block", (0.999, 2e-2, 2.0 ** -6))
    assert rt.get_stat("CapturedTrace") == 1 and rt.get_stat("ExecutedTrace") == 2
