"""tt::runtime API semantics on the GPU, in the spirit of the reference's
runtime/test/ttnn/python/n150/test_runtime_api.py and test_debug_hooks.py."""

import ctypes

import pytest
import torch

from helpers import assert_matches, oracle_results, run_program
from ttmlir_b200 import graphs

pytestmark = pytest.mark.gpu


def test_to_layout_round_trip_and_cast(rt, device):
    buf = graphs.build_binary(graphs.quant_chain_graph, rows=32, cols=32)
    binary = rt.Binary.load_from_memory(buf)
    layout = rt.get_layout(binary, 0, 0)
    x = torch.randn(32, 32)
    h = rt.from_torch(x)                      # f32 on host, program wants bf16 on device
    d = rt.to_layout(h, device, layout)
    assert d.is_on_device() and d.get_dtype() == rt.DataType.BFloat16 and rt.has_layout(d, layout)
    back = rt.to_torch(rt.to_host(d, untilize=True)[0])
    assert torch.equal(back, x.to(torch.bfloat16))


def test_memcpy_between_tensors(rt, device):
    buf = graphs.build_binary(graphs.mlp_graph)
    binary = rt.Binary.load_from_memory(buf)
    x = torch.randn(128, 784)
    d = rt.to_layout(rt.from_torch(x), device, rt.get_layout(binary, 0, 0))
    y = torch.randn(128, 784)
    rt.memcpy(d, rt.from_torch(y))            # host -> device tensor
    out = torch.empty_like(y)
    rt.memcpy(rt.from_torch(out), d)          # device -> host tensor
    assert torch.equal(out, y)


def test_retain_and_deallocate(rt, device):
    buf = graphs.build_binary(graphs.mlp_graph)
    binary = rt.Binary.load_from_memory(buf)
    ins = graphs.mlp_inputs()
    dev_in = [rt.to_layout(rt.from_torch(t), device, rt.get_layout(binary, 0, i), retain=True) for i, t in enumerate(ins)]
    o1 = rt.to_torch(rt.to_host(rt.submit(device, binary, 0, dev_in)[0])[0])
    o2 = rt.to_torch(rt.to_host(rt.submit(device, binary, 0, dev_in)[0])[0])   # inputs survive a submit
    assert torch.equal(o1, o2)
    rt.deallocate_tensor(dev_in[0])           # retained: ignored
    assert dev_in[0].is_allocated()
    rt.deallocate_tensor(dev_in[0], force=True)
    assert not dev_in[0].is_allocated()
    with pytest.raises(RuntimeError, match="deallocated"):
        rt.submit(device, binary, 0, dev_in)


def test_submit_argument_errors(rt, device):
    buf = graphs.build_binary(graphs.mlp_graph)
    binary = rt.Binary.load_from_memory(buf)
    ins = graphs.mlp_inputs()
    with pytest.raises(RuntimeError, match="expects 5 inputs"):
        rt.submit(device, binary, 0, [rt.from_torch(ins[0])])
    bad = [rt.from_torch(t) for t in ins]
    bad[1] = rt.from_torch(torch.randn(10, 10))
    with pytest.raises(RuntimeError, match="elements"):
        rt.submit(device, binary, 0, bad)
    with pytest.raises(RuntimeError, match="out of range"):
        rt.submit(device, binary, 3, [rt.from_torch(t) for t in ins])
    two = graphs.build_binary(graphs.mlp_graph, mesh_shape=(1, 2))
    with pytest.raises(RuntimeError, match="mesh"):
        rt.submit(device, rt.Binary.load_from_memory(two), 0, [rt.from_torch(t) for t in ins])


def test_host_inputs_are_uploaded(rt, device):
    # Callers normally run to_layout first; host tensors of the right dtype are accepted too.
    buf = graphs.build_binary(graphs.mlp_graph)
    binary = rt.Binary.load_from_memory(buf)
    ins = graphs.mlp_inputs()
    out = rt.to_torch(rt.to_host(rt.submit(device, binary, 0, [rt.from_torch(t) for t in ins])[0])[0])
    assert_matches(out, oracle_results(graphs.mlp_graph, ins)[0], "mlp via host inputs")


def test_cpu_op_is_rejected_not_emulated(rt, device):
    def g(b):
        x = b.input([4, 4], "Float32")
        b.output(b.cpu_op([x], [4, 4], "Float32", "hoisted_add_helper"))
    buf = graphs.build_binary(g)
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        run_program(rt, device, buf, [torch.randn(4, 4)])


def test_unsupported_op_names_itself(rt, device):
    from ttmlir_b200.schema.fbs import Writer
    from ttmlir_b200.schema.ttnn_schema import FILE_IDENTIFIER, S, SCHEMA_HASH
    w = Writer(S)
    prog = {"name": "main", "inputs": [], "outputs": [], "mesh_shape": (1, 1),
            "operations": [{"type": ("MoeComputeOp", {}), "debug_info": "", "loc_info": "loc(\"moe\")"}]}
    root = w.create_table("TTNNBinary", {"version": (0, 1, 0), "schema_hash": SCHEMA_HASH, "programs": [prog]})
    binary = rt.Binary.load_from_memory(w.finish(root, FILE_IDENTIFIER))
    with pytest.raises(RuntimeError, match="MoeComputeOp"):
        rt.submit(device, binary, 0, [])


def test_debug_hooks_see_every_op_and_do_not_change_results(rt, device):
    kw = dict(rows=64, cols=48, keep_intermediates=False)
    buf = graphs.build_binary(graphs.quant_chain_graph, **kw)
    ins = graphs.quant_chain_inputs(64, 48)
    fused = run_program(rt, device, buf, ins)[0]
    seen, outputs = [], {}

    def post(_bin, ctx, op):
        loc = rt.get_op_loc_info(op)
        seen.append(loc)
        t = rt.get_op_output_tensor(op, ctx)
        if t is not None:
            outputs[loc] = rt.to_torch(t)
    rt.DebugHooks.get(None, post)
    try:
        unfused = run_program(rt, device, buf, ins)[0]
    finally:
        rt.unregister_hooks()
    assert torch.equal(fused, unfused)        # the fused launch equals the op-by-op execution
    assert 'loc("quantize")' in seen and 'loc("requantize")' in seen and 'loc("dequantize")' in seen
    want = oracle_results(graphs.quant_chain_graph, ins, rows=64, cols=48, keep_intermediates=True)
    assert torch.equal(outputs['loc("quantize")'], want[1])      # intermediates visible to callbacks
    assert torch.equal(outputs['loc("requantize")'], want[2])
    after = run_program(rt, device, buf, ins)[0]
    assert torch.equal(after, fused)


def test_launch_counter_moves(rt, device):
    buf = graphs.build_binary(graphs.quant_chain_graph, rows=64, cols=64)
    before = rt.launch_count()
    run_program(rt, device, buf, graphs.quant_chain_inputs(64, 64))
    assert rt.launch_count() > before


def test_pipelined_steps_with_pinned_buffers(rt, device):
    """Uploads from page-locked memory and non-blocking downloads run on their own streams.
    A pipelined loop (upload i+1 and download i-1 around compute i) must give exactly what
    the blocking calls give, step by step, with a different input every step."""
    import ctypes
    buf = graphs.build_binary(graphs.mlp_graph)
    binary = rt.Binary.load_from_memory(buf)
    ins = graphs.mlp_inputs()
    weights = [rt.to_layout(rt.from_torch(t), device, rt.get_layout(binary, 0, i), retain=True)
               for i, t in enumerate(ins)][1:]
    layout = rt.get_layout(binary, 0, 0)
    steps = 6
    xs = [(ins[0] + 0.25 * k).clone().pin_memory() for k in range(steps)]
    # blocking reference results
    want = []
    for x in xs:
        d = rt.to_layout(rt.from_torch(x.clone()), device, layout)   # pageable copy: blocking upload
        out = rt.submit(device, binary, 0, [d] + weights)[0]
        want.append(rt.to_torch(rt.to_host(out, untilize=True)[0]))
    # pipelined
    got, pending = [], None

    def read(h, like):
        rt.wait(h)
        n = like.numel() * like.element_size()
        raw = (ctypes.c_char * n).from_address(h.host_ptr())
        return torch.frombuffer(raw, dtype=like.dtype).reshape(like.shape).clone()

    for x in xs:
        d = rt.to_layout(rt.from_torch(x), device, layout)
        out = rt.submit(device, binary, 0, [d] + weights)[0]
        h = rt.to_host(out, untilize=True, blocking=False)[0]
        if pending is not None:
            got.append(read(pending, want[len(got)]))
        pending = h
    got.append(read(pending, want[len(got)]))
    for k in range(steps):
        assert torch.equal(got[k], want[k]), f"step {k} differs"
    assert not torch.equal(got[0], got[1])


def test_wait_on_blocking_host_tensor_is_harmless(rt, device):
    buf = graphs.build_binary(graphs.quant_chain_graph, rows=32, cols=32)
    binary = rt.Binary.load_from_memory(buf)
    x = torch.randn(32, 32).pin_memory()
    d = rt.to_layout(rt.from_torch(x), device, rt.get_layout(binary, 0, 0))
    h = rt.to_host(d, untilize=True)[0]
    rt.wait(h)
    rt.wait(d)
    assert torch.equal(rt.to_torch(h), x.to(torch.bfloat16))


def test_a_timed_out_tensor_core_launch_is_reported_by_wait(rt, device):
    """Every wait inside the tensor-core kernels is bounded; a launch that gave up leaves a status
    word behind and incomplete output.  wait() must turn that word into an error, once, and the
    device must stay usable.  The word is written from the host here (ttb_tcgen05_set_status): no
    GPU wait is made to run out."""
    kw = dict(m=256, k=512, n=384)
    ins = graphs.w8_linear_inputs(**kw)
    binary = rt.Binary.load_from_memory(graphs.build_binary(graphs.w8_linear_graph, **kw))
    dev_in = [rt.to_layout(rt.from_torch(t), device, rt.get_layout(binary, 0, i), retain=True) for i, t in enumerate(ins)]
    good = rt.to_torch(rt.to_host(rt.submit(device, binary, 0, dev_in)[0], untilize=True)[0])
    for gemm, sdpa, text in ((0x0401, 0, "GEMM"), (0, 0x0901, "attention")):
        out = rt.submit(device, binary, 0, dev_in)[0]
        assert rt.lib.ttb_tcgen05_set_status(gemm, sdpa) == 0
        with pytest.raises(RuntimeError, match=text):
            rt.wait(out)
        rt.wait(out)                                   # reported once: the word was cleared
        again = rt.to_torch(rt.to_host(rt.submit(device, binary, 0, dev_in)[0], untilize=True)[0])
        assert torch.equal(again, good)


def test_tensor_core_wait_limit_can_be_set_and_restored(rt, device):
    """The limit of the bounded waits is a setting, not a constant: a short limit that no healthy
    launch reaches leaves results unchanged, and the default comes back with a non-positive value."""
    kw = dict(m=256, k=512, n=384)
    ins = graphs.w8_linear_inputs(**kw)
    buf = graphs.build_binary(graphs.w8_linear_graph, **kw)
    before = run_program(rt, device, buf, ins)[0]
    assert rt.lib.ttb_tcgen05_set_wait_limit(ctypes.c_longlong(200_000_000)) == 0   # ~0.1 s
    try:
        after = run_program(rt, device, buf, ins)[0]
    finally:
        assert rt.lib.ttb_tcgen05_set_wait_limit(ctypes.c_longlong(0)) == 0
    assert torch.equal(before, after)
    g, a = ctypes.c_int(-1), ctypes.c_int(-1)
    assert rt.lib.ttb_tcgen05_status(ctypes.byref(g), ctypes.byref(a), 0) == 0
    assert (g.value, a.value) == (0, 0)
