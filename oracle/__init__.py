"""CPU oracle for the TTNN-flatbuffer hot path.  TEST INFRASTRUCTURE ONLY.

Nothing in the product (tt-mlir_b200/) imports this package; only tests/, the smoke check in
__graft_entry__.py and bench.py's CPU-baseline / reference arms do.

What it restates, and from where (paths inside tenstorrent/tt-mlir):
  * the reference's CPU path for TTIR ops: its TTIR->Linalg->LLVM "CPU-hoist" lowering, whose
    torch twin is tools/tt-alchemist/templates/python/local/ttir_cpu.py (one function per op);
  * the CPU-hoist rounding model: every op widens its operands to f32 (integers to i32),
    computes, and narrows the result back (lib/Dialect/TTIR/Transforms/HoistCPUOps/HoistCPUOps.cpp:78-93,
    171-245), one op per hoisted function (:614-631).  `ops.py` applies exactly that around
    each op, so a bf16 graph is "f32 math per op, one rounding to bf16 after each op";
  * the torch goldens of tools/golden/mapping.py for ops that have no CPU-hoist lowering:
    quantize / dequantize / requantize (:2534-2582), rms_norm (:1221-1290), scaled dot product
    attention (:8398-8500), mesh_shard and the collectives (:4189-4235, 5658-5794), and the
    rotary-embedding definition (lib/Dialect/TTNN/Transforms/Fusing/RoPEFusingPattern.cpp:49-51).

Pinning: the reference ships no stored vectors for this path.  tests/golden/generate.py imports,
unmodified and in the development container where the reference tree is mounted, the reference's
ttir_cpu.py and its tools/golden/mapping.py (the latter with stand-in classes for the compiler's
Python bindings, tests/golden/ttmlir_standin.py) and records what their functions return on seeded
inputs; tests/test_oracle_golden.py checks this package against those fixtures bit for bit.  That
covers every op restated here, the kv-cache ops, decode and paged attention, gather / scatter /
sort / top-k and the collectives included.  Not pinned by a reference function, because the
reference has none: per-axis quantization (pinned on torch.quantize_per_channel instead) and the
rotary embedding (one formula in RoPEFusingPattern.cpp:49-51, restated).  The int8-storage
quantization variant has no runnable reference test (the reference skips it), so for that storage
width parity is pinned only through the torch golden.
"""
