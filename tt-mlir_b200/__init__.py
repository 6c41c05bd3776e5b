"""B200-native execution backend for TTNN flatbuffers (tt-mlir's compiled-graph hot path).

The directory name contains a hyphen, so the package is loaded under the import name
`ttmlir_b200` by `__graft_entry__.load_package()` (also used by tests and bench.py).
"""
