"""CPU oracle for the sync-free MoE forward path. TEST INFRASTRUCTURE, not product code.

A restatement of the reference's own CPU algorithms for this path (SparseBench's
sparsebench/topology.py and sparsebench/reference.py), written from their behaviour: numpy for the
integer layout, CPU PyTorch for the floating-point layer. It is pinned against golden vectors that
were produced by the reference itself (tests/golden/, generator script beside them).

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this package, and only
as the checker or the timed baseline. Nothing in sparsebench_b200 imports it.
"""
