"""sparsebench.spmm (reference: sparsebench/spmm.py): sdd and dsd; plus combine."""

from sparsebench_b200.spmm import combine, dsd, sdd  # noqa: F401
