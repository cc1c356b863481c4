"""The reference's extension module `sparsebench._C` (csrc/bindings.cpp:5-16): the same four
functions, positional order and keyword names, served by libsparsebench_b200."""

from sparsebench_b200._C import (  # noqa: F401
    arch_probe,
    build_topology_cuda,
    combine_cuda,
    dsd_cuda,
    router_topk_cuda,
    sdd_cuda,
)
