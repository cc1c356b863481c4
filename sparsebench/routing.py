"""sparsebench.routing (reference: sparsebench/routing.py): DeviceTopology, route_device,
build_topology_cuda; plus route(), the on-device top-k router."""

from sparsebench_b200.routing import DeviceTopology, build_topology_cuda, route, route_device  # noqa: F401
