"""CPU-affinity helpers; the reference's version excludes the cores of its accelerator runtime (``utils/cann_cores_utils.py:27``), here the cores follow the GPU's NUMA node."""
from ..utils.cpu_affinity import bind_rank_to_cores, cores_for_rank, format_cpu_list, gpu_numa_node, numa_nodes, parse_cpu_list  # noqa: F401

__all__ = ["bind_rank_to_cores", "cores_for_rank", "format_cpu_list", "gpu_numa_node", "numa_nodes", "parse_cpu_list"]
