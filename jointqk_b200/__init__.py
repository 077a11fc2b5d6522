"""jointqk_b200: the compress-then-attend key path of JointQK on NVIDIA B200 (sm_100a).

Host objects keep the reference toolkit's names (``PerCoordCompressor``, ``batched_roundtrip``,
``water_fill``, ``solve_lloyd_max``, moment accumulators ...); the work runs in the CUDA
kernels of ``libjointqk_b200.so`` (C ABI in ``include/jointqk_b200.h``).
"""

from .allocation import allocate_bits, allocate_bits_for_budget, round_bits_to_integer, water_fill
from .basis import eigvec_desc, jointqk_basis, regularize_batch, repeat_kv_states
from .codebooks import generate_rotation_matrix, solve_lloyd_max, unit_gaussian_centroids
from .layout import KeyLayout, plan_key_layout

__all__ = [
    "allocate_bits", "allocate_bits_for_budget", "round_bits_to_integer", "water_fill",
    "eigvec_desc", "jointqk_basis", "regularize_batch", "repeat_kv_states",
    "generate_rotation_matrix", "solve_lloyd_max", "unit_gaussian_centroids",
    "KeyLayout", "plan_key_layout",
    "PerCoordCompressor", "batched_roundtrip", "stack_per_head", "build_method_compressor",
    "HeadTables", "PackedKeys", "PagedKVCache",
    "QueryMomentsAccumulator", "CrossMomentsAccumulator", "KeyPathMoments",
    "compute_moments_from_tensors", "compute_query_moments", "compute_grouped_query_second_moment",
    "compute_attention_metrics", "CenteredCompressor", "build_v_compressor", "V_METHOD_NAMES", "PagePool", "JointQKPressB200",
]

_LAZY = {
    "PerCoordCompressor": "compressor", "batched_roundtrip": "compressor", "stack_per_head": "compressor",
    "build_method_compressor": "compressor", "HeadTables": "tables", "PackedKeys": "paged",
    "PagedKVCache": "paged", "QueryMomentsAccumulator": "moments", "CrossMomentsAccumulator": "moments",
    "KeyPathMoments": "moments", "compute_moments_from_tensors": "moments",
    "compute_query_moments": "moments", "compute_grouped_query_second_moment": "moments",
    "compute_attention_metrics": "eval", "CenteredCompressor": "v_compressor", "build_v_compressor": "v_compressor",
    "V_METHOD_NAMES": "v_compressor", "PagePool": "paged", "JointQKPressB200": "press",
}


def __getattr__(name):
    # Modules that bind the CUDA library load on first use, so that the pure host-side fit
    # objects stay importable on machines that only prepare calibration artefacts.
    mod = _LAZY.get(name)
    if mod is None:
        raise AttributeError(name)
    import importlib

    return getattr(importlib.import_module(f".{mod}", __name__), name)
