"""Operation layer: launch plans over the CUDA library, capability checks and the CPU oracle.

Names of the reference's op layer (nvls/torch_symm_triton/__init__.py:3-10, nvls/metadata.py) and
their counterparts here:

    fused_metadata_update            -> MetadataPlan
    multimem_all_gather_v            -> AllGatherVPlan (one tensor)
    multimem_all_gatherv_3tensor     -> AllGatherVPlan (up to four tensors, one barrier)
    multimem_reduce_scatter_v        -> ReduceScatterVPlan
    multimem_all_gather[_fused]      -> UniformAllGatherPlan
    multimem_reduce_scatter          -> UniformReduceScatterPlan
    fused_multimem_rs_add_norm_ag    -> RsAddNormAgPlan
    (DeepEP ElasticBuffer)           -> A2ADispatchPlan / A2ACombinePlan
    (no counterpart)                 -> RoutePlan, GroupedGemmPlan, ExpertCombinePlan,
                                        DispatchRouteFc1Plan, Fc2CombinePlan
"""
import importlib

# Resolved on first use: the plan modules import the symmetric heap, which imports ``ops._ext``;
# importing them here eagerly would close that loop.
_EXPORTS = {
    "a2a": ["A2ABuffers", "A2ACombinePlan", "A2ADispatchPlan", "a2a_decode_step"],
    "capability": ["are_tensors_gather_eligible", "are_tensors_reduce_eligible", "heap_has_multicast",
                   "is_device_multimem_capable", "is_device_tcgen05_capable", "row_access_bytes"],
    "dense": ["AllGatherVPlan", "MetadataPlan", "ReduceScatterVPlan", "UniformAllGatherPlan",
              "UniformReduceScatterPlan", "dense_decode_step"],
    "experts": ["DispatchRouteFc1Plan", "ExpertCombinePlan", "ExpertWeights", "Fc2CombinePlan", "GroupedGemmPlan",
                "RouteBuffers", "RoutePlan"],
    "norm": ["RsAddNormAgPlan"],
}
_WHERE = {name: mod for mod, names in _EXPORTS.items() for name in names}
__all__ = sorted(_WHERE)


def __getattr__(name):
    if name in _WHERE:
        return getattr(importlib.import_module(f"{__name__}.{_WHERE[name]}"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
