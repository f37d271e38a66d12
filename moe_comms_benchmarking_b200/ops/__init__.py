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
from .a2a import A2ABuffers, A2ACombinePlan, A2ADispatchPlan, a2a_decode_step  # noqa: F401
from .capability import (are_tensors_gather_eligible, are_tensors_reduce_eligible, heap_has_multicast,  # noqa: F401
                         is_device_multimem_capable, is_device_tcgen05_capable, row_access_bytes)
from .dense import (AllGatherVPlan, MetadataPlan, ReduceScatterVPlan, UniformAllGatherPlan,  # noqa: F401
                    UniformReduceScatterPlan, dense_decode_step)
from .experts import (DispatchRouteFc1Plan, ExpertCombinePlan, ExpertWeights, Fc2CombinePlan,  # noqa: F401
                      GroupedGemmPlan, RouteBuffers, RoutePlan)
from .norm import RsAddNormAgPlan  # noqa: F401
