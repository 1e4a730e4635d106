"""Expert parallelism: see ``asystem_amem_b200.ops.moe.MoeDispatcher`` (fused dispatch /
combine) and ``asystem_amem_b200.models.moe_layer.MoELayer`` which uses it."""
from ..ops.moe import DispatchResult, MoeDispatcher  # noqa: F401
