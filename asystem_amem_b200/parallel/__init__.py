"""Parallelism wrappers built on the library's collectives and fused kernels:
data parallel / fully sharded (fsdp), tensor + sequence parallel (tp), expert parallel (ep),
pipeline parallel (pp), context parallel attention (cp: Ulysses all-to-all and ring send/recv), and
hybrid layouts through split communicators (hybrid)."""
from .cp import ring_attention, ulysses_attention  # noqa: F401
from .fsdp import FSDP, ShardedAdamW  # noqa: F401
from .hybrid import make_grid  # noqa: F401
from .pp import PipelineStage  # noqa: F401
from .tp import ColumnParallelLinear, RowParallelLinear  # noqa: F401
