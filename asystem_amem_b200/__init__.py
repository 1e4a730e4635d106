"""B200-native pausable collective library (AMem capabilities, built from scratch).

Layers: ``bindings`` (ctypes over ``lib/libamem_b200.so``), ``comm`` (Communicator and the
process-wide pause/resume calls), ``ops`` (fused compute+collective operations),
``parallel`` (DP/FSDP, TP, EP, PP wrappers), ``models`` (Llama decoder, TP MLP, MoE layer),
``utils``.
"""
from .bindings import NcclError, load_library  # noqa: F401
from .comm import (Communicator, backend_usage, paused, get_group_id, get_unique_id, group_end, group_start, inject,  # noqa: F401
                   mem_alloc, mem_free, mem_stats, pause_all, process_pause_resume_stats, resume_all, set_group_id)

__version__ = "0.1.0"
