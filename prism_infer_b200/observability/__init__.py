"""No-op-by-default observability facades (reference ``prism_infer/observability``).

Runtime code calls ``profile_region(name)`` and the KV-trace hooks unconditionally; they do
nothing until a provider is installed (``prism_infer_b200.analysis.performance_profile``
installs the profiling provider when a session is opened).
"""

from .kv_trace import emit_kv_event, install_kv_trace_provider
from .performance import install_profile_provider, profile_region, profile_step_metadata

__all__ = [
    "profile_region", "profile_step_metadata", "install_profile_provider",
    "emit_kv_event", "install_kv_trace_provider",
]
