from .memory_auditor import MemoryAuditor, MemorySnapshot
from .runtime_component_factory import LiteRuntimeAssembler, RuntimeAssemblyContext

__all__ = ["MemoryAuditor", "MemorySnapshot", "LiteRuntimeAssembler", "RuntimeAssemblyContext"]
