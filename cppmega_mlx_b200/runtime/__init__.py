from .env import RuntimeEnvironment, detect_runtime_environment
from .kernel_policy import KernelPath, clear_dispatch_log, get_dispatch_log, record_dispatch, selected_path
from .memory import MemoryLimitPlan, MemorySnapshot, apply_memory_limit_plan, memory_limit_plan
from .memory_audit import audit_memory
from .seed import capture_rng_state, restore_rng_state, seed_all
