"""Context parallelism: strategy registry and the built-in strategies."""

from titan_b200.parallel.context_parallel.registry import (  # noqa: F401
    adjust_cp_mask,
    apply_cp_to_attention_module,
    register_cp_mask_handler,
    register_cp_strategy,
    registered_strategies,
)
from titan_b200.parallel.context_parallel import ulysses  # noqa: F401,E402  (registers itself)
from titan_b200.parallel.context_parallel import varlen_cp  # noqa: F401,E402  (registers itself)
