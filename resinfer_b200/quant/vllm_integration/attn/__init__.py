"""ResAttn attention adapter for vLLM: ``decode`` (the decode launches, no vLLM import), ``backend`` (backend,
metadata builder and implementation classes), ``register`` (CUSTOM backend registration), ``warmup``, ``runtime``.
Only the decode mixin is imported here, so the package loads without vLLM."""
from .decode import ResAttnDecodeMixin  # noqa: F401
