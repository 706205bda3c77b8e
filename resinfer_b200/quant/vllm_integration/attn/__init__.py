"""Decode half of the ResAttn attention adapter (the part that needs no vLLM import)."""
from .decode import ResAttnDecodeMixin  # noqa: F401
