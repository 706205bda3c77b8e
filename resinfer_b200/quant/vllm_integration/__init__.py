"""Adapters on the vLLM side of the hot path: the ``residue::nvfp4_linear`` op and the
tensor-parallel shard plan for K-extended tensors."""
