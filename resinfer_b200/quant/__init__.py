"""Linear-method registry, the ``residue::*`` custom ops and the tensor-parallel shard plan."""
