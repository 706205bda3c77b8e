"""Top-level ``quant`` package name of the reference (ShawRong/ResInfer quant/): handed over to
``resinfer_b200.quant`` on import (see ``resinfer_b200._compat.nvfp4``)."""
import resinfer_b200

resinfer_b200.install_aliases(overwrite=True)
