"""Top-level ``nvfp4`` distribution name of the reference wheel (ShawRong/ResInfer csrc/setup.py:113-127:
packages ``nvfp4``, ``nvfp4.mxfp4``, ``nvfp4.cute_fold``, ``nvfp4.cute_attn``).  Importing it hands the name
over to ``resinfer_b200.nvfp4`` -- after this module has run, ``sys.modules["nvfp4"]`` and its sub-packages
are the real ones, so ``import nvfp4.mxfp4`` and ``from nvfp4.cute_attn import host`` resolve there."""
import resinfer_b200

resinfer_b200.install_aliases(overwrite=True)
