"""CPU oracle for the MEXT / KEXT / ResAttn hot paths.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package imports this directory: only the test-suite, the smoke
check and the ``cpu_baseline`` / ``--impl reference`` legs of the benchmark may use it,
and only as the checker or as the timed CPU baseline.

What it restates (file:line are paths inside the ShawRong/ResInfer reference project):

* FP4 / scale codecs          csrc/common/fp4/nvfp4_utils.cuh:143-238, 402-429
* NVFP4 MEXT block maths      csrc/common/fp4/nvfp4_utils.cuh:467-556, 614-713
* NVFP4 MEXT layouts          csrc/common/fp4/nvfp4_utils.cuh:1109-1160,
                              csrc/nvfp4/cuda/nvfp4_quant_kernels.cu:113-262
* NVFP4 KEXT (masked residue) csrc/common/fp4/nvfp4_utils.cuh:895-1045, 1185-1217,
                              csrc/nvfp4/cuda/nvfp4_residue_pack8.cu:102-304
* MXFP4 MEXT / selective      csrc/mxfp4/cuda/mxfp4_residue_quant.cu:19-29, 55-81, 84-265
* grouped-Q quantiser         csrc/nvfp4/cuda/nvfp4_quant_kernels.cu:616-689
* 128x4 scale swizzle         csrc/common/fp4/nvfp4_utils.cuh:1080-1107,
                              csrc/nvfp4/scale_layout.py:8-33
* torch-eager linear          quant/modelopt_integration/residue_linear.py:53-136
* ResAttn decode semantics    csrc/resattn/kernel_paged_decode.py:1888-1969, 2193-2203,
                              2822-2834

Pinning.  The reference ships no tests, golden vectors or fixtures.  The quantiser part of
the oracle is pinned against the reference's own compiled CUDA kernels (``oracle/_ref``,
built by ``oracle/build_ref.py`` from the reference sources) on a B200: the fixtures under
``tests/golden`` hold outputs of those reference kernels on seeded inputs, and the oracle
reproduces them bit for bit once it is given the device's ``rcp.approx.ftz.f32`` results for
the handful of reciprocals the algorithm takes (stored with each fixture).  The GEMM and
attention parts have no runnable reference on this toolchain (the reference kernels need a
newer CUTLASS DSL / CUDA 13.4 PTX) and the eager path needs NVIDIA ModelOpt, which is not
vendored: for those two parts parity is UNPINNED and is stated as a tolerance against the
FP32 product of the dequantised operands.
"""
from .fp4_codec import *  # noqa: F401,F403
from .nvfp4_quant import *  # noqa: F401,F403
from .mxfp4_quant import *  # noqa: F401,F403
from .linear import *  # noqa: F401,F403
from .resattn import *  # noqa: F401,F403
