"""B200-native kernels for the per-layer PTQ encode path of hi2.

Modules mirror the reference's: ``hessian``, ``encode``, ``ladder_kernel``, ``gptq_kernel``,
``refine_kernel``, ``refine``, ``format``, ``stats``, ``allocate``, ``calibrate``; ``dist`` holds the
multi-GPU plan and ``install`` the wiring that makes an unmodified hi2 call these modules.
"""

__version__ = "0.1.0"
