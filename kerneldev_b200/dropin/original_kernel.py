"""Drop-in module: put this directory ahead of the reference checkout on ``sys.path`` and the
reference's ``model.py`` (``from original_kernel import flash_attention``, model.py:24) binds the
sm_100a operator instead of the Triton one."""
from kerneldev_b200.original_kernel import (flash_attention, generate_hadamard_signs,  # noqa: F401
                                             hadamard_transform)
