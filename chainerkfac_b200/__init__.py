"""chainerkfac_b200: the K-FAC curvature path of chainerkfac on B200 GPUs.

Layout: ``csrc/`` CUDA kernels and the C ABI (``include/kfac_b200.h``),
``_lib``/``ops`` the ctypes binding, ``optimizers``/``communicators`` the
host-side mirror of the reference's Python interface.
"""

__version__ = '0.1.0'

from chainerkfac_b200 import communicators  # NOQA
from chainerkfac_b200 import optimizers  # NOQA

from chainerkfac_b200.communicators import create_communicator  # NOQA
from chainerkfac_b200.optimizers import fisher_blocks  # NOQA
from chainerkfac_b200.optimizers.kfac import KFAC  # NOQA
from chainerkfac_b200.optimizers.kfac import DistributedKFAC  # NOQA
