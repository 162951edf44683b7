from chainerkfac_b200.optimizers import fisher_blocks  # NOQA

from chainerkfac_b200.optimizers.kfac import KFAC  # NOQA
from chainerkfac_b200.optimizers.kfac import DistributedKFAC  # NOQA
