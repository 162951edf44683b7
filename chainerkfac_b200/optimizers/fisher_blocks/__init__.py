from chainerkfac_b200.optimizers.fisher_blocks.connection import FisherBlockConnection  # NOQA
from chainerkfac_b200.optimizers.fisher_blocks.connections.linear import FisherBlockLinear  # NOQA
from chainerkfac_b200.optimizers.fisher_blocks.connections.convolution_2d import FisherBlockConvolution2D  # NOQA
from chainerkfac_b200.optimizers.fisher_blocks.normalizations.batch_normalization import FisherBlockBatchNormalization  # NOQA
