"""Communicator base; mirrors ``chainerkfac/communicators/base.py`` with
``torch.distributed`` in the place of ChainerMN's MPI communicator."""

import os
import warnings

import torch
import torch.distributed as dist


class KfacCommunicatorBase(object):

    def __init__(self, group=None):
        if not dist.is_initialized():
            if 'RANK' in os.environ and 'WORLD_SIZE' in os.environ:
                backend = 'nccl' if torch.cuda.is_available() else 'gloo'
                dist.init_process_group(backend)
            else:
                raise RuntimeError(
                    'torch.distributed is not initialised and no torchrun '
                    'environment (RANK/WORLD_SIZE) was found')
        self.group = group
        self.indices = None

    @property
    def rank(self):
        return dist.get_rank(self.group)

    @property
    def size(self):
        return dist.get_world_size(self.group)

    @property
    def intra_rank(self):
        return int(os.environ.get('LOCAL_RANK', self.rank))

    def global_rank(self, group_rank):
        if self.group is None:
            return group_rank
        return dist.get_global_rank(self.group, group_rank)

    def bcast_data(self, model):
        """Broadcast every parameter from rank 0 (ChainerMN's ``bcast_data``,
        used by ``kfac.py:376-377``)."""
        for _, param in sorted(model.namedparams(), key=lambda kv: kv[0]):
            if param.data is not None:
                dist.broadcast(param.data, src=self.global_rank(0),
                               group=self.group)

    def allreduce_grad(self, model=None):
        # We don't use AllReduce for training K-FAC
        warnings.warn('AllReduce called, skipping...')

    def reduce_scatter_v_arrays(self, arrays, stream=None):
        raise NotImplementedError

    def all_gather_v_arrays(self, arrays, stream=None):
        raise NotImplementedError
