def create_communicator(communicator_name='pure_nccl', mpi_comm=None):
    """Same call as ``chainerkfac.create_communicator``
    (``communicators/__init__.py:1-12``).  ``mpi_comm`` is accepted for
    compatibility: processes are launched by ``torchrun`` (one per GPU) and
    bootstrap through ``torch.distributed``; pass a torch process group to use
    a sub-group, or None for the world."""
    if communicator_name == 'pure_nccl':
        from chainerkfac_b200.communicators.pure_nccl_communicator \
            import PureNcclCommunicator
        return PureNcclCommunicator(mpi_comm)
    else:
        raise ValueError(
            'Unrecognized communicator_name: {}'.format(communicator_name))
