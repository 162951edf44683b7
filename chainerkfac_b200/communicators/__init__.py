def create_communicator(communicator_name='pure_nccl', mpi_comm=None,
                        wire_dtype='float32'):
    """Same call as ``chainerkfac.create_communicator``
    (``communicators/__init__.py:1-12``).  ``mpi_comm`` is accepted for
    compatibility: processes are launched by ``torchrun`` (one per GPU) and
    bootstrap through ``torch.distributed``; pass a torch process group to use
    a sub-group, or None for the world.

    'pure_nccl' is the reference's name and moves the wire buffer with NCCL;
    'peer_memory' (an addition) has the same interface and results and moves
    it with this library's own kernels over NVLink peer mappings.

    ``wire_dtype`` ('float32' as in the reference, 'float16' or 'bfloat16')
    is the element type of the wire buffer; the 16-bit types halve the
    exchanged bytes and deliver 16-bit-accurate factors and gradients."""
    if communicator_name == 'pure_nccl':
        from chainerkfac_b200.communicators.pure_nccl_communicator \
            import PureNcclCommunicator
        return PureNcclCommunicator(mpi_comm, wire_dtype)
    elif communicator_name == 'peer_memory':
        from chainerkfac_b200.communicators.peer_memory_communicator \
            import PeerMemoryCommunicator
        return PeerMemoryCommunicator(mpi_comm, wire_dtype)
    else:
        raise ValueError(
            'Unrecognized communicator_name: {}'.format(communicator_name))
