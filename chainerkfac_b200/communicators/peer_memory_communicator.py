"""The 'peer_memory' communicator: the two collectives of
``chainerkfac/communicators/pure_nccl_communicator.py`` with the transfer done
by this library's own unpack kernel reading the other GPUs' wire buffers over
NVLink, instead of by a library collective.

Interface, wire format (arrays concatenated in (owner rank, array) order,
factors as packed lower triangles) and results are those of the 'pure_nccl'
communicator.  Mechanism:

* every rank packs into a wire buffer that all ranks of the group have mapped
  (symmetric memory), then all ranks meet at a stream-ordered barrier;
* reduce-scatter: the owner's unpack kernel sums its segment of every rank's
  buffer in rank order (``kfac_wire_unpack_sum``: peer loads, scale 1/size,
  mirror) - reduction and unpack are one kernel, and nothing is staged in
  between;
* all-gather: every rank unpacks each other owner's segment straight from that
  owner's buffer.

Two wire buffers alternate between successive collective calls.  A rank
packs into a buffer again only after the barrier of the call in between, which
every peer reaches only after its kernels that read the buffer's previous
content, so one barrier per call is enough.  The barrier is a one-element
all-reduce of the process group (stream-ordered, no host synchronisation).
All ranks must issue the same sequence of calls with the same array shapes,
as with any collective.
"""

import torch
import torch.distributed as dist

from chainerkfac_b200.communicators.pure_nccl_communicator import \
    PureNcclCommunicator


class PeerMemoryCommunicator(PureNcclCommunicator):

    def __init__(self, group=None, wire_dtype='float32'):
        super(PeerMemoryCommunicator, self).__init__(group, wire_dtype)
        self._wires = [None, None]    # (tensor, device addresses by rank)
        self._turn = 0
        self._flag = None

    # -- pieces a test can replace ------------------------------------------
    def _map_wire(self, nelems, device):
        """A wire buffer of ``nelems`` floats mapped by every rank of the
        group; returns (local tensor, device addresses of all ranks' buffers
        in rank order).  Collective."""
        import torch.distributed._symmetric_memory as symm
        t = symm.empty(nelems, dtype=self.wire_dtype, device=device)
        group = self.group if self.group is not None else dist.group.WORLD
        handle = symm.rendezvous(t, group)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        if len(ptrs) != self.size or ptrs[self.rank] != t.data_ptr():
            raise RuntimeError('symmetric memory rendezvous returned an '
                               'unexpected mapping')
        self._handles = getattr(self, '_handles', []) + [handle]
        return t, ptrs

    def _barrier(self, device):
        if self._flag is None or self._flag.device != device:
            self._flag = torch.zeros(1, dtype=torch.float32, device=device)
        dist.all_reduce(self._flag, group=self.group)

    def _unpack_sum(self, flat, tri, ptrs, select, scale):
        from chainerkfac_b200 import ops
        ops.wire_unpack_sum(flat, tri, ptrs, select=select, scale=scale,
                            wire_dtype=self.wire_dtype)

    # -------------------------------------------------------------------------
    def reserve(self, nelems, device):
        """Map both wire buffers for calls of up to ``nelems`` wire elements
        now.  Collective; otherwise the buffers are mapped (and re-mapped when
        a larger call comes) on demand."""
        for k in (0, 1):
            ent = self._wires[k]
            if ent is None or ent[0].numel() < nelems:
                if ent is not None:
                    # peers may still read the old mapping
                    self._barrier(device)
                    if device.type == 'cuda':
                        torch.cuda.synchronize(device)
                self._wires[k] = self._map_wire(max(int(nelems), 1), device)

    def _next_wire(self, nelems, device):
        k = self._turn
        self._turn ^= 1
        ent = self._wires[k]
        if ent is None or ent[0].numel() < nelems:
            self.reserve(nelems, device)
            ent = self._wires[k]
        return ent

    def reduce_scatter_v_arrays(self, arrays, stream=None, debug=False):
        """``arrays[r]`` lists (array, triangular) owned by rank r.  On return
        this rank's own arrays hold the mean over ranks; arrays of other
        owners are left as they were
        (``communicators/pure_nccl_communicator.py:47-108``)."""
        if len(arrays) != self.size:
            raise ValueError('arrays must have one entry per rank')
        flat, tri, owner, seg, total = self._layout(arrays)
        if total == 0:
            return
        me = self.rank
        device = flat[0].device

        def body():
            wire, ptrs = self._next_wire(total, device)
            self._pack(flat, tri, wire[:total], None)
            self._barrier(device)
            select = [1 if o == me else 0 for o in owner]
            if any(select):
                self._unpack_sum(flat, tri, ptrs, select, 1.0 / self.size)
        self._run(stream, body)

    def all_gather_v_arrays(self, arrays, stream=None, debug=False):
        """Every rank ends with each owner's version of ``arrays[owner]``
        (``communicators/pure_nccl_communicator.py:150-218``)."""
        if len(arrays) != self.size:
            raise ValueError('arrays must have one entry per rank')
        flat, tri, owner, seg, total = self._layout(arrays)
        if total == 0:
            return
        me = self.rank
        device = flat[0].device

        def body():
            wire, ptrs = self._next_wire(total, device)
            mine = [1 if o == me else 0 for o in owner]
            if any(mine):
                self._pack(flat, tri, wire[:total], mine)
            self._barrier(device)
            for r, (_, n) in enumerate(seg):
                if r != me and n > 0:
                    self._unpack_sum(flat, tri, [ptrs[r]],
                                     [1 if o == r else 0 for o in owner], 1.0)
        self._run(stream, body)
