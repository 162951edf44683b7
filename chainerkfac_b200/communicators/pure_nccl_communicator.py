"""The 'pure_nccl' communicator; mirrors the interface of
``chainerkfac/communicators/pure_nccl_communicator.py``.

Wire format and results are the reference's (arrays concatenated in
(owner rank, array) order, factors as packed lower triangles, owner receives
the mean over ranks; all-gather delivers each owner's arrays to everyone).
The mechanism differs: the reference all-reduces the whole buffer for both
collectives (``:98,209``); here each owner's segment is reduced to that owner
only, and gathered by a broadcast from it, so a rank receives only what it
keeps.  Pack and unpack are the library's kernels (``kfac_wire_pack`` /
``kfac_wire_unpack``); the transport is NCCL through ``torch.distributed``.
"""

import torch
import torch.distributed as dist

from chainerkfac_b200.communicators import _utility
from chainerkfac_b200.communicators import base


class PureNcclCommunicator(base.KfacCommunicatorBase):

    def __init__(self, group=None, wire_dtype='float32'):
        super(PureNcclCommunicator, self).__init__(group)
        self.gpu_buf_a = None   # grow-only wire buffer
        # element type of the wire buffer.  The reference's pack kernels can
        # cast to fp16 (:354-375,438-461) but its communicator fixes fp32
        # (:32-33); 'float16' / 'bfloat16' halve the bytes on the wire at
        # 16-bit accuracy of what arrives (the arrays themselves stay fp32).
        self.wire_dtype = _utility.wire_torch_dtype(wire_dtype)

    # -- pieces a test can replace (pack/unpack need the CUDA library) ------
    def _wire_buffer(self, nelems, like):
        if self.gpu_buf_a is None or self.gpu_buf_a.numel() < nelems or \
                self.gpu_buf_a.device != like.device or \
                self.gpu_buf_a.dtype != self.wire_dtype:
            self.gpu_buf_a = torch.empty(max(nelems, 1), dtype=self.wire_dtype,
                                         device=like.device)
        return self.gpu_buf_a[:nelems]

    def _pack(self, flat, tri, wire, select):
        from chainerkfac_b200 import ops
        ops.wire_pack(flat, tri, wire, select=select)

    def _unpack(self, flat, tri, wire, select, scale):
        from chainerkfac_b200 import ops
        ops.wire_unpack(flat, tri, wire, select=select, scale=scale)

    # -- layout ----------------------------------------------------------------
    @staticmethod
    def _layout(arrays):
        flat, tri, owner, seg = [], [], [], []
        off = 0
        for rank, local in enumerate(arrays):
            n = _utility.get_local_nelems(local)
            seg.append((off, n))
            off += n
            for a, t in local:
                if a.dtype != torch.float32:
                    raise ValueError('dtype must be float32.')
                if not a.is_contiguous():
                    raise ValueError('non contiguous array detected')
                flat.append(a)
                tri.append(bool(t))
                owner.append(rank)
        return flat, tri, owner, seg, off

    def _run(self, stream, fn):
        if stream is None or not torch.cuda.is_available():
            return fn()
        with torch.cuda.stream(stream):
            return fn()

    def reduce_scatter_v_arrays(self, arrays, stream=None, debug=False):
        """``arrays[r]`` lists (array, triangular) owned by rank r.  On return
        this rank's own arrays hold the mean over ranks; arrays of other
        owners are left as they were (``:47-108``)."""
        if len(arrays) != self.size:
            raise ValueError('arrays must have one entry per rank')
        flat, tri, owner, seg, total = self._layout(arrays)
        if total == 0:
            return
        me = self.rank

        def body():
            wire = self._wire_buffer(total, flat[0])
            self._pack(flat, tri, wire, None)
            works = []
            for r, (off, n) in enumerate(seg):
                if n > 0:
                    works.append(dist.reduce(
                        wire[off:off + n], dst=self.global_rank(r),
                        op=dist.ReduceOp.SUM, group=self.group, async_op=True))
            for w in works:
                w.wait()
            select = [1 if o == me else 0 for o in owner]
            if any(select):
                self._unpack(flat, tri, wire, select, 1.0 / self.size)
        self._run(stream, body)

    def all_gather_v_arrays(self, arrays, stream=None, debug=False):
        """Every rank ends with each owner's version of ``arrays[owner]``
        (``:150-218``)."""
        if len(arrays) != self.size:
            raise ValueError('arrays must have one entry per rank')
        flat, tri, owner, seg, total = self._layout(arrays)
        if total == 0:
            return
        me = self.rank

        def body():
            wire = self._wire_buffer(total, flat[0])
            mine = [1 if o == me else 0 for o in owner]
            if any(mine):
                self._pack(flat, tri, wire, mine)
            works = []
            for r, (off, n) in enumerate(seg):
                if n > 0:
                    works.append(dist.broadcast(
                        wire[off:off + n], src=self.global_rank(r),
                        group=self.group, async_op=True))
            for w in works:
                w.wait()
            others = [1 - m for m in mine]
            if any(others):
                self._unpack(flat, tri, wire, others, 1.0)
        self._run(stream, body)
