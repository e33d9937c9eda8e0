"""Carry exchange of the split-along-T scan over peer-mapped memory (one box, NVLink/NVSwitch).

``PeerCarryExchange`` owns this rank's exchange buffer, allocated as torch symmetric memory so
that every rank of the group has it mapped, and drives the two C-ABI calls
``fms_peer_publish`` (peer stores + flag) and ``fms_peer_wait_fold`` (bounded wait on local flags
+ carry fold).  It replaces the NCCL all-gather, the carry fold kernel and the tensor slicing of
the default path of ``fm_b200.time_split`` by two small kernels per direction.

All ranks must create the object together and then perform the same sequence of forward and
backward exchanges (the usual SPMD discipline): exchange numbers are counted per direction.
Consumers acknowledge every fold and publishers wait for the acknowledgement of the exchange two
before theirs, so any sequence is safe -- forward-only loops (inference) included: a fast rank
runs at most one exchange ahead of the slowest rank that reads its carries.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from . import capi

_P, _I64, _I, _U32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_uint32


def _bind():
    L = capi.lib()
    if not getattr(L, "_fms_peer_bound", False):
        L.fms_peer_exchange_bytes.restype = ctypes.c_size_t
        L.fms_peer_exchange_bytes.argtypes = [_I64, _I]
        L.fms_peer_exchange_status_offset.restype = ctypes.c_size_t
        L.fms_peer_exchange_status_offset.argtypes = [_I64, _I]
        L.fms_peer_publish.restype = _I
        L.fms_peer_publish.argtypes = [_P, _P, _I64, ctypes.POINTER(_P), _I, _I, _I, _U32, ctypes.c_double, _P]
        L.fms_peer_wait_fold.restype = _I
        L.fms_peer_wait_fold.argtypes = [ctypes.POINTER(_P), _P, _P, _I64, _I, _I, _I, _U32, ctypes.c_double, _P]
        L._fms_peer_bound = True
    return L


class PeerExchangeTimeout(RuntimeError):
    pass


_FAULTS = {1: "a block this rank depends on was not published in time (forward exchange)",
           2: "a block this rank depends on was not published in time (reverse exchange)",
           3: "a slot already held a later exchange than the one waited for (numbering broken)",
           4: "a reader did not acknowledge the exchange two before this one in time"}


def _bind_fused():
    L = capi.lib()
    if not getattr(L, "_fms_tsplit_bound", False):
        L.fms_tsplit_exchange_bytes.restype = ctypes.c_size_t
        L.fms_tsplit_exchange_bytes.argtypes = [_I64, _I]
        L.fms_tsplit_exchange_status_offset.restype = ctypes.c_size_t
        L.fms_tsplit_exchange_status_offset.argtypes = [_I64, _I]
        L.fms_tsplit_forward.restype = _I
        L.fms_tsplit_forward.argtypes = [_P, _P, _P, _P, _P, _I64, _I64, _I, ctypes.POINTER(_P), _I, _I, _U32,
                                         ctypes.c_double, _P]
        L.fms_tsplit_backward.restype = _I
        L.fms_tsplit_backward.argtypes = [_P, _P, _P, _P, _P, _P, _P, _I64, _I64, _I, ctypes.POINTER(_P), _I, _I,
                                          _U32, ctypes.c_double, _P]
        L._fms_tsplit_bound = True
    return L


class FusedTimeSplit:
    """The split-along-T scan as ONE kernel per direction (``fms_tsplit_forward`` / ``_backward``).

    Owns this rank's exchange buffer in torch symmetric memory.  Carry pass, exchange of the
    carries (peer stores, bounded local polls) and scan pass run fused row by row inside the kernel,
    so a row's operands are re-read from L2 and the block moves the HBM bytes of an unsplit scan.
    All ranks create the object together and call ``forward`` / ``backward`` in the same order.
    Needs 16-byte aligned rows (``T_k * element size % 16 == 0``); ``applies()`` tells.
    """

    def __init__(self, rows: int, group=None, device=None, max_wait_seconds: float = 2.0):
        import torch.distributed._symmetric_memory as symm_mem

        self._L = _bind_fused()
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("the fused split covers one box: at most 8 ranks")
        self.rows = int(rows)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_wait_seconds = float(max_wait_seconds)
        nbytes = int(self._L.fms_tsplit_exchange_bytes(self.rows, self.world))
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every buffer is zeroed before anyone publishes
        self._peers = (_P * self.world)(*[int(p) for p in self.handle.buffer_ptrs])
        off = int(self._L.fms_tsplit_exchange_status_offset(self.rows, self.world))
        self.status = self.buffer[off:off + 4].view(torch.int32)
        self._count = [0, 0]

    @staticmethod
    def applies(gates: torch.Tensor) -> bool:
        T = gates.shape[-1]
        return gates.is_cuda and T >= 1 and (T * gates.element_size()) % 16 == 0 and gates.data_ptr() % 16 == 0

    @staticmethod
    def pays(gates: torch.Tensor) -> bool:
        """Whether the fused kernels are expected to beat the three-launch path for this block.

        Their advantage is that a row's second pass re-reads the row from L2, which holds while the
        rows in flight (one per SM) fit: 148 rows x 2 operands x T_k x element size well inside the
        126 MB L2.  Measured on B200 with fp32 rows: T_k = 32768 (38 MB in flight) 0.72 ms fused
        against 1.01 ms; T_k = 131072 (155 MB) slower than three launches.  The bound used is 48 MB.
        """
        if not FusedTimeSplit.applies(gates):
            return False
        sms = torch.cuda.get_device_properties(gates.device).multi_processor_count
        return sms * 2 * gates.shape[-1] * gates.element_size() <= 48 * (1 << 20)

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def _raise(self, what, rc):
        raise capi.FmsError(what, rc, capi.status_string(rc), int(self._L.fms_last_cuda_error()))

    def forward(self, gates, tokens, h0=None):
        """-> (states, h_in): this block's states and the fp32 carry (rows) that entered the block."""
        T = gates.shape[-1]
        states = torch.empty_like(gates)
        h_in = torch.empty(self.rows, device=self.device, dtype=torch.float32)
        self._count[0] += 1
        with torch.cuda.device(self.device):
            rc = self._L.fms_tsplit_forward(gates.data_ptr(), tokens.data_ptr(), capi.ptr(h0), states.data_ptr(),
                                            h_in.data_ptr(), self.rows, T, capi.dtype_tag(gates.dtype), self._peers,
                                            self.world, self.rank, self._count[0], self.max_wait_seconds,
                                            self._stream())
        if rc != capi.FMS_OK:
            self._raise("fms_tsplit_forward", rc)
        return states, h_in

    def backward(self, gates, states, grad_states, h_in, want_grad_h0=False):
        T = gates.shape[-1]
        grad_gates, grad_tokens = torch.empty_like(gates), torch.empty_like(gates)
        grad_h0 = torch.empty(self.rows, device=self.device, dtype=torch.float32) if want_grad_h0 else None
        self._count[1] += 1
        with torch.cuda.device(self.device):
            rc = self._L.fms_tsplit_backward(gates.data_ptr(), states.data_ptr(), grad_states.data_ptr(),
                                             h_in.data_ptr(), grad_gates.data_ptr(), grad_tokens.data_ptr(),
                                             capi.ptr(grad_h0), self.rows, T, capi.dtype_tag(gates.dtype),
                                             self._peers, self.world, self.rank, self._count[1],
                                             self.max_wait_seconds, self._stream())
        if rc != capi.FMS_OK:
            self._raise("fms_tsplit_backward", rc)
        return grad_gates, grad_tokens, grad_h0

    def check(self) -> None:
        """Synchronise and raise if a kernel recorded a fault (a wait ran out, numbering broken)."""
        code = int(self.status.item())
        if code != 0:
            raise PeerExchangeTimeout(
                f"rank {self.rank}: {_FAULTS.get(code, 'unknown fault %d' % code)} (bound {self.max_wait_seconds} s)")


class PeerCarryExchange:
    def __init__(self, rows: int, group=None, device=None, max_wait_seconds: float = 2.0):
        import torch.distributed._symmetric_memory as symm_mem

        self._L = _bind()
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.world = dist.get_world_size(self.group)
        if self.world > 8:
            raise ValueError("the peer exchange covers one box: at most 8 ranks")
        self.rows = int(rows)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.max_wait_seconds = float(max_wait_seconds)
        nbytes = int(self._L.fms_peer_exchange_bytes(self.rows, self.world))
        self.buffer = symm_mem.empty(nbytes, dtype=torch.uint8, device=self.device)
        self.buffer.zero_()
        self.handle = symm_mem.rendezvous(self.buffer, self.group)
        torch.cuda.synchronize(self.device)
        dist.barrier(self.group)  # every buffer is zeroed before anyone publishes
        self._peers = (_P * self.world)(*[int(p) for p in self.handle.buffer_ptrs])
        off = int(self._L.fms_peer_exchange_status_offset(self.rows, self.world))
        self.status = self.buffer[off:off + 4].view(torch.int32)
        self._count = [0, 0]  # exchanges done so far: forward, reverse

    def _stream(self):
        return torch.cuda.current_stream(self.device).cuda_stream

    def exchange(self, P: torch.Tensor, S: torch.Tensor, carry0=None, reverse: bool = False) -> torch.Tensor:
        """Publish this block's (P, S) and return the carry entering this block (fp32, rows)."""
        for t in (P, S):
            if not (t.is_cuda and t.dtype == torch.float32 and t.is_contiguous() and t.numel() == self.rows):
                raise RuntimeError("P and S must be contiguous fp32 CUDA tensors with one element per row")
        if carry0 is not None and not (carry0.is_cuda and carry0.dtype == torch.float32
                                       and carry0.is_contiguous() and carry0.numel() == self.rows):
            raise RuntimeError("carry0 must be a contiguous fp32 CUDA tensor with one element per row")
        d = 1 if reverse else 0
        self._count[d] += 1
        number = self._count[d]
        out = torch.empty(self.rows, device=self.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            rc = self._L.fms_peer_publish(P.data_ptr(), S.data_ptr(), self.rows, self._peers, self.world, self.rank,
                                          d, number, self.max_wait_seconds, self._stream())
            if rc == capi.FMS_OK:
                rc = self._L.fms_peer_wait_fold(self._peers, capi.ptr(carry0), out.data_ptr(), self.rows,
                                                self.world, self.rank, d, number, self.max_wait_seconds,
                                                self._stream())
        if rc != capi.FMS_OK:
            raise capi.FmsError("fms_peer_publish/wait_fold", rc, capi.status_string(rc),
                                int(self._L.fms_last_cuda_error()))
        return out

    def check(self) -> None:
        """Synchronise and raise if an exchange recorded a fault.  After a fault the ranks'
        exchange numbers no longer agree: build a new ``PeerCarryExchange``."""
        code = int(self.status.item())
        if code != 0:
            raise PeerExchangeTimeout(
                f"rank {self.rank}: {_FAULTS.get(code, 'unknown fault %d' % code)} "
                f"(bound {self.max_wait_seconds} s)")
