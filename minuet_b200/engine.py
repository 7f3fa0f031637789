"""Torch-facing glue over the C ABI: pointers, streams, workspaces, key specs.

PyTorch is used here only for device memory, the current stream and the final
device-to-host reads.  All compute is in ``libminuet_b200.so``.
"""
import ctypes
import weakref
from typing import Optional, Sequence

import numpy as np
import torch

from minuet_b200 import _lib
from minuet_b200._lib import KeySpec

DEFAULT_MARGIN = 64
# When set to a list, every convolution appends a dict with its shape (S, T, O, E,
# c_in, c_out, algorithm); benchmarks use it to compute per-layer rooflines.
LAYER_LOG = None
_DTYPE_CODE = {torch.float32: _lib.MN_F32, torch.float16: _lib.MN_F16,
               torch.bfloat16: _lib.MN_BF16}


def event_pair_begin(device):
    """Two timing events, the first recorded now on the current stream (per-layer
    times for LAYER_LOG)."""
    pair = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
    pair[0].record(torch.cuda.current_stream(device))
    return pair


def event_pair_end(pair, device):
    pair[1].record(torch.cuda.current_stream(device))


def lib():
    return _lib.load()


def require_cuda(*tensors):
    """The reference raises NotImplementedError for non-CUDA tensors
    (minuet/nn/functional/indexing.py:56,127); so does this engine."""
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise NotImplementedError("minuet_b200 runs on CUDA tensors only (no CPU path)")


def ptr(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def np_ptr(a: Optional[np.ndarray]):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _device_index(device) -> int:
    if isinstance(device, int):
        return device
    if not isinstance(device, torch.device):
        device = torch.device(device)
    return torch.cuda.current_device() if device.index is None else device.index


def raw_stream(device) -> int:
    """The current stream of ``device`` as an integer handle (the raw query costs a
    fraction of a microsecond; building a ``torch.cuda.Stream`` object costs several, and
    the map step asks for the stream a dozen times per build)."""
    return torch._C._cuda_getCurrentRawStream(_device_index(device))


def stream_ptr(device) -> ctypes.c_void_p:
    return ctypes.c_void_p(raw_stream(device))


def dtype_code(dtype: torch.dtype) -> int:
    if dtype not in _DTYPE_CODE:
        raise RuntimeError(f"Cannot find implementation of sparse convolution for {dtype}")
    return _DTYPE_CODE[dtype]


_WORKSPACE_CACHE_BYTES = 64 << 20
_workspaces = {}


def workspace(nbytes: int, device) -> torch.Tensor:
    """Scratch bytes for one library call.  Requests up to 64 MiB share one grow-only
    buffer per (device, stream): calls on one stream run in order, so the next call may
    overwrite what the previous one left.  Larger requests get a buffer of their own."""
    nbytes = max(int(nbytes), 256)
    if nbytes > _WORKSPACE_CACHE_BYTES:
        return torch.empty(nbytes, dtype=torch.uint8, device=device)
    key = (_device_index(device), raw_stream(device))
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8,
                          device=torch.device("cuda", key[0]))
        _workspaces[key] = buf
    return buf


def as_i32_coords(coords: torch.Tensor) -> torch.Tensor:
    """The kernels read int32 coordinates; int64 tensors are narrowed (their
    values must fit, as the reference's subtraction-based comparisons already
    require |c| < 2**30, csrc/minuet/common/functions.h:94-105)."""
    if coords.dtype == torch.int32:
        return coords.contiguous()
    if coords.dtype == torch.int64:
        return coords.to(torch.int32).contiguous()
    raise ValueError(f"The coordinates tensor must be int32 or int64 but found {coords.dtype}")


def as_i64(t: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if t is None:
        return None
    return t.to(torch.int64).contiguous()


# ---------------------------------------------------------------------------
# device status word
#   bit 1 (value 2): a coordinate fell outside the box the keys were built for
#   bit 2 (value 4): a bounded wait inside a tensor-core kernel ran out; the
#                    features that kernel wrote are invalid
#   bit 3 (value 8): the bounding box needs more than 63 key bits
# ---------------------------------------------------------------------------
STATUS_KEY_BOX = 2
STATUS_TC_TIMEOUT = 4
STATUS_KEY_BITS = 8
STATUS_GRID_TIMEOUT = 16
_status = {}
_pending_status = {}


def control_block(device) -> torch.Tensor:
    """The ``MN_CTRL_WORDS`` int32 control block of (device, current stream): word 0
    is the status word, the rest is grid-barrier state of the cooperative kernels.
    One block per stream, because kernels of different streams may overlap."""
    index = _device_index(device)
    key = (index, raw_stream(index))
    block = _status.get(key)
    if block is None:
        block = torch.zeros(_lib.MN_CTRL_WORDS, dtype=torch.int32,
                            device=torch.device("cuda", index))
        _status[key] = block
    return block


def status_word(device) -> torch.Tensor:
    """One-element view of the status word (the start of the control block)."""
    return control_block(device)[:1]


def decode_status(value: int) -> Optional[Exception]:
    """The exception a non-zero status word stands for (None for 0)."""
    value = int(value)
    if value == 0:
        return None
    parts = []
    if value & STATUS_TC_TIMEOUT:
        parts.append("a tensor-core kernel gave up waiting on one of its barriers: the "
                     "features it wrote are invalid (MN_ERR_DEVICE)")
    if value & STATUS_KEY_BITS:
        parts.append("the bounding box of the coordinates needs more than 63 key bits")
    if value & STATUS_KEY_BOX:
        parts.append("a coordinate lies outside the bounding box the sort/search keys were "
                     "built for (call KernelMapCache.reset() before feeding unrelated "
                     "coordinates)")
    if value & STATUS_GRID_TIMEOUT:
        parts.append("a grid-wide barrier of a cooperative kernel timed out: its outputs are "
                     "invalid (MN_ERR_DEVICE)")
    if value & ~(STATUS_KEY_BOX | STATUS_TC_TIMEOUT | STATUS_KEY_BITS | STATUS_GRID_TIMEOUT):
        parts.append(f"unknown device status bits 0x{value:x}")
    if value & STATUS_KEY_BITS and not value & (STATUS_TC_TIMEOUT | STATUS_GRID_TIMEOUT):
        return NotImplementedError("; ".join(parts))
    return RuntimeError("; ".join(parts))


def raise_on_status(value: int, device):
    error = decode_status(value)
    if error is not None:
        control_block(device).zero_()      # also resets the barrier state after a timeout
        raise error


def check_status(device):
    """Blocking read of the status word."""
    raise_on_status(int(status_word(device).item()), device)


def poll_status(device):
    """Non-blocking check for the forward path: queues an asynchronous copy of the
    status word into pinned memory and raises for any earlier copy that has
    landed with a non-zero value.  An error therefore surfaces at the latest one
    call after the kernel that raised it, without a host-device synchronisation."""
    dev = torch.device(device)
    key = dev.index if dev.index is not None else torch.cuda.current_device()
    queue = _pending_status.setdefault(key, [])
    while queue and queue[0][1].query():
        pinned, _ = queue.pop(0)
        raise_on_status(int(pinned[0]), device)
    if len(queue) < 8:
        pinned = torch.empty(1, dtype=torch.int32, pin_memory=True)
        pinned.copy_(status_word(device), non_blocking=True)
        event = torch.cuda.Event()
        event.record(torch.cuda.current_stream(device))
        queue.append((pinned, event))


# ---------------------------------------------------------------------------
# key specs and keys
# ---------------------------------------------------------------------------

def make_keyspec(coord_tensors: Sequence[torch.Tensor], ndim: int, num_clouds: int,
                 margin: int) -> KeySpec:
    """Bounding box on the device, one small D2H read, layout on the host."""
    tensors = [t for t in coord_tensors if t is not None and t.shape[0] > 0]
    spec = KeySpec()
    if not tensors:
        mm = np.array([0, 0, 0, 0, 0, 0, 0, 0], dtype=np.int32)
    else:
        device = tensors[0].device
        assert len(tensors) <= 2
        a = tensors[0]
        b = tensors[1] if len(tensors) > 1 else None
        out = torch.empty(8, dtype=torch.int32, device=device)
        ws = workspace(lib().mn_map_workspace_bytes(0, 0, 0), device)
        _lib.check(lib().mn_bbox(ptr(a), a.shape[0], ptr(b), 0 if b is None else b.shape[0], ndim,
                                 ptr(out), ptr(ws), ws.numel(), stream_ptr(device)), "bbox")
        mm = out.cpu().numpy()
    _lib.check(lib().mn_keyspec_make(np_ptr(mm), ndim, max(int(num_clouds), 1), int(margin),
                                     ctypes.byref(spec)), "keyspec")
    return spec


def make_keyspec_device(coords: torch.Tensor, batch_dims: Optional[torch.Tensor], ndim: int,
                        num_clouds: int, margin: int, with_keys: bool = True):
    """Bounding box, key layout and (optionally) the keys of ``coords`` in one launch,
    all left on the device (no read-back).  Returns ``(spec, spec_dev, keys)``: the
    host struct only carries ndim, margin and the pointer to ``spec_dev``, which
    must stay alive for as long as the spec is used."""
    device = coords.device
    spec = KeySpec()
    spec_dev = torch.empty(256, dtype=torch.uint8, device=device)
    keys = torch.empty(coords.shape[0], dtype=torch.int64, device=device) if with_keys else None
    ws = workspace(lib().mn_map_workspace_bytes(0, 0, 0), device)
    _lib.check(lib().mn_keyspec_device(ptr(coords), coords.shape[0], ndim, ptr(batch_dims),
                                       max(int(num_clouds), 1), int(margin), ptr(spec_dev),
                                       ctypes.byref(spec), ptr(keys), ptr(control_block(device)),
                                       ptr(ws), ws.numel(), stream_ptr(device)), "keyspec_device")
    return spec, spec_dev, keys


def read_small(t: torch.Tensor) -> np.ndarray:
    """Blocking device-to-host read of a small tensor through pinned memory (one DMA
    transfer, no kernel)."""
    pinned = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
    pinned.copy_(t, non_blocking=True)
    torch.cuda.current_stream(t.device).synchronize()
    return pinned.numpy().copy()


def pack_keys(coords: torch.Tensor, batch_dims: Optional[torch.Tensor], spec: KeySpec,
              tstride: Optional[Sequence[int]] = None) -> torch.Tensor:
    n, ndim = coords.shape
    keys = torch.empty(n, dtype=torch.int64, device=coords.device)
    ts = None if tstride is None else np.asarray(tstride, dtype=np.int32)
    nb = 1 if batch_dims is None else batch_dims.numel() - 1
    _lib.check(lib().mn_pack_keys(ptr(coords), n, ndim, ptr(batch_dims), nb, np_ptr(ts),
                                  ctypes.byref(spec), ptr(keys), ptr(status_word(coords.device)),
                                  stream_ptr(coords.device)), "pack_keys")
    return keys


# ---------------------------------------------------------------------------
# host copies of small device tensors (kernel-map sizes), keyed by tensor
# ---------------------------------------------------------------------------
_host_copies = {}


class PendingHostCopy:
    """Asynchronous device-to-host copy of a small int32 tensor whose LAST element
    is a snapshot of the status word (one DMA transfer into pinned memory, no
    kernel); the wait happens when (and if) the host needs the values."""

    _pool = []

    def __init__(self, values_and_status: torch.Tensor):
        device = values_and_status.device
        self.device = device
        n = values_and_status.numel()
        pinned = None
        for i, buf in enumerate(self._pool):
            if buf.numel() >= n:
                pinned = self._pool.pop(i)
                break
        if pinned is None:
            pinned = torch.empty(max(n, 160), dtype=torch.int32, pin_memory=True)
        self.pinned = pinned
        self.n = n
        pinned[:n].copy_(values_and_status, non_blocking=True)
        self.event = torch.cuda.Event()
        self.event.record(torch.cuda.current_stream(device))
        self.values = None

    def get(self) -> np.ndarray:
        if self.values is None:
            self.event.synchronize()
            host = self.pinned[:self.n].numpy().copy()
            if len(self._pool) < 64:
                self._pool.append(self.pinned)
            self.pinned = None
            raise_on_status(int(host[-1]), self.device)
            self.values = np.ascontiguousarray(host[:-1])
        return self.values


def remember_host(t: torch.Tensor, values):
    """``values``: a numpy array or a PendingHostCopy of the tensor's contents."""
    key = id(t)
    _host_copies[key] = (weakref.ref(t, lambda _r, k=key: _host_copies.pop(k, None)), values)


def host_copy(t: torch.Tensor, dtype=np.int32) -> np.ndarray:
    """Host values of ``t``: the remembered copy when the tensor came from this
    engine, otherwise a blocking device-to-host read."""
    hit = _host_copies.get(id(t))
    if hit is not None and hit[0]() is t:
        values = hit[1].get() if isinstance(hit[1], PendingHostCopy) else hit[1]
        return np.ascontiguousarray(values.astype(dtype, copy=False))
    return np.ascontiguousarray(t.detach().cpu().numpy().astype(dtype, copy=False))


# ---------------------------------------------------------------------------
# per-row hit words of kernel maps, keyed by the mask tensors they belong to
# ---------------------------------------------------------------------------
_hit_bits = {}


def remember_bits(source_masks, target_masks, source_bits, target_bits):
    """Keep the per-row hit words (bit p set <=> mask row p has an entry for the row)
    that the fused map build produced, for as long as the masks live."""
    for masks, bits in ((source_masks, source_bits), (target_masks, target_bits)):
        key = id(masks)
        _hit_bits[key] = (weakref.ref(masks, lambda _r, k=key: _hit_bits.pop(k, None)), bits)


def hit_bits(masks: torch.Tensor) -> Optional[torch.Tensor]:
    """Hit words of a mask tensor that came from the fused map build, else None."""
    hit = _hit_bits.get(id(masks))
    if hit is not None and hit[0]() is masks:
        return hit[1]
    return None


# ---------------------------------------------------------------------------
# neighbour tables of kernel maps (fused forward), keyed by the mask tensors
# ---------------------------------------------------------------------------
_neighbor_tables = {}


def neighbor_table(source_masks: torch.Tensor, target_masks: torch.Tensor,
                   sizes_host: np.ndarray, reorder: bool = True):
    """``(nbr [O, T] int32, tile_bits [ceil(T/128)] int32, perm [T] int32 or None)`` of
    the kernel map that the two mask tensors describe; built on first use and kept for
    as long as the masks live (a transposed convolution passes the same masks swapped
    and gets its own table).  With ``reorder`` and a map that carries hit words, the
    table's rows are the targets sorted by hit word (``perm[r]`` = target at position
    ``r``), so that 128-row tiles skip the offsets none of their rows has."""
    bits = hit_bits(target_masks) if reorder else None
    key = (id(source_masks), id(target_masks), bits is not None)
    hit = _neighbor_tables.get(key)
    if hit is not None and hit[0]() is source_masks and hit[1]() is target_masks:
        return hit[2], hit[3], hit[4]
    O, S = source_masks.shape
    T = target_masks.shape[1]
    device = source_masks.device
    nbr = torch.empty((O, T), dtype=torch.int32, device=device)
    tile_bits = torch.empty((T + 127) // 128, dtype=torch.int32, device=device)
    perm = torch.empty(T, dtype=torch.int32, device=device) if bits is not None else None
    ws = workspace(lib().mn_neighbor_table_workspace_bytes(np_ptr(sizes_host), O, T), device)
    _lib.check(lib().mn_build_neighbor_table(ptr(source_masks), ptr(target_masks),
                                             np_ptr(sizes_host), O, S, T,
                                             ptr(hit_bits(source_masks) if bits is not None else None),
                                             ptr(bits), ptr(nbr),
                                             ptr(tile_bits), ptr(perm), ptr(control_block(device)),
                                             ptr(ws), ws.numel(), stream_ptr(device)),
               "build_neighbor_table")

    def drop(_ref, k=key):
        _neighbor_tables.pop(k, None)

    _neighbor_tables[key] = (weakref.ref(source_masks, drop), weakref.ref(target_masks, drop),
                             nbr, tile_bits, perm)
    return nbr, tile_bits, perm


# ---------------------------------------------------------------------------
# pair lists of kernel maps (pair-list forward), keyed by the mask tensors
# ---------------------------------------------------------------------------
_pair_lists = {}


def pair_list(source_masks: torch.Tensor, target_masks: torch.Tensor, sizes_host: np.ndarray,
              allow_shortcut: bool):
    """``pair_src`` int32 ``[R]`` (the source row of every product row, -1 in the
    padding) of the kernel map the masks describe, or None when the map did not come
    with hit words; built on first use and kept for as long as the masks live."""
    bits = hit_bits(source_masks)
    if bits is None or hit_bits(target_masks) is None:
        return None
    key = (id(source_masks), id(target_masks), bool(allow_shortcut))
    hit = _pair_lists.get(key)
    if hit is not None and hit[0]() is source_masks and hit[1]() is target_masks:
        return hit[2]
    O, S = source_masks.shape
    T = target_masks.shape[1]
    device = source_masks.device
    rows = int(lib().mn_pair_rows(np_ptr(sizes_host), O, S, T, int(bool(allow_shortcut))))
    pair_src = torch.empty(max(rows, 1), dtype=torch.int32, device=device)
    _lib.check(lib().mn_build_pair_list(ptr(source_masks), ptr(bits), np_ptr(sizes_host), O, S, T,
                                        int(bool(allow_shortcut)), ptr(pair_src),
                                        stream_ptr(device)), "build_pair_list")

    def drop(_ref, k=key):
        _pair_lists.pop(k, None)

    _pair_lists[key] = (weakref.ref(source_masks, drop), weakref.ref(target_masks, drop), pair_src)
    return pair_src
