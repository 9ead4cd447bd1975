"""Host <-> device staging around the op front end: a three-stream pipeline
(upload, compute, download) over the device runtime.

TensorFlow's executor drives the reference plugin the same way: feeds go up on
the host-to-device stream, kernels run on the compute stream, fetches come
down on the device-to-host stream, and stream dependencies order the three
(musa_ext/mu/musa_se_plugin.cc:127-212 copies, :362-432 dependencies; pinned
staging blocks from musa_ext/mu/device/pinned_memory_pool.h).  This module is
that driver for callers that hold HOST tensors: `StagedPipeline.submit(op,
*args)` returns at once, the upload of call k+1 overlaps the kernels of call k
and the download of call k-1, and `StagedCall.result()` hands back the host
results.

Streams, events, copies and pinned blocks all come from the runtime's C ABI
(include/musa_plugin_runtime.h); torch supplies device memory only.
"""
import collections
import ctypes
import threading
import weakref

import numpy as np
import torch

from . import raw_ops as _r
from .errors import InternalError, InvalidArgumentError

try:
    import ml_dtypes
    _NP_BF16 = np.dtype(ml_dtypes.bfloat16)
except Exception:  # pragma: no cover
    _NP_BF16 = None


def _to_host_tensor(a):
    """numpy array -> CPU torch tensor sharing its memory."""
    a = np.ascontiguousarray(a)
    if _NP_BF16 is not None and a.dtype == _NP_BF16:
        return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16)
    return torch.from_numpy(a)


def _free_pinned_block(lib, ordinal, ptr, nbytes, stream, alive):
    # After close() the stream is gone: a null stream makes the pool wait for
    # the device instead of following a stream.
    lib.MusaRtPinnedFreeAsync(ordinal, ptr, nbytes, stream if alive[0] else None)


class _DevicePool:
    """Device staging buffers, recycled by exact size.  A buffer is handed out
    again only after every call that touched it has been seen to finish, so
    reuse needs no stream ordering."""

    def __init__(self, device):
        self.device = device
        self.free = collections.defaultdict(list)
        self.bytes_held = 0
        self.lock = threading.Lock()

    def get(self, nbytes):
        with self.lock:
            bucket = self.free.get(nbytes)
            if bucket:
                return bucket.pop()
            self.bytes_held += nbytes
        return torch.empty(max(nbytes, 1), dtype=torch.uint8, device=self.device)

    def put(self, buf, nbytes):
        with self.lock:
            self.free[nbytes].append(buf)


class _Lease:
    """One device staging buffer in use; goes back to the pool when the last
    holder (a call in flight or a StagedValue) lets go of it."""

    def __init__(self, pool, nbytes):
        self.pool = pool
        self.nbytes = nbytes
        self.buf = pool.get(nbytes)

    def __del__(self):
        try:
            self.pool.put(self.buf, self.nbytes)
        except Exception:  # interpreter shutdown
            pass


class StagedValue:
    """A device-resident tensor of the pipeline: an uploaded input or an output
    of an earlier call.  Pass it to a later `submit()` to use the tensor
    without another trip over PCIe."""

    def __init__(self, tensor, keep):
        self.tensor = tensor
        self._keep = keep   # lease (inputs) or None (outputs own their memory)

    @property
    def shape(self):
        return tuple(self.tensor.shape)


class StagedCall:
    """One submitted op.  `result()` waits for its downloads and returns the
    fetched outputs as host tensors.  Each host tensor lives in a pinned
    staging block that goes back to the runtime's pool when the last reference
    to the tensor (or a view of it) is gone; `release()` drops the references
    that this object holds."""

    def __init__(self, pipe):
        self._pipe = pipe
        self._inputs = []       # StagedValue per positional argument (or None)
        self._outputs = []      # StagedValue per op output (or None)
        self._host = {}         # output index -> host tensor (owns its pinned block)
        self._hold = []         # leases, host sources and device tensors in use
        self._events = []
        self._done_event = None
        self._finished = False
        self._released = False
        self.error = None

    def input(self, i):
        """Device copy of positional argument i (a host tensor that this call
        uploaded)."""
        v = self._inputs[i]
        if v is None:
            raise InvalidArgumentError("argument %d was not a tensor" % i)
        return v

    def output(self, i):
        v = self._outputs[i]
        if v is None:
            raise InvalidArgumentError("output %d is not a tensor" % i)
        return v

    def done(self):
        return self._finished or self._pipe._poll(self)

    def result(self):
        self._pipe._wait(self)
        if self._released:
            raise InvalidArgumentError("the results of this call were released")
        n = len(self._outputs)
        return tuple(self._host.get(i) for i in range(n))

    def release(self):
        """Forgets the host results; their pinned blocks return to the pool
        once the caller has dropped its own references too.  The device
        handles (`input()`, `output()`) stay valid."""
        if self._released:
            return
        self._pipe._wait(self)
        self._released = True
        self._host = {}


class StagedPipeline:
    """Upload / compute / download pipeline for ops called with host tensors.

        pipe = StagedPipeline(depth=4)
        call = pipe.submit(raw_ops.FusedBatchNormV3, x_host, scale, offset, e, e, epsilon=1e-3)
        grad = pipe.submit(raw_ops.FusedBatchNormGradV3, dy_host, call.input(0), scale,
                           call.output(3), call.output(4), None, epsilon=1e-3)
        y, *_ = call.result()

    `depth` bounds the calls in flight (and with them the staging memory).
    Submission is thread-safe; results may be collected in any order.  Host
    sources may be pinned (copied by DMA straight from the caller's memory,
    which must stay untouched until the call is done) or pageable (staged
    through pinned chunks by the runtime, reusable as soon as submit returns).
    """

    def __init__(self, device=None, depth=4):
        _r._require_cuda()
        if depth < 1:
            raise InvalidArgumentError("depth must be at least 1")
        self.device = torch.device("cuda", torch.cuda.current_device() if device is None
                                   else torch.device(device).index or 0)
        self.ordinal = self.device.index
        self.depth = depth
        self._lib = _r._lib()
        self._check(self._lib.MusaRtCreateDevice(self.ordinal), "create_device")
        self._streams = []
        for _ in range(3):
            s = ctypes.c_void_p()
            self._check(self._lib.MusaRtCreateStream(self.ordinal, ctypes.byref(s)), "create_stream")
            self._streams.append(s)
        self._up, self._compute, self._down = self._streams
        self._compute_torch = torch.cuda.ExternalStream(
            self._lib.MusaRtRawStream(self._compute), device=self.device)
        self._pool = _DevicePool(self.device)
        self._inflight = collections.deque()
        self._lock = threading.RLock()
        self._closed = False
        self._alive = [True]     # shared with the finalizers of the host results
        self.stats = {"calls": 0, "h2d_bytes": 0, "d2h_bytes": 0, "retire_waits": 0}

    # ---- runtime plumbing ----
    def _check(self, rc, what):
        if rc != 0:
            raise InternalError("staging %s failed (%d): %s" % (
                what, rc, (self._lib.MusaRtLastError() or b"").decode()))

    def _event(self, call, stream):
        e = ctypes.c_void_p()
        self._check(self._lib.MusaRtCreateEvent(self.ordinal, ctypes.byref(e)), "create_event")
        call._events.append(e)
        self._check(self._lib.MusaRtRecordEvent(self.ordinal, stream, e), "record_event")
        return e

    def _pinned_tensor(self, nbytes, dtype, shape):
        """A host tensor in a pinned block of the runtime's pool; the block is
        freed when the tensor and all of its views are gone."""
        ptr = self._lib.MusaRtPinnedAllocate(self.ordinal, nbytes)
        if not ptr:
            raise InternalError("out of pinned staging memory (%d bytes)" % nbytes)
        block = (ctypes.c_char * nbytes).from_address(ptr)
        # The copy that filled the block is long done when the last reference
        # dies, but the free follows the download stream all the same.
        fin = weakref.finalize(block, _free_pinned_block, self._lib, self.ordinal, ptr, nbytes,
                               self._down, self._alive)
        fin.atexit = False
        return ptr, torch.frombuffer(block, dtype=dtype).view(shape)

    # ---- submission ----
    def _stage_in(self, call, arg):
        """-> (value for the op, StagedValue or None)."""
        if isinstance(arg, StagedValue):
            call._hold.append(arg)
            return arg.tensor, arg
        if isinstance(arg, np.ndarray):
            arg = _to_host_tensor(arg)
        if not isinstance(arg, torch.Tensor):
            return arg, None
        if arg.is_cuda:
            # A device tensor of the caller: whatever the caller's current
            # stream still has queued for it is ordered before this call.
            with torch.cuda.device(self.device):
                ready = torch.cuda.current_stream().record_event()
                self._compute_torch.wait_event(ready)
            call._hold.append(arg)
            return arg, StagedValue(arg, None)
        src = arg.contiguous()
        nbytes = src.numel() * src.element_size()
        lease = _Lease(self._pool, nbytes)
        dev = lease.buf[:nbytes].view(src.dtype).view(src.shape) if nbytes else \
            torch.empty(src.shape, dtype=src.dtype, device=self.device)
        if nbytes:
            self._check(self._lib.MusaRtMemcpyHtoD(self.ordinal, self._up, dev.data_ptr(),
                                                   src.data_ptr(), nbytes), "memcpy_htod")
            self.stats["h2d_bytes"] += nbytes
        value = StagedValue(dev, lease)
        call._hold.append(src)      # a pinned source is read by DMA until the call is done
        call._hold.append(value)
        return dev, value

    def submit(self, fn, *args, fetch=None, **kwargs):
        """Queues fn(*args, **kwargs).  Host tensors / arrays among the
        arguments are uploaded, StagedValues are used in place.  `fetch` lists
        the output indices to download (default: every tensor output)."""
        with self._lock:
            if self._closed:
                raise InvalidArgumentError("the pipeline is closed")
            self._retire(block=len(self._inflight) >= self.depth)
            call = StagedCall(self)
            try:
                dev_args = []
                for a in args:
                    v, handle = self._stage_in(call, a)
                    dev_args.append(v)
                    call._inputs.append(handle)
                dev_kwargs = {k: self._stage_in(call, v)[0] for k, v in kwargs.items()}
                uploaded = self._event(call, self._up)
                self._check(self._lib.MusaRtWaitForEvent(self.ordinal, self._compute, uploaded),
                            "wait_for_event")
                with torch.cuda.device(self.device), torch.cuda.stream(self._compute_torch):
                    outs = fn(*dev_args, **dev_kwargs)
                if outs is None:
                    outs = ()
                elif isinstance(outs, torch.Tensor):
                    outs = (outs,)
                computed = self._event(call, self._compute)
                self._check(self._lib.MusaRtWaitForEvent(self.ordinal, self._down, computed),
                            "wait_for_event")
                for i, o in enumerate(outs):
                    if isinstance(o, torch.Tensor) and o.is_cuda:
                        call._outputs.append(StagedValue(o, None))
                    else:
                        call._outputs.append(None)
                wanted = range(len(outs)) if fetch is None else fetch
                for i in wanted:
                    v = call._outputs[i]
                    if v is None:
                        continue
                    t = v.tensor.contiguous()
                    nbytes = t.numel() * t.element_size()
                    if nbytes == 0:
                        call._host[i] = torch.empty(t.shape, dtype=t.dtype)
                        continue
                    ptr, host = self._pinned_tensor(nbytes, t.dtype, t.shape)
                    call._host[i] = host
                    call._hold.append(t)
                    self._check(self._lib.MusaRtMemcpyDtoH(self.ordinal, self._down, ptr,
                                                           t.data_ptr(), nbytes), "memcpy_dtoh")
                    self.stats["d2h_bytes"] += nbytes
                call._done_event = self._event(call, self._down)
            except Exception:
                # Whatever was queued still runs: drain before the buffers go.
                for s in self._streams:
                    self._lib.MusaRtBlockHostUntilDone(self.ordinal, s)
                call._done_event = None
                call._host = {}
                self._finish(call)
                raise
            self._inflight.append(call)
            self.stats["calls"] += 1
            return call

    # ---- completion ----
    def _finish(self, call):
        if call._finished:
            return
        call._finished = True
        call._hold = []
        for e in call._events:
            self._lib.MusaRtDestroyEvent(self.ordinal, e)
        call._events = []

    def _poll(self, call):
        with self._lock:
            if call._finished:
                return True
            if self._lib.MusaRtGetEventStatus(self.ordinal, call._done_event) == 0:
                self._finish(call)
                return True
            return False

    def _wait(self, call):
        with self._lock:
            if not call._finished:
                self._check(self._lib.MusaRtBlockHostForEvent(self.ordinal, call._done_event),
                            "block_host_for_event")
                self._finish(call)
            self._retire(block=False)

    def _retire(self, block):
        """Drops finished calls from the head of the queue; with `block`, waits
        for the oldest one first."""
        if block and self._inflight:
            head = self._inflight[0]
            if not head._finished:
                self.stats["retire_waits"] += 1
                self._check(self._lib.MusaRtBlockHostForEvent(self.ordinal, head._done_event),
                            "block_host_for_event")
                self._finish(head)
        while self._inflight and (self._inflight[0]._finished or self._poll(self._inflight[0])):
            self._inflight.popleft()

    def synchronize(self):
        """Waits until every submitted call has finished."""
        with self._lock:
            while self._inflight:
                self._retire(block=True)

    def close(self):
        with self._lock:
            if self._closed:
                return
            self.synchronize()
            for s in self._streams:
                self._lib.MusaRtBlockHostUntilDone(self.ordinal, s)
                self._lib.MusaRtDestroyStream(self.ordinal, s)
            self._alive[0] = False
            self._closed = True

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()
        return False
