"""Gradient allreduce for data-parallel training: flat buckets over NCCL, overlapped with compute.

Takes the place of hetr's GPU allreduce, CudaAllReduceKernel
(ngraph/transformers/gpu/tensor_ops.py:428-618): per gradient tensor, a reduce-scatter by
peer-to-peer memcpy into peer scratch, a float_accum kernel, an all-gather by peer-to-peer memcpy,
three MPI barriers and host synchronisations, with no overlap with back-propagation.

Here every tensor that goes through an allreduce lives inside one flat arena, cut into buckets of at
most `bucket_bytes` (25 MB by default; at least four buckets per step) in the order the tensors are produced.  When the last tensor
of a bucket has been produced, ONE collective is started for the whole bucket on the communication
stream (torch.distributed: NCCL over NVLink/NVSwitch on GPUs, gloo in CPU tests); the compute
stream only waits for it right before the first consumer of a reduced tensor, so the exchange
overlaps the remaining back-propagation.  `reduce_func` is 'sum' or 'mean' as in the reference's
kernel (tensor_ops.py:95-108).

One process per GPU; the process group is created by the caller (torchrun) and handed in.
"""
import datetime
import threading
import time

import numpy as np


class CommError(RuntimeError):
    """A collective failed or did not finish within its time limit (B2_ERR_COMM of the C ABI's
    error codes): a peer raised, left, or never joined.  The exchange state of the call is
    undefined afterwards; the computation's weights have not been updated with a partial sum."""


DEFAULT_BUCKET_BYTES = 25 * 1024 * 1024
DEFAULT_TIMEOUT_S = 120.0
ALIGN_ELEMS = 64          # every tensor starts on a 256-byte boundary inside the arena


class BucketPlan(object):
    """Assigns tensors (given in production order as (key, n_elements)) to arena offsets and
    buckets.  A tensor never straddles two buckets; a tensor larger than the limit gets a bucket
    of its own.  `bucket_bytes` is the upper bound of a bucket; `min_buckets` > 1 lowers the limit
    to an even share of the total, so that a small model (ResNet-20: 1.1 MB of gradients, far below
    25 MB) still exchanges in several pieces, each started as its last gradient lands, instead
    of in one piece after back-propagation has ended."""

    def __init__(self, sizes, bucket_bytes=DEFAULT_BUCKET_BYTES, itemsize=4, min_buckets=1):
        self.offsets = {}
        self.bucket_of = {}
        self.buckets = []          # (start_elem, end_elem, [keys])
        sizes = list(sizes)
        limit = max(1, int(bucket_bytes) // itemsize)
        if min_buckets > 1:
            total = sum(-(-int(n) // ALIGN_ELEMS) * ALIGN_ELEMS for _, n in sizes)
            limit = max(1, min(limit, -(-total // int(min_buckets))))
        cur_start, cur_end, cur_keys = 0, 0, []
        for key, n in sizes:
            n_pad = -(-int(n) // ALIGN_ELEMS) * ALIGN_ELEMS
            if cur_keys and (cur_end - cur_start) + n_pad > limit:
                self.buckets.append((cur_start, cur_end, cur_keys))
                cur_start, cur_keys = cur_end, []
            self.offsets[key] = cur_end
            self.bucket_of[key] = len(self.buckets)
            cur_keys.append(key)
            cur_end += n_pad
        if cur_keys:
            self.buckets.append((cur_start, cur_end, cur_keys))
        self.total = cur_end


class TorchDistComm(object):
    """Thin wrapper over an initialised torch.distributed process group."""

    def __init__(self, group=None, timeout_s=DEFAULT_TIMEOUT_S):
        """timeout_s: how long a collective may take before the wait gives up with CommError
        (a replica that raised or left never joins; without a limit the others wait for ever)."""
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised: launch one process per GPU "
                               "(torchrun) and call init_process_group first")
        self.dist = dist
        self.group = group
        self.rank = dist.get_rank(group)
        self.size = dist.get_world_size(group)
        self.timeout_s = float(timeout_s)

    def Get_rank(self):          # the reference passes an mpi4py-style comm (hetrtransform.py:38-57)
        return self.rank

    def Get_size(self):
        return self.size

    def all_reduce_async(self, flat, reduce_func="sum"):
        """Starts an in-place allreduce of a flat tensor; returns a handle with .wait()."""
        if reduce_func not in ("sum", "mean"):
            raise ValueError("unsupported reduce_func %r" % (reduce_func,))
        work = self.dist.all_reduce(flat, op=self.dist.ReduceOp.SUM, group=self.group,
                                    async_op=True)
        return _Pending(work, flat, self.size if reduce_func == "mean" else 1, self.timeout_s)


    def all_gather_host(self, array, axis):
        """Host arrays of all replicas joined along `axis` (every replica gets the whole)."""
        import torch
        t = torch.from_numpy(np.ascontiguousarray(array))
        if self.dist.get_backend(self.group) == "nccl":
            t = t.cuda()
        parts = [torch.empty_like(t) for _ in range(self.size)]
        self.dist.all_gather(parts, t, group=self.group)
        return np.concatenate([p.cpu().numpy() for p in parts], axis=axis)


class _Pending(object):
    def __init__(self, work, flat, divisor, timeout_s=DEFAULT_TIMEOUT_S):
        self.work, self.flat, self.divisor = work, flat, divisor
        self.timeout_s = timeout_s
        self.done = False

    def poll_error(self):
        """Raises CommError if the collective has failed so far; True once it has completed."""
        try:
            finished = self.work.is_completed()
        except RuntimeError as e:                     # the backend reports the failure by raising
            raise CommError("collective failed: %s" % e)
        exc = None
        if finished:
            try:
                exc = self.work.exception()
            except RuntimeError as e:
                raise CommError("collective failed: %s" % e)
            except TypeError:
                # the NCCL backend's work object cannot hand its (empty) exception slot to
                # Python; a failed NCCL collective raises from is_completed / wait instead
                exc = None
        if exc is not None:
            raise CommError("collective failed: %s" % (exc,))
        return finished

    def wait(self):
        """Makes the current stream wait for the collective (does not block the host on GPUs; on
        CPU tensors the host waits, at most timeout_s)."""
        if self.done:
            return
        try:
            if self.flat.is_cuda:
                # the device-side wait is queued; completion is checked, with the time limit, by
                # BucketedAllReduce.finish before the call's stream synchronisation
                self.work.wait()
            else:
                self.work.wait(datetime.timedelta(seconds=self.timeout_s))
        except RuntimeError as e:
            raise CommError("collective did not complete: %s" % e)
        if self.divisor != 1:
            self.flat.div_(self.divisor)
        self.done = True


class NcclComm(object):
    """The library's own communicator (C ABI: b2_comm_*): one NCCL communicator per process,
    collectives on a communication stream of its own, ordered against the compute stream by
    events, asynchronous NCCL errors polled instead of waited for.

    The 128-byte identifier made by replica 0 has to reach the others once; `exchange` is any
    callable (bytes or None) -> bytes that does that.  `from_torch_distributed` uses an already
    initialised torch.distributed group (any backend) for it."""
    capturable = True      # its collectives may be recorded into a CUDA graph with the step list

    def __init__(self, rank, size, device, exchange, timeout_s=DEFAULT_TIMEOUT_S):
        import ctypes as C
        import torch
        from . import lib
        self.lib, self.torch = lib, torch
        self.rank, self.size, self.device = int(rank), int(size), int(device)
        self.timeout_s = float(timeout_s)
        raw = lib.raw()
        ident = C.create_string_buffer(128)
        if self.rank == 0:
            lib.check(raw.b2_comm_unique_id(ident))
        blob = exchange(bytes(ident.raw) if self.rank == 0 else None)
        handle = C.c_void_p()
        torch.cuda.set_device(self.device)
        lib.check(raw.b2_comm_init(C.create_string_buffer(blob, 128), self.rank, self.size,
                                   self.device, C.byref(handle)))
        self.handle = handle
        self.stream = torch.cuda.Stream(device=self.device)
        # watchdog (see watch): armed between the launch of a step and its synchronisation
        self._deadline = None
        self._failed = None
        self._stop = threading.Event()
        self._watcher = None

    @classmethod
    def from_torch_distributed(cls, device, group=None, timeout_s=DEFAULT_TIMEOUT_S):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("torch.distributed is not initialised")

        def exchange(blob):
            box = [blob]
            dist.broadcast_object_list(box, src=0, group=group)
            return box[0]
        return cls(dist.get_rank(group), dist.get_world_size(group), device, exchange, timeout_s)

    def Get_rank(self):
        return self.rank

    def Get_size(self):
        return self.size

    def all_reduce_async(self, flat, reduce_func="sum"):
        if reduce_func not in ("sum", "mean"):
            raise ValueError("unsupported reduce_func %r" % (reduce_func,))
        torch = self.torch
        cur = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        self.stream.wait_event(ready)          # the bucket's producers have run
        rc = self.lib.raw().b2_comm_allreduce_f32(self.handle, flat.data_ptr(), flat.numel(),
                                                  int(reduce_func == "mean"),
                                                  self.stream.cuda_stream)
        if rc < 0:
            raise CommError(self.lib.raw().b2_last_error().decode(errors="replace"))
        done = torch.cuda.Event()
        done.record(self.stream)
        return _NcclPending(self, done)

    def poll_error(self):
        rc = self.lib.raw().b2_comm_poll_error(self.handle)
        if rc < 0:
            raise CommError(self.lib.raw().b2_last_error().decode(errors="replace"))

    # -- watchdog ----------------------------------------------------------------------------
    # The host must not sit in a stream synchronisation for ever when a replica has failed, and
    # it must not spin on the driver either while its own step runs (a query loop on the main
    # thread competes with the driver's work submission: measured 0.1 - 0.3 ms per 2.7 ms
    # training step on four GPUs).  So the main thread synchronises as usual and a background
    # thread looks at NCCL's asynchronous error state and at the clock every 20 ms; when a
    # collective has failed or the time limit has passed it aborts the communicator, which makes
    # the kernels in flight return, so the synchronisation ends and `unwatch` raises CommError.
    def watch(self, timeout_s=None):
        """Arms the watchdog for the collectives in flight (call before synchronising)."""
        if self._failed is not None:
            raise CommError(self._failed)
        if self._watcher is None:
            self._watcher = threading.Thread(target=self._watch_loop, name="b2-comm-watchdog",
                                             daemon=True)
            self._watcher.start()
        self._deadline = time.monotonic() + (self.timeout_s if timeout_s is None else timeout_s)

    def unwatch(self):
        """Disarms the watchdog (call after the synchronisation); CommError if it had to act."""
        self._deadline = None
        if self._failed is not None:
            raise CommError(self._failed)

    def _watch_loop(self):
        while not self._stop.wait(0.02):
            deadline = self._deadline
            if deadline is None or self.handle is None:
                continue
            reason = None
            try:
                self.poll_error()
            except CommError as e:
                reason = str(e)
            if reason is None and time.monotonic() > deadline:
                reason = ("a collective did not complete within its time limit: a replica has "
                          "failed or left")
            if reason is not None and self._deadline is not None:
                self._failed = reason
                self._deadline = None
                self.abort()

    def all_gather_host(self, array, axis):
        import torch.distributed as dist
        if not dist.is_initialized():
            raise RuntimeError("gathering results needs torch.distributed")
        return TorchDistComm(timeout_s=self.timeout_s).all_gather_host(array, axis)

    def abort(self):
        self.lib.raw().b2_comm_abort(self.handle)

    def close(self):
        self._stop.set()
        self._deadline = None
        if self._watcher is not None:
            self._watcher.join(timeout=1.0)
            self._watcher = None
        if self.handle is not None:
            self.lib.raw().b2_comm_destroy(self.handle)
            self.handle = None


class _NcclPending(object):
    def __init__(self, comm, done):
        self.comm, self.done_event = comm, done
        self.timeout_s = comm.timeout_s
        self.waited = False

    def wait(self):
        """The current stream waits for the collective; the host does not."""
        if not self.waited:
            self.comm.torch.cuda.current_stream(self.comm.device).wait_event(self.done_event)
            self.waited = True

    def poll_error(self):
        self.comm.poll_error()
        return self.done_event.query()


class SingleProcessComm(object):
    """World of one: the allreduce is the identity.  Lets a graph with allreduce ops run
    unchanged on a single GPU."""
    rank, size = 0, 1

    def Get_rank(self):
        return 0

    def Get_size(self):
        return 1

    def all_reduce_async(self, flat, reduce_func="sum"):
        if reduce_func not in ("sum", "mean"):
            raise ValueError("unsupported reduce_func %r" % (reduce_func,))
        return _Done()


    def all_gather_host(self, array, axis):
        return array


class _Done(object):
    def wait(self):
        return


class _InGraph(object):
    """Stands for the collectives a replayed CUDA graph holds."""
    poll_error = None


_IN_GRAPH = _InGraph()


class BucketedAllReduce(object):
    """Run-time state of the bucketed exchange for one computation.

    Tensors are produced in arena order.  A bucket's collective normally starts when its last
    tensor has been produced; if a consumer needs a reduced tensor earlier (an optimizer update
    whose result feeds the rest of back-propagation), the part of the bucket produced so far is
    exchanged at that point and the remainder later.  Every replica runs the same step list, so
    all of them issue the same sequence of collectives."""

    def __init__(self, comm, plan, arena, reduce_funcs):
        self.comm = comm
        self.plan = plan
        self.arena = arena                      # flat fp32 torch tensor of plan.total elements
        self.reduce_funcs = reduce_funcs        # key -> 'sum' | 'mean'
        self.sizes = {}
        for start, end, keys in plan.buckets:
            for i, k in enumerate(keys):
                nxt = plan.offsets[keys[i + 1]] if i + 1 < len(keys) else end
                self.sizes[k] = nxt - plan.offsets[k]
        self.started = 0
        self.last_sizes = []
        self._watched = False
        self.begin_call()

    def begin_call(self):
        self._sizes_now = []
        self.graph_handle = None
        self.pending = [[] for _ in self.plan.buckets]          # (start, end, handle)
        self.launched_upto = [b[0] for b in self.plan.buckets]
        self.produced_upto = [b[0] for b in self.plan.buckets]
        self.produced_keys = [[] for _ in self.plan.buckets]

    def produced(self, key):
        b = self.plan.bucket_of[key]
        self.produced_upto[b] = self.plan.offsets[key] + self.sizes[key]
        self.produced_keys[b].append(key)

    def flush(self, b):
        start, end = self.launched_upto[b], self.produced_upto[b]
        if end <= start:
            return
        funcs = set(self.reduce_funcs[k] for k in self.produced_keys[b]
                    if self.plan.offsets[k] >= start)
        if len(funcs) != 1:
            raise ValueError("tensors exchanged together must share a reduce_func")
        self.pending[b].append((start, end,
                                self.comm.all_reduce_async(self.arena[start:end], funcs.pop())))
        self._sizes_now.append(end - start)
        self.last_sizes = self._sizes_now       # elements per collective of the last exchanging call
        self.launched_upto[b] = end
        self.started += 1

    def bucket_ready(self, index):
        """All tensors of bucket `index` have been produced: exchange what is left of it."""
        self.flush(index)

    def join_all(self):
        """The current stream waits for every collective started in this call (the end of a CUDA
        graph recording: all forked streams have to be back)."""
        for bucket in self.pending:
            for _, _, handle in bucket:
                handle.wait()

    def graph_launched(self, stream):
        """A replayed graph held this call's collectives: `finish` has something to watch."""
        if hasattr(self.comm, "watch"):
            self.graph_handle = _IN_GRAPH
        else:
            event = self.comm.torch.cuda.Event()
            event.record(stream)
            self.graph_handle = _NcclPending(self.comm, event)

    def finish(self, timeout_s=None):
        """Before the call's stream synchronisation: every collective started in this call must
        complete within the time limit, else CommError (a synchronisation on a stream that waits
        for a collective nobody else joins would never return)."""
        handles = [h for bucket in self.pending for _, _, h in bucket if hasattr(h, "poll_error")]
        if self.graph_handle is not None:
            handles.append(self.graph_handle)
        if not handles:
            return
        if hasattr(self.comm, "watch"):
            # a communicator with a watchdog: the caller synchronises, the watchdog ends a
            # synchronisation that would not end by itself (after_sync reports it)
            self.comm.watch(timeout_s)
            self._watched = True
            return
        limit = handles[0].timeout_s if timeout_s is None else timeout_s
        start = time.monotonic()
        for h in handles:
            while not h.poll_error():
                waited = time.monotonic() - start
                if waited > limit:
                    raise CommError("a collective did not complete within %.1f s: a replica "
                                    "has failed or left" % limit)
                if waited > 0.05:
                    time.sleep(0.0005)      # a healthy step ends within the spinning phase

    def after_sync(self):
        """After the call's stream synchronisation: CommError if the watchdog had to end it."""
        if self._watched:
            self._watched = False
            self.comm.unwatch()

    def wait_for(self, key):
        """Called before the first consumer of the reduced tensor `key`.  A tensor that another
        computation exchanged (and finished with) needs no waiting here."""
        if key not in self.plan.bucket_of:
            return
        b = self.plan.bucket_of[key]
        off = self.plan.offsets[key]
        if off >= self.launched_upto[b]:
            self.flush(b)
        for start, end, handle in self.pending[b]:
            if start <= off < end:
                handle.wait()
