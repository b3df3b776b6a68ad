"""DistributedDataParallel communication hook: gradient buckets are averaged with the compressed
allreduce instead of NCCL.

    state = CompressedHookState(eb=1e-5, max_bucket_elems=...)
    ddp_model.register_comm_hook(state, compressed_allreduce_hook)

CUDA buckets run on a side stream (``state.stream``) so the collective of bucket k overlaps the
backward pass that fills bucket k+1.  The hook returns a CUDA-aware future whose result is set
under the side stream: the backward stream is never made to wait, only whoever consumes the bucket
(DDP's finalisation, through ``Future.wait``) is ordered behind the collective, and the host never
blocks.  ``state.check()`` reads the sticky device status (time-outs, missing peers) when the
trainer wants to know.  fp32 buckets only (the codec is fp32); other dtypes fall back to a plain
allreduce.  CPU buckets (gloo groups) go through the host-rank ring, which keeps the hook testable
without a GPU.  The reference ships the collective only; a trainer integration is the motivating
use case of its thesis (section 7.1), not part of its code.
"""
import torch
import torch.distributed as dist

from .comm import CompressedAllreduce
from .cpu_ring import cpu_compressed_allreduce


class CompressedHookState:
    def __init__(self, eb: float = 1e-5, max_bucket_elems: int = 8 * 1024 * 1024, group=None,
                 min_compress_elems: int = 4096):
        self.eb = float(eb)
        self.group = group
        self.max_bucket_elems = int(max_bucket_elems)
        self.min_compress_elems = int(min_compress_elems)
        self._ar = None
        self.stream = None
        self.calls = 0
        self.compressed_calls = 0

    def engine(self) -> CompressedAllreduce:
        if self._ar is None:
            self._ar = CompressedAllreduce(self.max_bucket_elems, group=self.group)
            self.stream = torch.cuda.Stream()
        return self._ar

    def check(self):
        """Synchronises and raises if a collective of this hook reported a device-side error
        (``kErrTimeout`` / ``kErrPeer`` / ``kErrCapacity``) since the last check."""
        if self._ar is not None:
            st = self._ar.status(clear=True)
            if st != 0:
                from .. import _lib

                raise _lib.HomCompError(st, "compressed gradient allreduce")

    def close(self):
        if self._ar is not None:
            self._ar.close()
            self._ar = None


def compressed_allreduce_hook(state: CompressedHookState, bucket: dist.GradBucket) -> torch.futures.Future[torch.Tensor]:
    buf = bucket.buffer()
    world = dist.get_world_size(state.group)
    state.calls += 1
    fut = torch.futures.Future()

    if buf.dtype != torch.float32 or buf.numel() < state.min_compress_elems or buf.numel() > state.max_bucket_elems:
        work = dist.all_reduce(buf, group=state.group, async_op=True)

        def done(_):
            return buf.div_(world)

        return work.get_future().then(lambda f: done(f))

    state.compressed_calls += 1
    if not buf.is_cuda:
        out = cpu_compressed_allreduce(buf.numpy(), state.eb, group=state.group)
        buf.copy_(torch.from_numpy(out)).div_(world)
        fut.set_result(buf)
        return fut

    return launch_bucket(state, buf, world)


def launch_bucket(state: CompressedHookState, buf: torch.Tensor, world: int) -> torch.futures.Future[torch.Tensor]:
    """Averages ``buf`` in place over the ranks on ``state.stream`` and returns a CUDA-aware future.
    The stream that calls this is not blocked: kernels queued on it afterwards run concurrently with
    the collective."""
    ar = state.engine()
    cur = torch.cuda.current_stream()
    state.stream.wait_stream(cur)  # the bucket's gradients are complete on the backward stream
    fut = torch.futures.Future(devices=[buf.device])
    with torch.cuda.stream(state.stream):
        ar.allreduce(buf, buf, state.eb)
        buf.div_(world)
        buf.record_stream(state.stream)
        # records an event on state.stream; Future.wait() / then() order their stream behind it
        fut.set_result(buf)
    return fut
