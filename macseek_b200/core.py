"""Stand-ins for the reference's core handles (src/core/metal.hpp:11-18,43-71): a Buffer is a torch CUDA tensor (a
sub-range is a slice), an Enc is a CUDA stream that work is enqueued on."""
import torch


class Enc:
    """One in-order CUDA stream.  barrier() is a no-op (the stream already orders dependent launches); wait() blocks
    until the enqueued work is done and raises if a kernel reported a device-side failure."""

    def __init__(self, stream=None):
        self.stream = stream if stream is not None else torch.cuda.current_stream()

    @property
    def handle(self):
        return self.stream.cuda_stream

    def barrier(self):
        return None

    def wait(self):
        from . import _lib
        self.stream.synchronize()
        st = _lib.device_status()
        if st:
            raise _lib.MsbError("device-side failure word = %d" % st)


def ptr(t, offset_bytes=0):
    """Device address of a tensor (or None -> 0)."""
    if t is None:
        return None
    assert t.is_cuda, "device tensor expected"
    return t.data_ptr() + offset_bytes
