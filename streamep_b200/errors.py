"""Exception types of the library."""


class StreamEPError(RuntimeError):
    """Invalid use of the library or an unrecoverable runtime failure."""


class StreamEPTimeout(StreamEPError):
    """A bounded wait gave up: a device-side wait reported through the status
    block, or the host poll for dispatch metadata.  The CUDA context stays usable
    (the reference traps the device instead: csrc/kernels/intranode.cu:68-72,
    csrc/kernels/utils.cuh:643-646)."""
