"""Exception types of the library."""


class StreamEPError(RuntimeError):
    """Invalid use of the library or an unrecoverable runtime failure."""


class StreamEPTimeout(StreamEPError):
    """A bounded wait gave up: a device-side wait reported through the status
    block, or the host poll for dispatch metadata.  The CUDA context stays usable
    (the reference traps the device instead: csrc/kernels/intranode.cu:68-72,
    csrc/kernels/utils.cuh:643-646)."""


class StreamEPOverflow(StreamEPError):
    """A capacity-mode dispatch needed more pool tiles or recv tokens than the fixed regions hold on some rank.
    Every rank ran that dispatch as an empty one (outputs and gradients of that layer are zero); the step is
    invalid and the capacity factor has to be raised.  The reference is dropless by always sizing exactly, at the
    price of a host read per forward (csrc/stream_ep.cpp:741-759)."""
