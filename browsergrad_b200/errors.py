"""Error types of the CUDA bridge, named after the reference's
(packages/browsergrad-kernels/src/types.ts:86-91 ``KernelError``;
packages/browsergrad-jit/src/python/_errors.py ``RealizationError`` / ``JitNotImplementedError`` /
``BufferTableError``)."""


class KernelError(RuntimeError):
    """Raised by a bridge method; the message starts with ``CUDA bridge: <op>``."""

    def __init__(self, message: str, status: int = 0) -> None:
        super().__init__(message)
        self.status = status


class RealizationError(RuntimeError):
    """Raised by the realizer front when a node cannot be realized."""


class JitNotImplementedError(NotImplementedError):
    """Raised for opcodes outside the forward path."""


class BufferTableError(RuntimeError):
    """Raised by the device buffer table for a buffer id that is registered twice or not at all."""
