"""Host logic of the device buffer table against a bridge that only counts: the methods and the error behaviour of
``GpuBufferTable`` (packages/browsergrad-jit/src/python/_gpu_buffer_table.py:63-113)."""
import numpy as np
import pytest

from browsergrad_b200.errors import BufferTableError
from browsergrad_b200.front import DeviceBufferTable


class CountingBridge:
    def __init__(self):
        self.next = 1
        self.alive = set()
        self.released = []

    def upload(self, array, shape, dtype):
        h = self.next
        self.next += 1
        self.alive.add(h)
        return h

    def release(self, handle):
        self.alive.discard(handle)
        self.released.append(handle)


def test_register_twice_raises_and_replace_releases_the_old_handle():
    bridge = CountingBridge()
    table = DeviceBufferTable(bridge)
    a = bridge.upload(None, (), "float32")
    b = bridge.upload(None, (), "float32")
    table.register("kv", a)
    assert table.has("kv") and table.get("kv") == a and not table.has("other") and table.get("other") is None
    with pytest.raises(BufferTableError):
        table.register("kv", b)
    assert table.get("kv") == a and bridge.released == []
    table.replace("kv", b)                       # the old handle is released, the id names the new one
    assert table.get("kv") == b and bridge.released == [a]
    table.replace("kv", b)                       # the same handle again: nothing is released
    assert bridge.released == [a]
    table.replace("fresh", a + 100)              # an unknown id is simply bound
    assert table.get("fresh") == a + 100


def test_detach_hands_the_handle_over_without_releasing_it():
    bridge = CountingBridge()
    table = DeviceBufferTable(bridge)
    h = table.upload("w", np.zeros(3, np.float32))
    assert table.upload("w", np.zeros(3, np.float32)) == h and table.stats() == {"resident": 1, "uploads": 1}
    assert table.detach("w") == h
    assert not table.has("w") and bridge.released == [] and h in bridge.alive
    with pytest.raises(BufferTableError):
        table.detach("w")
    table.release("w")                           # releasing an unknown id is a no-op, as in the reference
    table.register("x", h)
    table.release_all()
    assert bridge.released == [h] and table.stats()["resident"] == 0
